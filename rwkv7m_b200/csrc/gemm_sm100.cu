// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with
// the fp32 accumulator in tensor memory -> tcgen05.ld epilogue.
//
// Persistent, warp-specialised CTA of 192 threads (one CTA per SM):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane)
//   warps 2..5  epilogue: each reads its 32-lane quarter of the accumulator
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue
// of tile i overlaps the main loop of tile i+1.  Operands may be K-major or
// MN-major in global memory; the three layouts cover y = x W^T, dx = dy W and
// dW = dy^T x without any transposition pass.  Every wait is bounded: when a
// limit runs out the CTA records an error code, drains and frees TMEM.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kEpiWarp0 = 2;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded mbarrier wait with an explicit suspend hint; gives up after ~2 s or when
// another role of this CTA already gave up.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(2000u)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u) {
      if (*abort_flag != 0) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
  return false;
}

// Activation of the kEpiStoreBf16 epilogue (act 1 = tanh, 2 = sigmoid) and the factor of the kEpiMulSqrt2Bf16 epilogue,
// the derivative of the producing activation expressed through its saved output h: act 0 = relu(.)^2 -> 2 sqrt(h),
// 1 = tanh -> 1 - h^2, 2 = sigmoid -> h (1 - h).
__device__ __forceinline__ float act_apply(float x, int act) {
  if (act == 1) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return __fdividef(1.f, 1.f + __expf(-x));
}
__device__ __forceinline__ float act_grad(float h, int act) {
  return act == 0 ? 2.f * sqrtf(h) : (act == 1 ? 1.f - h * h : h * (1.f - h));
}

// Write one 32-column chunk of an accumulator row (thread = row) with the selected epilogue.
template <int EPI>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], void* __restrict__ Dptr, int row, int col0, int M,
                                            int N, int ldd, bool atomic = false, const void* __restrict__ aux = nullptr,
                                            int ldaux = 0, int act = 0) {
  if (EPI == kEpiScatterAddBf16) {
    // Reduce-scatter over time fused into the epilogue: the row belongs to the rank that owns its time slice; the
    // partial result is added straight into that rank's output buffer (peer memory over NVLink, bf16x2 atomics).
    if (row < M && col0 + 32 <= N) {
      const GemmScatter* sc = reinterpret_cast<const GemmScatter*>(Dptr);
      const int T = sc->T, Tl = sc->Tl;
      const int bi = row / T, t = row - bi * T;
      const int owner = t / Tl;
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(sc->out[owner]) + ((size_t)bi * Tl + (t - owner * Tl)) * ldd + col0;
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        pk[j] = *reinterpret_cast<uint32_t*>(&h);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(out + 8 * j), "r"(pk[4 * j]),
                     "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]), "r"(pk[4 * j + 3])
                     : "memory");
    }
    return;
  }
  if (EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16) {
    // second input tile read with the same 16-byte pieces as the output is written
    if (row < M && col0 < N) {
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Dptr) + (size_t)row * ldd + col0;
      const __nv_bfloat16* ax = reinterpret_cast<const __nv_bfloat16*>(aux) + (size_t)row * ldaux + col0;
      if (col0 + 32 <= N) {
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) raw[j] = __ldg(reinterpret_cast<const uint4*>(ax) + j);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(raw);
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 hx = __bfloat1622float2(h2[j]);
          float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
          if (EPI == kEpiMulSqrt2Bf16) { x0 *= act_grad(hx.x, act); x1 *= act_grad(hx.y, act); }
          else { x0 += hx.x; x1 += hx.y; }
          __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
        for (int j = 0; j < 4; ++j) o4[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < N) {
            const float hx = __bfloat162float(ax[j]);
            float x0 = __uint_as_float(v[j]);
            x0 = EPI == kEpiMulSqrt2Bf16 ? x0 * act_grad(hx, act) : x0 + hx;
            out[j] = f2bf(x0);
          }
        }
      }
    }
    return;
  }
  if (row < M && col0 < N) {
          if (EPI == kEpiStoreBf16 || EPI == kEpiReluSqBf16) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Dptr) + (size_t)row * ldd + col0;
            if (col0 + 32 <= N) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
                if (EPI == kEpiReluSqBf16) { x0 = fmaxf(x0, 0.f); x0 *= x0; x1 = fmaxf(x1, 0.f); x1 *= x1; }
                else if (act != 0) { x0 = act_apply(x0, act); x1 = act_apply(x1, act); }
                __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
                pk[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
              for (int j = 0; j < 4; ++j) o4[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            } else {
              // ragged right edge: fully unrolled with a per-element guard so that v stays in registers
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x0 = __uint_as_float(v[j]);
                if (EPI == kEpiReluSqBf16) { x0 = fmaxf(x0, 0.f); x0 *= x0; }
                else if (act != 0) x0 = act_apply(x0, act);
                if (col0 + j < N) out[j] = f2bf(x0);
              }
            }
          } else {
            float* out = reinterpret_cast<float*>(Dptr) + (size_t)row * ldd + col0;
            if (EPI == kEpiAccumF32 && atomic) {
              // split-K: several CTAs hold partial sums of this tile
              if (col0 + 32 <= N) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + 4 * j),
                               "f"(__uint_as_float(v[4 * j])), "f"(__uint_as_float(v[4 * j + 1])),
                               "f"(__uint_as_float(v[4 * j + 2])), "f"(__uint_as_float(v[4 * j + 3]))
                               : "memory");
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < N) atomicAdd(out + j, __uint_as_float(v[j]));
              }
            } else if (col0 + 32 <= N) {
              float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 t = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                if (EPI == kEpiAccumF32) { float4 o = o4[j]; t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w; }
                o4[j] = t;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < N) {
                  float t = __uint_as_float(v[j]);
                  if (EPI == kEpiAccumF32) t += out[j];
                  out[j] = t;
                }
              }
            }
          }
        }
}

// Cross-entropy statistics of one output row over the columns of a tile (kEpiCeStats): the logits are rounded to bf16
// first, so the numbers equal those of a pass over a stored bf16 logits matrix, which the backward recomputes.
struct CeRow { float m, s, tl; int am; };

__device__ __forceinline__ void ce_row_update(CeRow& st, const uint32_t (&v)[32], int col0, int N, int tgt) {
  if (col0 >= N) return;
  float x[32];
  float cm = -INFINITY;
  int ci = col0;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float f = __bfloat162float(__float2bfloat16(__uint_as_float(v[j])));
    if (col0 + j >= N) f = -INFINITY;
    x[j] = f;
    if (f > cm) { cm = f; ci = col0 + j; }      // strict: the lowest column among equal values
    if (col0 + j == tgt) st.tl = f;
  }
  if (cm > st.m) { st.s *= __expf(st.m - cm); st.m = cm; st.am = ci; }   // first chunk: s = 0 and exp(-inf) = 0
#pragma unroll
  for (int j = 0; j < 32; ++j) st.s += __expf(x[j] - st.m);
}

// bf16 output through shared memory: the four epilogue warps write their 128 rows x 64 columns (two accumulator chunks
// per thread = 128 bytes = one row of the box) into a 16 KB staging buffer in the 128-byte-swizzled layout, and one
// thread hands the box to the copy engine (cp.async.bulk.tensor store), which writes full lines and clips at the matrix
// edge.  Two buffers alternate; the issuing thread lets the previous store finish reading its buffer before the barrier
// that precedes the next one, so a buffer is free again by the time the warps return to it.
constexpr int kOutStageBytes = 128 * 128;   // 128 rows x 64 bf16

__device__ __forceinline__ void epilogue_named_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// aux_row (two-input epilogues): this thread's 64 bf16 of the second input, or nullptr for a row past the matrix edge
template <int EPI>
__device__ __forceinline__ void stage_round(const uint32_t (&v0)[32], const uint32_t (&v1)[32], uint8_t* buf, int tile_row,
                                            int act, const __nv_bfloat16* aux_row) {
  uint32_t pk[32];
  uint4 raw[8];
  if (EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      raw[j] = aux_row != nullptr ? __ldg(reinterpret_cast<const uint4*>(aux_row) + j) : make_uint4(0u, 0u, 0u, 0u);
  }
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(raw);   // pairs 0-15: first chunk, 16-31: second
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float x0 = __uint_as_float(v0[2 * j]), x1 = __uint_as_float(v0[2 * j + 1]);
    float y0 = __uint_as_float(v1[2 * j]), y1 = __uint_as_float(v1[2 * j + 1]);
    if (EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16) {
      const float2 a = __bfloat1622float2(h2[j]), b = __bfloat1622float2(h2[16 + j]);
      if (EPI == kEpiMulSqrt2Bf16) {
        x0 *= act_grad(a.x, act); x1 *= act_grad(a.y, act); y0 *= act_grad(b.x, act); y1 *= act_grad(b.y, act);
      } else {
        x0 += a.x; x1 += a.y; y0 += b.x; y1 += b.y;
      }
    } else if (EPI == kEpiReluSqBf16) {
      x0 = fmaxf(x0, 0.f); x0 *= x0; x1 = fmaxf(x1, 0.f); x1 *= x1;
      y0 = fmaxf(y0, 0.f); y0 *= y0; y1 = fmaxf(y1, 0.f); y1 *= y1;
    } else if (act != 0) {
      x0 = act_apply(x0, act); x1 = act_apply(x1, act); y0 = act_apply(y0, act); y1 = act_apply(y1, act);
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1), g = __floats2bfloat162_rn(y0, y1);
    pk[j] = *reinterpret_cast<uint32_t*>(&h);
    pk[16 + j] = *reinterpret_cast<uint32_t*>(&g);
  }
  uint8_t* dst = buf + tile_row * 128;
  const int sw = tile_row & 7;   // 16-byte piece j of row r sits at piece j ^ (r mod 8)
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(dst + ((j ^ sw) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
  fence_proxy_async_smem();
}

// Tile order: blocks of kRasterM consecutive m-tiles sweep all n-tiles before the next block starts, so the
// CTAs that run at the same time share a few A row-panels and B column-panels and both stay in L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int raster_m, int& tm, int& tn) {
  const int group_size = raster_m * tiles_n;
  const int group = tile / group_size;
  const int first = group * raster_m;
  const int rows = min(raster_m, tiles_m - first);
  const int within = tile - group * group_size;
  tm = first + within % rows;
  tn = within / rows;
}

template <int BN>
struct Tile {
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = BN == 256 ? 512 : (BN == 128 ? 256 : 128);
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * 16384 /*output staging*/ + 1024 /*align slack*/ + 256 /*barriers*/;
};

template <int BN, int A_MN, int B_MN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, int tma_out,
                 void* __restrict__ Dptr, int M, int N, int K, int ldd, int raster_m, int splits,
                 const void* __restrict__ aux, int ldaux, int act, int* __restrict__ err) {
  using TL = Tile<BN>;
  constexpr int kStages = TL::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* out_stage = smem + kStages * TL::kStageBytes;   // 2 x 16 KB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * kOutStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K (accumulating epilogue only): work item w covers k-blocks [kb0, kb1) of tile w % num_tiles
  const int num_work = num_tiles * splits;
  const int kb_per = (num_kb + splits - 1) / splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); if (tma_out) tma_prefetch_desc(&tmD); }
  if (warp == 1) { tmem_alloc(tmem_slot, TL::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        const int tile = work % num_tiles, split = work / num_tiles;
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, raster_m, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = split * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_bar(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + stage * TL::kStageBytes;
          uint8_t* sb = sa + TL::kABytes;
          mbar_expect_tx(&full_bar[stage], TL::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[stage], m0 + 64 * c, k0);
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[stage], n0 + 64 * c, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x10000 | 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        if (!wait_bar(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = (work / num_tiles) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_bar(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * TL::kStageBytes);
          const uint32_t sb = sa + TL::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN == 0 ? umma_smem_desc_sw128(sa + k * 32, 16, 1024)
                                          : umma_smem_desc_sw128(sa + k * 2048, BK * 128, 1024);
            const uint64_t db = B_MN == 0 ? umma_smem_desc_sw128(sb + k * 32, 16, 1024)
                                          : umma_smem_desc_sw128(sb + k * 2048, BK * 128, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x10000 | 2); }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    const bool atomic = splits > 1;
    constexpr bool kTwoInput = EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16;
    constexpr bool kCanStage = (EPI == kEpiStoreBf16 || EPI == kEpiReluSqBf16 || kTwoInput) && BN >= 64;
    const bool staged = kCanStage && tma_out != 0;
    const bool issuer = warp == 2 && lane == 0;   // the one thread whose bulk groups track the output stores
    int obuf = 0;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      int tm, tn;
      tile_coords(work % num_tiles, tiles_m, tiles_n, raster_m, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      if (!wait_bar(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      if constexpr (EPI == kEpiCeStats) {
        CeRow st{-INFINITY, 0.f, -INFINITY, 0};
        const int tgt = row < M ? reinterpret_cast<const int*>(aux)[row] : -1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(t0 + c * 32, v0);
          tmem_ld_32x32(t0 + c * 32 + 32, v1);
          tmem_ld_wait();
          ce_row_update(st, v0, n0 + c * 32, N, tgt);
          ce_row_update(st, v1, n0 + c * 32 + 32, N, tgt);
        }
        if (row < M)
          reinterpret_cast<float4*>(Dptr)[(size_t)row * (ldd / 4) + tn] = make_float4(st.m, st.s, __int_as_float(st.am), st.tl);
      } else if constexpr (BN >= 64) {
        // two 32-column chunks per round: the second load is in flight while the first chunk is converted and stored
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(t0 + c * 32, v0);
          tmem_ld_32x32(t0 + c * 32 + 32, v1);
          tmem_ld_wait();
          if (kCanStage && staged) {
            if (n0 + c * 32 < N) {   // same for all 128 threads
              uint8_t* buf = out_stage + obuf * kOutStageBytes;
              const __nv_bfloat16* ax = nullptr;   // the host stages two-input epilogues only when N is a multiple of 64
              if (kTwoInput && row < M) ax = reinterpret_cast<const __nv_bfloat16*>(aux) + (size_t)row * ldaux + n0 + c * 32;
              stage_round<EPI>(v0, v1, buf, q * 32 + lane, act, ax);
              if (issuer) tma_store_wait_read<0>();
              epilogue_named_barrier();
              if (issuer) { tma_store_2d(&tmD, buf, n0 + c * 32, m0); tma_store_commit(); }
              obuf ^= 1;
            }
          } else {
            store_chunk<EPI>(v0, Dptr, row, n0 + c * 32, M, N, ldd, atomic, aux, ldaux, act);
            store_chunk<EPI>(v1, Dptr, row, n0 + c * 32 + 32, M, N, ldd, atomic, aux, ldaux, act);
          }
        }
      } else {
        uint32_t v[32];
        tmem_ld_32x32(t0, v);
        tmem_ld_wait();
        store_chunk<EPI>(v, Dptr, row, n0, M, N, ldd, atomic, aux, ldaux, act);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    if (staged && issuer) tma_store_wait<0>();   // the staging buffers are read until the last store has drained
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 0x10000 | 3); }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // give copies and MMAs that were already issued time to land before TMEM/smem are released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) { }
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TL::kTmemCols); }
}

// ---------------------------------------------------------------------------------------------
// Grouped variant: up to four y_i = act_i(x_i W_i^T) problems with the same number of rows in one persistent launch
// (layout TN, bf16 store epilogue).  The low-rank pairs of the time-mix block are four skinny GEMMs of 30-40 us each; one
// launch walks the tiles of all of them (problem after problem), so there is one ramp-up and one tail instead of four
// and the short problems fill the SMs that the tail of a longer one leaves idle.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxGroup = 4;
struct GroupProblem {
  void* D;
  int N, K, ldd, act;
  int tiles_n, tile_begin, tma_out, pad;
};
struct GroupParams {
  CUtensorMap tmA[kMaxGroup];
  CUtensorMap tmB[kMaxGroup];
  CUtensorMap tmD[kMaxGroup];
  GroupProblem pr[kMaxGroup];
  int count, M, total_tiles, raster_m;
};

__device__ __forceinline__ int group_find(const GroupParams& g, int work) {
  int p = 0;
#pragma unroll
  for (int i = 1; i < kMaxGroup; ++i)
    if (i < g.count && work >= g.pr[i].tile_begin) p = i;
  return p;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_group_kernel(const __grid_constant__ GroupParams g, int* __restrict__ err) {
  using TL = Tile<BN>;
  constexpr int kStages = TL::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* out_stage = smem + kStages * TL::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * kOutStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = g.M;
  const int tiles_m = (M + BM - 1) / BM;
  const int num_work = g.total_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < g.count; ++i) {
      tma_prefetch_desc(&g.tmA[i]); tma_prefetch_desc(&g.tmB[i]);
      if (g.pr[i].tma_out) tma_prefetch_desc(&g.tmD[i]);
    }
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TL::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        const int p = group_find(g, work);
        int tm, tn;
        tile_coords(work - g.pr[p].tile_begin, tiles_m, g.pr[p].tiles_n, g.raster_m, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int num_kb = (g.pr[p].K + BK - 1) / BK;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bar(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + stage * TL::kStageBytes;
          uint8_t* sb = sa + TL::kABytes;
          mbar_expect_tx(&full_bar[stage], TL::kStageBytes);
          tma_load_2d(sa, &g.tmA[p], &full_bar[stage], kb * BK, m0);
          tma_load_2d(sb, &g.tmB[p], &full_bar[stage], kb * BK, n0);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x10000 | 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
        const int num_kb = (g.pr[group_find(g, work)].K + BK - 1) / BK;
        if (!wait_bar(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bar(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * TL::kStageBytes);
          const uint32_t sb = sa + TL::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(d_tmem, umma_smem_desc_sw128(sa + k * 32, 16, 1024), umma_smem_desc_sw128(sb + k * 32, 16, 1024), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x10000 | 2); }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    const bool issuer = warp == 2 && lane == 0;
    bool stored = false;
    int obuf = 0;
    for (int work = blockIdx.x; work < num_work && ok; work += gridDim.x) {
      const int p = group_find(g, work);
      const GroupProblem pr = g.pr[p];
      int tm, tn;
      tile_coords(work - pr.tile_begin, tiles_m, pr.tiles_n, g.raster_m, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      if (!wait_bar(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c += 2) {
        if (n0 + c * 32 >= pr.N) break;   // the same for all 128 threads: nothing of this tile lies further right
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(t0 + c * 32, v0);
        tmem_ld_32x32(t0 + c * 32 + 32, v1);
        tmem_ld_wait();
        if (pr.tma_out) {
          uint8_t* buf = out_stage + obuf * kOutStageBytes;
          stage_round<kEpiStoreBf16>(v0, v1, buf, q * 32 + lane, pr.act, nullptr);
          if (issuer) tma_store_wait_read<0>();
          epilogue_named_barrier();
          if (issuer) { tma_store_2d(&g.tmD[p], buf, n0 + c * 32, m0); tma_store_commit(); stored = true; }
          obuf ^= 1;
        } else {
          store_chunk<kEpiStoreBf16>(v0, pr.D, row, n0 + c * 32, M, pr.N, pr.ldd, false, nullptr, 0, pr.act);
          store_chunk<kEpiStoreBf16>(v1, pr.D, row, n0 + c * 32 + 32, M, pr.N, pr.ldd, false, nullptr, 0, pr.act);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    if (stored) tma_store_wait<0>();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 0x10000 | 3); }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) { }
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TL::kTmemCols); }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster compute one 256 x 256 tile with tcgen05.mma.cta_group::2.
// Each CTA loads only its own 128 rows of A and 128 columns of B per k-block (32 KB instead of the
// 48 KB a lone 128 x 256 CTA needs for the same FLOPs) and keeps the 128 x 256 half of the accumulator
// that belongs to its rows in its own tensor memory.  The even CTA of the pair ("leader") owns the
// full-stage barriers and issues every MMA; completions are signalled to both CTAs.
//   full[s]   leader only, count 1 (leader's expect_tx) + bytes of both CTAs' TMA loads
//   empty[s]  one per CTA, count 1 (commit from the leader's MMA thread, delivered to both CTAs)
//   tfull[a]  one per CTA, count 1 (same mechanism)
//   tempty[a] leader only, count 8 (4 epilogue warps of each CTA; the peer's arrive remotely)
// ---------------------------------------------------------------------------------------------
struct PairTile {
  static constexpr int kStages = 6;
  static constexpr int kABytes = BM * BK * 2;        // this CTA's 128 rows of A
  static constexpr int kBBytes = 128 * BK * 2;       // this CTA's 128 columns of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 512;              // two 256-column accumulators
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * 16384 /*output staging*/ + 1024 + 256;
};

template <int A_MN, int B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmD, int tma_out,
                      void* __restrict__ Dptr, int M, int N, int K, int ldd, int raster_m, int splits,
                      const void* __restrict__ aux, int ldaux, int act, int* __restrict__ err) {
  using TL = PairTile;
  constexpr int kStages = TL::kStages;
  constexpr int BN2 = 256;  // tile width of the pair
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* out_stage = smem + kStages * TL::kStageBytes;   // 2 x 16 KB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * kOutStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const bool leader = cta == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K (accumulating epilogue only): work item w covers k-blocks [kb0, kb1) of tile w % num_tiles, so the pairs
  // that run at the same time work on the same k-range of different tiles and share operand panels in L2
  const int num_work = num_tiles * splits;
  const int kb_per = (num_kb + splits - 1) / splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); if (tma_out) tma_prefetch_desc(&tmD); }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TL::kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int work = pair_id; work < num_work && ok; work += num_pairs) {
        const int tile = work % num_tiles, split = work / num_tiles;
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, raster_m, tm, tn);
        const int m0 = tm * 2 * BM + (int)cta * BM;   // this CTA's rows
        const int n0 = tn * BN2 + (int)cta * 128;     // this CTA's columns of B
        const int kb0 = split * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_bar(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + stage * TL::kStageBytes;
          uint8_t* sb = sa + TL::kABytes;
          // completion of both CTAs' copies is counted on the leader's barrier
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * TL::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tmA, bar, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (BK * 128), &tmA, bar, m0 + 64 * c, k0);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sb, &tmB, bar, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sb + c * (BK * 128), &tmB, bar, n0 + 64 * c, k0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x30000 | 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN2, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = pair_id; work < num_work && ok; work += num_pairs) {
        if (!wait_bar(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        const int kb0 = (work / num_tiles) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_bar(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * TL::kStageBytes);
          const uint32_t sb = sa + TL::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN == 0 ? umma_smem_desc_sw128(sa + k * 32, 16, 1024)
                                          : umma_smem_desc_sw128(sa + k * 2048, BK * 128, 1024);
            const uint64_t db = B_MN == 0 ? umma_smem_desc_sw128(sb + k * 32, 16, 1024)
                                          : umma_smem_desc_sw128(sb + k * 2048, BK * 128, 1024);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc], 3);
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x30000 | 2); }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows x 256 columns) ----------------
    const int q = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    constexpr bool kTwoInput = EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16;
    constexpr bool kCanStage = EPI == kEpiStoreBf16 || EPI == kEpiReluSqBf16 || kTwoInput;
    const bool staged = kCanStage && tma_out != 0;
    const bool issuer = warp == 2 && lane == 0;
    int obuf = 0;
    const bool atomic = splits > 1;
    for (int work = pair_id; work < num_work && ok; work += num_pairs) {
      int tm, tn;
      tile_coords(work % num_tiles, tiles_m, tiles_n, raster_m, tm, tn);
      const int m0 = tm * 2 * BM + (int)cta * BM, n0 = tn * BN2;
      if (!wait_bar(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16) + acc * BN2;
      if constexpr (EPI == kEpiCeStats) {
        CeRow st{-INFINITY, 0.f, -INFINITY, 0};
        const int tgt = row < M ? reinterpret_cast<const int*>(aux)[row] : -1;
#pragma unroll 1
        for (int c = 0; c < BN2 / 32; c += 2) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(t0 + c * 32, v0);
          tmem_ld_32x32(t0 + c * 32 + 32, v1);
          tmem_ld_wait();
          ce_row_update(st, v0, n0 + c * 32, N, tgt);
          ce_row_update(st, v1, n0 + c * 32 + 32, N, tgt);
        }
        if (row < M)
          reinterpret_cast<float4*>(Dptr)[(size_t)row * (ldd / 4) + tn] = make_float4(st.m, st.s, __int_as_float(st.am), st.tl);
      } else
#pragma unroll 1
      for (int c = 0; c < BN2 / 32; c += 2) {   // two chunks per round: the second load overlaps the first chunk's stores
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(t0 + c * 32, v0);
        tmem_ld_32x32(t0 + c * 32 + 32, v1);
        tmem_ld_wait();
        if (kCanStage && staged) {
          if (n0 + c * 32 < N && m0 < M) {   // same for all 128 threads
            uint8_t* buf = out_stage + obuf * kOutStageBytes;
            const __nv_bfloat16* ax = nullptr;
            if (kTwoInput && row < M) ax = reinterpret_cast<const __nv_bfloat16*>(aux) + (size_t)row * ldaux + n0 + c * 32;
            stage_round<EPI>(v0, v1, buf, q * 32 + lane, act, ax);
            if (issuer) tma_store_wait_read<0>();
            epilogue_named_barrier();
            if (issuer) { tma_store_2d(&tmD, buf, n0 + c * 32, m0); tma_store_commit(); }
            obuf ^= 1;
          }
        } else {
          store_chunk<EPI>(v0, Dptr, row, n0 + c * 32, M, N, ldd, atomic, aux, ldaux, act);
          store_chunk<EPI>(v1, Dptr, row, n0 + c * 32 + 32, M, N, ldd, atomic, aux, ldaux, act);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
    if (staged && issuer) tma_store_wait<0>();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 0x30000 | 3); }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) { }
    __syncthreads();
  }
  cluster_sync_all();  // neither CTA leaves while the other may still signal into its shared memory
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TL::kTmemCols); }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr; int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull + (size_t)k.cols * 0xC2B2AE3D27D4EB4Full;
    h ^= ((size_t)k.ld << 20) ^ (size_t)k.box_rows;
    return h;
  }
};

// Row-major bf16 matrix [rows, cols] with leading dimension ld; box = 64 columns x box_rows rows, 128B swizzle.
// The cache stores the 128 descriptor bytes as a plain byte array: CUtensorMap is 64-byte aligned and
// node-based containers do not honour that alignment under every host compiler configuration.
struct MapBytes { unsigned char raw[sizeof(CUtensorMap)]; };

bool make_map(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::unordered_map<MapKey, MapBytes, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { memcpy(out, it->second.raw, sizeof(CUtensorMap)); return true; }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  // The driver entry point needs the primary context bound to the calling thread.  A worker
  // thread (e.g. an autograd thread) whose first CUDA action is this call has none yet.
  // Done once per thread, so later calls are legal while a stream of this thread is being captured into a graph.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)
      return false;
    context_bound = true;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  MapBytes mb;
  memcpy(mb.raw, out, sizeof(CUtensorMap));
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache[key] = mb;
  return true;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Height (in m-tiles) of the raster groups; RWKV7M_B200_GEMM_RASTER overrides the default for experiments.
int raster_rows(const GemmArgs& p) {
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("RWKV7M_B200_GEMM_RASTER"); forced = e != nullptr ? atoi(e) : 0; }
  if (forced > 0) return forced;
  (void)p;
  return 16;
}

// RWKV7M_B200_GEMM_TMA_STORE=0 keeps the per-thread 16-byte stores of the bf16 epilogues (for comparisons).
bool tma_store_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("RWKV7M_B200_GEMM_TMA_STORE"); on = (e != nullptr && e[0] == '0') ? 0 : 1; }
  return on == 1;
}

// RWKV7M_B200_GEMM_PAIR_SPLITK=0 keeps one CTA pair per output tile of the accumulating epilogue (for comparisons).
bool pair_splitk_enabled() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("RWKV7M_B200_GEMM_PAIR_SPLITK"); on = (e != nullptr && e[0] == '0') ? 0 : 1; }
  return on == 1;
}

#define RK_TRACE(...) do { if (trace_on()) { fprintf(stderr, "[gemm] " __VA_ARGS__); fflush(stderr); } } while (0)
bool trace_on() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("RWKV7M_B200_TRACE"); on = (e != nullptr && e[0] == '1') ? 1 : 0; }
  return on == 1;
}

template <int BN, int A_MN, int B_MN, int EPI>
int launch(const GemmArgs& p, cudaStream_t st) {
  using TL = Tile<BN>;
  RK_TRACE("launch BN=%d A_MN=%d B_MN=%d EPI=%d M=%d N=%d K=%d lda=%d ldb=%d ldd=%d A=%p B=%p D=%p err=%p\n", BN, A_MN,
           B_MN, EPI, p.M, p.N, p.K, p.lda, p.ldb, p.ldd, p.A, p.B, p.D, (void*)p.error_flag);
  alignas(64) CUtensorMap ta;
  alignas(64) CUtensorMap tb;
  bool ok;
  if (A_MN == 0) ok = make_map(&ta, p.A, p.M, p.K, p.lda, BM); else ok = make_map(&ta, p.A, p.K, p.M, p.lda, BK);
  if (!ok) return 2;
  if (B_MN == 0) ok = make_map(&tb, p.B, p.N, p.K, p.ldb, BN); else ok = make_map(&tb, p.B, p.K, p.N, p.ldb, BK);
  if (!ok) return 2;
  // bf16 store epilogues hand finished boxes to the copy engine when the output rows are 16-byte aligned
  alignas(64) CUtensorMap td = ta;
  int tma_out = 0;
  constexpr bool kTwoInput = EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16;
  if ((EPI == kEpiStoreBf16 || EPI == kEpiReluSqBf16 || kTwoInput) && BN >= 64 && tma_store_enabled() &&
      (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 && p.ldd % 8 == 0 &&
      (!kTwoInput || (p.N % 64 == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0 && p.ldaux % 8 == 0)))
    tma_out = make_map(&td, p.D, p.M, p.N, p.ldd, BM) ? 1 : 0;
  RK_TRACE("maps ok\n");
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::kSmemBytes) != cudaSuccess) return 3;
    attr_set = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  // split-K: a weight gradient with few output tiles and a long reduction (LoRA factors, K = tokens) would leave most
  // SMs idle; the accumulating epilogue lets several CTAs add their partial sums to the same tile
  int splits = 1;
  if (EPI == kEpiAccumF32 && tiles * 2 <= sm_count()) {
    const int num_kb = (p.K + BK - 1) / BK;
    splits = sm_count() / tiles;
    if (splits > num_kb / 8) splits = num_kb / 8;
    if (splits < 1) splits = 1;
    const int per = (num_kb + splits - 1) / splits;
    splits = (num_kb + per - 1) / per;   // no empty split
  }
  const int work = tiles * splits;
  const int grid = work < sm_count() ? work : sm_count();
  RK_TRACE("attr ok grid=%d smem=%d splits=%d\n", grid, TL::kSmemBytes, splits);
  kern<<<grid, kThreads, TL::kSmemBytes, st>>>(ta, tb, td, tma_out, p.D, p.M, p.N, p.K, p.ldd, raster_rows(p), splits, p.aux,
                                               p.ldaux, p.act, p.error_flag);
  RK_TRACE("launched\n");
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <int BN, int A_MN, int B_MN>
int launch_epi(const GemmArgs& p, cudaStream_t st) {
  switch (p.epilogue) {
    case kEpiStoreBf16: return launch<BN, A_MN, B_MN, kEpiStoreBf16>(p, st);
    case kEpiReluSqBf16: return launch<BN, A_MN, B_MN, kEpiReluSqBf16>(p, st);
    case kEpiStoreF32: return launch<BN, A_MN, B_MN, kEpiStoreF32>(p, st);
    case kEpiAccumF32: return launch<BN, A_MN, B_MN, kEpiAccumF32>(p, st);
    case kEpiMulSqrt2Bf16: return launch<BN, A_MN, B_MN, kEpiMulSqrt2Bf16>(p, st);
    case kEpiAddBf16: return launch<BN, A_MN, B_MN, kEpiAddBf16>(p, st);
  }
  return 5;
}

template <int BN>
int launch_layout(const GemmArgs& p, cudaStream_t st) {
  switch (p.layout) {
    case kGemmTN: return launch_epi<BN, 0, 0>(p, st);
    case kGemmNN: return launch_epi<BN, 0, 1>(p, st);
    case kGemmNT_wgrad: return launch_epi<BN, 1, 1>(p, st);
  }
  return 5;
}

template <int BN>
int launch_group(const GemmArgs* ps, int count, cudaStream_t st) {
  using TL = Tile<BN>;
  alignas(64) GroupParams g;
  memset(&g, 0, sizeof(g));
  g.count = count;
  g.M = ps[0].M;
  g.raster_m = raster_rows(ps[0]);
  const int tiles_m = (g.M + BM - 1) / BM;
  int total = 0;
  for (int i = 0; i < count; ++i) {
    const GemmArgs& p = ps[i];
    if (!make_map(&g.tmA[i], p.A, p.M, p.K, p.lda, BM)) return 2;
    if (!make_map(&g.tmB[i], p.B, p.N, p.K, p.ldb, BN)) return 2;
    g.tmD[i] = g.tmA[i];
    GroupProblem& q = g.pr[i];
    q.D = p.D; q.N = p.N; q.K = p.K; q.ldd = p.ldd; q.act = p.act;
    q.tiles_n = (p.N + BN - 1) / BN;
    q.tile_begin = total;
    q.tma_out = 0;
    if (tma_store_enabled() && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 && p.ldd % 8 == 0)
      q.tma_out = make_map(&g.tmD[i], p.D, p.M, p.N, p.ldd, BM) ? 1 : 0;
    total += tiles_m * q.tiles_n;
  }
  for (int i = count; i < kMaxGroup; ++i) { g.tmA[i] = g.tmA[0]; g.tmB[i] = g.tmB[0]; g.tmD[i] = g.tmD[0]; g.pr[i].tile_begin = total; }
  g.total_tiles = total;
  auto kern = gemm_bf16_group_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::kSmemBytes) != cudaSuccess) return 3;
    attr_set = true;
  }
  const int grid = total < sm_count() ? total : sm_count();
  kern<<<grid, kThreads, TL::kSmemBytes, st>>>(g, ps[0].error_flag);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <int A_MN, int B_MN, int EPI>
int launch_pair(const GemmArgs& p, cudaStream_t st) {
  using TL = PairTile;
  alignas(64) CUtensorMap ta;
  alignas(64) CUtensorMap tb;
  bool ok;
  if (A_MN == 0) ok = make_map(&ta, p.A, p.M, p.K, p.lda, BM); else ok = make_map(&ta, p.A, p.K, p.M, p.lda, BK);
  if (!ok) return 2;
  if (B_MN == 0) ok = make_map(&tb, p.B, p.N, p.K, p.ldb, 128); else ok = make_map(&tb, p.B, p.K, p.N, p.ldb, BK);
  if (!ok) return 2;
  alignas(64) CUtensorMap td = ta;
  int tma_out = 0;
  constexpr bool kTwoInput = EPI == kEpiMulSqrt2Bf16 || EPI == kEpiAddBf16;
  if ((EPI == kEpiStoreBf16 || EPI == kEpiReluSqBf16 || kTwoInput) && tma_store_enabled() &&
      (reinterpret_cast<uintptr_t>(p.D) & 15) == 0 && p.ldd % 8 == 0 &&
      (!kTwoInput || (p.N % 64 == 0 && (reinterpret_cast<uintptr_t>(p.aux) & 15) == 0 && p.ldaux % 8 == 0)))
    tma_out = make_map(&td, p.D, p.M, p.N, p.ldd, BM) ? 1 : 0;
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL::kSmemBytes) != cudaSuccess) return 3;
    attr_set = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256);
  const int max_pairs = sm_count() / 2;
  // split-K for the accumulating epilogue: a weight gradient has few tiles and a long reduction, and 64 or 256 tiles
  // on 74 pairs leave the last wave of tiles mostly idle.  The split count that minimises waves / splits wins (ties
  // to the smaller count: every split adds one pass of atomic adds over the output).
  int splits = 1;
  if (EPI == kEpiAccumF32 && pair_splitk_enabled()) {
    const int num_kb = (p.K + BK - 1) / BK;
    double best = (double)((tiles + max_pairs - 1) / max_pairs);
    for (int s = 2; s <= 8 && num_kb / s >= 32; ++s) {
      const double cost = (double)((tiles * s + max_pairs - 1) / max_pairs) / s;
      if (cost < best * 0.97) { best = cost; splits = s; }
    }
    const int per = (num_kb + splits - 1) / splits;
    splits = (num_kb + per - 1) / per;   // no empty split
  }
  const int work = tiles * splits;
  const int pairs = work < max_pairs ? work : max_pairs;
  kern<<<2 * pairs, kThreads, TL::kSmemBytes, st>>>(ta, tb, td, tma_out, p.D, p.M, p.N, p.K, p.ldd, raster_rows(p), splits,
                                                    p.aux, p.ldaux, p.act, p.error_flag);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <int A_MN, int B_MN>
int launch_pair_epi(const GemmArgs& p, cudaStream_t st) {
  switch (p.epilogue) {
    case kEpiStoreBf16: return launch_pair<A_MN, B_MN, kEpiStoreBf16>(p, st);
    case kEpiReluSqBf16: return launch_pair<A_MN, B_MN, kEpiReluSqBf16>(p, st);
    case kEpiStoreF32: return launch_pair<A_MN, B_MN, kEpiStoreF32>(p, st);
    case kEpiAccumF32: return launch_pair<A_MN, B_MN, kEpiAccumF32>(p, st);
    case kEpiMulSqrt2Bf16: return launch_pair<A_MN, B_MN, kEpiMulSqrt2Bf16>(p, st);
    case kEpiAddBf16: return launch_pair<A_MN, B_MN, kEpiAddBf16>(p, st);
  }
  return 5;
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode-sized GEMM: y[M <= 64, N] = x[M, K] W[N, K]^T, the shape of every projection of a T = 1 serving step.  The work
// is streaming the weight matrix once, and with one m-tile a long reduction is a serial chain of dependent MMAs, so the
// roles of the operands are swapped and the reduction is split: a CTA takes 128 rows of W as the 128-row tensor-core
// operand, the (zero-padded) 64 activation rows as the 64-column operand and one slice of K; the CTAs that share an
// n-tile form a thread-block cluster (up to 8) and meet their partial sums through distributed shared memory: every
// CTA parks its fp32 tile in its own shared memory, and after a cluster barrier CTA r sums rows [r 64/S, (r+1) 64/S)
// over all members, applies the epilogue (activation, relu^2 or the second input) and writes bf16.  No global
// workspace, no atomics, and no CTA spins on another one (cluster barriers are hardware barriers between co-scheduled
// CTAs).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kDecStages = 4;
constexpr int kDecWBytes = 128 * BK * 2, kDecXBytes = 64 * BK * 2, kDecStageBytes = kDecWBytes + kDecXBytes;
constexpr int kDecSmemBytes = kDecStages * kDecStageBytes + 1024 + 256;
constexpr int kDecRStride = 132;   // floats per activation row of the parked tile [64][128]
static_assert(64 * kDecRStride * 4 <= kDecStages * kDecStageBytes, "the parked tile reuses the pipeline stages");

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads, 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   __nv_bfloat16* __restrict__ out, int ldd, const __nv_bfloat16* __restrict__ aux, int ldaux, int M, int N,
                   int K, int kb_per, int splits, int epi, int act, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDecStages * kDecStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kDecStages;
  uint64_t* tfull_bar = bars + 2 * kDecStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kDecStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* R = reinterpret_cast<float*>(smem);     // parked partial tile, valid once this CTA's MMAs have completed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = blockIdx.x / splits, split = blockIdx.x - tn * splits;   // consecutive CTAs = one cluster = one n-tile
  const int n0 = tn * 128;
  const int num_kb = (K + BK - 1) / BK;
  const int kb0 = split * kb_per, kb1 = min(num_kb, kb0 + kb_per);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX); }
  if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!wait_bar(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
        uint8_t* sw = smem + stage * kDecStageBytes;
        mbar_expect_tx(&full_bar[stage], kDecStageBytes);
        tma_load_2d(sw, &tmW, &full_bar[stage], kb * BK, n0);
        tma_load_2d(sw + kDecWBytes, &tmX, &full_bar[stage], kb * BK, 0);
        if (++stage == kDecStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(err, 0x60000 | 1); }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!wait_bar(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + stage * kDecStageBytes);
        const uint32_t sx = sw + kDecWBytes;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(tmem_base, umma_smem_desc_sw128(sw + k * 32, 16, 1024), umma_smem_desc_sw128(sx + k * 32, 16, 1024),
                    idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == kDecStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
      else { *abort_flag = 1; atomicExch(err, 0x60000 | 2); }
    }
  } else {
    // ---- epilogue warps: lane = output channel, 64 accumulator columns = the activation rows; park the tile ----------------
    const int q = warp & 3;
    const int nl = q * 32 + lane;
    const bool ok = wait_bar(tfull_bar, 0, abort_flag);
    uint32_t v0[32], v1[32];
    if (ok) {
      tc_fence_after();
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16);
      tmem_ld_32x32(t0, v0);
      tmem_ld_32x32(t0 + 32, v1);
      tmem_ld_wait();
    } else {
      if (lane == 0) { *abort_flag = 1; atomicExch(err, 0x60000 | 3); }
#pragma unroll
      for (int m = 0; m < 32; ++m) { v0[m] = 0u; v1[m] = 0u; }
    }
    // every MMA of this CTA has completed (or was given up), so the pipeline stages are free to hold the tile
#pragma unroll
    for (int m = 0; m < 32; ++m) { R[m * kDecRStride + nl] = __uint_as_float(v0[m]); R[(32 + m) * kDecRStride + nl] = __uint_as_float(v1[m]); }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                   // every member's tile is parked and visible
  if (warp >= kEpiWarp0) {
    const int nl = (warp & 3) * 32 + lane, n = n0 + nl;
    const int rows = 64 / splits, m_lo = split * rows;
    const uint32_t my = smem_u32(R);
    // four rows at a time, every member's values requested before the first one is used: the latency of a remote
    // shared-memory read is paid once per group, not once per element
#pragma unroll 1
    for (int mb = m_lo; mb < m_lo + rows && mb < M; mb += 4) {
      float part[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int r = 0; r < 8; ++r)
          part[j][r] = (r < splits && mb + j < m_lo + rows)
                           ? ld_cluster_f32(map_to_cta(my + (uint32_t)((mb + j) * kDecRStride + nl) * 4u, (uint32_t)r)) : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = mb + j;
        float acc = ((part[j][0] + part[j][1]) + (part[j][2] + part[j][3])) + ((part[j][4] + part[j][5]) + (part[j][6] + part[j][7]));
        if (n < N && m < M && m < m_lo + rows) {
          if (epi == kEpiReluSqBf16) { acc = fmaxf(acc, 0.f); acc *= acc; }
          else if (epi == kEpiAddBf16) acc += bf2f(aux[(size_t)m * ldaux + n]);
          else if (act != 0) acc = act_apply(acc, act);
          out[(size_t)m * ldd + n] = f2bf(acc);
        }
      }
    }
  }
  cluster_sync_all();                                   // nobody leaves while a peer may still read its tile
  if (warp == 1) tmem_dealloc(tmem_base, 64);
}

int launch_decode(const GemmArgs& p, cudaStream_t st) {
  alignas(64) CUtensorMap tw;
  alignas(64) CUtensorMap tx;
  if (!make_map(&tw, p.B, p.N, p.K, p.ldb, 128)) return 2;
  if (!make_map(&tx, p.A, p.M, p.K, p.lda, 64)) return 2;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes) != cudaSuccess)
      return 3;
    attr_set = true;
  }
  const int tiles_n = (p.N + 127) / 128;
  const int num_kb = (p.K + BK - 1) / BK;
  // cluster size = K slices per n-tile: a power of two up to 8, enough that about every SM streams part of W
  int splits = 1;
  while (splits < 8 && tiles_n * splits < sm_count() && 2 * splits <= num_kb) splits *= 2;
  const int kb_per = (num_kb + splits - 1) / splits;
  if ((splits - 1) * kb_per >= num_kb) return -1;   // a member would get no k-block: let the general kernel run
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles_n * splits, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kDecSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D);
  const __nv_bfloat16* aux = reinterpret_cast<const __nv_bfloat16*>(p.aux);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_decode_kernel, tw, tx, out, p.ldd, aux, p.ldaux, p.M, p.N, p.K, kb_per,
                                           splits, p.epilogue, p.act, p.error_flag);
  return e == cudaSuccess ? 0 : 4;
}

int launch_pair_layout(const GemmArgs& p, cudaStream_t st) {
  switch (p.layout) {
    case kGemmTN: return launch_pair_epi<0, 0>(p, st);
    case kGemmNN: return launch_pair_epi<0, 1>(p, st);
    case kGemmNT_wgrad: return launch_pair_epi<1, 1>(p, st);
  }
  return 5;
}

}  // namespace

bool tma_encode_bf16_3d(void* map, const void* ptr, unsigned long long d0, unsigned long long d1, unsigned long long d2,
                        unsigned long long stride1, unsigned long long stride2, unsigned box0, unsigned box1) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  static thread_local bool context_bound = false;   // the driver entry point needs a current context on this thread
  if (!context_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess)
      return false;
    context_bound = true;
  }
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
  cuuint64_t strides[2] = {(cuuint64_t)stride1, (cuuint64_t)stride2};
  cuuint32_t box[3] = {box0, box1, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  return fn(reinterpret_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int gemm_bf16_group(const GemmArgs* ps, int count, cudaStream_t st) {
  if (count < 1 || count > kMaxGroup) return 1;
  int max_n = 0;
  for (int i = 0; i < count; ++i) {
    const GemmArgs& p = ps[i];
    if (p.layout != kGemmTN || p.epilogue != kEpiStoreBf16 || p.M != ps[0].M || p.M <= 0 || p.N <= 0 || p.K <= 0) return 1;
    if (p.K % 8 != 0 || p.lda % 8 != 0 || p.ldb % 8 != 0) return 1;
    if ((reinterpret_cast<uintptr_t>(p.A) | reinterpret_cast<uintptr_t>(p.B) | reinterpret_cast<uintptr_t>(p.D)) & 15) return 1;
    if (p.ldd % 8 != 0 || p.error_flag == nullptr) return 1;
    if (p.N > max_n) max_n = p.N;
  }
  // narrow outputs (the down-projections) take 128-column tiles, wide ones 256-column tiles
  return max_n <= 256 ? launch_group<128>(ps, count, st) : launch_group<256>(ps, count, st);
}

bool gemm_decode_eligible(const GemmArgs& p) {
  const bool epi_ok = p.epilogue == kEpiStoreBf16 || p.epilogue == kEpiReluSqBf16 || p.epilogue == kEpiAddBf16;
  // with a short reduction (the up-projection of a low-rank pair) there is no chain of dependent MMAs to split and the
  // general kernel's single pass is faster (measured 3.8 against 7 us at K = 128)
  return p.layout == kGemmTN && p.M <= 64 && p.N >= 64 && p.K >= 512 && epi_ok;
}

int gemm_bf16(const GemmArgs& p, cudaStream_t st) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return 1;
  // TMA needs 16-byte aligned bases and row pitches.
  if ((reinterpret_cast<uintptr_t>(p.A) & 15) || (reinterpret_cast<uintptr_t>(p.B) & 15) ||
      (reinterpret_cast<uintptr_t>(p.D) & 15) || (p.lda & 7) || (p.ldb & 7))
    return 6;
  if (p.epilogue == kEpiScatterAddBf16) {
    // D is a device-resident GemmScatter; ldd is the row pitch of the per-rank output buffers
    if (p.layout != kGemmTN || (p.N & 31) || (p.ldd & 7)) return 6;
    if (p.error_flag == nullptr) return 7;
    if (p.pair != 0 && p.M >= 256 && p.N >= 256) return launch_pair<0, 0, kEpiScatterAddBf16>(p, st);
    return launch<256, 0, 0, kEpiScatterAddBf16>(p, st);
  }
  if (p.epilogue == kEpiCeStats) {
    // D is float [M, ceil(N / 256), 4] (row pitch ldd floats), aux the int32 targets: both tile shapes are 256 wide
    if (p.layout != kGemmTN || p.aux == nullptr || (p.ldd & 3) || p.ldd < 4 * ((p.N + 255) / 256)) return 6;
    if (p.error_flag == nullptr) return 7;
    if (p.pair != 0 && p.M >= 256 && p.N >= 256 && p.K >= 512) return launch_pair<0, 0, kEpiCeStats>(p, st);
    return launch<256, 0, 0, kEpiCeStats>(p, st);
  }
  const bool two_input = p.epilogue == kEpiMulSqrt2Bf16 || p.epilogue == kEpiAddBf16;
  if (two_input && (p.aux == nullptr || (reinterpret_cast<uintptr_t>(p.aux) & 15) || (p.ldaux & 7))) return 6;
  const bool out_bf16 = p.epilogue == kEpiStoreBf16 || p.epilogue == kEpiReluSqBf16 || two_input;
  if (p.ldd & (out_bf16 ? 7 : 3)) return 6;
  if (p.error_flag == nullptr) return 7;
  // the CTA-pair kernel needs at least one full 256-row tile and a wide N to pay off
  // (with a short reduction the epilogue dominates and two independent CTAs drain their tiles faster: measured 59 vs
  // 72 us at 32768 x 2048 x 128)
  if (p.pair != 0 && p.M >= 256 && p.N >= 256 && p.K >= 512) return launch_pair_layout(p, st);
  // decode-sized problems: swap-AB split-K kernel when the caller provided its workspace
  if (p.decode_kernel != 0 && gemm_decode_eligible(p)) {
    const int rc = launch_decode(p, st);
    if (rc >= 0) return rc;
  }
  // otherwise (one m-tile): narrow n-tiles so that the weight matrix is streamed by many SMs at once
  if (p.layout == kGemmTN && p.M <= BM && p.N >= 1024) return launch_epi<32, 0, 0>(p, st);
  if (p.N > 128) return launch_layout<256>(p, st);
  return launch_layout<128>(p, st);
}

}  // namespace rk
