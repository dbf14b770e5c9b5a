// WKV7 generalised delta rule, chunked form on the 5th-generation tensor cores (head size 64, bf16 vectors).
//
// With P_t = prod_{s<=t} d_s inside a chunk of L = 64 steps and the rescaled vectors
//   a~_t = a_t * P_{t-1},  r~_t = r_t * P_t,  b~_t = b_t / P_t,  k~_t = k_t / P_t,
//   b^_t = b_t * P_L / P_t,  k^_t = k_t * P_L / P_t
// the recurrence  S_t = S_{t-1} diag(d_t) + (S_{t-1} a_t) b_t^T + v_t k_t^T,  y_t = S_t r_t  becomes, per chunk,
//   A_ab = tril<(A~ B~^T)   A_ak = tril<(A~ K~^T)   A_rb = tril<=(R~ B~^T)   A_rk = tril<=(R~ K~^T)      (one MMA)
//   Z    = A~ S0^T + A_ak V                                                                            (MMA)
//   U    = (I - A_ab)^-1 Z          the inverse is formed blockwise in fp32 (CUDA cores, overlapped with the Z
//                                   product) and applied as one more MMA; U_t = S_{t-1} a_t
//   Y    = R~ S0^T + A_rk V + A_rb U                                                                   (MMA)
//   S1^T = diag(P_L) S0^T + B^^T U + K^^T V                                                            (MMA)
// One CTA of 8 warps per (batch, head) walks the chunks in order; two CTAs share an SM.  Every product is a
// tcgen05.mma with M = 128 (two 64-row operands stacked, or 64 useful rows plus 64 ignored ones), bf16
// operands written into shared memory in the 128-byte-swizzled canonical layout, fp32 accumulators in tensor
// memory.  The raw [64 steps][64 channels] tiles of the next chunk are requested as soon as the last product that
// reads a slot has completed, so their latency hides behind the rest of the current chunk: one thread issues
// cp.async.bulk.tensor loads over 3-D tensor maps of the [B, T, H * 64] inputs (the copy engine writes the 128-byte
// swizzled operand layout directly and zero-fills steps past the end of the sequence) and an mbarrier counts the
// bytes; a cp.async variant with per-thread 16-byte copies remains as the fallback when no tensor map can be made.  The fp32 master copy of the state lives in registers (thread (k, half) holds 32 values of row k of
// S^T); its bf16 image is the B operand of the next chunk.  Decay is bounded below by exp(-exp(-0.5)) = 0.545
// per step, so every scale factor stays inside the fp32 / bf16 exponent range over 64 steps.
//
// In training mode the kernel also writes U (the `sa` vectors, bf16) and the state after every chunk, which is what
// the chunked backward kernel consumes.  Reference semantics: src/rwkv7m/model/rwkv_core.py:54-86,
// src/rwkv7m/kernels/wkv_pallas_gpu.py:66-164.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "wkv7_chunk.cuh"

namespace rk {

using namespace chunk;

namespace {

constexpr int L = 64;        // chunk length
constexpr int NH = 64;       // head size
constexpr int kThreads = 256;
constexpr int kFStride = 68; // row stride (floats) of the fp32 scratch matrices: 16-byte aligned, conflict-light

// shared memory map (byte offsets from a 1024-byte aligned base)
constexpr uint32_t kOffAR = 0;                    // [128][64] bf16: rows 0-63 A~, 64-127 R~
constexpr uint32_t kOffBK = kOffAR + 16384;       // [128][64] bf16: B~ | K~; later A_ak | A_rk; later Z (rows 0-63)
constexpr uint32_t kOffBKe = kOffBK + 16384;      // [128][64] bf16: rows 0-63 B^, 64-127 K^
constexpr uint32_t kOffUV = kOffBKe + 16384;      // [128][64] bf16: rows 0-63 (I - A_ab)^-1, then U; rows 64-127 V
constexpr uint32_t kOffX2 = kOffUV + 16384;       // [64][64] bf16: A_rb (rows 64-127 of an operand that starts 8 KB earlier)
constexpr uint32_t kOffS = kOffX2 + 8192;         // [64][64] bf16: S^T
constexpr uint32_t kOffF = kOffS + 8192;          // fp32 [64][68]: A_ab, overwritten by its inverse
constexpr uint32_t kOffW = kOffF + L * kFStride * 4;    // fp32 scratch of the blocked inverse
constexpr uint32_t kOffPL = kOffW + kInvWorkFloats * 4; // fp32 [64]: P_L
constexpr uint32_t kOffBar = kOffPL + NH * 4;     // 5 mbarriers (4 MMA groups, tile loads), tmem slot, failure flag
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;    // + alignment slack

static_assert(kFStride == kInvStride, "the inverse routine reads the A_ab scratch with its own row stride");

constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColD1 = 0;    // 128 columns: A matrices; then U (first 64, lanes 0-63); then the state products
constexpr uint32_t kColD2 = 128;  // 64 columns: Z (lanes 0-63) and Y (lanes 64-127)

__device__ int g_wkv_chunk_error = 0;

#ifdef RK_WKV_PROF
__device__ long long g_wkv_chunk_prof[16];
#define PROF_MARK(i)                                                          \
  do {                                                                        \
    if (blockIdx.x == 0 && tid == 0) {                                        \
      const long long now_ = clock64();                                       \
      g_wkv_chunk_prof[i] += now_ - prof_t;                                   \
      prof_t = now_;                                                          \
    }                                                                         \
  } while (0)
#else
#define PROF_MARK(i) do { } while (0)
#endif

// tensor maps of the six inputs in slot order: a, r, b, k, w, v
struct ChunkMaps { CUtensorMap m[6]; };

struct ChunkPtrs {
  const __nv_bfloat16 *r, *w, *k, *v, *a, *b;
  __nv_bfloat16* y;
  const float* s0;
  float *sT, *ckpt;
  __nv_bfloat16* sa;
};

template <bool SAVE>
__global__ void __launch_bounds__(kThreads, 2) wkv7_chunk_fwd_kernel(ChunkPtrs g, const __grid_constant__ ChunkMaps maps,
                                                                     int use_tma, int T, int H, int BH) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by adding an offset (not by casting through an integer) so accesses stay in the shared address space
  uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(sm);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 48);
  volatile int* failed = reinterpret_cast<volatile int*>(sm + kOffBar + 56);
  float* F = reinterpret_cast<float*>(sm + kOffF);
  float* Wk = reinterpret_cast<float*>(sm + kOffW);
  float* PL = reinterpret_cast<float*>(sm + kOffPL);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, bi = bh / H, hi = bh - bi * H;
  const size_t stride_t = (size_t)H * NH;
  const size_t base = (size_t)bi * T * stride_t + (size_t)hi * NH;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
    mbar_init(&bars[4], 3);   // tile loads: three request groups per chunk, each one arrival plus its bytes
    *failed = 0;
    mbar_fence_init();
    if (use_tma) {
#pragma unroll
      for (int i = 0; i < 6; ++i) tma_prefetch_desc(&maps.m[i]);
    }
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // tensor-memory view of this thread: row m of the 128-row accumulators, column half ch
  const int wq = warp & 3, ch = warp >> 2;
  const int m = wq * 32 + lane;
  const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
  const bool lower = wq < 2;            // rows 0-63 (A~ rows, Z, state) vs rows 64-127 (R~ rows, Y)
  const int trow = m & 63;

  // fp32 master copy of the state: thread (k = trow, ch) of the lower warps holds S[v][k] for v in [32 ch, 32 ch + 32)
  float st[32];
  if (lower) {
#pragma unroll
    for (int j = 0; j < 32; ++j) st[j] = g.s0 != nullptr ? g.s0[((size_t)bh * NH + 32 * ch + j) * NH + trow] : 0.f;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = st[8 * p + j];
      *reinterpret_cast<uint4*>(sm + kOffS + sw128(trow, 4 * ch + p)) = pack8(x);
    }
  }

  const int nchunks = (T + L - 1) / L;
  bool ok = true;
  // Coalesced asynchronous copy of one raw [64][64] bf16 tile of chunk cc straight into an operand slot (8 lanes per
  // 128-byte row, swizzled like the operand tiles; rows past the end of the sequence are zero-filled).  Each slot of
  // the next chunk is requested as soon as the last product that reads the current contents has completed.
  // bulk-tensor variant: one thread announces the bytes of a request group and issues one copy per tile
  auto fetch_group = [&](int cc, int first, int count) {   // tiles first .. first + count - 1 in the order a, r, b, k, w, v
    constexpr uint32_t slot_of[6] = {kOffAR, kOffAR + 8192, kOffBK, kOffBK + 8192, kOffBKe, kOffUV + 8192};
    if (tid == 0) {
      mbar_expect_tx(&bars[4], (uint32_t)count * 8192u);
      for (int i = first; i < first + count; ++i) tma_load_3d(sm + slot_of[i], &maps.m[i], &bars[4], hi * NH, cc * L, bi);
    }
  };
  auto fetch_tile = [&](uint32_t slot, const __nv_bfloat16* src, int cc) {
    const int p8 = tid & 7;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = (tid >> 3) + 32 * i;
      const uint32_t off = sw128(row, p8);
      if (cc * L + row < T) cp_async16(sm + slot + off, src + base + (size_t)(cc * L + row) * stride_t + p8 * 8);
      else *reinterpret_cast<uint4*>(sm + slot + off) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  if (use_tma) {
    fetch_group(0, 0, 2);   // the same three groups as inside the loop: (a, r, k), (b), (w, v)
    fetch_group(0, 2, 2);
    fetch_group(0, 4, 2);
  } else {
    fetch_tile(kOffAR, g.a, 0);
    fetch_tile(kOffAR + 8192, g.r, 0);
    fetch_tile(kOffBK, g.b, 0);
    fetch_tile(kOffBK + 8192, g.k, 0);
    fetch_tile(kOffBKe, g.w, 0);
    fetch_tile(kOffUV + 8192, g.v, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
#ifdef RK_WKV_PROF
  long long prof_t = clock64();
#endif
  for (int c = 0; c < nchunks; ++c) {
    const bool more = c + 1 < nchunks;
    const int t0 = c * L;
    const uint32_t par = (uint32_t)(c & 1);
    // ---- raw tiles: requested during the previous chunk (before the loop for the first one) -------------------------
    if (use_tma) {
      if (!mbar_wait(&bars[4], par, failed)) { *failed = 1; }
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(8);
    // ---- rescale in place: warp w owns the 16-byte column piece w, lane l owns rows l and l + 32 ----------------------
    {
      const int piece = warp;
      uint4 rw[2], ra[2], rr[2], rb[2], rk[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t off = sw128(lane + 32 * i, piece);
        rw[i] = *reinterpret_cast<const uint4*>(sm + kOffBKe + off);
        ra[i] = *reinterpret_cast<const uint4*>(sm + kOffAR + off);
        rr[i] = *reinterpret_cast<const uint4*>(sm + kOffAR + 8192 + off);
        rb[i] = *reinterpret_cast<const uint4*>(sm + kOffBK + off);
        rk[i] = *reinterpret_cast<const uint4*>(sm + kOffBK + 8192 + off);
      }
      // cumulative log decay: one warp scan per half (rows 0-31, rows 32-63), the second offset by the first total
      float ld[2][8], lp[2][8], ptot[8];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float x[8];
        unpack8(rw[i], x);
        const bool valid = t0 + lane + 32 * i < T;
#pragma unroll
        for (int j = 0; j < 8; ++j) ld[i][j] = valid ? -__expf(x[j]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s0_ = ld[0][j], s1_ = ld[1][j];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const float o0 = __shfl_up_sync(0xffffffffu, s0_, off);
          const float o1 = __shfl_up_sync(0xffffffffu, s1_, off);
          if (lane >= off) { s0_ += o0; s1_ += o1; }
        }
        const float tot0 = __shfl_sync(0xffffffffu, s0_, 31);
        lp[0][j] = s0_;
        lp[1][j] = tot0 + s1_;
        ptot[j] = __expf(tot0 + __shfl_sync(0xffffffffu, s1_, 31));  // P_L of the column
      }
      if (lane == 31) {
        float* dst = PL + piece * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(ptot[0], ptot[1], ptot[2], ptot[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(ptot[4], ptot[5], ptot[6], ptot[7]);
      }
      PROF_MARK(9);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t off = sw128(lane + 32 * i, piece);
        float e1[8], e0[8], inv[8], x[8], y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          e1[j] = __expf(lp[i][j]);                 // P_t
          e0[j] = __expf(lp[i][j] - ld[i][j]);      // P_{t-1}
          inv[j] = __expf(-lp[i][j]);
        }
        unpack8(ra[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * e0[j];
        *reinterpret_cast<uint4*>(sm + kOffAR + off) = pack8(y);
        unpack8(rr[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * e1[j];
        *reinterpret_cast<uint4*>(sm + kOffAR + 8192 + off) = pack8(y);
        unpack8(rb[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * inv[j];
        *reinterpret_cast<uint4*>(sm + kOffBK + off) = pack8(y);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] *= ptot[j];
        *reinterpret_cast<uint4*>(sm + kOffBKe + off) = pack8(y);
        unpack8(rk[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * inv[j];
        *reinterpret_cast<uint4*>(sm + kOffBK + 8192 + off) = pack8(y);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] *= ptot[j];
        *reinterpret_cast<uint4*>(sm + kOffBKe + 8192 + off) = pack8(y);
      }
    }
    PROF_MARK(10);
    fence_proxy_async_smem();
    __syncthreads();
    PROF_MARK(0);
    // ---- MMA 1: the four triangular score matrices ------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kColD1, desc_k(sbase + kOffAR + k * 32), desc_k(sbase + kOffBK + k * 32), idesc, k > 0);
      umma_commit(&bars[0]);
    }
    if (!mbar_wait(&bars[0], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(1);
    // thread (row m, half ch) reads 64 columns: ch = 0 -> products with B~ (A_ab | A_rb), ch = 1 -> with K~ (A_ak | A_rk)
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kColD1 + ch * 64 + q * 32, v);
      tmem_ld_wait();
      const int s0 = q * 32;
      if (lower) {
        if (ch == 0) {  // A_ab, strictly lower, fp32: F[t][s], the input of the blocked inverse
          float* dst = F + trow * kFStride + s0;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(
                s0 + j < trow ? __uint_as_float(v[j]) : 0.f, s0 + j + 1 < trow ? __uint_as_float(v[j + 1]) : 0.f,
                s0 + j + 2 < trow ? __uint_as_float(v[j + 2]) : 0.f, s0 + j + 3 < trow ? __uint_as_float(v[j + 3]) : 0.f);
        } else {        // A_ak, strictly lower
          store_masked_bf16(sm + kOffBK, trow, q * 4, v, s0, [&](int s) { return s < trow; });
        }
      } else {
        if (ch == 0) store_masked_bf16(sm + kOffX2, trow, q * 4, v, s0, [&](int s) { return s <= trow; });           // A_rb
        else store_masked_bf16(sm + kOffBK + 8192, trow, q * 4, v, s0, [&](int s) { return s <= trow; });           // A_rk
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(2);
    // ---- MMA 2: Z = A~ S0^T + A_ak V (lanes 0-63),  Y = R~ S0^T + A_rk V (lanes 64-127) -------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kColD2, desc_k(sbase + kOffAR + k * 32), desc_mn(sbase + kOffS + k * 2048, 8192), idesc, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kColD2, desc_k(sbase + kOffBK + k * 32), desc_mn(sbase + kOffUV + 8192 + k * 2048, 8192), idesc, 1);
      umma_commit(&bars[1]);
    }
    // the inverse of I - A_ab on the CUDA cores while the tensor cores form Z; it lands in the U slot as a bf16 operand
    unit_lower_inverse_64(F, Wk, sm + kOffUV, tid);
    PROF_MARK(11);
    if (!mbar_wait(&bars[1], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(3);
    if (more) {   // A~, R~ and A_rk have been consumed: their slots take the next chunk's raw a, r and k
      if (use_tma) {
        if (tid == 0) {
          mbar_expect_tx(&bars[4], 3u * 8192u);
          tma_load_3d(sm + kOffAR, &maps.m[0], &bars[4], hi * NH, (c + 1) * L, bi);
          tma_load_3d(sm + kOffAR + 8192, &maps.m[1], &bars[4], hi * NH, (c + 1) * L, bi);
          tma_load_3d(sm + kOffBK + 8192, &maps.m[3], &bars[4], hi * NH, (c + 1) * L, bi);
        }
      } else {
        fetch_tile(kOffAR, g.a, c + 1);
        fetch_tile(kOffAR + 8192, g.r, c + 1);
        fetch_tile(kOffBK + 8192, g.k, c + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }
    if (lower) {  // Z rows -> bf16 operand tile over the dead A_ak slot, 32 columns per thread
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kColD2 + ch * 32, v);
      tmem_ld_wait();
      store_masked_bf16(sm + kOffBK, trow, ch * 4, v, 0, [](int) { return true; });
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(4);
    // ---- MMA U: U = (I - A_ab)^-1 Z (lanes 0-63; lanes 64-127 multiply the V rows that follow the inverse: ignored) ------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kColD1, desc_k(sbase + kOffUV + k * 32), desc_mn(sbase + kOffBK + k * 2048, 8192), idesc, k > 0);
      umma_commit(&bars[3]);
    }
    if (!mbar_wait(&bars[3], par, failed)) { *failed = 1; }
    tc_fence_after();
    if (more) {   // Z has been consumed: its slot takes the next chunk's raw b
      if (use_tma) {
        fetch_group(c + 1, 2, 1);
      } else {
        fetch_tile(kOffBK, g.b, c + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }
    if (lower) {  // U rows -> bf16 operand tile (over the inverse, which the finished MMA no longer reads) and, in
                  // training, the same bf16 rows for the backward pass
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kColD1 + ch * 32, v);
      tmem_ld_wait();
      const bool keep = SAVE && t0 + trow < T;
      __nv_bfloat16* dst = g.sa + base + (size_t)(t0 + trow) * stride_t + ch * 32;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
        const uint4 packed = pack8(x);
        *reinterpret_cast<uint4*>(sm + kOffUV + sw128(trow, ch * 4 + p)) = packed;
        if (keep) *reinterpret_cast<uint4*>(dst + 8 * p) = packed;
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(5);
    // ---- MMA 3: Y += A_rb U;  MMA 4: state products B^^T U + K^^T V -------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc3 = umma_idesc_bf16(128, 64, 0, 1);
      constexpr uint32_t idesc4 = umma_idesc_bf16(128, 64, 1, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kColD2, desc_k(sbase + kOffX2 - 8192 + k * 32), desc_mn(sbase + kOffUV + k * 2048, 8192), idesc3, 1);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        umma_bf16(tmem + kColD1, desc_mn(sbase + kOffBKe + k * 2048, 16384), desc_mn(sbase + kOffUV + k * 2048, 8192),
                  idesc4, k > 0);
      umma_commit(&bars[2]);
    }
    if (!mbar_wait(&bars[2], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(6);
    if (more) {   // B^ and V have been consumed: their slots take the next chunk's raw w and v
      if (use_tma) {
        fetch_group(c + 1, 4, 2);
      } else {
        fetch_tile(kOffBKe, g.w, c + 1);
        fetch_tile(kOffUV + 8192, g.v, c + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }
    {
      uint32_t v[32];
      if (!lower) {  // output row t, columns [32 ch, 32 ch + 32)
        tmem_ld_32x32(tmem + lane_base + kColD2 + ch * 32, v);
        tmem_ld_wait();
        const int t = t0 + trow;
        if (t < T) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
            *reinterpret_cast<uint4*>(g.y + base + (size_t)t * stride_t + ch * 32 + p * 8) = pack8(x);
          }
        }
      } else {       // state row k = trow, value columns [32 ch, 32 ch + 32)
        tmem_ld_32x32(tmem + lane_base + kColD1 + ch * 32, v);
        tmem_ld_wait();
        const float pl = PL[trow];
#pragma unroll
        for (int j = 0; j < 32; ++j) st[j] = fmaf(pl, st[j], __uint_as_float(v[j]));
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          float x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = st[8 * p + j];
          *reinterpret_cast<uint4*>(sm + kOffS + sw128(trow, 4 * ch + p)) = pack8(x);
        }
        if (SAVE) {  // state after this chunk, [v][k] layout
          float* dst = g.ckpt + ((size_t)c * BH + bh) * NH * NH + (size_t)(32 * ch) * NH + trow;
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[(size_t)j * NH] = st[j];
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(7);
  }
  if (lower && g.sT != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) g.sT[((size_t)bh * NH + 32 * ch + j) * NH + trow] = st[j];
  }
  if (!ok && tid == 0) atomicExch(&g_wkv_chunk_error, 0x30000 | (bh & 0xffff));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool wkv7_chunk_supported(const WkvArgs& p) { return p.is_bf16 && p.N == NH && (p.sa == nullptr || p.interval == L); }

int wkv7_chunk_forward(const WkvArgs& p, cudaStream_t st) {
  if (!wkv7_chunk_supported(p)) return 1;
  ChunkPtrs g;
  g.r = (const __nv_bfloat16*)p.r; g.w = (const __nv_bfloat16*)p.w; g.k = (const __nv_bfloat16*)p.k;
  g.v = (const __nv_bfloat16*)p.v; g.a = (const __nv_bfloat16*)p.a; g.b = (const __nv_bfloat16*)p.b;
  g.y = (__nv_bfloat16*)p.y; g.s0 = p.s0; g.sT = p.sT; g.sa = (__nv_bfloat16*)p.sa; g.ckpt = p.ckpt;
  const int BH = p.B * p.H;
  // tensor maps over the [B, T, H * 64] inputs; RWKV7M_B200_WKV_TMA=0 keeps the per-thread copies (for comparisons)
  alignas(64) ChunkMaps maps;
  static const bool want_tma = [] { const char* e = getenv("RWKV7M_B200_WKV_TMA"); return e == nullptr || e[0] != '0'; }();
  int use_tma = want_tma ? 1 : 0;
  const void* src[6] = {p.a, p.r, p.b, p.k, p.w, p.v};
  const unsigned long long row_bytes = (unsigned long long)p.H * NH * 2;
  for (int i = 0; i < 6 && use_tma; ++i) {
    if ((reinterpret_cast<uintptr_t>(src[i]) & 15) != 0 ||
        !tma_encode_bf16_3d(&maps.m[i], src[i], (unsigned long long)p.H * NH, (unsigned long long)p.T, (unsigned long long)p.B,
                            row_bytes, row_bytes * p.T, NH, L))
      use_tma = 0;
  }
  if (!use_tma) memset(&maps, 0, sizeof(maps));
  if (p.sa != nullptr) {
    auto kern = wkv7_chunk_fwd_kernel<true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    kern<<<BH, kThreads, kSmemBytes, st>>>(g, maps, use_tma, p.T, p.H, BH);
  } else {
    auto kern = wkv7_chunk_fwd_kernel<false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    kern<<<BH, kThreads, kSmemBytes, st>>>(g, maps, use_tma, p.T, p.H, BH);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

#ifdef RK_WKV_PROF
void wkv7_chunk_prof(long long* out, bool reset) {
  cudaMemcpyFromSymbol(out, g_wkv_chunk_prof, 16 * sizeof(long long));
  if (reset) { long long z[16] = {0}; cudaMemcpyToSymbol(g_wkv_chunk_prof, z, sizeof(z)); }
}
#endif

int wkv7_chunk_error(bool reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_wkv_chunk_error, sizeof(int));
  if (reset && v != 0) { const int z = 0; cudaMemcpyToSymbol(g_wkv_chunk_error, &z, sizeof(int)); }
  return v;
}

}  // namespace rk
