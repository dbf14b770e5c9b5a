// WKV7 generalised delta rule, chunked form on the 5th-generation tensor cores (head size 64, bf16 vectors).
//
// With P_t = prod_{s<=t} d_s inside a chunk of L = 64 steps and the rescaled vectors
//   a~_t = a_t * P_{t-1},  r~_t = r_t * P_t,  b~_t = b_t / P_t,  k~_t = k_t / P_t,
//   b^_t = b_t * P_L / P_t,  k^_t = k_t * P_L / P_t
// the recurrence  S_t = S_{t-1} diag(d_t) + (S_{t-1} a_t) b_t^T + v_t k_t^T,  y_t = S_t r_t  becomes, per chunk,
//   A_ab = tril<(A~ B~^T)   A_ak = tril<(A~ K~^T)   A_rb = tril<=(R~ B~^T)   A_rk = tril<=(R~ K~^T)      (one MMA)
//   Z    = A~ S0^T + A_ak V                                                                            (MMA)
//   U    = (I - A_ab)^-1 Z          forward substitution in fp32 on the CUDA cores; U_t = S_{t-1} a_t
//   Y    = R~ S0^T + A_rk V + A_rb U                                                                   (MMA)
//   S1^T = diag(P_L) S0^T + B^^T U + K^^T V                                                            (MMA)
// One CTA per (batch, head) walks the chunks in order.  Every product is a tcgen05.mma with M = 128 (two
// 64-row operands stacked, or 64 useful rows plus 64 ignored ones), bf16 operands written into shared memory in
// the 128-byte-swizzled canonical layout, fp32 accumulators in tensor memory.  The fp32 master copy of the
// state lives in the registers of 64 threads (thread k holds row k of S^T); its bf16 image is the B operand
// of the next chunk.  Decay is bounded below by exp(-exp(-0.5)) = 0.545 per step, so every scale factor stays
// inside the fp32 / bf16 exponent range over 64 steps.
//
// In training mode the kernel also writes what the time-sequential backward kernel consumes: U (as `sa`) and
// the state after every 16th step.  Reference semantics: src/rwkv7m/model/rwkv_core.py:54-86,
// src/rwkv7m/kernels/wkv_pallas_gpu.py:66-164.
#include "common.cuh"
#include "kernels.h"
#include "wkv7_chunk.cuh"

namespace rk {

using namespace chunk;

namespace {

constexpr int L = 64;        // chunk length
constexpr int NH = 64;       // head size
constexpr int kThreads = 128;
constexpr int kFStride = 68; // row stride (floats) of the fp32 scratch matrices: 16-byte aligned, conflict-light

// shared memory map (byte offsets from a 1024-byte aligned base)
constexpr uint32_t kOffAR = 0;                    // [128][64] bf16: rows 0-63 A~, 64-127 R~
constexpr uint32_t kOffBK = kOffAR + 16384;       // [128][64] bf16: B~ | K~; later A_ak | A_rk; later Z fp32 [64][68]
constexpr uint32_t kOffBKe = kOffBK + 18432;      // [128][64] bf16: rows 0-63 B^, 64-127 K^
constexpr uint32_t kOffUV = kOffBKe + 16384;      // [128][64] bf16: rows 0-63 U, 64-127 V
constexpr uint32_t kOffX2 = kOffUV + 16384;       // [64][64] bf16: A_rb (rows 64-127 of an operand that starts 8 KB earlier)
constexpr uint32_t kOffS = kOffX2 + 8192;         // [64][64] bf16: S^T
constexpr uint32_t kOffF = kOffS + 8192;          // fp32 [64][68]: cumulative log decay, later A_ab
constexpr uint32_t kOffPL = kOffF + L * kFStride * 4;   // fp32 [4][64]: P at steps 15, 31, 47, 63
constexpr uint32_t kOffBar = kOffPL + 4 * NH * 4; // 4 mbarriers, tmem slot, failure flag
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;    // + alignment slack

constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColD1 = 0;    // 128 columns: A matrices; later the state products
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

struct ChunkPtrs {
  const __nv_bfloat16 *r, *w, *k, *v, *a, *b;
  __nv_bfloat16* y;
  const float* s0;
  float *sT, *sa, *ckpt;
};

}  // namespace

namespace {

template <bool SAVE>
__global__ void __launch_bounds__(kThreads, 2) wkv7_chunk_fwd_kernel(ChunkPtrs g, int T, int H, int BH) {
  extern __shared__ uint8_t smem_raw[];
  // aligned by adding an offset (not by casting through an integer) so accesses stay in the shared address space
  uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(sm);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 32);
  volatile int* failed = reinterpret_cast<volatile int*>(sm + kOffBar + 40);
  float* F = reinterpret_cast<float*>(sm + kOffF);
  float* Zs = reinterpret_cast<float*>(sm + kOffBK);
  float* PL = reinterpret_cast<float*>(sm + kOffPL);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int bh = blockIdx.x, bi = bh / H, hi = bh - bi * H;
  const size_t stride_t = (size_t)H * NH;
  const size_t base = (size_t)bi * T * stride_t + (size_t)hi * NH;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
    *failed = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const int trow = tid & 63;

  // fp32 master copy of the state: thread k (< 64) holds row k of S^T, i.e. S[v][k] for all v
  float st[NH];
  if (tid < 64) {
#pragma unroll
    for (int v = 0; v < NH; ++v) st[v] = g.s0 != nullptr ? g.s0[((size_t)bh * NH + v) * NH + tid] : 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = st[8 * p + j];
      *reinterpret_cast<uint4*>(sm + kOffS + sw128(tid, p)) = pack8(x);
    }
  }

  const int nchunks = (T + L - 1) / L;
  const int nck = (T + 15) / 16;
  const int piece = 2 * warp + ((tid >> 4) & 1), lq = tid & 15;  // operand preparation: column piece, row quad
  bool ok = true;
#ifdef RK_WKV_PROF
  long long prof_t = clock64();
#endif
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * L;
    const uint32_t par = (uint32_t)(c & 1);
    // ---- operands: every warp owns two 16-byte column pieces, lane l' of a 16-lane group owns rows 4l'..4l'+3 --
    {
      const size_t go0 = base + (size_t)(t0 + 4 * lq) * stride_t + piece * 8;
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      uint4 rw[4], ra[4], rr[4], rb[4], rk[4], rv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool valid = t0 + 4 * lq + i < T;
        const size_t go = go0 + (size_t)i * stride_t;
        rw[i] = valid ? *reinterpret_cast<const uint4*>(g.w + go) : zero;
        ra[i] = valid ? *reinterpret_cast<const uint4*>(g.a + go) : zero;
        rr[i] = valid ? *reinterpret_cast<const uint4*>(g.r + go) : zero;
        rb[i] = valid ? *reinterpret_cast<const uint4*>(g.b + go) : zero;
        rk[i] = valid ? *reinterpret_cast<const uint4*>(g.k + go) : zero;
        rv[i] = valid ? *reinterpret_cast<const uint4*>(g.v + go) : zero;
      }
      if (c + 1 < nchunks) {  // pull the next chunk's rows into L2 while this chunk is being processed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = t0 + L + 4 * lq + i;
          if (t < T && (piece & 1) == 0) {  // one prefetch per 32-byte sector pair is enough: pieces 2w and 2w+1 share it
            const size_t go = go0 + (size_t)(L + i) * stride_t;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.w + go));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.a + go));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.r + go));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.b + go));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.k + go));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(g.v + go));
          }
        }
      }
      // inclusive cumulative log decay of the lane's four rows, then a 16-lane scan of the lane totals
      float lp[4][8], ex[8], ptot[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float x[8];
        unpack8(rw[i], x);
        const bool valid = t0 + 4 * lq + i < T;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ld = valid ? -__expf(x[j]) : 0.f;
          lp[i][j] = i == 0 ? ld : lp[i - 1][j] + ld;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float tot = lp[3][j];
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) {
          const float o = __shfl_up_sync(0xffffffffu, tot, off, 16);
          if (lq >= off) tot += o;
        }
        ex[j] = tot - lp[3][j];                                   // cumulative log decay before this lane's rows
        ptot[j] = __expf(__shfl_sync(0xffffffffu, tot, 15, 16));  // P_L of the column
      }
      PROF_MARK(8);
      float eprev[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) eprev[j] = __expf(ex[j]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * lq + i;
        const uint32_t off = sw128(row, piece);
        float e1[8], inv[8], x[8], y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          e1[j] = __expf(ex[j] + lp[i][j]);
          inv[j] = __frcp_rn(e1[j]);
        }
        unpack8(ra[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * eprev[j];
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
        *reinterpret_cast<uint4*>(sm + kOffUV + 8192 + off) = rv[i];
        if (i == 3 && (lq & 3) == 3) {  // P at steps 15, 31, 47, 63
          float* dst = PL + (lq >> 2) * NH + piece * 8;
          *reinterpret_cast<float4*>(dst) = make_float4(e1[0], e1[1], e1[2], e1[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(e1[4], e1[5], e1[6], e1[7]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) eprev[j] = e1[j];
      }
    }
    PROF_MARK(9);
    fence_proxy_async_smem();
    __syncthreads();
    PROF_MARK(1);
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
    PROF_MARK(2);
#pragma unroll
    for (int hq = 0; hq < 4; ++hq) {  // hq>>1: which matrix of the row, hq&1: which half of its columns
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kColD1 + hq * 32, v);
      tmem_ld_wait();
      const int s0 = (hq & 1) * 32;
      if (tid < 64) {
        if (hq < 2) {  // A_ab, strictly lower, fp32, stored transposed (column s contiguous over t) for the substitution
#pragma unroll
          for (int j = 0; j < 32; ++j) F[(s0 + j) * kFStride + trow] = s0 + j < trow ? __uint_as_float(v[j]) : 0.f;
        } else {       // A_ak, strictly lower
          store_masked_bf16(sm + kOffBK, trow, (hq & 1) * 4, v, s0, [&](int s) { return s < trow; });
        }
      } else {
        if (hq < 2) store_masked_bf16(sm + kOffX2, trow, (hq & 1) * 4, v, s0, [&](int s) { return s <= trow; });          // A_rb
        else store_masked_bf16(sm + kOffBK + 8192, trow, (hq & 1) * 4, v, s0, [&](int s) { return s <= trow; });          // A_rk
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(3);
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
    if (!mbar_wait(&bars[1], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(4);
    if (tid < 64) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + kColD2 + q * 32, v);
        tmem_ld_wait();
        float* dst = Zs + trow * kFStride + q * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                            __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
      asm volatile("bar.sync 1, 64;" ::: "memory");
      PROF_MARK(10);
      // forward substitution, thread = value column, right-looking: once u_s is final it is pushed into
      // every later row, so all updates of one step are independent of each other
      float u[L];
#pragma unroll
      for (int t = 0; t < L; ++t) u[t] = Zs[t * kFStride + tid];
#pragma unroll
      for (int s_ = 0; s_ < L - 1; ++s_) {
#pragma unroll
        for (int t4 = 0; t4 < L / 4; ++t4) {
          if (4 * t4 + 3 > s_) {
            const float4 A = *reinterpret_cast<const float4*>(F + s_ * kFStride + 4 * t4);
            if (4 * t4 + 0 > s_) u[4 * t4 + 0] = fmaf(A.x, u[s_], u[4 * t4 + 0]);
            if (4 * t4 + 1 > s_) u[4 * t4 + 1] = fmaf(A.y, u[s_], u[4 * t4 + 1]);
            if (4 * t4 + 2 > s_) u[4 * t4 + 2] = fmaf(A.z, u[s_], u[4 * t4 + 2]);
            if (4 * t4 + 3 > s_) u[4 * t4 + 3] = fmaf(A.w, u[s_], u[4 * t4 + 3]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < L; ++t) {
        *reinterpret_cast<__nv_bfloat16*>(sm + kOffUV + sw128(t, tid >> 3) + (tid & 7) * 2) = f2bf(u[t]);
        if (SAVE && t0 + t < T) g.sa[base + (size_t)(t0 + t) * stride_t + tid] = u[t];
      }
      PROF_MARK(11);
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
      if (!SAVE) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tmem + kColD1, desc_mn(sbase + kOffBKe + k * 2048, 16384), desc_mn(sbase + kOffUV + k * 2048, 8192),
                    idesc4, k > 0);
      } else {  // one accumulator per 16-step block so the intermediate states can be written out
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          umma_bf16(tmem + kColD1 + 64 * q, desc_mn(sbase + kOffBKe + q * 2048, 16384),
                    desc_mn(sbase + kOffUV + q * 2048, 8192), idesc4, 0);
          umma_bf16(tmem + kColD1 + 64 * q, desc_mn(sbase + kOffBKe + (4 + q) * 2048, 16384),
                    desc_mn(sbase + kOffUV + (4 + q) * 2048, 8192), idesc4, 1);
        }
      }
      umma_commit(&bars[2]);
    }
    if (!mbar_wait(&bars[2], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(6);
    if (tid >= 64) {  // output rows
      const int t = t0 + trow;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + kColD2 + q * 32, v);
        tmem_ld_wait();
        if (t < T) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
            *reinterpret_cast<uint4*>(g.y + base + (size_t)t * stride_t + q * 32 + p * 8) = pack8(x);
          }
        }
      }
    }
    if (!SAVE) {
      if (tid < 64) {
        const float pl = PL[3 * NH + tid];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + lane_base + kColD1 + q * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) st[q * 32 + j] = fmaf(pl, st[q * 32 + j], __uint_as_float(v[j]));
        }
      }
    } else {
      float acc[NH];
      const float p63 = PL[3 * NH + (tid & 63)];
      const float ip63 = 1.0f / p63;
#pragma unroll
      for (int round = 0; round < 2; ++round) {
        if (round == 1) {
          tc_fence_before();
          __syncthreads();
          if (tid == 0) {
            tc_fence_after();
            constexpr uint32_t idesc4 = umma_idesc_bf16(128, 64, 1, 1);
#pragma unroll
            for (int q = 2; q < 4; ++q) {
              umma_bf16(tmem + kColD1 + 64 * (q - 2), desc_mn(sbase + kOffBKe + q * 2048, 16384),
                        desc_mn(sbase + kOffUV + q * 2048, 8192), idesc4, 0);
              umma_bf16(tmem + kColD1 + 64 * (q - 2), desc_mn(sbase + kOffBKe + (4 + q) * 2048, 16384),
                        desc_mn(sbase + kOffUV + (4 + q) * 2048, 8192), idesc4, 1);
            }
            umma_commit(&bars[3]);
          }
          if (!mbar_wait(&bars[3], par, failed)) { *failed = 1; }
          tc_fence_after();
        }
        if (tid < 64) {
#pragma unroll
          for (int qq = 0; qq < 2; ++qq) {
            const int q = round * 2 + qq;  // 16-step block inside the chunk
            const float pq = PL[q * NH + tid];
            const float ratio = pq * ip63;
            const int ck = c * 4 + q;
            float* dst = g.ckpt + ((size_t)ck * BH + bh) * NH * NH + tid;
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
              uint32_t v[32];
              tmem_ld_32x32(tmem + lane_base + kColD1 + 64 * qq + hlf * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int vi = hlf * 32 + j;
                acc[vi] = (q == 0 ? 0.f : acc[vi]) + __uint_as_float(v[j]);
                if (ck < nck) dst[(size_t)vi * NH] = fmaf(pq, st[vi], ratio * acc[vi]);
              }
            }
          }
        }
      }
      if (tid < 64) {
#pragma unroll
        for (int vi = 0; vi < NH; ++vi) st[vi] = fmaf(p63, st[vi], acc[vi]);
      }
    }
    if (tid < 64) {  // bf16 image of the new state for the next chunk
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = st[8 * p + j];
        *reinterpret_cast<uint4*>(sm + kOffS + sw128(tid, p)) = pack8(x);
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(7);
  }
  if (tid < 64 && g.sT != nullptr) {
#pragma unroll
    for (int v = 0; v < NH; ++v) g.sT[((size_t)bh * NH + v) * NH + tid] = st[v];
  }
  if (!ok && tid == 0) atomicExch(&g_wkv_chunk_error, 0x30000 | (bh & 0xffff));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool wkv7_chunk_supported(const WkvArgs& p) {
  return p.is_bf16 && p.N == NH && (p.sa == nullptr || p.interval == 16);
}

int wkv7_chunk_forward(const WkvArgs& p, cudaStream_t st) {
  if (!wkv7_chunk_supported(p)) return 1;
  ChunkPtrs g;
  g.r = (const __nv_bfloat16*)p.r; g.w = (const __nv_bfloat16*)p.w; g.k = (const __nv_bfloat16*)p.k;
  g.v = (const __nv_bfloat16*)p.v; g.a = (const __nv_bfloat16*)p.a; g.b = (const __nv_bfloat16*)p.b;
  g.y = (__nv_bfloat16*)p.y; g.s0 = p.s0; g.sT = p.sT; g.sa = p.sa; g.ckpt = p.ckpt;
  const int BH = p.B * p.H;
  if (p.sa != nullptr) {
    auto kern = wkv7_chunk_fwd_kernel<true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    kern<<<BH, kThreads, kSmemBytes, st>>>(g, p.T, p.H, BH);
  } else {
    auto kern = wkv7_chunk_fwd_kernel<false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    kern<<<BH, kThreads, kSmemBytes, st>>>(g, p.T, p.H, BH);
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
