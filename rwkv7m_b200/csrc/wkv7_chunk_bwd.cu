// Backward of the chunked WKV7 recurrence on the 5th-generation tensor cores (head size 64, bf16 vectors).
//
// Per chunk of 64 steps (notation of wkv7_chunk.cu; S0 / S1 = state before / after the chunk, U saved by the
// forward pass, G = diag(P_L) dS1^T):
//   dUdir = A_rb^T dY + B~ G            dVp = A_rk^T dY + K~ G                         (one accumulator, M = 128)
//   dZ    = (I - A_ab)^-T dUdir         backward substitution in fp32 on the CUDA cores
//   dV    = dVp + A_ak^T dZ
//   dA_ab = tril<(dZ U^T)  dA_ak = tril<(dZ V^T)  dA_rb = tril<=(dY U^T)  dA_rk = tril<=(dY V^T)   (one MMA)
//   dA~   = dZ S0 + dA_ab B~ + dA_ak K~      dR~ = dY S0 + dA_rb B~ + dA_rk K~
//   DB    = dA_ab^T A~ + dA_rb^T R~ + U G^T  DK  = dA_ak^T A~ + dA_rk^T R~ + V G^T
//   dS0^T = G + R~^T dY + A~^T dZ
//   dr = dR~ P_t,  da = dA~ P_{t-1},  db = DB / P_t,  dk = DK / P_t
//   dlogP_t = r~ dR~ - b~ DB - k~ DK + (a~ dA~)_{t+1}  (+ <dS1, S1> per key channel at the last step)
//   dw_t = logd_t * sum_{t' >= t} dlogP_t'
// One CTA per (batch, head) walks the chunks from last to first; the fp32 master copy of dS lives in the
// registers of 64 threads.  Every product is a tcgen05.mma with M = 128 over 128-byte-swizzled bf16 tiles in
// shared memory, accumulators in tensor memory.  All waits are bounded.
#include "common.cuh"
#include "kernels.h"
#include "wkv7_chunk.cuh"

namespace rk {

using namespace chunk;

namespace {

constexpr int L = 64;
constexpr int NH = 64;
constexpr int kThreads = 128;
constexpr int kFStride = 68;

constexpr uint32_t kOffAR = 0;                       // [128][64] bf16: A~ | R~
constexpr uint32_t kOffBK = kOffAR + 16384;          // [128][64] bf16: B~ | K~
constexpr uint32_t kOffUV = kOffBK + 16384;          // [128][64] bf16: U | V
constexpr uint32_t kOffZY = kOffUV + 16384;          // [128][64] bf16: dZ | dY
constexpr uint32_t kOffS0 = kOffZY + 16384;          // [64][64] bf16: S0^T  (row = key channel)
constexpr uint32_t kOffG = kOffS0 + 8192;            // [64][64] bf16: G = diag(P_L) dS1^T
constexpr uint32_t kOffX = kOffG + 8192;             // [128][128] bf16 as two [128][64] column blocks: A then dA matrices
constexpr uint32_t kOffF = kOffX + 32768;            // fp32 [64][68]: A_ab; later (a~ dA~)
constexpr uint32_t kOffZ = kOffF + L * kFStride * 4; // fp32 [64][68]: dUdir; later the dlogP terms
constexpr uint32_t kOffLP = kOffZ + L * kFStride * 4;// fp32 [64][68]: inclusive cumulative log decay
constexpr uint32_t kOffPL = kOffLP + L * kFStride * 4; // fp32 [64]: P_L
constexpr uint32_t kOffBar = kOffPL + NH * 4;
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kC1 = 0;     // 128: A matrices, later dA matrices
constexpr uint32_t kC2 = 128;   // 64: dUdir (lanes 0-63) | dV (lanes 64-127)
constexpr uint32_t kC3 = 192;   // 64: dA~ | dR~
constexpr uint32_t kC4 = 256;   // 64: DB | DK
constexpr uint32_t kC6 = 320;   // 64: R~^T dY + A~^T dZ (lanes 0-63)

struct BwdPtrs {
  const __nv_bfloat16 *r, *w, *k, *v, *a, *b, *dy;
  const float *sa, *s0, *ckpt, *dsT;
  __nv_bfloat16 *dr, *dw, *dk, *dv, *da, *db;
  float* ds0;
};

__device__ int g_wkv_chunk_bwd_error = 0;

#ifdef RK_WKV_PROF
__device__ long long g_wkv_chunk_bwd_prof[16];
#define PROF_MARK(i)                                                          \
  do {                                                                        \
    if (blockIdx.x == 0 && tid == 0) {                                        \
      const long long now_ = clock64();                                       \
      g_wkv_chunk_bwd_prof[i] += now_ - prof_t;                               \
      prof_t = now_;                                                          \
    }                                                                         \
  } while (0)
#else
#define PROF_MARK(i) do { } while (0)
#endif

}  // namespace

namespace {

__global__ void __launch_bounds__(kThreads, 1) wkv7_chunk_bwd_kernel(BwdPtrs g, int T, int H, int BH) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(sm);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 32);
  volatile int* failed = reinterpret_cast<volatile int*>(sm + kOffBar + 40);
  float* F = reinterpret_cast<float*>(sm + kOffF);
  float* Zs = reinterpret_cast<float*>(sm + kOffZ);
  float* LP = reinterpret_cast<float*>(sm + kOffLP);
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
  const int piece = 2 * warp + ((tid >> 4) & 1), lq = tid & 15;

  // fp32 master copy of dS: thread k (< 64) holds row k of dS^T, i.e. dS[v][k] for all v
  float ds[NH];
  if (tid < 64) {
#pragma unroll
    for (int v = 0; v < NH; ++v) ds[v] = g.dsT != nullptr ? g.dsT[((size_t)bh * NH + v) * NH + tid] : 0.f;
  }

  const int nchunks = (T + L - 1) / L;
  const int nck = (T + 15) / 16;
  bool ok = true;
#ifdef RK_WKV_PROF
  long long prof_t = clock64();
#endif
  uint32_t par = 0;
  for (int c = nchunks - 1; c >= 0; --c, par ^= 1u) {
    const int t0 = c * L;
    const float* S0g = c == 0 ? g.s0 + (size_t)bh * NH * NH : g.ckpt + ((size_t)(c * 4 - 1) * BH + bh) * NH * NH;
    const float* S1g = g.ckpt + ((size_t)min(c * 4 + 3, nck - 1) * BH + bh) * NH * NH;
    // ---- P0: operand tiles ------------------------------------------------------------------------------------
    {
      const size_t go0 = base + (size_t)(t0 + 4 * lq) * stride_t + piece * 8;
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      // v and dy are copied unchanged: asynchronous 16-byte copies straight into the swizzled tiles
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * lq + i;
        const uint32_t off = sw128(row, piece);
        if (t0 + row < T) {
          cp_async16(sm + kOffUV + 8192 + off, g.v + go0 + (size_t)i * stride_t);
          cp_async16(sm + kOffZY + 8192 + off, g.dy + go0 + (size_t)i * stride_t);
        } else {
          *reinterpret_cast<uint4*>(sm + kOffUV + 8192 + off) = zero;
          *reinterpret_cast<uint4*>(sm + kOffZY + 8192 + off) = zero;
        }
      }
      uint4 rw[4], ra[4], rr[4], rb[4], rk[4];
      float4 u0[4], u1[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool valid = t0 + 4 * lq + i < T;
        const size_t go = go0 + (size_t)i * stride_t;
        rw[i] = valid ? *reinterpret_cast<const uint4*>(g.w + go) : zero;
        ra[i] = valid ? *reinterpret_cast<const uint4*>(g.a + go) : zero;
        rr[i] = valid ? *reinterpret_cast<const uint4*>(g.r + go) : zero;
        rb[i] = valid ? *reinterpret_cast<const uint4*>(g.b + go) : zero;
        rk[i] = valid ? *reinterpret_cast<const uint4*>(g.k + go) : zero;
        u0[i] = valid ? *reinterpret_cast<const float4*>(g.sa + go) : make_float4(0.f, 0.f, 0.f, 0.f);
        u1[i] = valid ? *reinterpret_cast<const float4*>(g.sa + go + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float lp[4][8], ex[8];
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
        ex[j] = tot - lp[3][j];
        if (lq == 15) PL[piece * 8 + j] = __expf(tot);
      }
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
          const float c_ = ex[j] + lp[i][j];
          e1[j] = __expf(c_);
          inv[j] = __frcp_rn(e1[j]);
          y[j] = c_;
        }
        float* lpd = LP + row * kFStride + piece * 8;
        *reinterpret_cast<float4*>(lpd) = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4*>(lpd + 4) = make_float4(y[4], y[5], y[6], y[7]);
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
        unpack8(rk[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * inv[j];
        *reinterpret_cast<uint4*>(sm + kOffBK + 8192 + off) = pack8(y);
        y[0] = u0[i].x; y[1] = u0[i].y; y[2] = u0[i].z; y[3] = u0[i].w;
        y[4] = u1[i].x; y[5] = u1[i].y; y[6] = u1[i].z; y[7] = u1[i].w;
        *reinterpret_cast<uint4*>(sm + kOffUV + off) = pack8(y);
#pragma unroll
        for (int j = 0; j < 8; ++j) eprev[j] = e1[j];
      }
    }
    PROF_MARK(0);
    // S0^T tile and the <dS1, S1> term of the decay gradient (thread = key channel)
    float lterm = 0.f;
    if (tid < 64) {
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int v = 8 * p + j;
          x[j] = S0g[(size_t)v * NH + tid];
          lterm = fmaf(ds[v], S1g[(size_t)v * NH + tid], lterm);
        }
        *reinterpret_cast<uint4*>(sm + kOffS0 + sw128(tid, p)) = pack8(x);
      }
    }
    PROF_MARK(1);
    cp_async_wait_all();
    fence_proxy_async_smem();
    __syncthreads();
    PROF_MARK(2);
    // ---- MMA 1: forward score matrices ------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kC1, desc_k(sbase + kOffAR + k * 32), desc_k(sbase + kOffBK + k * 32), idesc, k > 0);
      umma_commit(&bars[0]);
    }
    if (tid < 64) {  // G = diag(P_L) dS1^T while the MMA runs
      const float pl = PL[tid];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = pl * ds[8 * p + j];
        *reinterpret_cast<uint4*>(sm + kOffG + sw128(tid, p)) = pack8(x);
      }
    }
    if (!mbar_wait(&bars[0], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(3);
#pragma unroll
    for (int hq = 0; hq < 4; ++hq) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kC1 + hq * 32, v);
      tmem_ld_wait();
      const int s0 = (hq & 1) * 32;
      uint8_t* blk = sm + kOffX + (hq >> 1) * 16384;
      if (tid < 64) {
        if (hq < 2) {  // A_ab also in fp32 (row t contiguous over s) for the substitution
          float* dst = F + trow * kFStride + s0;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) =
                make_float4(s0 + j < trow ? __uint_as_float(v[j]) : 0.f, s0 + j + 1 < trow ? __uint_as_float(v[j + 1]) : 0.f,
                            s0 + j + 2 < trow ? __uint_as_float(v[j + 2]) : 0.f, s0 + j + 3 < trow ? __uint_as_float(v[j + 3]) : 0.f);
        }
        store_masked_bf16(blk, trow, (hq & 1) * 4, v, s0, [&](int s) { return s < trow; });
      } else {
        store_masked_bf16(blk, 64 + trow, (hq & 1) * 4, v, s0, [&](int s) { return s <= trow; });
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(4);
    // ---- MMA 2: dUdir = A_rb^T dY + B~ G (lanes 0-63),  dVp = A_rk^T dY + K~ G (lanes 64-127) ---------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 64, 1, 1);
      constexpr uint32_t id_km = umma_idesc_bf16(128, 64, 0, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // A = rows 64-127 of the score tile read M-major (both column blocks), K = t
        umma_bf16(tmem + kC2, desc_mn(sbase + kOffX + 8192 + k * 2048, 16384), desc_mn(sbase + kOffZY + 8192 + k * 2048, 8192),
                  id_mm, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // A = [B~; K~] K-major, B = G read N-major, K = key channel
        umma_bf16(tmem + kC2, desc_k(sbase + kOffBK + k * 32), desc_mn(sbase + kOffG + k * 2048, 8192), id_km, 1);
      umma_commit(&bars[1]);
    }
    if (!mbar_wait(&bars[1], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(5);
    if (tid < 64) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + kC2 + q * 32, v);
        tmem_ld_wait();
        float* dst = Zs + trow * kFStride + q * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                            __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
      asm volatile("bar.sync 1, 64;" ::: "memory");
      PROF_MARK(6);
      // backward substitution, thread = value column: once dZ_t is final it is pushed into every earlier row
      float z[L];
#pragma unroll
      for (int t = 0; t < L; ++t) z[t] = Zs[t * kFStride + tid];
#pragma unroll
      for (int t = L - 1; t > 0; --t) {
#pragma unroll
        for (int s4 = 0; s4 < L / 4; ++s4) {
          if (4 * s4 < t) {
            const float4 A = *reinterpret_cast<const float4*>(F + t * kFStride + 4 * s4);
            if (4 * s4 + 0 < t) z[4 * s4 + 0] = fmaf(A.x, z[t], z[4 * s4 + 0]);
            if (4 * s4 + 1 < t) z[4 * s4 + 1] = fmaf(A.y, z[t], z[4 * s4 + 1]);
            if (4 * s4 + 2 < t) z[4 * s4 + 2] = fmaf(A.z, z[t], z[4 * s4 + 2]);
            if (4 * s4 + 3 < t) z[4 * s4 + 3] = fmaf(A.w, z[t], z[4 * s4 + 3]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < L; ++t)
        *reinterpret_cast<__nv_bfloat16*>(sm + kOffZY + sw128(t, tid >> 3) + (tid & 7) * 2) = f2bf(z[t]);
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(7);
    // ---- MMA 3-7: everything that needs dZ but not the dA matrices ------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 64, 1, 1);
      constexpr uint32_t id_kk64 = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t id_kk128 = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // dV += A_ak^T dZ (lanes 64-127; lanes 0-63 receive A_ab^T dZ, unused)
        umma_bf16(tmem + kC2, desc_mn(sbase + kOffX + k * 2048, 16384), desc_mn(sbase + kOffZY + k * 2048, 8192), id_mm, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // dA matrices = [dZ; dY] [U; V]^T
        umma_bf16(tmem + kC1, desc_k(sbase + kOffZY + k * 32), desc_k(sbase + kOffUV + k * 32), id_kk128, k > 0);
#pragma unroll
      for (int k = 0; k < 8; ++k)   // A~^T dZ + R~^T dY  (A = [A~; R~] read M-major; second M block is ignored)
        umma_bf16(tmem + kC6, desc_mn(sbase + kOffAR + k * 2048, 16384), desc_mn(sbase + kOffZY + k * 2048, 8192), id_mm, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // [dZ; dY] S0
        umma_bf16(tmem + kC3, desc_k(sbase + kOffZY + k * 32), desc_k(sbase + kOffS0 + k * 32), id_kk64, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // [U; V] G^T
        umma_bf16(tmem + kC4, desc_k(sbase + kOffUV + k * 32), desc_k(sbase + kOffG + k * 32), id_kk64, k > 0);
      umma_commit(&bars[2]);
    }
    if (!mbar_wait(&bars[2], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(8);
#pragma unroll
    for (int hq = 0; hq < 4; ++hq) {   // dA matrices, masked, into the two column blocks of X
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kC1 + hq * 32, v);
      tmem_ld_wait();
      const int s0 = (hq & 1) * 32;
      uint8_t* blk = sm + kOffX + (hq >> 1) * 16384;
      if (tid < 64) store_masked_bf16(blk, trow, (hq & 1) * 4, v, s0, [&](int s) { return s < trow; });
      else store_masked_bf16(blk, 64 + trow, (hq & 1) * 4, v, s0, [&](int s) { return s <= trow; });
    }
    if (tid >= 64) {   // dV rows
      const int t = t0 + trow;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + kC2 + q * 32, v);
        tmem_ld_wait();
        if (t < T) {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
            *reinterpret_cast<uint4*>(g.dv + base + (size_t)t * stride_t + q * 32 + p * 8) = pack8(x);
          }
        }
      }
    } else {           // dS0^T = G + R~^T dY + A~^T dZ
      const float pl = PL[tid];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + kC6 + q * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) ds[q * 32 + j] = fmaf(pl, ds[q * 32 + j], __uint_as_float(v[j]));
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(9);
    // ---- MMA 8-9: the products with the dA matrices ----------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_km = umma_idesc_bf16(128, 64, 0, 1);
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 64, 1, 1);
#pragma unroll
      for (int jb = 0; jb < 2; ++jb)
#pragma unroll
        for (int k = 0; k < 4; ++k)   // [dA~; dR~] += dA(:, block jb) [B~ or K~]
          umma_bf16(tmem + kC3, desc_k(sbase + kOffX + jb * 16384 + k * 32),
                    desc_mn(sbase + kOffBK + jb * 8192 + k * 2048, 8192), id_km, 1);
#pragma unroll
      for (int k = 0; k < 8; ++k)     // [DB; DK] += dA^T [A~; R~]
        umma_bf16(tmem + kC4, desc_mn(sbase + kOffX + k * 2048, 16384), desc_mn(sbase + kOffAR + k * 2048, 8192), id_mm, 1);
      umma_commit(&bars[3]);
    }
    if (!mbar_wait(&bars[3], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(10);
    // ---- epilogue: undo the rescaling, write dr/dk/da/db, assemble the decay gradient --------------------------------
    {
      const int t = t0 + trow;
      const bool lower = tid < 64;          // lanes 0-63: (dA~, DB) of row t;  lanes 64-127: (dR~, DK) of row t
      float e1r[NH];                        // upper lanes keep r~ dR~ - k~ DK until the lower lanes have stored their term
      const uint8_t* arow = sm + kOffAR + (lower ? 0 : 8192);
      const uint8_t* brow = sm + kOffBK + (lower ? 0 : 8192);
      __nv_bfloat16* g3 = (lower ? g.da : g.dr) + base + (size_t)t * stride_t;
      __nv_bfloat16* g4 = (lower ? g.db : g.dk) + base + (size_t)t * stride_t;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        float d3[32], d4[32];
        tmem_ld_f32(tmem + lane_base + kC3 + q * 32, d3);
        tmem_ld_f32(tmem + lane_base + kC4 + q * 32, d4);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int k0 = q * 32 + p * 8;
          float av[8], bv[8], s3[8], s4[8], o3[8], o4[8];
          unpack8(*reinterpret_cast<const uint4*>(arow + sw128(trow, q * 4 + p)), av);
          unpack8(*reinterpret_cast<const uint4*>(brow + sw128(trow, q * 4 + p)), bv);
          const float* lp = LP + trow * kFStride + k0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float x = lp[j];
            s4[j] = __expf(-x);                                                   // 1 / P_t
            s3[j] = lower ? (trow > 0 ? __expf(lp[j - kFStride]) : 1.f) : __expf(x);  // P_{t-1} or P_t
            o3[j] = d3[p * 8 + j] * s3[j];
            o4[j] = d4[p * 8 + j] * s4[j];
          }
          if (t < T) {
            *reinterpret_cast<uint4*>(g3 + k0) = pack8(o3);
            *reinterpret_cast<uint4*>(g4 + k0) = pack8(o4);
          }
          if (lower) {
            float* zq = Zs + trow * kFStride + k0;
            float* fq = F + trow * kFStride + k0;
            *reinterpret_cast<float4*>(zq) = make_float4(-bv[0] * d4[p * 8 + 0], -bv[1] * d4[p * 8 + 1], -bv[2] * d4[p * 8 + 2], -bv[3] * d4[p * 8 + 3]);
            *reinterpret_cast<float4*>(zq + 4) = make_float4(-bv[4] * d4[p * 8 + 4], -bv[5] * d4[p * 8 + 5], -bv[6] * d4[p * 8 + 6], -bv[7] * d4[p * 8 + 7]);
            *reinterpret_cast<float4*>(fq) = make_float4(av[0] * d3[p * 8 + 0], av[1] * d3[p * 8 + 1], av[2] * d3[p * 8 + 2], av[3] * d3[p * 8 + 3]);
            *reinterpret_cast<float4*>(fq + 4) = make_float4(av[4] * d3[p * 8 + 4], av[5] * d3[p * 8 + 5], av[6] * d3[p * 8 + 6], av[7] * d3[p * 8 + 7]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) e1r[k0 + j] = av[j] * d3[p * 8 + j] - bv[j] * d4[p * 8 + j];
          }
        }
      }
      PROF_MARK(11);
      __syncthreads();
      if (!lower) {
#pragma unroll
        for (int k4 = 0; k4 < NH; k4 += 4) {
          float4* zq = reinterpret_cast<float4*>(Zs + trow * kFStride + k4);
          float4 o = *zq;
          o.x += e1r[k4]; o.y += e1r[k4 + 1]; o.z += e1r[k4 + 2]; o.w += e1r[k4 + 3];
          *zq = o;
        }
      }
      __syncthreads();
      PROF_MARK(12);
      if (lower) {   // thread = key channel: reverse cumulative sum over the steps of the chunk
        float run = lterm;
#pragma unroll 8
        for (int tt = L - 1; tt >= 0; --tt) {
          run += Zs[tt * kFStride + tid] + (tt < L - 1 ? F[(tt + 1) * kFStride + tid] : 0.f);
          const float logd = LP[tt * kFStride + tid] - (tt > 0 ? LP[(tt - 1) * kFStride + tid] : 0.f);
          if (t0 + tt < T) g.dw[base + (size_t)(t0 + tt) * stride_t + tid] = f2bf(run * logd);
        }
      }
    }
    PROF_MARK(13);
    tc_fence_before();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(14);
  }
  if (tid < 64 && g.ds0 != nullptr) {
#pragma unroll
    for (int v = 0; v < NH; ++v) g.ds0[((size_t)bh * NH + v) * NH + tid] = ds[v];
  }
  if (!ok && tid == 0) atomicExch(&g_wkv_chunk_bwd_error, 0x40000 | (bh & 0xffff));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool wkv7_chunk_bwd_supported(const WkvArgs& p) { return p.is_bf16 && p.N == NH && p.interval == 16; }

int wkv7_chunk_backward(const WkvArgs& p, cudaStream_t st) {
  if (!wkv7_chunk_bwd_supported(p)) return 1;
  BwdPtrs g;
  g.r = (const __nv_bfloat16*)p.r; g.w = (const __nv_bfloat16*)p.w; g.k = (const __nv_bfloat16*)p.k;
  g.v = (const __nv_bfloat16*)p.v; g.a = (const __nv_bfloat16*)p.a; g.b = (const __nv_bfloat16*)p.b;
  g.dy = (const __nv_bfloat16*)p.dy; g.sa = p.sa; g.s0 = p.s0; g.ckpt = p.ckpt; g.dsT = p.dsT;
  g.dr = (__nv_bfloat16*)p.dr; g.dw = (__nv_bfloat16*)p.dw; g.dk = (__nv_bfloat16*)p.dk;
  g.dv = (__nv_bfloat16*)p.dv; g.da = (__nv_bfloat16*)p.da; g.db = (__nv_bfloat16*)p.db; g.ds0 = p.ds0;
  const int BH = p.B * p.H;
  auto kern = wkv7_chunk_bwd_kernel;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  kern<<<BH, kThreads, kSmemBytes, st>>>(g, p.T, p.H, BH);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

#ifdef RK_WKV_PROF
void wkv7_chunk_bwd_prof(long long* out, bool reset) {
  cudaMemcpyFromSymbol(out, g_wkv_chunk_bwd_prof, 16 * sizeof(long long));
  if (reset) { long long z[16] = {0}; cudaMemcpyToSymbol(g_wkv_chunk_bwd_prof, z, sizeof(z)); }
}
#endif

int wkv7_chunk_bwd_error(bool reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_wkv_chunk_bwd_error, sizeof(int));
  if (reset && v != 0) { const int z = 0; cudaMemcpyToSymbol(g_wkv_chunk_bwd_error, &z, sizeof(int)); }
  return v;
}

}  // namespace rk
