// Backward of the chunked WKV7 recurrence on the 5th-generation tensor cores (head size 64, bf16 vectors).
//
// Per chunk of 64 steps (notation of wkv7_chunk.cu; S0 / S1 = state before / after the chunk, U saved by the
// forward pass, G = diag(P_L) dS1^T):
//   dUdir = A_rb^T dY + B~ G            dVp = A_rk^T dY + K~ G                         (one accumulator, M = 128)
//   dZ    = (I - A_ab)^-T dUdir         the inverse is formed blockwise in fp32 on the CUDA cores (while the tensor
//                                       cores form dUdir) and applied, transposed, by one more MMA
//   dV    = dVp + A_ak^T dZ
//   dA_ab = tril<(dZ U^T)  dA_ak = tril<(dZ V^T)  dA_rb = tril<=(dY U^T)  dA_rk = tril<=(dY V^T)   (one MMA)
//   dA~   = dZ S0 + dA_ab B~ + dA_ak K~      dR~ = dY S0 + dA_rb B~ + dA_rk K~
//   DB    = dA_ab^T A~ + dA_rb^T R~ + U G^T  DK  = dA_ak^T A~ + dA_rk^T R~ + V G^T
//   dS0^T = G + R~^T dY + A~^T dZ
//   dr = dR~ P_t,  da = dA~ P_{t-1},  db = DB / P_t,  dk = DK / P_t
//   dlogP_t = r~ dR~ - b~ DB - k~ DK + (a~ dA~)_{t+1}  (+ <dS1, S1> per key channel at the last step)
//   dw_t = logd_t * sum_{t' >= t} dlogP_t'
// One CTA of 16 warps per (batch, head) walks the chunks from last to first; the fp32 master copy of dS lives in
// registers (16 values per thread: a warp reaches one 32-lane quarter of tensor memory, four warps share a quarter
// and split the accumulator columns).  Every product is a tcgen05.mma with M = 128 over 128-byte-swizzled bf16 tiles in
// shared memory, accumulators in tensor memory.  The raw tiles of the next chunk (the previous one in time) are
// fetched with asynchronous copies while the second half of the current chunk runs: dY, V and U land directly in
// their operand slots, which the remaining products no longer read, the five tiles that are rescaled go to a
// staging area.  All waits are bounded.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "wkv7_chunk.cuh"

namespace rk {

using namespace chunk;

namespace {

constexpr int L = 64;
constexpr int NH = 64;
constexpr int kThreads = 512;   // 16 warps: four per tensor-memory lane quarter, each on a quarter of the columns
constexpr int kFStride = 68;

constexpr uint32_t kOffAR = 0;                       // [128][64] bf16: A~ | R~
constexpr uint32_t kOffBK = kOffAR + 16384;          // [128][64] bf16: B~ | K~
constexpr uint32_t kOffUV = kOffBK + 16384;          // [128][64] bf16: U | V
constexpr uint32_t kOffZY = kOffUV + 16384;          // [128][64] bf16: dZ | dY
constexpr uint32_t kOffS0 = kOffZY + 16384;          // [64][64] bf16: S0^T  (row = key channel)
constexpr uint32_t kOffG = kOffS0 + 8192;            // [64][64] bf16: G = diag(P_L) dS1^T
constexpr uint32_t kOffX = kOffG + 8192;             // [128][128] bf16 as two [128][64] column blocks: A then dA matrices
                                                     // (rows 0-63 of block 0 hold (I - A_ab)^-1 instead of A_ab)
constexpr uint32_t kOffF = kOffX + 32768;            // fp32 [64][68]: A_ab, then its inverse; later (a~ dA~)
constexpr uint32_t kOffZ = kOffF + L * kFStride * 4; // fp32 [64][68]: the dlogP terms
constexpr uint32_t kOffLP = kOffZ + L * kFStride * 4;// fp32 [64][68]: inclusive cumulative log decay
constexpr uint32_t kOffPL = kOffLP + L * kFStride * 4; // fp32 [64]: P_L
constexpr uint32_t kOffLT = kOffPL + NH * 4;         // fp32 [4][64]: quarters of <dS1, S1>
constexpr uint32_t kOffBS = kOffLT + 4 * NH * 4;     // fp32 [8][64]: block sums of the decay-gradient scan
constexpr uint32_t kOffTot = kOffBS + 8 * NH * 4;    // fp32 [64]: cumulative log decay after the first 32 rows
constexpr uint32_t kOffW = kOffTot + NH * 4;         // fp32 scratch of the blocked inverse
constexpr uint32_t kOffStage = (kOffW + kInvWorkFloats * 4 + 1023u) & ~1023u;   // raw a | r | b | k | w tiles of the next chunk
constexpr uint32_t kOffBar = kOffStage + 5 * 8192;
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kC1 = 0;     // 128: A matrices, later dA matrices
constexpr uint32_t kC2 = 128;   // 64: dUdir (lanes 0-63) | dV (lanes 64-127)
constexpr uint32_t kC3 = 192;   // 64: dA~ | dR~
constexpr uint32_t kC4 = 256;   // 64: DB | DK
constexpr uint32_t kC6 = 320;   // 64: dZ (lanes 0-63), then R~^T dY + A~^T dZ (lanes 0-63)

static_assert(kFStride == kInvStride, "the inverse routine reads the A_ab scratch with its own row stride");

// tensor maps of the eight per-chunk tiles in destination order: a, r, b, k, w (staging area), saved U, v, dY
struct BwdMaps { CUtensorMap m[8]; };

struct BwdPtrs {
  const __nv_bfloat16 *r, *w, *k, *v, *a, *b, *dy, *sa;
  const __nv_bfloat16 *dr_add, *dk_add, *dv_add;   // optional: gradients that reach r, k, v by another path, summed here
  const float *s0, *ckpt, *dsT;
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

// 16 accumulator values of one row -> two swizzled 16-byte bf16 pieces (pieces p0, p0 + 1 of `row`)
__device__ __forceinline__ void store16_bf16(uint8_t* tile, int row, int p0, const uint32_t (&v)[16]) {
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
    *reinterpret_cast<uint4*>(tile + sw128(row, p0 + p)) = pack8(x);
  }
}

__global__ void __launch_bounds__(kThreads, 1) wkv7_chunk_bwd_kernel(BwdPtrs g, const __grid_constant__ BwdMaps maps,
                                                                     int use_tma, int T, int H, int BH) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(sm);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 48);
  volatile int* failed = reinterpret_cast<volatile int*>(sm + kOffBar + 56);
  float* F = reinterpret_cast<float*>(sm + kOffF);
  float* Wk = reinterpret_cast<float*>(sm + kOffW);
  float* Zs = reinterpret_cast<float*>(sm + kOffZ);
  float* LP = reinterpret_cast<float*>(sm + kOffLP);
  float* PL = reinterpret_cast<float*>(sm + kOffPL);
  float* LT = reinterpret_cast<float*>(sm + kOffLT);
  float* BS = reinterpret_cast<float*>(sm + kOffBS);
  float* TOT = reinterpret_cast<float*>(sm + kOffTot);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, bi = bh / H, hi = bh - bi * H;
  const size_t stride_t = (size_t)H * NH;
  const size_t base = (size_t)bi * T * stride_t + (size_t)hi * NH;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
    mbar_init(&bars[5], 1);   // tile loads: one request per chunk, its arrival plus the bytes of eight tiles
    if (use_tma) {
#pragma unroll
      for (int i = 0; i < 8; ++i) tma_prefetch_desc(&maps.m[i]);
    }
    *failed = 0;
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // tensor-memory view of this thread: row m of the 128-row accumulators (a warp reaches the 32 lanes of its quarter),
  // column quarter ch: 16 of the 64 columns of the narrow accumulators, 32 of the 128 columns of the score matrices
  const int wq = warp & 3, ch = warp >> 2;
  const int m = wq * 32 + lane;
  const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
  const bool lower = wq < 2;
  const int trow = m & 63;
  const int cb = ch >> 1, cq = ch & 1;      // score matrices: column block (products with B~ / with K~) and its half

  // fp32 master copy of dS: thread (k = trow, ch) of the lower warps holds dS[v][k] for v in [16 ch, 16 ch + 16)
  float ds[16];
  if (lower) {
#pragma unroll
    for (int j = 0; j < 16; ++j) ds[j] = g.dsT != nullptr ? g.dsT[((size_t)bh * NH + 16 * ch + j) * NH + trow] : 0.f;
  }

  const int nchunks = (T + L - 1) / L;
  bool ok = true;
  float lt_next = 0.f;
#ifdef RK_WKV_PROF
  long long prof_t = clock64();
#endif
  // Asynchronous copies of one chunk's raw tiles (8 lanes per 128-byte row, swizzled like the operand tiles): dY, V
  // and the saved U rows go straight into their operand slots, a / r / b / k / w into the staging area.
  auto fetch_chunk = [&](int cc) {
    const int tc = cc * L;
    if (use_tma) {
      // one thread hands the eight [64 steps][64 channels] boxes to the copy engine, which writes the swizzled operand
      // layout and zero-fills steps past the end of the sequence; the mbarrier counts the bytes
      if (tid == 0) {
        mbar_expect_tx(&bars[5], 8u * 8192u);
        const int x = hi * NH;
        tma_load_3d(sm + kOffStage, &maps.m[0], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffStage + 8192, &maps.m[1], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffStage + 16384, &maps.m[2], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffStage + 24576, &maps.m[3], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffStage + 32768, &maps.m[4], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffUV, &maps.m[5], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffUV + 8192, &maps.m[6], &bars[5], x, tc, bi);
        tma_load_3d(sm + kOffZY + 8192, &maps.m[7], &bars[5], x, tc, bi);
      }
    } else {
    const int p8 = tid & 7, row = tid >> 3;
    const uint32_t off = sw128(row, p8);
    const size_t go = base + (size_t)(tc + row) * stride_t + p8 * 8;
    if (tc + row < T) {
      cp_async16(sm + kOffStage + off, g.a + go);
      cp_async16(sm + kOffStage + 8192 + off, g.r + go);
      cp_async16(sm + kOffStage + 16384 + off, g.b + go);
      cp_async16(sm + kOffStage + 24576 + off, g.k + go);
      cp_async16(sm + kOffStage + 32768 + off, g.w + go);
      cp_async16(sm + kOffUV + off, g.sa + go);
      cp_async16(sm + kOffUV + 8192 + off, g.v + go);
      cp_async16(sm + kOffZY + 8192 + off, g.dy + go);
    } else {
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(sm + kOffStage + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffStage + 8192 + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffStage + 16384 + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffStage + 24576 + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffStage + 32768 + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffUV + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffUV + 8192 + off) = zero;
      *reinterpret_cast<uint4*>(sm + kOffZY + 8192 + off) = zero;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (tid < 128) {   // the state before that chunk (fp32, converted at the top of its iteration): pull it into L2
      const float* s_in = cc == 0 ? g.s0 + (size_t)bh * NH * NH : g.ckpt + ((size_t)(cc - 1) * BH + bh) * NH * NH;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(s_in + tid * 32));
    }
  };
  fetch_chunk(nchunks - 1);
  uint32_t par = 0;
  for (int c = nchunks - 1; c >= 0; --c, par ^= 1u) {
    const int t0 = c * L;
    const float* S0g = c == 0 ? g.s0 + (size_t)bh * NH * NH : g.ckpt + ((size_t)(c - 1) * BH + bh) * NH * NH;
    const float* S1g = g.ckpt + ((size_t)c * BH + bh) * NH * NH;
    // ---- the raw tiles of this chunk were requested one chunk ago (before the loop for the first one) -------------------
    {
      // S0^T tile: thread (k, vq) converts S0[8 vq .. 8 vq + 7][k]
      {
        const int k = tid & 63, vq = tid >> 6;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = S0g[(size_t)(8 * vq + j) * NH + k];
        *reinterpret_cast<uint4*>(sm + kOffS0 + sw128(k, vq)) = pack8(x);
      }
      if (lower) {   // <dS1, S1> per key channel, one quarter of the value columns per thread
        if (c == nchunks - 1) {   // last chunk: S1 is the final state; later chunks took it from the bf16 S0 tile
          lt_next = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) lt_next = fmaf(ds[j], S1g[(size_t)(16 * ch + j) * NH + trow], lt_next);
        }
        LT[ch * NH + trow] = lt_next;
      }
      if (use_tma) {
        if (!mbar_wait(&bars[5], par, failed)) { *failed = 1; }
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
    }
    if (*failed) { ok = false; break; }
    PROF_MARK(12);
    // ---- rescale: warp w owns the 16-byte column piece w % 8 of rows 32 (w / 8) .. 32 (w / 8) + 31, lane = row ---------
    {
      const int piece = warp & 7, half = warp >> 3;
      const int row = lane + 32 * half;
      const uint32_t off = sw128(row, piece);
      const uint4 ra = *reinterpret_cast<const uint4*>(sm + kOffStage + off);
      const uint4 rr = *reinterpret_cast<const uint4*>(sm + kOffStage + 8192 + off);
      const uint4 rb = *reinterpret_cast<const uint4*>(sm + kOffStage + 16384 + off);
      const uint4 rk = *reinterpret_cast<const uint4*>(sm + kOffStage + 24576 + off);
      const uint4 rw = *reinterpret_cast<const uint4*>(sm + kOffStage + 32768 + off);
      float ld[8], lp[8];
      {
        float x[8];
        unpack8(rw, x);
        const bool valid = t0 + row < T;
#pragma unroll
        for (int j = 0; j < 8; ++j) ld[j] = valid ? -__expf(x[j]) : 0.f;
      }
      // cumulative log decay: a warp scan over its 32 rows; the warps of the second half add the first half's totals
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s_ = ld[j];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float up = __shfl_up_sync(0xffffffffu, s_, o);
          if (lane >= o) s_ += up;
        }
        lp[j] = s_;
      }
      if (half == 0 && lane == 31) {
        float* dst = TOT + piece * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(lp[0], lp[1], lp[2], lp[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(lp[4], lp[5], lp[6], lp[7]);
      }
      __syncthreads();
      if (half == 1) {
        const float4 t0v = *reinterpret_cast<const float4*>(TOT + piece * 8), t1v = *reinterpret_cast<const float4*>(TOT + piece * 8 + 4);
        lp[0] += t0v.x; lp[1] += t0v.y; lp[2] += t0v.z; lp[3] += t0v.w;
        lp[4] += t1v.x; lp[5] += t1v.y; lp[6] += t1v.z; lp[7] += t1v.w;
        if (lane == 31) {
#pragma unroll
          for (int j = 0; j < 8; ++j) PL[piece * 8 + j] = __expf(lp[j]);
        }
      }
      float e1[8], e0[8], inv[8], x[8], y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        e1[j] = __expf(lp[j]);
        e0[j] = __expf(lp[j] - ld[j]);
        inv[j] = __expf(-lp[j]);
      }
      float* lpd = LP + row * kFStride + piece * 8;
      *reinterpret_cast<float4*>(lpd) = make_float4(lp[0], lp[1], lp[2], lp[3]);
      *reinterpret_cast<float4*>(lpd + 4) = make_float4(lp[4], lp[5], lp[6], lp[7]);
      unpack8(ra, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[j] * e0[j];
      *reinterpret_cast<uint4*>(sm + kOffAR + off) = pack8(y);
      unpack8(rr, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[j] * e1[j];
      *reinterpret_cast<uint4*>(sm + kOffAR + 8192 + off) = pack8(y);
      unpack8(rb, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[j] * inv[j];
      *reinterpret_cast<uint4*>(sm + kOffBK + off) = pack8(y);
      unpack8(rk, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = x[j] * inv[j];
      *reinterpret_cast<uint4*>(sm + kOffBK + 8192 + off) = pack8(y);
    }
    fence_proxy_async_smem();
    __syncthreads();
    PROF_MARK(0);
    // ---- MMA 1: forward score matrices ------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kC1, desc_k(sbase + kOffAR + k * 32), desc_k(sbase + kOffBK + k * 32), idesc, k > 0);
      umma_commit(&bars[0]);
    }
    if (lower) {  // G = diag(P_L) dS1^T while the MMA runs
      const float pl = PL[trow];
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = pl * ds[8 * p + j];
        *reinterpret_cast<uint4*>(sm + kOffG + sw128(trow, 2 * ch + p)) = pack8(x);
      }
    }
    if (!mbar_wait(&bars[0], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(1);
    // thread (row m, quarter ch) reads 32 columns: block cb = 0 -> products with B~ (A_ab | A_rb), 1 -> with K~ (A_ak | A_rk)
    {
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kC1 + cb * 64 + cq * 32, v);
      tmem_ld_wait();
      const int s0 = cq * 32;
      uint8_t* blk = sm + kOffX + cb * 16384;
      if (lower) {
        if (cb == 0) {  // A_ab in fp32, F[t][s]: the input of the blocked inverse (its bf16 slot receives the inverse)
          float* dst = F + trow * kFStride + s0;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(
                s0 + j < trow ? __uint_as_float(v[j]) : 0.f, s0 + j + 1 < trow ? __uint_as_float(v[j + 1]) : 0.f,
                s0 + j + 2 < trow ? __uint_as_float(v[j + 2]) : 0.f, s0 + j + 3 < trow ? __uint_as_float(v[j + 3]) : 0.f);
        } else {
          store_masked_bf16(blk, trow, cq * 4, v, s0, [&](int s) { return s < trow; });   // A_ak
        }
      } else {
        store_masked_bf16(blk, 64 + trow, cq * 4, v, s0, [&](int s) { return s <= trow; });
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(2);
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
    // the inverse of I - A_ab on the CUDA cores while the tensor cores form dUdir; it lands in the A_ab operand slot
    unit_lower_inverse_64(F, Wk, sm + kOffX, tid);
    if (!mbar_wait(&bars[1], par, failed)) { *failed = 1; }
    tc_fence_after();
    PROF_MARK(3);
    if (lower) {   // dUdir rows -> bf16 operand tile in the dZ slot
      uint32_t v[16];
      tmem_ld_32x16(tmem + lane_base + kC2 + ch * 16, v);
      tmem_ld_wait();
      store16_bf16(sm + kOffZY, trow, ch * 2, v);
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(4);
    // ---- MMA dZ: dZ = (I - A_ab)^-T dUdir (lanes 0-63; lanes 64-127 receive A_ak^T dUdir, ignored) ----------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 64, 1, 1);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem + kC6, desc_mn(sbase + kOffX + k * 2048, 16384), desc_mn(sbase + kOffZY + k * 2048, 8192), id_mm, k > 0);
      umma_commit(&bars[4]);
    }
    if (!mbar_wait(&bars[4], par, failed)) { *failed = 1; }
    tc_fence_after();
    if (lower) {   // dZ rows -> bf16 operand tile, over dUdir (the finished MMA no longer reads it)
      uint32_t v[16];
      tmem_ld_32x16(tmem + lane_base + kC6 + ch * 16, v);
      tmem_ld_wait();
      store16_bf16(sm + kOffZY, trow, ch * 2, v);
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(5);
    // ---- MMA 3-7: everything that needs dZ but not the dA matrices ------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 64, 1, 1);
      constexpr uint32_t id_kk64 = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t id_kk128 = umma_idesc_bf16(128, 128, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)   // dV += A_ak^T dZ (lanes 64-127; lanes 0-63 receive T^-T dZ, unused)
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
    PROF_MARK(6);
    // U, V and dY are dead from here on (the products still to come read the score tiles and A~ / R~ / B~ / K~ only)
    // and the staging area was emptied by the rescale pass: request the previous chunk's tiles now
    if (c > 0) fetch_chunk(c - 1);
    {   // dA matrices, masked, into column block cb of X
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + kC1 + cb * 64 + cq * 32, v);
      tmem_ld_wait();
      uint8_t* blk = sm + kOffX + cb * 16384;
      if (lower) store_masked_bf16(blk, trow, cq * 4, v, cq * 32, [&](int s) { return s < trow; });
      else store_masked_bf16(blk, 64 + trow, cq * 4, v, cq * 32, [&](int s) { return s <= trow; });
    }
    {
      uint32_t v[16];
      if (!lower) {   // dV row t, columns [16 ch, 16 ch + 16)
        tmem_ld_32x16(tmem + lane_base + kC2 + ch * 16, v);
        tmem_ld_wait();
        const int t = t0 + trow;
        if (t < T) {
          const size_t go = base + (size_t)t * stride_t + ch * 16;
          uint4 extra[2];
          if (g.dv_add != nullptr) {
#pragma unroll
            for (int p = 0; p < 2; ++p) extra[p] = *reinterpret_cast<const uint4*>(g.dv_add + go + p * 8);
          }
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(v[8 * p + j]);
            if (g.dv_add != nullptr) {
              float e[8];
              unpack8(extra[p], e);
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] += e[j];
            }
            *reinterpret_cast<uint4*>(g.dv + go + p * 8) = pack8(x);
          }
        }
      } else {        // dS0^T = G + R~^T dY + A~^T dZ
        tmem_ld_32x16(tmem + lane_base + kC6 + ch * 16, v);
        tmem_ld_wait();
        const float pl = PL[trow];
#pragma unroll
        for (int j = 0; j < 16; ++j) ds[j] = fmaf(pl, ds[j], __uint_as_float(v[j]));
        // <dS0, S0> of this chunk is the <dS1, S1> term of the next one: S0 is still in its operand tile (bf16)
        lt_next = 0.f;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          float x[8];
          unpack8(*reinterpret_cast<const uint4*>(sm + kOffS0 + sw128(trow, 2 * ch + p)), x);
#pragma unroll
          for (int j = 0; j < 8; ++j) lt_next = fmaf(ds[8 * p + j], x[j], lt_next);
        }
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(7);
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
    PROF_MARK(8);
    // ---- epilogue: undo the rescaling, write dr/dk/da/db, assemble the decay gradient --------------------------------
    {
      const int t = t0 + trow;
      float e1r[16];   // upper lanes keep r~ dR~ - k~ DK until the lower lanes have stored their term
      const uint8_t* arow = sm + kOffAR + (lower ? 0 : 8192);
      const uint8_t* brow = sm + kOffBK + (lower ? 0 : 8192);
      __nv_bfloat16* g3 = (lower ? g.da : g.dr) + base + (size_t)t * stride_t;
      __nv_bfloat16* g4 = (lower ? g.db : g.dk) + base + (size_t)t * stride_t;
      const __nv_bfloat16* a3 = (lower || g.dr_add == nullptr) ? nullptr : g.dr_add + base + (size_t)t * stride_t;
      const __nv_bfloat16* a4 = (lower || g.dk_add == nullptr) ? nullptr : g.dk_add + base + (size_t)t * stride_t;
      uint32_t d3[16], d4[16];
      tmem_ld_32x16(tmem + lane_base + kC3 + ch * 16, d3);
      tmem_ld_32x16(tmem + lane_base + kC4 + ch * 16, d4);
      tmem_ld_wait();
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int k0 = ch * 16 + p * 8;
        float av[8], bv[8], o3[8], o4[8], x3[8], x4[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { x3[j] = __uint_as_float(d3[p * 8 + j]); x4[j] = __uint_as_float(d4[p * 8 + j]); }
        unpack8(*reinterpret_cast<const uint4*>(arow + sw128(trow, ch * 2 + p)), av);
        unpack8(*reinterpret_cast<const uint4*>(brow + sw128(trow, ch * 2 + p)), bv);
        const float* lp = LP + trow * kFStride + k0;
        const float4 c0 = *reinterpret_cast<const float4*>(lp), c1 = *reinterpret_cast<const float4*>(lp + 4);
        const float cur[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float prv[8];   // cumulative log decay of the row before (lower lanes: da needs P_{t-1}); row 0 has none
        if (lower && trow > 0) {
          const float4 q0 = *reinterpret_cast<const float4*>(lp - kFStride), q1 = *reinterpret_cast<const float4*>(lp - kFStride + 4);
          prv[0] = q0.x; prv[1] = q0.y; prv[2] = q0.z; prv[3] = q0.w; prv[4] = q1.x; prv[5] = q1.y; prv[6] = q1.z; prv[7] = q1.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) prv[j] = lower ? 0.f : cur[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float s4 = __expf(-cur[j]);     // 1 / P_t
          const float s3 = __expf(prv[j]);      // P_{t-1} (da) or P_t (dr)
          o3[j] = x3[j] * s3;
          o4[j] = x4[j] * s4;
        }
        if (t < T) {
          if (!lower && a3 != nullptr) {   // dr, dk: add the gradients that arrive by the other path
            float e3[8], e4[8];
            unpack8(*reinterpret_cast<const uint4*>(a3 + k0), e3);
            unpack8(*reinterpret_cast<const uint4*>(a4 + k0), e4);
#pragma unroll
            for (int j = 0; j < 8; ++j) { o3[j] += e3[j]; o4[j] += e4[j]; }
          }
          *reinterpret_cast<uint4*>(g3 + k0) = pack8(o3);
          *reinterpret_cast<uint4*>(g4 + k0) = pack8(o4);
        }
        if (lower) {
          float* zq = Zs + trow * kFStride + k0;
          float* fq = F + trow * kFStride + k0;
          *reinterpret_cast<float4*>(zq) = make_float4(-bv[0] * x4[0], -bv[1] * x4[1], -bv[2] * x4[2], -bv[3] * x4[3]);
          *reinterpret_cast<float4*>(zq + 4) = make_float4(-bv[4] * x4[4], -bv[5] * x4[5], -bv[6] * x4[6], -bv[7] * x4[7]);
          *reinterpret_cast<float4*>(fq) = make_float4(av[0] * x3[0], av[1] * x3[1], av[2] * x3[2], av[3] * x3[3]);
          *reinterpret_cast<float4*>(fq + 4) = make_float4(av[4] * x3[4], av[5] * x3[5], av[6] * x3[6], av[7] * x3[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) e1r[p * 8 + j] = av[j] * x3[j] - bv[j] * x4[j];
        }
      }
      PROF_MARK(9);
      __syncthreads();
      if (!lower) {
#pragma unroll
        for (int k4 = 0; k4 < 16; k4 += 4) {
          float4* zq = reinterpret_cast<float4*>(Zs + trow * kFStride + ch * 16 + k4);
          float4 o = *zq;
          o.x += e1r[k4]; o.y += e1r[k4 + 1]; o.z += e1r[k4 + 2]; o.w += e1r[k4 + 3];
          *zq = o;
        }
      }
      __syncthreads();
      PROF_MARK(10);
      {   // decay gradient: thread (k, blk) scans rows 8 blk .. 8 blk + 7 from the end, then adds the later blocks
        const int k = tid & 63, blk = tid >> 6;
        float part[8];
        float run = 0.f;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          const int tt = 8 * blk + j;
          run += Zs[tt * kFStride + k] + (tt < L - 1 ? F[(tt + 1) * kFStride + k] : 0.f);
          part[j] = run;
        }
        BS[blk * NH + k] = run;
        __syncthreads();
        float offs = (LT[k] + LT[NH + k]) + (LT[2 * NH + k] + LT[3 * NH + k]);
#pragma unroll
        for (int b2 = 1; b2 < 8; ++b2) offs += b2 > blk ? BS[b2 * NH + k] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int tt = 8 * blk + j;
          const float logd = LP[tt * kFStride + k] - (tt > 0 ? LP[(tt - 1) * kFStride + k] : 0.f);
          if (t0 + tt < T) g.dw[base + (size_t)(t0 + tt) * stride_t + k] = f2bf((part[j] + offs) * logd);
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    if (*failed) { ok = false; break; }
    PROF_MARK(11);
  }
  if (lower && g.ds0 != nullptr) {
#pragma unroll
    for (int j = 0; j < 16; ++j) g.ds0[((size_t)bh * NH + 16 * ch + j) * NH + trow] = ds[j];
  }
  if (!ok && tid == 0) atomicExch(&g_wkv_chunk_bwd_error, 0x40000 | (bh & 0xffff));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool wkv7_chunk_bwd_supported(const WkvArgs& p) { return p.is_bf16 && p.N == NH && p.interval == L; }

int wkv7_chunk_backward(const WkvArgs& p, cudaStream_t st) {
  if (!wkv7_chunk_bwd_supported(p)) return 1;
  BwdPtrs g;
  g.r = (const __nv_bfloat16*)p.r; g.w = (const __nv_bfloat16*)p.w; g.k = (const __nv_bfloat16*)p.k;
  g.v = (const __nv_bfloat16*)p.v; g.a = (const __nv_bfloat16*)p.a; g.b = (const __nv_bfloat16*)p.b;
  g.dy = (const __nv_bfloat16*)p.dy; g.sa = (const __nv_bfloat16*)p.sa; g.s0 = p.s0; g.ckpt = p.ckpt; g.dsT = p.dsT;
  g.dr = (__nv_bfloat16*)p.dr; g.dw = (__nv_bfloat16*)p.dw; g.dk = (__nv_bfloat16*)p.dk;
  g.dv = (__nv_bfloat16*)p.dv; g.da = (__nv_bfloat16*)p.da; g.db = (__nv_bfloat16*)p.db; g.ds0 = p.ds0;
  g.dr_add = (const __nv_bfloat16*)p.dr_add; g.dk_add = (const __nv_bfloat16*)p.dk_add; g.dv_add = (const __nv_bfloat16*)p.dv_add;
  const int BH = p.B * p.H;
  // tensor maps over the [B, T, H * 64] tensors; RWKV7M_B200_WKV_TMA=0 keeps the per-thread copies (for comparisons)
  alignas(64) BwdMaps maps;
  static const bool want_tma = [] { const char* e = getenv("RWKV7M_B200_WKV_TMA"); return e == nullptr || e[0] != '0'; }();
  int use_tma = want_tma ? 1 : 0;
  const void* src[8] = {p.a, p.r, p.b, p.k, p.w, p.sa, p.v, p.dy};
  const unsigned long long row_bytes = (unsigned long long)p.H * NH * 2;
  for (int i = 0; i < 8 && use_tma; ++i) {
    if ((reinterpret_cast<uintptr_t>(src[i]) & 15) != 0 ||
        !tma_encode_bf16_3d(&maps.m[i], src[i], (unsigned long long)p.H * NH, (unsigned long long)p.T, (unsigned long long)p.B,
                            row_bytes, row_bytes * p.T, NH, L))
      use_tma = 0;
  }
  if (!use_tma) memset(&maps, 0, sizeof(maps));
  auto kern = wkv7_chunk_bwd_kernel;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  kern<<<BH, kThreads, kSmemBytes, st>>>(g, maps, use_tma, p.T, p.H, BH);
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
