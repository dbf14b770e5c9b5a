// Memory-bound fused kernels around the GEMMs of an RWKV-7 block (bf16 activations,
// fp32 parameters and statistics).  Each forward has an explicit backward; per-channel
// parameter gradients are produced as partial sums [parts, C] that the caller reduces.
//
//   layernorm            fp32 statistics, saves mean / rstd
//   shift_mix            K token-shift lerps of one input in one pass
//   tmix_pre             decay clamp, in-context rate, value residual, per-head key normalisation
//   gn_bonus_gate        per-head GroupNorm + (r.k.r_k) v bonus + output gate
//   relusq_bwd           derivative of relu(x)^2 from the saved output
//
// Math: src/rwkv7m/model/nnx_model.py:592-798 of the reference.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace rk {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// read-only path: lets the compiler hoist the loads of the next unrolled rows above this row's stores
__device__ __forceinline__ float2 ld2(const bf16* p) {
  const unsigned int raw = __ldg(reinterpret_cast<const unsigned int*>(p));
  return __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw));
}
__device__ __forceinline__ void st2(bf16* p, float a, float b) { *reinterpret_cast<bf162*>(p) = __floats2bfloat162_rn(a, b); }

// ---------------------------------------------------------------------------------
// LayerNorm: one warp per row.
// ---------------------------------------------------------------------------------
__global__ void layernorm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                                     const float* __restrict__ b, bf16* __restrict__ y, float* __restrict__ mean,
                                     float* __restrict__ rstd, int M, int C, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < M; row += gridDim.x * warps_per_block) {
    const bf16* xr = x + (size_t)row * C;
    float s = 0.f, ss = 0.f;
    for (int c = lane * 2; c < C; c += 64) {
      float2 v = ld2(xr + c);
      s += v.x + v.y;
      ss += v.x * v.x + v.y * v.y;
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float mu = s / C;
    const float var = fmaxf(ss / C - mu * mu, 0.f);
    const float rs = rsqrtf(var + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    bf16* yr = y + (size_t)row * C;
    for (int c = lane * 2; c < C; c += 64) {
      float2 v = ld2(xr + c);
      st2(yr + c, (v.x - mu) * rs * w[c] + b[c], (v.y - mu) * rs * w[c + 1] + b[c + 1]);
    }
  }
}

// Single-pass forward for the common widths: one warp per row, the row stays in registers (16-byte accesses), weight and
// bias are staged in shared memory once per block.
template <int NCH>   // C = NCH * 256
__global__ void __launch_bounds__(256) layernorm_fwd_wide_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                                                                 const float* __restrict__ b, bf16* __restrict__ y,
                                                                 float* __restrict__ mean, float* __restrict__ rstd, int M,
                                                                 float eps) {
  constexpr int C = NCH * 256;
  __shared__ float s_w[C], s_b[C];
  for (int c = threadIdx.x; c < C; c += 256) { s_w[c] = w[c]; s_b[c] = b[c]; }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * 8 + warp; row < M; row += gridDim.x * 8) {
    const bf16* xr = x + (size_t)row * C + lane * 8;
    uint4 raw[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i) raw[i] = __ldg(reinterpret_cast<const uint4*>(xr + i * 256));
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint32_t* xp = reinterpret_cast<const uint32_t*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(&xp[j]));
        s += v.x + v.y;
        ss += v.x * v.x + v.y * v.y;
      }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float mu = s / C;
    const float var = fmaxf(ss / C - mu * mu, 0.f);
    const float rs = rsqrtf(var + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    bf16* yr = y + (size_t)row * C + lane * 8;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const uint32_t* xp = reinterpret_cast<const uint32_t*>(&raw[i]);
      const int cb = i * 256 + lane * 8;
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(&xp[j]));
        bf162 h = __floats2bfloat162_rn((v.x - mu) * rs * s_w[cb + 2 * j] + s_b[cb + 2 * j],
                                        (v.y - mu) * rs * s_w[cb + 2 * j + 1] + s_b[cb + 2 * j + 1]);
        op[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(yr + i * 256) = o;
    }
  }
}

__global__ void layernorm_bwd_dx_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                        const float* __restrict__ w, const float* __restrict__ mean,
                                        const float* __restrict__ rstd, bf16* __restrict__ dx, int M, int C) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < M; row += gridDim.x * warps_per_block) {
    const bf16* xr = x + (size_t)row * C;
    const bf16* gr = dy + (size_t)row * C;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane * 2; c < C; c += 64) {
      float2 v = ld2(xr + c), g = ld2(gr + c);
      const float g0 = g.x * w[c], g1 = g.y * w[c + 1];
      s1 += g0 + g1;
      s2 += g0 * (v.x - mu) * rs + g1 * (v.y - mu) * rs;
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    bf16* dr = dx + (size_t)row * C;
    for (int c = lane * 2; c < C; c += 64) {
      float2 v = ld2(xr + c), g = ld2(gr + c);
      const float xh0 = (v.x - mu) * rs, xh1 = (v.y - mu) * rs;
      st2(dr + c, rs * (g.x * w[c] - s1 - xh0 * s2), rs * (g.y * w[c + 1] - s1 - xh1 * s2));
    }
  }
}

// Column sums for dw/db: block (32 columns x 8 row lanes), grid (C/32, parts).
__global__ void layernorm_bwd_wb_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                        const float* __restrict__ mean, const float* __restrict__ rstd,
                                        float* __restrict__ dw_part, float* __restrict__ db_part, int M, int C) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int parts = gridDim.y;
  const int rows_per = (M + parts - 1) / parts;
  const int r0 = blockIdx.y * rows_per;
  const int r1 = min(M, r0 + rows_per);
  float aw = 0.f, ab = 0.f;
  if (c < C) {
    for (int r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      const float g = bf2f(dy[(size_t)r * C + c]);
      const float xh = (bf2f(x[(size_t)r * C + c]) - mean[r]) * rstd[r];
      aw += g * xh;
      ab += g;
    }
  }
  __shared__ float sw[8][33], sb[8][33];
  sw[threadIdx.y][threadIdx.x] = aw;
  sb[threadIdx.y][threadIdx.x] = ab;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    for (int j = 1; j < 8; ++j) { aw += sw[j][threadIdx.x]; ab += sb[j][threadIdx.x]; }
    dw_part[(size_t)blockIdx.y * C + c] = aw;
    db_part[(size_t)blockIdx.y * C + c] = ab;
  }
}

// LayerNorm backward in one pass over dy and x: a block of C / 8 threads walks rows two at a time, every thread owns 8
// consecutive channels of every row its block sees, so the input gradient (row statistics through one block reduction
// per row pair), the optional residual-path gradient and the per-block partial sums of the weight / bias gradients
// (16 registers per thread) all come from the same 16-byte loads.  dw_part / db_part receive one row per block.
template <int NT, bool RES>
__global__ void __launch_bounds__(NT, (NT >= 256 ? 3 : 4)) layernorm_bwd_onepass_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                                   const float* __restrict__ w, const float* __restrict__ mean,
                                                                   const float* __restrict__ rstd, bf16* __restrict__ dx,
                                                                   float* __restrict__ dw_part, float* __restrict__ db_part,
                                                                   int M, const bf16* __restrict__ dres) {
  constexpr int C = NT * 8, NW = NT / 32;
  __shared__ float red[2][NW][4];
  const int c = threadIdx.x * 8, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float w8[8], aw[8], ab[8];
  {
    const float4 a = *reinterpret_cast<const float4*>(w + c), b = *reinterpret_cast<const float4*>(w + c + 4);
    w8[0] = a.x; w8[1] = a.y; w8[2] = a.z; w8[3] = a.w; w8[4] = b.x; w8[5] = b.y; w8[6] = b.z; w8[7] = b.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { aw[j] = 0.f; ab[j] = 0.f; }
  int it = 0;
  for (int row = 2 * blockIdx.x; row < M; row += 2 * gridDim.x, it ^= 1) {
    const bool two = row + 1 < M;
    const size_t o0 = (size_t)row * C + c, o1 = o0 + C;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4 g0r = __ldg(reinterpret_cast<const uint4*>(dy + o0)), x0r = __ldg(reinterpret_cast<const uint4*>(x + o0));
    const uint4 g1r = two ? __ldg(reinterpret_cast<const uint4*>(dy + o1)) : zero;
    const uint4 x1r = two ? __ldg(reinterpret_cast<const uint4*>(x + o1)) : zero;
    uint4 d0r = zero, d1r = zero;
    if (RES) {
      d0r = __ldg(reinterpret_cast<const uint4*>(dres + o0));
      if (two) d1r = __ldg(reinterpret_cast<const uint4*>(dres + o1));
    }
    const float mu0 = mean[row], rs0 = rstd[row];
    const float mu1 = two ? mean[row + 1] : 0.f, rs1 = two ? rstd[row + 1] : 0.f;
    float g0[8], h0[8], g1[8], h1[8];
    {
      const bf162* gp = reinterpret_cast<const bf162*>(&g0r);
      const bf162* xp = reinterpret_cast<const bf162*>(&x0r);
      const bf162* gq = reinterpret_cast<const bf162*>(&g1r);
      const bf162* xq = reinterpret_cast<const bf162*>(&x1r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = __bfloat1622float2(gp[j]), b = __bfloat1622float2(xp[j]);
        g0[2 * j] = a.x; g0[2 * j + 1] = a.y; h0[2 * j] = (b.x - mu0) * rs0; h0[2 * j + 1] = (b.y - mu0) * rs0;
        a = __bfloat1622float2(gq[j]); b = __bfloat1622float2(xq[j]);
        g1[2 * j] = a.x; g1[2 * j + 1] = a.y; h1[2 * j] = (b.x - mu1) * rs1; h1[2 * j + 1] = (b.y - mu1) * rs1;
      }
    }
    float s[4] = {0.f, 0.f, 0.f, 0.f};   // sum(g w), sum(g w xhat) of the two rows
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = g0[j] * w8[j], b = g1[j] * w8[j];
      s[0] += a; s[1] = fmaf(a, h0[j], s[1]);
      s[2] += b; s[3] = fmaf(b, h1[j], s[3]);
      aw[j] = fmaf(g0[j], h0[j], aw[j]); aw[j] = fmaf(g1[j], h1[j], aw[j]);
      ab[j] += g0[j] + g1[j];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = warp_sum(s[i]);
    if (NW > 1) {
      if (lane == 0) { red[it][warp][0] = s[0]; red[it][warp][1] = s[1]; red[it][warp][2] = s[2]; red[it][warp][3] = s[3]; }
      __syncthreads();   // one barrier per row pair: the buffer alternates, and the barrier of the next pair separates
                         // these reads from the writes of the pair after it
      s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
      for (int k = 0; k < NW; ++k) { s[0] += red[it][k][0]; s[1] += red[it][k][1]; s[2] += red[it][k][2]; s[3] += red[it][k][3]; }
    }
    const float inv = 1.f / C;
    const float a1 = s[0] * inv, a2 = s[1] * inv, b1 = s[2] * inv, b2 = s[3] * inv;
    uint4 o0r, o1r;
    {
      bf162* op = reinterpret_cast<bf162*>(&o0r);
      bf162* oq = reinterpret_cast<bf162*>(&o1r);
      const bf162* dp = reinterpret_cast<const bf162*>(&d0r);
      const bf162* dq = reinterpret_cast<const bf162*>(&d1r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 r0 = __bfloat1622float2(dp[j]), r1 = __bfloat1622float2(dq[j]);
        op[j] = __floats2bfloat162_rn(r0.x + rs0 * (g0[2 * j] * w8[2 * j] - a1 - h0[2 * j] * a2),
                                      r0.y + rs0 * (g0[2 * j + 1] * w8[2 * j + 1] - a1 - h0[2 * j + 1] * a2));
        oq[j] = __floats2bfloat162_rn(r1.x + rs1 * (g1[2 * j] * w8[2 * j] - b1 - h1[2 * j] * b2),
                                      r1.y + rs1 * (g1[2 * j + 1] * w8[2 * j + 1] - b1 - h1[2 * j + 1] * b2));
      }
    }
    *reinterpret_cast<uint4*>(dx + o0) = o0r;
    if (two) *reinterpret_cast<uint4*>(dx + o1) = o1r;
  }
  float* dwp = dw_part + (size_t)blockIdx.x * C + c;
  float* dbp = db_part + (size_t)blockIdx.x * C + c;
  *reinterpret_cast<float4*>(dwp) = make_float4(aw[0], aw[1], aw[2], aw[3]);
  *reinterpret_cast<float4*>(dwp + 4) = make_float4(aw[4], aw[5], aw[6], aw[7]);
  *reinterpret_cast<float4*>(dbp) = make_float4(ab[0], ab[1], ab[2], ab[3]);
  *reinterpret_cast<float4*>(dbp + 4) = make_float4(ab[4], ab[5], ab[6], ab[7]);
}

template <int NCH>
static void launch_ln_bwd_fused(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                                float* dw_part, float* db_part, int parts, int M, cudaStream_t st, const void* dres) {
  constexpr int NT = NCH * 32;   // C / 8 threads
  if (dres != nullptr)
    layernorm_bwd_onepass_kernel<NT, true><<<parts, NT, 0, st>>>((const bf16*)dy, (const bf16*)x, w, mean, rstd, (bf16*)dx,
                                                                 dw_part, db_part, M, (const bf16*)dres);
  else
    layernorm_bwd_onepass_kernel<NT, false><<<parts, NT, 0, st>>>((const bf16*)dy, (const bf16*)x, w, mean, rstd, (bf16*)dx,
                                                                  dw_part, db_part, M, nullptr);
}

void layernorm_fwd(const void* x, const float* w, const float* b, void* y, float* mean, float* rstd, int M, int C,
                   float eps, cudaStream_t st) {
  int blocks = (M + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  // few, long-lived blocks: every block stages weight and bias (8 C bytes) before its first row
  const int wide_blocks = blocks > 148 * 4 ? 148 * 4 : blocks;
#define RK_LN_FWD(NCH) \
  layernorm_fwd_wide_kernel<NCH><<<wide_blocks, 256, 0, st>>>((const bf16*)x, w, b, (bf16*)y, mean, rstd, M, eps)
  if (aligned) {
    switch (C) {
      case 256: RK_LN_FWD(1); return;
      case 512: RK_LN_FWD(2); return;
      case 768: RK_LN_FWD(3); return;
      case 1024: RK_LN_FWD(4); return;
      case 2048: RK_LN_FWD(8); return;
      case 4096: RK_LN_FWD(16); return;
      default: break;
    }
  }
#undef RK_LN_FWD
  layernorm_fwd_kernel<<<blocks, 256, 0, st>>>((const bf16*)x, w, b, (bf16*)y, mean, rstd, M, C, eps);
}

// dres (optional, bf16 [M, C]): gradient arriving through the residual connection around the normalisation; dx = dres +
// the LayerNorm input gradient in the same pass.  Returns false when the width has no fused kernel (the caller adds).
bool layernorm_bwd_res(const void* dy, const void* x, const float* w, const float* mean, const float* rstd,
                       const void* dres, void* dx, float* dw_part, float* db_part, int parts, int M, int C,
                       cudaStream_t st) {
  // the single-pass kernel reads dy, x, dres and the weight and writes dx with 16-byte accesses
  const bool aligned = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) |
                         reinterpret_cast<uintptr_t>(dres) | reinterpret_cast<uintptr_t>(w) |
                         reinterpret_cast<uintptr_t>(dw_part) | reinterpret_cast<uintptr_t>(db_part)) & 15) == 0;
  switch (aligned ? C : 0) {   // single-pass kernel for the common widths
    case 256: launch_ln_bwd_fused<1>(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, st, dres); return true;
    case 512: launch_ln_bwd_fused<2>(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, st, dres); return true;
    case 768: launch_ln_bwd_fused<3>(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, st, dres); return true;
    case 1024: launch_ln_bwd_fused<4>(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, st, dres); return true;
    case 2048: launch_ln_bwd_fused<8>(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, st, dres); return true;
    default: break;
  }
  if (dres != nullptr) return false;
  int blocks = (M + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  layernorm_bwd_dx_kernel<<<blocks, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, w, mean, rstd, (bf16*)dx, M, C);
  dim3 grid((C + 31) / 32, parts), block(32, 8);
  layernorm_bwd_wb_kernel<<<grid, block, 0, st>>>((const bf16*)dy, (const bf16*)x, mean, rstd, dw_part, db_part, M, C);
  return true;
}

void layernorm_bwd(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                   float* dw_part, float* db_part, int parts, int M, int C, cudaStream_t st) {
  layernorm_bwd_res(dy, x, w, mean, rstd, nullptr, dx, dw_part, db_part, parts, M, C, st);
}

// ---------------------------------------------------------------------------------
// shift_mix: out[z][b,t,c] = x[b,t,c] + (xprev - x[b,t,c]) * mix[z][c], xprev = x[b,t-1,c] or prev[b,c] at t = 0.
// Thread = one column pair; block walks a segment of SEG consecutive tokens of one batch row.
// ---------------------------------------------------------------------------------
constexpr int kShiftSeg = 64;

template <int K>
__global__ void shift_mix_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ prev,
                                     const float* __restrict__ mix, bf16* __restrict__ out, int B, int T, int C) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * kShiftSeg;
  const int t1 = min(T, t0 + kShiftSeg);
  float m0[K], m1[K];
#pragma unroll
  for (int z = 0; z < K; ++z) { m0[z] = mix[z * C + c]; m1[z] = mix[z * C + c + 1]; }
  float2 p;
  if (t0 == 0) p = make_float2(prev[(size_t)b * C + c], prev[(size_t)b * C + c + 1]);
  else p = ld2(x + ((size_t)b * T + t0 - 1) * C + c);
  const size_t plane = (size_t)B * T * C;
  for (int t = t0; t < t1; ++t) {
    const size_t o = ((size_t)b * T + t) * C + c;
    const float2 v = ld2(x + o);
    const float d0 = p.x - v.x, d1 = p.y - v.y;
#pragma unroll
    for (int z = 0; z < K; ++z) st2(out + z * plane + o, v.x + d0 * m0[z], v.y + d1 * m1[z]);
    p = v;
  }
}

// dx[t] = sum_z dout_z[t] (1 - mix_z) + sum_z dout_z[t+1] mix_z ;  dmix_z = sum_t dout_z[t] (xprev_t - x_t) ;
// dprev = sum_z dout_z[0] mix_z.  Segment walked backwards in time.
template <int K> struct ShiftGrads { const bf16* p[K]; };

template <int K>
__global__ void shift_mix_bwd_kernel(ShiftGrads<K> dout, const bf16* __restrict__ x,
                                     const float* __restrict__ prev, const float* __restrict__ mix,
                                     bf16* __restrict__ dx, float* __restrict__ dprev, float* __restrict__ dmix_part,
                                     int B, int T, int C) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * kShiftSeg;
  const int t1 = min(T, t0 + kShiftSeg);
  float m0[K], m1[K], a0[K], a1[K];
#pragma unroll
  for (int z = 0; z < K; ++z) { m0[z] = mix[z * C + c]; m1[z] = mix[z * C + c + 1]; a0[z] = 0.f; a1[z] = 0.f; }
  // carry = sum_z dout_z[t+1] * mix_z
  float c0 = 0.f, c1 = 0.f;
  if (t1 < T) {
    const size_t o = ((size_t)b * T + t1) * C + c;
#pragma unroll
    for (int z = 0; z < K; ++z) { float2 g = ld2(dout.p[z] + o); c0 += g.x * m0[z]; c1 += g.y * m1[z]; }
  }
  float2 cur = ld2(x + ((size_t)b * T + t1 - 1) * C + c);
  for (int t = t1 - 1; t >= t0; --t) {
    const size_t o = ((size_t)b * T + t) * C + c;
    float2 pv;
    if (t == 0) pv = make_float2(prev[(size_t)b * C + c], prev[(size_t)b * C + c + 1]);
    else pv = ld2(x + o - C);
    const float d0 = pv.x - cur.x, d1 = pv.y - cur.y;
    float s0 = 0.f, s1 = 0.f, n0 = 0.f, n1 = 0.f;
#pragma unroll
    for (int z = 0; z < K; ++z) {
      float2 g = ld2(dout.p[z] + o);
      s0 += g.x * (1.f - m0[z]); s1 += g.y * (1.f - m1[z]);
      n0 += g.x * m0[z]; n1 += g.y * m1[z];
      a0[z] += g.x * d0; a1[z] += g.y * d1;
    }
    st2(dx + o, s0 + c0, s1 + c1);
    c0 = n0; c1 = n1;
    cur = pv;
  }
  if (t0 == 0) { dprev[(size_t)b * C + c] = c0; dprev[(size_t)b * C + c + 1] = c1; }
  const int part = blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
  for (int z = 0; z < K; ++z) {
    dmix_part[((size_t)part * K + z) * C + c] = a0[z];
    dmix_part[((size_t)part * K + z) * C + c + 1] = a1[z];
  }
}

// Wide variant of the backward: thread = 4 consecutive channels (8-byte accesses).  Tokens are handled two per iteration
// and the packed loads of the pair after it are issued first, so every thread keeps 14 loads in flight; the mixing
// coefficients sit in shared memory to leave the registers to those loads and to the K x 4 coefficient-gradient sums.
__device__ __forceinline__ void unpack4(const uint2 raw, float (&x)[4]) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
__device__ __forceinline__ uint2 ldraw4(const bf16* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

template <int K>
__global__ void __launch_bounds__(128, 4) shift_mix_bwd_wide_kernel(ShiftGrads<K> dout, const bf16* __restrict__ x,
                                                                    const float* __restrict__ prev, const float* __restrict__ mix,
                                                                    bf16* __restrict__ dx, float* __restrict__ dprev,
                                                                    float* __restrict__ dmix_part, int B, int T, int C) {
  __shared__ __align__(16) float s_m[K][512];
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;   // no block-wide barrier below: every thread reads only the coefficients it stored itself
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * kShiftSeg;
  const int t1 = min(T, t0 + kShiftSeg);
  float acc[K][4];
#pragma unroll
  for (int z = 0; z < K; ++z) {
    *reinterpret_cast<float4*>(&s_m[z][threadIdx.x * 4]) = *reinterpret_cast<const float4*>(mix + (size_t)z * C + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[z][j] = 0.f;
  }
  float carry[4] = {0.f, 0.f, 0.f, 0.f};   // sum_z dout_z[t+1] * mix_z
  if (t1 < T) {
    const size_t o = ((size_t)b * T + t1) * C + c;
#pragma unroll
    for (int z = 0; z < K; ++z) {
      float g[4];
      unpack4(ldraw4(dout.p[z] + o), g);
      const float4 m = *reinterpret_cast<const float4*>(&s_m[z][threadIdx.x * 4]);
      carry[0] = fmaf(g[0], m.x, carry[0]); carry[1] = fmaf(g[1], m.y, carry[1]);
      carry[2] = fmaf(g[2], m.z, carry[2]); carry[3] = fmaf(g[3], m.w, carry[3]);
    }
  }
  const bf16* xb = x + (size_t)b * T * C + c;
  float cur[4];
  unpack4(ldraw4(xb + (size_t)(t1 - 1) * C), cur);
  const uint2 zero2 = make_uint2(0u, 0u);
  // ga / xa: gradients of token t and x[t-1]; gb / xq: gradients of token t-1 and x[t-2]
  uint2 ga[K], gb[K], xa = zero2, xq = zero2;
  auto fetch = [&](int t, uint2 (&g)[K], uint2& xp) {
    if (t < t0) return;
    const size_t o = ((size_t)b * T + t) * C + c;
#pragma unroll
    for (int z = 0; z < K; ++z) g[z] = ldraw4(dout.p[z] + o);
    if (t > 0) xp = ldraw4(xb + (size_t)(t - 1) * C);
  };
  auto step = [&](int t, const uint2 (&g)[K], const uint2 xp) {
    float pv[4];
    if (t == 0) {
      const float4 p = *reinterpret_cast<const float4*>(prev + (size_t)b * C + c);
      pv[0] = p.x; pv[1] = p.y; pv[2] = p.z; pv[3] = p.w;
    } else {
      unpack4(xp, pv);
    }
    float s[4] = {0.f, 0.f, 0.f, 0.f}, n[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int z = 0; z < K; ++z) {
      float gv[4];
      unpack4(g[z], gv);
      const float4 m4 = *reinterpret_cast<const float4*>(&s_m[z][threadIdx.x * 4]);
      const float m[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[j] += gv[j];
        n[j] = fmaf(gv[j], m[j], n[j]);
        acc[z][j] = fmaf(gv[j], pv[j] - cur[j], acc[z][j]);
      }
    }
    // sum_z g (1 - mix) = sum_z g - sum_z g mix
    bf162 h0 = __floats2bfloat162_rn(s[0] - n[0] + carry[0], s[1] - n[1] + carry[1]);
    bf162 h1 = __floats2bfloat162_rn(s[2] - n[2] + carry[2], s[3] - n[3] + carry[3]);
    uint2 o2;
    o2.x = *reinterpret_cast<uint32_t*>(&h0); o2.y = *reinterpret_cast<uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(dx + ((size_t)b * T + t) * C + c) = o2;
#pragma unroll
    for (int j = 0; j < 4; ++j) { carry[j] = n[j]; cur[j] = pv[j]; }
  };
  fetch(t1 - 1, ga, xa);
  fetch(t1 - 2, gb, xq);
  for (int t = t1 - 1; t >= t0; t -= 2) {
    uint2 na[K], nb[K], nxa = zero2, nxq = zero2;
#pragma unroll
    for (int z = 0; z < K; ++z) { na[z] = zero2; nb[z] = zero2; }
    fetch(t - 2, na, nxa);
    fetch(t - 3, nb, nxq);
    step(t, ga, xa);
    if (t - 1 >= t0) step(t - 1, gb, xq);
#pragma unroll
    for (int z = 0; z < K; ++z) { ga[z] = na[z]; gb[z] = nb[z]; }
    xa = nxa; xq = nxq;
  }
  if (t0 == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) dprev[(size_t)b * C + c + j] = carry[j];
  }
  const int part = blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
  for (int z = 0; z < K; ++z)
    *reinterpret_cast<float4*>(dmix_part + ((size_t)part * K + z) * C + c) = make_float4(acc[z][0], acc[z][1], acc[z][2], acc[z][3]);
}

int shift_mix_parts(int B, int T) { return B * ((T + kShiftSeg - 1) / kShiftSeg); }

void shift_mix_fwd(const void* x, const float* prev, const float* mix, void* out, int K, int B, int T, int C,
                   cudaStream_t st) {
  dim3 block(128), grid((C / 2 + 127) / 128, (T + kShiftSeg - 1) / kShiftSeg, B);
  if (K == 6) shift_mix_fwd_kernel<6><<<grid, block, 0, st>>>((const bf16*)x, prev, mix, (bf16*)out, B, T, C);
  else shift_mix_fwd_kernel<1><<<grid, block, 0, st>>>((const bf16*)x, prev, mix, (bf16*)out, B, T, C);
}

void shift_mix_bwd(const void* const* dout, const void* x, const float* prev, const float* mix, void* dx,
                   float* dprev, float* dmix_part, int K, int B, int T, int C, cudaStream_t st) {
  dim3 block(128), grid((C / 2 + 127) / 128, (T + kShiftSeg - 1) / kShiftSeg, B);
  if (C % 4 == 0) {   // 8-byte accesses
    dim3 gridw((C / 4 + 127) / 128, (T + kShiftSeg - 1) / kShiftSeg, B);
    if (K == 6) {
      ShiftGrads<6> g;
      for (int z = 0; z < 6; ++z) g.p[z] = (const bf16*)dout[z];
      shift_mix_bwd_wide_kernel<6><<<gridw, block, 0, st>>>(g, (const bf16*)x, prev, mix, (bf16*)dx, dprev, dmix_part, B, T, C);
    } else {
      ShiftGrads<1> g;
      g.p[0] = (const bf16*)dout[0];
      shift_mix_bwd_wide_kernel<1><<<gridw, block, 0, st>>>(g, (const bf16*)x, prev, mix, (bf16*)dx, dprev, dmix_part, B, T, C);
    }
    return;
  }
  if (K == 6) {
    ShiftGrads<6> g;
    for (int z = 0; z < 6; ++z) g.p[z] = (const bf16*)dout[z];
    shift_mix_bwd_kernel<6><<<grid, block, 0, st>>>(g, (const bf16*)x, prev, mix, (bf16*)dx, dprev, dmix_part, B, T, C);
  } else {
    ShiftGrads<1> g;
    g.p[0] = (const bf16*)dout[0];
    shift_mix_bwd_kernel<1><<<grid, block, 0, st>>>(g, (const bf16*)x, prev, mix, (bf16*)dx, dprev, dmix_part, B, T, C);
  }
}

// ---------------------------------------------------------------------------------
// tmix_pre: one warp per (row, head), head size 64 (two channels per lane).  A block of
// 8 warps covers 8 heads; blocks walk kRowsPerBlock rows so per-channel parameter
// gradients accumulate in registers before the partial write.
// ---------------------------------------------------------------------------------
constexpr int kRowsPerPart = 64;

struct TmixPreParams {
  const bf16 *k_raw, *v_raw, *w_lora, *a_lora, *vg_lora, *v_first;  // vg_lora / v_first null on layer 0
  const float *w0, *a0, *v0, *k_k, *k_a;
  bf16 *w, *k_mod, *v, *neg_kk, *kka;
  // backward
  const bf16 *dw, *dk_mod, *dv, *dneg_kk, *dkka;
  bf16 *dk_raw, *dv_raw, *dw_lora, *da_lora, *dvg_lora, *dv_first;
  float *dw0_part, *da0_part, *dv0_part, *dkk_part, *dka_part;  // [parts, C]
  int M, C;
  int rows_per_part;  // forward only: rows walked by one block (small for decode-sized M so the grid stays wide)
};

// Rows per block of the forward head-wise kernels: 128 at training sizes, fewer when there are few rows.
static int fwd_rows_per_part(int M) { return M >= 16384 ? kRowsPerPart : (M >= 1024 ? 16 : 1); }

__global__ void tmix_pre_fwd_kernel(TmixPreParams p) {
  const int H = p.C / 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * 8 + warp;
  if (head >= H) return;
  const int c = head * 64 + lane * 2;
  const float w0a = p.w0[c], w0b = p.w0[c + 1], a0a = p.a0[c], a0b = p.a0[c + 1];
  const float kka_ = p.k_k[c], kkb_ = p.k_k[c + 1], kaa = p.k_a[c], kab = p.k_a[c + 1];
  const bool has_v = p.vg_lora != nullptr;
  float v0a = 0.f, v0b = 0.f;
  if (has_v) { v0a = p.v0[c]; v0b = p.v0[c + 1]; }
  const int r0 = blockIdx.y * p.rows_per_part, r1 = min(p.M, r0 + p.rows_per_part);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    const float2 k = ld2(p.k_raw + o), v = ld2(p.v_raw + o), wl = ld2(p.w_lora + o), al = ld2(p.a_lora + o);
    const float wa = -softplusf_(-(w0a + wl.x)) - 0.5f, wb = -softplusf_(-(w0b + wl.y)) - 0.5f;
    const float aa = sigmoidf_(a0a + al.x), ab = sigmoidf_(a0b + al.y);
    float va = v.x, vb = v.y;
    if (has_v) {
      const float2 vg = ld2(p.vg_lora + o), vf = ld2(p.v_first + o);
      va = v.x + (vf.x - v.x) * sigmoidf_(v0a + vg.x);
      vb = v.y + (vf.y - v.y) * sigmoidf_(v0b + vg.y);
    }
    const float x0 = k.x * kka_, x1 = k.y * kkb_;
    const float inv = rsqrtf(warp_sum(x0 * x0 + x1 * x1) + 1e-24f);
    const float kk0 = x0 * inv, kk1 = x1 * inv;
    st2(p.w + o, wa, wb);
    st2(p.k_mod + o, k.x * (1.f + (aa - 1.f) * kaa), k.y * (1.f + (ab - 1.f) * kab));
    st2(p.v + o, va, vb);
    st2(p.neg_kk + o, -kk0, -kk1);
    st2(p.kka + o, kk0 * aa, kk1 * ab);
  }
}

__global__ void tmix_pre_bwd_kernel(TmixPreParams p) {
  const int H = p.C / 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * 8 + warp;
  if (head >= H) return;
  const int c = head * 64 + lane * 2;
  const float w0a = p.w0[c], w0b = p.w0[c + 1], a0a = p.a0[c], a0b = p.a0[c + 1];
  const float kka_ = p.k_k[c], kkb_ = p.k_k[c + 1], kaa = p.k_a[c], kab = p.k_a[c + 1];
  const bool has_v = p.vg_lora != nullptr;
  float v0a = 0.f, v0b = 0.f;
  if (has_v) { v0a = p.v0[c]; v0b = p.v0[c + 1]; }
  float gw0a = 0.f, gw0b = 0.f, ga0a = 0.f, ga0b = 0.f, gv0a = 0.f, gv0b = 0.f, gkka = 0.f, gkkb = 0.f, gkaa = 0.f,
        gkab = 0.f;
  const int r0 = blockIdx.y * kRowsPerPart, r1 = min(p.M, r0 + kRowsPerPart);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    const float2 k = ld2(p.k_raw + o), v = ld2(p.v_raw + o), wl = ld2(p.w_lora + o), al = ld2(p.a_lora + o);
    const float2 gw = ld2(p.dw + o), gk = ld2(p.dk_mod + o), gv = ld2(p.dv + o), gn = ld2(p.dneg_kk + o),
                 gb = ld2(p.dkka + o);
    // decay
    const float dwa = gw.x * sigmoidf_(-(w0a + wl.x)), dwb = gw.y * sigmoidf_(-(w0b + wl.y));
    st2(p.dw_lora + o, dwa, dwb);
    gw0a += dwa; gw0b += dwb;
    // key normalisation
    const float aa = sigmoidf_(a0a + al.x), ab = sigmoidf_(a0b + al.y);
    const float x0 = k.x * kka_, x1 = k.y * kkb_;
    const float inv = rsqrtf(warp_sum(x0 * x0 + x1 * x1) + 1e-24f);
    const float kk0 = x0 * inv, kk1 = x1 * inv;
    const float dkk0 = -gn.x + gb.x * aa, dkk1 = -gn.y + gb.y * ab;
    const float dot = warp_sum(dkk0 * kk0 + dkk1 * kk1);
    const float dx0 = (dkk0 - kk0 * dot) * inv, dx1 = (dkk1 - kk1 * dot) * inv;
    gkka += dx0 * k.x; gkkb += dx1 * k.y;
    // in-context rate
    const float da0 = gk.x * k.x * kaa + gb.x * kk0, da1 = gk.y * k.y * kab + gb.y * kk1;
    const float dar0 = da0 * aa * (1.f - aa), dar1 = da1 * ab * (1.f - ab);
    st2(p.da_lora + o, dar0, dar1);
    ga0a += dar0; ga0b += dar1;
    gkaa += gk.x * k.x * (aa - 1.f); gkab += gk.y * k.y * (ab - 1.f);
    st2(p.dk_raw + o, dx0 * kka_ + gk.x * (1.f + (aa - 1.f) * kaa), dx1 * kkb_ + gk.y * (1.f + (ab - 1.f) * kab));
    // value residual
    if (has_v) {
      const float2 vg = ld2(p.vg_lora + o), vf = ld2(p.v_first + o);
      const float g0 = sigmoidf_(v0a + vg.x), g1 = sigmoidf_(v0b + vg.y);
      st2(p.dv_raw + o, gv.x * (1.f - g0), gv.y * (1.f - g1));
      st2(p.dv_first + o, gv.x * g0, gv.y * g1);
      const float dg0 = gv.x * (vf.x - v.x) * g0 * (1.f - g0), dg1 = gv.y * (vf.y - v.y) * g1 * (1.f - g1);
      st2(p.dvg_lora + o, dg0, dg1);
      gv0a += dg0; gv0b += dg1;
    } else {
      st2(p.dv_raw + o, gv.x, gv.y);
    }
  }
  const size_t po = (size_t)blockIdx.y * p.C + c;
  p.dw0_part[po] = gw0a; p.dw0_part[po + 1] = gw0b;
  p.da0_part[po] = ga0a; p.da0_part[po + 1] = ga0b;
  p.dkk_part[po] = gkka; p.dkk_part[po + 1] = gkkb;
  p.dka_part[po] = gkaa; p.dka_part[po + 1] = gkab;
  if (has_v) { p.dv0_part[po] = gv0a; p.dv0_part[po + 1] = gv0b; }
}

// ---- wide variants: one block walks whole rows, thread = 8 consecutive channels (16-byte accesses), the 8 lanes of a
//      head reduce with three shuffles; per-channel parameter gradients stay in registers over the block's rows ----------
__device__ __forceinline__ void ld8(const bf16* p, float (&x)[8]) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&w[i]));
    x[2 * i] = f.x; x[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void st8(bf16* p, const float (&x)[8]) {
  uint4 o;
  bf162 h;
  h = __floats2bfloat162_rn(x[0], x[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[2], x[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[4], x[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[6], x[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ float head_sum8(float v) {   // sum over the 8 lanes that hold one 64-channel head
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__global__ void __launch_bounds__(256, 1) tmix_pre_bwd_wide_kernel(TmixPreParams p) {
  const int c = threadIdx.x * 8;
  float w0[8], a0[8], kk_[8], ka[8], v0[8];
  float gw0[8], ga0[8], gkk[8], gka[8], gv0[8];
  const bool has_v = p.vg_lora != nullptr;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    w0[j] = p.w0[c + j]; a0[j] = p.a0[c + j]; kk_[j] = p.k_k[c + j]; ka[j] = p.k_a[c + j];
    v0[j] = has_v ? p.v0[c + j] : 0.f;
    gw0[j] = ga0[j] = gkk[j] = gka[j] = gv0[j] = 0.f;
  }
  const int r0 = blockIdx.x * kRowsPerPart, r1 = min(p.M, r0 + kRowsPerPart);
  // software pipeline: the raw 16-byte pieces of the next row are in flight while this row is processed
  uint4 nx[11];
  auto fetch = [&](int row) {
    const size_t o = (size_t)row * p.C + c;
    nx[0] = __ldg(reinterpret_cast<const uint4*>(p.k_raw + o)); nx[1] = __ldg(reinterpret_cast<const uint4*>(p.v_raw + o));
    nx[2] = __ldg(reinterpret_cast<const uint4*>(p.w_lora + o)); nx[3] = __ldg(reinterpret_cast<const uint4*>(p.a_lora + o));
    nx[4] = __ldg(reinterpret_cast<const uint4*>(p.dw + o)); nx[5] = __ldg(reinterpret_cast<const uint4*>(p.dk_mod + o));
    nx[6] = __ldg(reinterpret_cast<const uint4*>(p.dv + o)); nx[7] = __ldg(reinterpret_cast<const uint4*>(p.dneg_kk + o));
    nx[8] = __ldg(reinterpret_cast<const uint4*>(p.dkka + o));
    if (has_v) {
      nx[9] = __ldg(reinterpret_cast<const uint4*>(p.vg_lora + o)); nx[10] = __ldg(reinterpret_cast<const uint4*>(p.v_first + o));
    }
  };
  auto cvt = [](const uint4& raw, float (&x)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  };
  if (r0 < r1) fetch(r0);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    float k[8], v[8], wl[8], al[8], gw[8], gk[8], gv[8], gn[8], gb[8];
    cvt(nx[0], k); cvt(nx[1], v); cvt(nx[2], wl); cvt(nx[3], al); cvt(nx[4], gw); cvt(nx[5], gk); cvt(nx[6], gv);
    cvt(nx[7], gn); cvt(nx[8], gb);
    float vg[8], vf[8];
    if (has_v) { cvt(nx[9], vg); cvt(nx[10], vf); }
    if (row + 1 < r1) fetch(row + 1);
    float out[8], aa[8], x[8], dkk[8];
    // decay
#pragma unroll
    for (int j = 0; j < 8; ++j) { out[j] = gw[j] * sigmoidf_(-(w0[j] + wl[j])); gw0[j] += out[j]; }
    st8(p.dw_lora + o, out);
    // key normalisation
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { aa[j] = sigmoidf_(a0[j] + al[j]); x[j] = k[j] * kk_[j]; ss = fmaf(x[j], x[j], ss); }
    const float inv = rsqrtf(head_sum8(ss) + 1e-24f);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { x[j] *= inv; dkk[j] = -gn[j] + gb[j] * aa[j]; dot = fmaf(dkk[j], x[j], dot); }
    dot = head_sum8(dot);
    float dal[8], dkr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float dx = (dkk[j] - x[j] * dot) * inv;
      gkk[j] += dx * k[j];
      const float da = gk[j] * k[j] * ka[j] + gb[j] * x[j];
      dal[j] = da * aa[j] * (1.f - aa[j]);
      ga0[j] += dal[j];
      gka[j] += gk[j] * k[j] * (aa[j] - 1.f);
      dkr[j] = dx * kk_[j] + gk[j] * (1.f + (aa[j] - 1.f) * ka[j]);
    }
    st8(p.da_lora + o, dal);
    st8(p.dk_raw + o, dkr);
    // value residual
    if (has_v) {
      float dvr[8], dvf[8], dvg[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = sigmoidf_(v0[j] + vg[j]);
        dvr[j] = gv[j] * (1.f - g);
        dvf[j] = gv[j] * g;
        dvg[j] = gv[j] * (vf[j] - v[j]) * g * (1.f - g);
        gv0[j] += dvg[j];
      }
      st8(p.dv_raw + o, dvr); st8(p.dv_first + o, dvf); st8(p.dvg_lora + o, dvg);
    } else {
      st8(p.dv_raw + o, gv);
    }
  }
  const size_t po = (size_t)blockIdx.x * p.C + c;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    p.dw0_part[po + j] = gw0[j]; p.da0_part[po + j] = ga0[j]; p.dkk_part[po + j] = gkk[j]; p.dka_part[po + j] = gka[j];
    if (has_v) p.dv0_part[po + j] = gv0[j];
  }
}

int row_parts(int M) { return (M + kRowsPerPart - 1) / kRowsPerPart; }

// Forward with 16-byte accesses: thread = 8 consecutive channels, 8 lanes per head, rows [r0, r1) of one part per block,
// the next row's pieces in flight while this row is processed.
template <bool HAS_V>
__global__ void __launch_bounds__(256) tmix_pre_fwd_wide_kernel(TmixPreParams p) {
  const int c = threadIdx.x * 8;
  float w0[8], a0[8], v0[8], kk_[8], ka[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    w0[j] = p.w0[c + j]; a0[j] = p.a0[c + j]; kk_[j] = p.k_k[c + j]; ka[j] = p.k_a[c + j];
    v0[j] = HAS_V ? p.v0[c + j] : 0.f;
  }
  const int r0 = blockIdx.x * p.rows_per_part, r1 = min(p.M, r0 + p.rows_per_part);
  uint4 nx[HAS_V ? 6 : 4];
  auto fetch = [&](int row) {
    const size_t o = (size_t)row * p.C + c;
    nx[0] = __ldg(reinterpret_cast<const uint4*>(p.k_raw + o)); nx[1] = __ldg(reinterpret_cast<const uint4*>(p.v_raw + o));
    nx[2] = __ldg(reinterpret_cast<const uint4*>(p.w_lora + o)); nx[3] = __ldg(reinterpret_cast<const uint4*>(p.a_lora + o));
    if (HAS_V) {
      nx[4] = __ldg(reinterpret_cast<const uint4*>(p.vg_lora + o));
      nx[5] = __ldg(reinterpret_cast<const uint4*>(p.v_first + o));
    }
  };
  auto cvt = [](const uint4& raw, float (&x)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  };
  if (r0 < r1) fetch(r0);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    float k[8], v[8], wl[8], al[8], vg[8], vf[8];
    cvt(nx[0], k); cvt(nx[1], v); cvt(nx[2], wl); cvt(nx[3], al);
    if (HAS_V) { cvt(nx[4], vg); cvt(nx[5], vf); }
    if (row + 1 < r1) fetch(row + 1);
    float out[8], aa[8], x[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      out[j] = -softplusf_(-(w0[j] + wl[j])) - 0.5f;
      aa[j] = sigmoidf_(a0[j] + al[j]);
      x[j] = k[j] * kk_[j];
      ss = fmaf(x[j], x[j], ss);
    }
    st8(p.w + o, out);
    const float inv = rsqrtf(head_sum8(ss) + 1e-24f);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = k[j] * (1.f + (aa[j] - 1.f) * ka[j]);
    st8(p.k_mod + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = HAS_V ? v[j] + (vf[j] - v[j]) * sigmoidf_(v0[j] + vg[j]) : v[j];
    st8(p.v + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) { x[j] *= inv; out[j] = -x[j]; }
    st8(p.neg_kk + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = x[j] * aa[j];
    st8(p.kka + o, out);
  }
}

void tmix_pre_fwd(const void* const* in, const float* const* par, void* const* out, int M, int C, cudaStream_t st) {
  TmixPreParams p{};
  p.k_raw = (const bf16*)in[0]; p.v_raw = (const bf16*)in[1]; p.w_lora = (const bf16*)in[2];
  p.a_lora = (const bf16*)in[3]; p.vg_lora = (const bf16*)in[4]; p.v_first = (const bf16*)in[5];
  p.w0 = par[0]; p.a0 = par[1]; p.v0 = par[2]; p.k_k = par[3]; p.k_a = par[4];
  p.w = (bf16*)out[0]; p.k_mod = (bf16*)out[1]; p.v = (bf16*)out[2]; p.neg_kk = (bf16*)out[3]; p.kka = (bf16*)out[4];
  p.M = M; p.C = C;
  p.rows_per_part = fwd_rows_per_part(M);
  if (C % 64 == 0 && C / 8 <= 256 && (C / 8) % 32 == 0) {
    const int parts = (M + p.rows_per_part - 1) / p.rows_per_part;
    if (p.vg_lora != nullptr) tmix_pre_fwd_wide_kernel<true><<<parts, C / 8, 0, st>>>(p);
    else tmix_pre_fwd_wide_kernel<false><<<parts, C / 8, 0, st>>>(p);
    return;
  }
  dim3 grid((C / 64 + 7) / 8, (M + p.rows_per_part - 1) / p.rows_per_part);
  tmix_pre_fwd_kernel<<<grid, 256, 0, st>>>(p);
}

void tmix_pre_bwd(const void* const* in, const float* const* par, const void* const* gout, void* const* gin,
                  float* const* gpar_part, int M, int C, cudaStream_t st) {
  TmixPreParams p{};
  p.k_raw = (const bf16*)in[0]; p.v_raw = (const bf16*)in[1]; p.w_lora = (const bf16*)in[2];
  p.a_lora = (const bf16*)in[3]; p.vg_lora = (const bf16*)in[4]; p.v_first = (const bf16*)in[5];
  p.w0 = par[0]; p.a0 = par[1]; p.v0 = par[2]; p.k_k = par[3]; p.k_a = par[4];
  p.dw = (const bf16*)gout[0]; p.dk_mod = (const bf16*)gout[1]; p.dv = (const bf16*)gout[2];
  p.dneg_kk = (const bf16*)gout[3]; p.dkka = (const bf16*)gout[4];
  p.dk_raw = (bf16*)gin[0]; p.dv_raw = (bf16*)gin[1]; p.dw_lora = (bf16*)gin[2]; p.da_lora = (bf16*)gin[3];
  p.dvg_lora = (bf16*)gin[4]; p.dv_first = (bf16*)gin[5];
  p.dw0_part = gpar_part[0]; p.da0_part = gpar_part[1]; p.dv0_part = gpar_part[2]; p.dkk_part = gpar_part[3];
  p.dka_part = gpar_part[4];
  p.M = M; p.C = C;
  if (C % 64 == 0 && C / 8 <= 256 && (C / 8) % 32 == 0) {
    tmix_pre_bwd_wide_kernel<<<row_parts(M), C / 8, 0, st>>>(p);
    return;
  }
  dim3 grid((C / 64 + 7) / 8, row_parts(M));
  tmix_pre_bwd_kernel<<<grid, 256, 0, st>>>(p);
}

// ---------------------------------------------------------------------------------
// gn_bonus_gate: out = (GroupNorm_head(y) * ln_w + ln_b + (sum_head r k r_k) v) * g
// ---------------------------------------------------------------------------------
struct GnParams {
  const bf16 *y, *r, *k, *v, *g;
  const float *ln_w, *ln_b, *r_k;
  bf16* out;
  const bf16* dout;
  bf16 *dy, *dr, *dk, *dv, *dg;
  float *dlnw_part, *dlnb_part, *drk_part;
  int M, C;
  float eps;
  int rows_per_part;  // forward only
};

__global__ void gn_bonus_gate_fwd_kernel(GnParams p) {
  const int H = p.C / 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * 8 + warp;
  if (head >= H) return;
  const int c = head * 64 + lane * 2;
  const float lw0 = p.ln_w[c], lw1 = p.ln_w[c + 1], lb0 = p.ln_b[c], lb1 = p.ln_b[c + 1];
  const float rk0 = p.r_k[c], rk1 = p.r_k[c + 1];
  const int r0 = blockIdx.y * p.rows_per_part, r1 = min(p.M, r0 + p.rows_per_part);
#pragma unroll 4
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    const float2 y = ld2(p.y + o), r = ld2(p.r + o), k = ld2(p.k + o), v = ld2(p.v + o), g = ld2(p.g + o);
    const float mu = warp_sum(y.x + y.y) * (1.f / 64.f);
    const float d0 = y.x - mu, d1 = y.y - mu;
    const float rs = rsqrtf(warp_sum(d0 * d0 + d1 * d1) * (1.f / 64.f) + p.eps);
    const float s = warp_sum(r.x * k.x * rk0 + r.y * k.y * rk1);
    st2(p.out + o, (d0 * rs * lw0 + lb0 + s * v.x) * g.x, (d1 * rs * lw1 + lb1 + s * v.y) * g.y);
  }
}

__global__ void gn_bonus_gate_bwd_kernel(GnParams p) {
  const int H = p.C / 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * 8 + warp;
  if (head >= H) return;
  const int c = head * 64 + lane * 2;
  const float lw0 = p.ln_w[c], lw1 = p.ln_w[c + 1], lb0 = p.ln_b[c], lb1 = p.ln_b[c + 1];
  const float rk0 = p.r_k[c], rk1 = p.r_k[c + 1];
  float aw0 = 0.f, aw1 = 0.f, ab0 = 0.f, ab1 = 0.f, ar0 = 0.f, ar1 = 0.f;
  const int r0 = blockIdx.y * kRowsPerPart, r1 = min(p.M, r0 + kRowsPerPart);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    const float2 y = ld2(p.y + o), r = ld2(p.r + o), k = ld2(p.k + o), v = ld2(p.v + o), g = ld2(p.g + o),
                 go = ld2(p.dout + o);
    const float mu = warp_sum(y.x + y.y) * (1.f / 64.f);
    const float d0 = y.x - mu, d1 = y.y - mu;
    const float rs = rsqrtf(warp_sum(d0 * d0 + d1 * d1) * (1.f / 64.f) + p.eps);
    const float xh0 = d0 * rs, xh1 = d1 * rs;
    const float s = warp_sum(r.x * k.x * rk0 + r.y * k.y * rk1);
    const float pre0 = xh0 * lw0 + lb0 + s * v.x, pre1 = xh1 * lw1 + lb1 + s * v.y;
    st2(p.dg + o, go.x * pre0, go.y * pre1);
    const float dp0 = go.x * g.x, dp1 = go.y * g.y;
    st2(p.dv + o, dp0 * s, dp1 * s);
    const float ds = warp_sum(dp0 * v.x + dp1 * v.y);
    st2(p.dr + o, ds * k.x * rk0, ds * k.y * rk1);
    st2(p.dk + o, ds * r.x * rk0, ds * r.y * rk1);
    ar0 += ds * r.x * k.x; ar1 += ds * r.y * k.y;
    aw0 += dp0 * xh0; aw1 += dp1 * xh1;
    ab0 += dp0; ab1 += dp1;
    const float dx0 = dp0 * lw0, dx1 = dp1 * lw1;
    const float m1 = warp_sum(dx0 + dx1) * (1.f / 64.f);
    const float m2 = warp_sum(dx0 * xh0 + dx1 * xh1) * (1.f / 64.f);
    st2(p.dy + o, rs * (dx0 - m1 - xh0 * m2), rs * (dx1 - m1 - xh1 * m2));
  }
  const size_t po = (size_t)blockIdx.y * p.C + c;
  p.dlnw_part[po] = aw0; p.dlnw_part[po + 1] = aw1;
  p.dlnb_part[po] = ab0; p.dlnb_part[po + 1] = ab1;
  p.drk_part[po] = ar0; p.drk_part[po + 1] = ar1;
}

// Wide variants (thread = 8 consecutive channels, 8 lanes per head, next row's pieces in flight while this row is processed).
__global__ void __launch_bounds__(256, 2) gn_bonus_gate_bwd_wide_kernel(GnParams p) {
  const int c = threadIdx.x * 8;
  float lw[8], lb[8], rk[8], aw[8], ab[8], ar[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { lw[j] = p.ln_w[c + j]; lb[j] = p.ln_b[c + j]; rk[j] = p.r_k[c + j]; aw[j] = ab[j] = ar[j] = 0.f; }
  const int r0 = blockIdx.x * kRowsPerPart, r1 = min(p.M, r0 + kRowsPerPart);
  uint4 nx[6];
  auto fetch = [&](int row) {
    const size_t o = (size_t)row * p.C + c;
    nx[0] = __ldg(reinterpret_cast<const uint4*>(p.y + o)); nx[1] = __ldg(reinterpret_cast<const uint4*>(p.r + o));
    nx[2] = __ldg(reinterpret_cast<const uint4*>(p.k + o)); nx[3] = __ldg(reinterpret_cast<const uint4*>(p.v + o));
    nx[4] = __ldg(reinterpret_cast<const uint4*>(p.g + o)); nx[5] = __ldg(reinterpret_cast<const uint4*>(p.dout + o));
  };
  auto cvt = [](const uint4& raw, float (&x)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  };
  if (r0 < r1) fetch(r0);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    float y[8], r[8], k[8], v[8], g[8], go[8];
    cvt(nx[0], y); cvt(nx[1], r); cvt(nx[2], k); cvt(nx[3], v); cvt(nx[4], g); cvt(nx[5], go);
    if (row + 1 < r1) fetch(row + 1);
    float sy = 0.f, srk = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { sy += y[j]; srk = fmaf(r[j] * k[j], rk[j], srk); }
    const float mu = head_sum8(sy) * (1.f / 64.f);
    const float s = head_sum8(srk);
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { y[j] -= mu; sv = fmaf(y[j], y[j], sv); }
    const float rs = rsqrtf(head_sum8(sv) * (1.f / 64.f) + p.eps);
    float dp[8], xh[8], out[8];
    float dsum = 0.f, m1 = 0.f, m2 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xh[j] = y[j] * rs;
      const float pre = xh[j] * lw[j] + lb[j] + s * v[j];
      out[j] = go[j] * pre;                       // d gate
      dp[j] = go[j] * g[j];
      dsum = fmaf(dp[j], v[j], dsum);
      const float dxn = dp[j] * lw[j];
      m1 += dxn; m2 = fmaf(dxn, xh[j], m2);
      aw[j] = fmaf(dp[j], xh[j], aw[j]); ab[j] += dp[j];
    }
    st8(p.dg + o, out);
    const float ds = head_sum8(dsum);
    m1 = head_sum8(m1) * (1.f / 64.f);
    m2 = head_sum8(m2) * (1.f / 64.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = dp[j] * s;
    st8(p.dv + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) { out[j] = ds * k[j] * rk[j]; ar[j] = fmaf(ds * r[j], k[j], ar[j]); }
    st8(p.dr + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = ds * r[j] * rk[j];
    st8(p.dk + o, out);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = rs * (dp[j] * lw[j] - m1 - xh[j] * m2);
    st8(p.dy + o, out);
  }
  const size_t po = (size_t)blockIdx.x * p.C + c;
#pragma unroll
  for (int j = 0; j < 8; ++j) { p.dlnw_part[po + j] = aw[j]; p.dlnb_part[po + j] = ab[j]; p.drk_part[po + j] = ar[j]; }
}

// Forward with the same layout as the wide backward: thread = 8 consecutive channels (16-byte accesses), 8 lanes per head,
// the next row's five pieces are in flight while this row is processed.  Rows [r0, r1) of one part per block.
__global__ void __launch_bounds__(256) gn_bonus_gate_fwd_wide_kernel(GnParams p) {
  const int c = threadIdx.x * 8;
  float lw[8], lb[8], rk[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { lw[j] = p.ln_w[c + j]; lb[j] = p.ln_b[c + j]; rk[j] = p.r_k[c + j]; }
  const int r0 = blockIdx.x * p.rows_per_part, r1 = min(p.M, r0 + p.rows_per_part);
  uint4 nx[5];
  auto fetch = [&](int row) {
    const size_t o = (size_t)row * p.C + c;
    nx[0] = __ldg(reinterpret_cast<const uint4*>(p.y + o)); nx[1] = __ldg(reinterpret_cast<const uint4*>(p.r + o));
    nx[2] = __ldg(reinterpret_cast<const uint4*>(p.k + o)); nx[3] = __ldg(reinterpret_cast<const uint4*>(p.v + o));
    nx[4] = __ldg(reinterpret_cast<const uint4*>(p.g + o));
  };
  auto cvt = [](const uint4& raw, float (&x)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  };
  if (r0 < r1) fetch(r0);
#pragma unroll 1
  for (int row = r0; row < r1; ++row) {
    const size_t o = (size_t)row * p.C + c;
    float y[8], r[8], k[8], v[8], g[8];
    cvt(nx[0], y); cvt(nx[1], r); cvt(nx[2], k); cvt(nx[3], v); cvt(nx[4], g);
    if (row + 1 < r1) fetch(row + 1);
    float sy = 0.f, srk = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { sy += y[j]; srk = fmaf(r[j] * k[j], rk[j], srk); }
    const float mu = head_sum8(sy) * (1.f / 64.f);
    const float s = head_sum8(srk);
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { y[j] -= mu; sv = fmaf(y[j], y[j], sv); }
    const float rs = rsqrtf(head_sum8(sv) * (1.f / 64.f) + p.eps);
    float out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = (y[j] * rs * lw[j] + lb[j] + s * v[j]) * g[j];
    st8(p.out + o, out);
  }
}

void gn_bonus_gate_fwd(const void* const* in, const float* const* par, void* out, int M, int C, float eps,
                       cudaStream_t st) {
  GnParams p{};
  p.y = (const bf16*)in[0]; p.r = (const bf16*)in[1]; p.k = (const bf16*)in[2]; p.v = (const bf16*)in[3];
  p.g = (const bf16*)in[4];
  p.ln_w = par[0]; p.ln_b = par[1]; p.r_k = par[2];
  p.out = (bf16*)out; p.M = M; p.C = C; p.eps = eps;
  p.rows_per_part = fwd_rows_per_part(M);
  if (C % 64 == 0 && C / 8 <= 256 && (C / 8) % 32 == 0) {
    gn_bonus_gate_fwd_wide_kernel<<<(M + p.rows_per_part - 1) / p.rows_per_part, C / 8, 0, st>>>(p);
    return;
  }
  dim3 grid((C / 64 + 7) / 8, (M + p.rows_per_part - 1) / p.rows_per_part);
  gn_bonus_gate_fwd_kernel<<<grid, 256, 0, st>>>(p);
}

void gn_bonus_gate_bwd(const void* const* in, const float* const* par, const void* dout, void* const* gin,
                       float* const* gpar_part, int M, int C, float eps, cudaStream_t st) {
  GnParams p{};
  p.y = (const bf16*)in[0]; p.r = (const bf16*)in[1]; p.k = (const bf16*)in[2]; p.v = (const bf16*)in[3];
  p.g = (const bf16*)in[4];
  p.ln_w = par[0]; p.ln_b = par[1]; p.r_k = par[2];
  p.dout = (const bf16*)dout;
  p.dy = (bf16*)gin[0]; p.dr = (bf16*)gin[1]; p.dk = (bf16*)gin[2]; p.dv = (bf16*)gin[3]; p.dg = (bf16*)gin[4];
  p.dlnw_part = gpar_part[0]; p.dlnb_part = gpar_part[1]; p.drk_part = gpar_part[2];
  p.M = M; p.C = C; p.eps = eps;
  if (C % 64 == 0 && C / 8 <= 256 && (C / 8) % 32 == 0) {
    gn_bonus_gate_bwd_wide_kernel<<<row_parts(M), C / 8, 0, st>>>(p);
    return;
  }
  dim3 grid((C / 64 + 7) / 8, row_parts(M));
  gn_bonus_gate_bwd_kernel<<<grid, 256, 0, st>>>(p);
}

// ---------------------------------------------------------------------------------
// relu(x)^2 backward from the saved output h: dpre = dh * 2 sqrt(h)
// ---------------------------------------------------------------------------------
__global__ void relusq_bwd_kernel(const bf16* __restrict__ dh, const bf16* __restrict__ h, bf16* __restrict__ out,
                                  int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 8;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    uint4 a = *reinterpret_cast<const uint4*>(dh + i);
    uint4 b = *reinterpret_cast<const uint4*>(h + i);
    const bf162* pa = reinterpret_cast<const bf162*>(&a);
    const bf162* pb = reinterpret_cast<const bf162*>(&b);
    uint4 o;
    bf162* po = reinterpret_cast<bf162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 g = __bfloat1622float2(pa[j]), hh = __bfloat1622float2(pb[j]);
      po[j] = __floats2bfloat162_rn(g.x * 2.f * sqrtf(hh.x), g.y * 2.f * sqrtf(hh.y));
    }
    *reinterpret_cast<uint4*>(out + i) = o;
  }
}

void relusq_bwd(const void* dh, const void* h, void* out, int64_t n, cudaStream_t st) {
  int64_t want = (n / 8 + 255) / 256;
  int blocks = (int)(want > 148 * 32 ? 148 * 32 : (want < 1 ? 1 : want));
  relusq_bwd_kernel<<<blocks, 256, 0, st>>>((const bf16*)dh, (const bf16*)h, (bf16*)out, n);
}

// ---------------------------------------------------------------------------------
// Embedding: out[m] = table[ids[m]] (bf16 out, bf16 or fp32 table) and its transpose, the scatter-add of the output
// gradient rows into the fp32 gradient of the table.  One warp per token row, 16-byte accesses; the scatter uses one
// vector reduction (red.global.add.v4.f32) per four channels, so rows that repeat a token id add up in any order.
// Ids outside [0, V) produce a zero row forward and are skipped backward.
// ---------------------------------------------------------------------------------
template <typename TT>
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const int* __restrict__ ids, const TT* __restrict__ table,
                                                            bf16* __restrict__ out, int M, int C, int V) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; m < M; m += warps) {
    const int id = ids[m];
    const bool ok = id >= 0 && id < V;
    const TT* src = table + (size_t)(ok ? id : 0) * C;
    bf16* dst = out + (size_t)m * C;
    for (int c = lane * 8; c < C; c += 256) {
      uint4 o = make_uint4(0u, 0u, 0u, 0u);
      if (ok) {
        if constexpr (sizeof(TT) == 2) {
          o = *reinterpret_cast<const uint4*>(src + c);
        } else {
          const float4 a = *reinterpret_cast<const float4*>(src + c), b = *reinterpret_cast<const float4*>(src + c + 4);
          bf162* po = reinterpret_cast<bf162*>(&o);
          po[0] = __floats2bfloat162_rn(a.x, a.y); po[1] = __floats2bfloat162_rn(a.z, a.w);
          po[2] = __floats2bfloat162_rn(b.x, b.y); po[3] = __floats2bfloat162_rn(b.z, b.w);
        }
      }
      *reinterpret_cast<uint4*>(dst + c) = o;
    }
  }
}

__global__ void __launch_bounds__(256) embedding_bwd_kernel(const int* __restrict__ ids, const bf16* __restrict__ dout,
                                                            float* __restrict__ grad, int M, int C, int V) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; m < M; m += warps) {
    const int id = ids[m];
    if (id < 0 || id >= V) continue;
    const bf16* src = dout + (size_t)m * C;
    float* dst = grad + (size_t)id * C;
    for (int c = lane * 8; c < C; c += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      const bf162* pr = reinterpret_cast<const bf162*>(&raw);
      const float2 a = __bfloat1622float2(pr[0]), b = __bfloat1622float2(pr[1]);
      const float2 e = __bfloat1622float2(pr[2]), f = __bfloat1622float2(pr[3]);
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c), "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y)
                   : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c + 4), "f"(e.x), "f"(e.y), "f"(f.x), "f"(f.y)
                   : "memory");
    }
  }
}

void embedding_fwd(const int* ids, const void* table, bool table_bf16, void* out, int M, int C, int V, cudaStream_t st) {
  const int blocks = std::min(148 * 8, (M + 7) / 8);
  if (table_bf16)
    embedding_fwd_kernel<bf16><<<blocks, 256, 0, st>>>(ids, (const bf16*)table, (bf16*)out, M, C, V);
  else
    embedding_fwd_kernel<float><<<blocks, 256, 0, st>>>(ids, (const float*)table, (bf16*)out, M, C, V);
}

void embedding_bwd(const int* ids, const void* dout, float* grad, int M, int C, int V, cudaStream_t st) {
  const int blocks = std::min(148 * 8, (M + 7) / 8);
  embedding_bwd_kernel<<<blocks, 256, 0, st>>>(ids, (const bf16*)dout, grad, M, C, V);
}

// ---------------------------------------------------------------------------------
// Sum of per-block partial rows: in [groups, parts, cols] (row stride `row_stride` floats, group stride `group_stride`)
// -> out [groups, cols].  One block owns 64 columns of one group: 16 threads across (16-byte loads) by 32 down, the 32
// row lanes meet in shared memory.  Fixed summation order, so a gradient does not depend on scheduling.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(512) partial_sum_kernel(const float* __restrict__ in, float* __restrict__ out, int parts,
                                                          int cols, size_t row_stride, size_t group_stride) {
  __shared__ float4 red[32][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int c = blockIdx.x * 64 + tx * 4;
  const float* src = in + (size_t)blockIdx.y * group_stride;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  if (c + 3 < cols) {
    int r = ty;
    for (; r + 32 < parts; r += 64) {
      const float4 u = __ldg(reinterpret_cast<const float4*>(src + (size_t)r * row_stride + c));
      const float4 v = __ldg(reinterpret_cast<const float4*>(src + (size_t)(r + 32) * row_stride + c));
      a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
      b.x += v.x; b.y += v.y; b.z += v.z; b.w += v.w;
    }
    if (r < parts) {
      const float4 u = __ldg(reinterpret_cast<const float4*>(src + (size_t)r * row_stride + c));
      a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
    }
  } else {
    for (int r = ty; r < parts; r += 32) {
      const float* p = src + (size_t)r * row_stride;
      if (c < cols) a.x += p[c];
      if (c + 1 < cols) a.y += p[c + 1];
      if (c + 2 < cols) a.z += p[c + 2];
    }
  }
  red[ty][tx] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
  __syncthreads();
  for (int half = 16; half >= 1; half >>= 1) {
    if (ty < half) {
      const float4 u = red[ty][tx], v = red[ty + half][tx];
      red[ty][tx] = make_float4(u.x + v.x, u.y + v.y, u.z + v.z, u.w + v.w);
    }
    __syncthreads();
  }
  if (ty == 0) {
    const float4 t = red[0][tx];
    float* o = out + (size_t)blockIdx.y * cols;
    if (c + 3 < cols) {
      *reinterpret_cast<float4*>(o + c) = t;
    } else {
      if (c < cols) o[c] = t.x;
      if (c + 1 < cols) o[c + 1] = t.y;
      if (c + 2 < cols) o[c + 2] = t.z;
    }
  }
}

// cols and both strides must be multiples of 4 floats and the pointers 16-byte aligned (the callers allocate them so)
void partial_sum(const float* in, float* out, int groups, int parts, int cols, size_t row_stride, size_t group_stride,
                 cudaStream_t st) {
  dim3 grid((cols + 63) / 64, groups);
  partial_sum_kernel<<<grid, 512, 0, st>>>(in, out, parts, cols, row_stride, group_stride);
}

}  // namespace rk
