// Cross-entropy + L2Wrap over a [rows, V] block of bf16 logits.
//
//   forward : per row  lse = logsumexp(x), max, argmax, nll = lse - x[target]          (fp32 math)
//   backward: in place dlogits = g_ce * mask * (softmax - onehot(target))
//                                + g_l2 * 1e-4 * max * onehot(argmax)
//             with lse / max / argmax as given: the caller may pass the statistics of a wider row of which these V
//             columns are a slice (vocabulary-parallel head)
// which is the gradient of  sum(mask * nll)  and  0.5e-4 * sum(max^2)
// (src/rwkv7m/model/losses.py:21-69 of the reference).  One CTA per row.
#include "common.cuh"
#include "kernels.h"

namespace rk {

using bf16 = __nv_bfloat16;

__global__ void __launch_bounds__(256) ce_fwd_kernel(const bf16* __restrict__ logits, const int* __restrict__ targets,
                                                     float* __restrict__ lse, float* __restrict__ maxv,
                                                     int* __restrict__ argmax, float* __restrict__ nll, int V) {
  const int row = blockIdx.x;
  const bf16* x = logits + (size_t)row * V;
  float m = -INFINITY, s = 0.f;
  int mi = 0x7fffffff;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float vals[8];
    if (c + 8 <= V) {
      uint4 raw = *reinterpret_cast<const uint4*>(x + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); vals[2 * j] = f.x; vals[2 * j + 1] = f.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) vals[j] = c + j < V ? bf2f(x[c + j]) : -INFINITY;
    }
    float cm = vals[0]; int ci = c;
#pragma unroll
    for (int j = 1; j < 8; ++j) if (vals[j] > cm) { cm = vals[j]; ci = c + j; }
    if (cm > m) { s *= __expf(m - cm); m = cm; mi = ci; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(vals[j] - m);
  }
  // block reduction of (m, s, mi): ties resolve to the lowest index
  __shared__ float sm_m[256], sm_s[256];
  __shared__ int sm_i[256];
  sm_m[threadIdx.x] = m; sm_s[threadIdx.x] = s; sm_i[threadIdx.x] = mi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const float m2 = sm_m[threadIdx.x + o], s2 = sm_s[threadIdx.x + o];
      const int i2 = sm_i[threadIdx.x + o];
      const float m1 = sm_m[threadIdx.x], s1 = sm_s[threadIdx.x];
      const int i1 = sm_i[threadIdx.x];
      const float mm = fmaxf(m1, m2);
      const float e1 = m1 == -INFINITY ? 0.f : s1 * __expf(m1 - mm);
      const float e2 = m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm);
      sm_m[threadIdx.x] = mm;
      sm_s[threadIdx.x] = e1 + e2;
      sm_i[threadIdx.x] = (m2 > m1 || (m2 == m1 && i2 < i1)) ? i2 : i1;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float l = sm_m[0] + logf(sm_s[0]);
    lse[row] = l;
    maxv[row] = sm_m[0];
    argmax[row] = sm_i[0];
    int t = targets[row];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    nll[row] = l - bf2f(x[t]);
  }
}

__global__ void __launch_bounds__(256) ce_bwd_kernel(bf16* __restrict__ logits, const int* __restrict__ targets,
                                                     const float* __restrict__ mask, const float* __restrict__ lse,
                                                     const float* __restrict__ maxv, const int* __restrict__ argmax,
                                                     const float* __restrict__ g_ce, const float* __restrict__ g_l2,
                                                     int V) {
  const int row = blockIdx.x;
  bf16* x = logits + (size_t)row * V;
  const float gce = g_ce[0] * (mask != nullptr ? mask[row] : 1.0f);
  const float l = lse[row];
  // a target or arg-max outside [0, V) matches no column: under a vocabulary split the row's target (or its largest
  // logit) may live on another rank, and this rank then contributes only the softmax term
  const int t = targets[row];
  const int am = argmax[row];
  const float gl2 = g_l2[0] * 1e-4f * maxv[row];
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    if (c + 8 <= V) {
      uint4 raw = *reinterpret_cast<const uint4*>(x + c);
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        float g0 = gce * __expf(f.x - l), g1 = gce * __expf(f.y - l);
        const int c0 = c + 2 * j, c1 = c0 + 1;
        if (c0 == t) g0 -= gce;
        if (c1 == t) g1 -= gce;
        if (c0 == am) g0 += gl2;
        if (c1 == am) g1 += gl2;
        h[j] = __floats2bfloat162_rn(g0, g1);
      }
      *reinterpret_cast<uint4*>(x + c) = raw;
    } else {
      for (int j = 0; j < 8 && c + j < V; ++j) {
        float g = gce * __expf(bf2f(x[c + j]) - l);
        if (c + j == t) g -= gce;
        if (c + j == am) g += gl2;
        x[c + j] = f2bf(g);
      }
    }
  }
}

// One warp per row folds the per-tile statistics of the head GEMM's epilogue: running maximum with rescaled sums, the
// lowest arg-max column among equal maxima, and the target logit (finite in exactly one tile).
__global__ void __launch_bounds__(256) ce_combine_kernel(const float4* __restrict__ stats, int tiles, float* __restrict__ lse,
                                                         float* __restrict__ maxv, int* __restrict__ argmax,
                                                         float* __restrict__ nll, int rows) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float m = -INFINITY, s = 0.f, tl = -INFINITY;
  int am = 0x7fffffff;
  for (int t = lane; t < tiles; t += 32) {
    const float4 v = stats[(size_t)row * tiles + t];
    const int vi = __float_as_int(v.z);
    if (v.x > m) { s = s * __expf(m - v.x) + v.y; m = v.x; am = vi; }
    else { s += v.y * __expf(v.x - m); if (v.x == m && vi < am) am = vi; }
    tl = fmaxf(tl, v.w);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float t2 = __shfl_xor_sync(0xffffffffu, tl, o);
    const int a2 = __shfl_xor_sync(0xffffffffu, am, o);
    const float mm = fmaxf(m, m2);
    const float e1 = m == -INFINITY ? 0.f : s * __expf(m - mm), e2 = m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm);
    am = (m2 > m || (m2 == m && a2 < am)) ? a2 : am;
    m = mm; s = e1 + e2; tl = fmaxf(tl, t2);
  }
  if (lane == 0) {
    const float l = m + logf(s);
    lse[row] = l; maxv[row] = m; argmax[row] = am; nll[row] = l - tl;
  }
}

void ce_combine(const float* stats, int tiles, float* lse, float* maxv, int* argmax, float* nll, int rows, cudaStream_t st) {
  if (rows <= 0) return;
  ce_combine_kernel<<<(rows + 7) / 8, 256, 0, st>>>(reinterpret_cast<const float4*>(stats), tiles, lse, maxv, argmax, nll, rows);
}

void ce_fwd(const void* logits, const int* targets, float* lse, float* maxv, int* argmax, float* nll, int rows, int V,
            cudaStream_t st) {
  if (rows <= 0) return;
  ce_fwd_kernel<<<rows, 256, 0, st>>>((const bf16*)logits, targets, lse, maxv, argmax, nll, V);
}

void ce_bwd(void* logits, const int* targets, const float* mask, const float* lse, const float* maxv,
            const int* argmax, const float* g_ce, const float* g_l2, int rows, int V, cudaStream_t st) {
  if (rows <= 0) return;
  ce_bwd_kernel<<<rows, 256, 0, st>>>((bf16*)logits, targets, mask, lse, maxv, argmax, g_ce, g_l2, V);
}

}  // namespace rk
