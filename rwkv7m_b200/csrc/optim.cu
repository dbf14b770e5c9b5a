// Fused optimizer kernels over the flat parameter buffer:
//  * grad_norm_sq: sum of squared gradients (for global-norm clipping),
//  * adamw_flat:   clip-scale * grad -> Adam moments -> decoupled weight decay on
//                  the decayed group -> x2 update on the w0 group -> master
//                  parameter, plus the bf16 compute copy and gradient zeroing,
//                  all in one pass over memory.
// Optimizer semantics: src/rwkv7m/train/train_state.py:69-124 of the reference.
#include "common.cuh"
#include "kernels.h"

namespace rk {

template <typename G>
__global__ void grad_norm_sq_kernel(const G* __restrict__ g, int64_t n, float* __restrict__ out) {
  float acc = 0.f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      if constexpr (sizeof(G) == 4) {
        float4 t = *reinterpret_cast<const float4*>(g + i);
        acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
      } else {
        uint2 raw = *reinterpret_cast<const uint2*>(g + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        acc += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
      }
    } else {
      for (int64_t j = i; j < n; ++j) { float t = to_float(g[j]); acc += t * t; }
    }
  }
  acc = warp_sum(acc);
  __shared__ float part[32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

void grad_norm_sq(const void* g, bool g_is_bf16, int64_t n, float* out, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (int)((n / 4 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (g_is_bf16)
    grad_norm_sq_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)g, n, out);
  else
    grad_norm_sq_kernel<float><<<blocks, 256, 0, st>>>((const float*)g, n, out);
}

template <typename P, typename G, typename S>
__global__ void adamw_kernel(AdamWArgs p) {
  P* param = (P*)p.param;
  G* grad = (G*)p.grad;
  S* m = (S*)p.m;
  S* v = (S*)p.v;
  __nv_bfloat16* shadow = (__nv_bfloat16*)p.shadow;
  const float norm = sqrtf(*p.norm_sq) * p.grad_scale;
  const float clip = (norm < p.max_norm ? 1.0f : p.max_norm / norm) * p.grad_scale;
  const float inv_bc1 = 1.0f / p.bc1, inv_bc2 = 1.0f / p.bc2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = p.begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.end; i += stride) {
    const float g = to_float(grad[i]) * clip;
    const float mi = p.beta1 * to_float(m[i]) + (1.0f - p.beta1) * g;
    const float vi = p.beta2 * to_float(v[i]) + (1.0f - p.beta2) * g * g;
    m[i] = from_float<S>(mi);
    v[i] = from_float<S>(vi);
    float w = to_float(param[i]);
    float upd = (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + p.eps);
    if (i < p.n_decay) upd += p.weight_decay * w;
    if (i >= p.n_nodecay_end) upd *= 2.0f;
    w -= p.lr * upd;
    param[i] = from_float<P>(w);
    if (shadow != nullptr) shadow[i] = f2bf(w);
    if (p.zero_grad) grad[i] = from_float<G>(0.f);
  }
}

void adamw_flat(const AdamWArgs& p, cudaStream_t st) {
  const int64_t n = p.end - p.begin;
  if (n <= 0) return;
  int64_t want = (n + 255) / 256;
  int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
#define RK_GO(P, G, S) adamw_kernel<P, G, S><<<blocks, 256, 0, st>>>(p)
  using bf = __nv_bfloat16;
  const int key = (p.param_bf16 ? 4 : 0) | (p.grad_bf16 ? 2 : 0) | (p.state_bf16 ? 1 : 0);
  switch (key) {
    case 0: RK_GO(float, float, float); break;
    case 1: RK_GO(float, float, bf); break;
    case 2: RK_GO(float, bf, float); break;
    case 3: RK_GO(float, bf, bf); break;
    case 4: RK_GO(bf, float, float); break;
    case 5: RK_GO(bf, float, bf); break;
    case 6: RK_GO(bf, bf, float); break;
    default: RK_GO(bf, bf, bf); break;
  }
#undef RK_GO
}

}  // namespace rk
