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

// Four consecutive elements as one 16-byte (fp32) or 8-byte (bf16) access.
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&o)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  }
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&o)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  } else {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(o[0], o[1]);
    h[1] = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}

struct AdamWScalars {
  float clip, inv_bc1, inv_bc2;
};

// One element of the update; returns the new master value.
__device__ __forceinline__ float adamw_one(const AdamWArgs& p, const AdamWScalars& c, int64_t i, float g, float w,
                                           float& mi, float& vi) {
  g *= c.clip;
  mi = p.beta1 * mi + (1.0f - p.beta1) * g;
  vi = p.beta2 * vi + (1.0f - p.beta2) * g * g;
  float upd = (mi * c.inv_bc1) / (sqrtf(vi * c.inv_bc2) + p.eps);
  if (i < p.n_decay) upd += p.weight_decay * w;
  if (i >= p.n_nodecay_end) upd *= 2.0f;
  return w - p.lr * upd;
}

// VEC: every thread owns groups of four consecutive elements (the launcher checks that all base pointers are
// 16-byte aligned); the ragged head and tail of [begin, end) are done one element at a time by block 0.
template <typename P, typename G, typename S, bool VEC>
__global__ void __launch_bounds__(256) adamw_kernel(AdamWArgs p) {
  P* param = (P*)p.param;
  G* grad = (G*)p.grad;
  S* m = (S*)p.m;
  S* v = (S*)p.v;
  __nv_bfloat16* shadow = (__nv_bfloat16*)p.shadow;
  const float norm = sqrtf(*p.norm_sq) * p.grad_scale;
  AdamWScalars c;
  c.clip = (norm < p.max_norm ? 1.0f : p.max_norm / norm) * p.grad_scale;
  c.inv_bc1 = 1.0f / p.bc1;
  c.inv_bc2 = 1.0f / p.bc2;
  auto scalar = [&](int64_t i) {
    float mi = to_float(m[i]), vi = to_float(v[i]);
    const float w = adamw_one(p, c, i, to_float(grad[i]), to_float(param[i]), mi, vi);
    m[i] = from_float<S>(mi);
    v[i] = from_float<S>(vi);
    param[i] = from_float<P>(w);
    if (shadow != nullptr) shadow[i] = f2bf(w);
    if (p.zero_grad) grad[i] = from_float<G>(0.f);
  };
  if constexpr (!VEC) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = p.begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.end; i += stride) scalar(i);
  } else {
    const int64_t v0 = (p.begin + 3) & ~(int64_t)3, v1 = p.end & ~(int64_t)3;
    if (blockIdx.x == 0) {
      const int64_t head_end = v0 < p.end ? v0 : p.end;
      for (int64_t i = p.begin + threadIdx.x; i < head_end; i += blockDim.x) scalar(i);
      for (int64_t i = (v1 > v0 ? v1 : head_end) + threadIdx.x; i < p.end; i += blockDim.x) scalar(i);
    }
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    const float zero[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t i = v0 + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < v1; i += stride) {
      float g[4], mi[4], vi[4], w[4];
      load4(grad + i, g);
      load4(m + i, mi);
      load4(v + i, vi);
      load4(param + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = adamw_one(p, c, i + j, g[j], w[j], mi[j], vi[j]);
      store4(m + i, mi);
      store4(v + i, vi);
      store4(param + i, w);
      if (shadow != nullptr) store4(shadow + i, w);
      if (p.zero_grad) store4(grad + i, zero);
    }
  }
}

void adamw_flat(const AdamWArgs& p, cudaStream_t st) {
  const int64_t n = p.end - p.begin;
  if (n <= 0) return;
  const uintptr_t bits = (uintptr_t)p.param | (uintptr_t)p.grad | (uintptr_t)p.m | (uintptr_t)p.v | (uintptr_t)p.shadow;
  const bool vec = (bits & 15) == 0;
  int64_t want = ((vec ? n / 4 : n) + 255) / 256 + 1;
  int blocks = (int)(want > 148 * 8 ? 148 * 8 : want);
#define RK_GO(P, G, S)                                      \
  do {                                                      \
    if (vec) adamw_kernel<P, G, S, true><<<blocks, 256, 0, st>>>(p);  \
    else adamw_kernel<P, G, S, false><<<blocks, 256, 0, st>>>(p);     \
  } while (0)
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
