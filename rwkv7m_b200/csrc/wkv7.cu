// WKV7 generalised delta-rule recurrence, time-sequential form.
//
//   d_t  = exp(-exp(w_t))
//   sa_t = S_{t-1} a_t
//   S_t  = S_{t-1} diag(d_t) + sa_t b_t^T + v_t k_t^T        (S is [value row i, key column j])
//   y_t  = S_t r_t
//
// One CTA per (batch, head).  Forward: four threads share row i of S (16 columns each
// for N = 64), so a mat-vec product is a short thread-local dot plus two shuffles and
// the per-step vectors are broadcast from double-buffered shared memory (one barrier
// per step).  Backward: 8N threads; the first 4N own rows of the state cotangent, the
// other 4N own columns of both the state and its cotangent, so every reduction is
// again a local dot plus two shuffles.  The previous state is re-derived by undoing
// one step (division by the decay, which the soft clamp keeps above 0.545) and
// is re-anchored from an exact checkpoint at every chunk boundary.
//
// Reference semantics: src/rwkv7m/model/rwkv_core.py:54-86 and
// src/rwkv7m/kernels/wkv_pallas_gpu.py:66-282 (forward with aux, backward).
#include "common.cuh"
#include "kernels.h"

namespace rk {

// Element e = 4*q + x of a thread with part index p covers position 16*q + 4*p + x, so the four
// threads that share a row (or column) read four consecutive float4 of a broadcast vector.
template <int N> __device__ __forceinline__ int pos_of(int q, int p, int x) { return 16 * q + 4 * p + x; }

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

template <typename T, int N, bool SAVE>
__global__ void __launch_bounds__(4 * N) wkv7_fwd_kernel(const T* __restrict__ r, const T* __restrict__ w,
                                                         const T* __restrict__ k, const T* __restrict__ v,
                                                         const T* __restrict__ a, const T* __restrict__ b,
                                                         const float* __restrict__ s0, T* __restrict__ y,
                                                         float* __restrict__ sT, float* __restrict__ sa_out,
                                                         float* __restrict__ ckpt, int Tlen, int H, int interval) {
  constexpr int NQ = N / 16;
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const int i = tid >> 2, p = tid & 3;
  const int BH = gridDim.x;
  __shared__ __align__(16) float sm[2][6][N];  // r, d, k, a, b, v

  float S[4 * NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    float4 t4 = *reinterpret_cast<const float4*>(s0 + ((size_t)bh * N + i) * N + pos_of<N>(q, p, 0));
    S[4 * q] = t4.x; S[4 * q + 1] = t4.y; S[4 * q + 2] = t4.z; S[4 * q + 3] = t4.w;
  }
  // staging: thread loads element (tid % N) of vector (tid / N) in {r,w,k,a}; the first 2N threads also load {b,v}
  const int vec0 = tid / N, elem = tid % N;
  const T* src0 = vec0 == 0 ? r : (vec0 == 1 ? w : (vec0 == 2 ? k : a));
  const int dst0 = vec0 == 0 ? 0 : (vec0 == 1 ? 1 : (vec0 == 2 ? 2 : 3));
  const bool second = tid < 2 * N;
  const T* src1 = vec0 == 0 ? b : v;
  const int dst1 = vec0 == 0 ? 4 : 5;
  const size_t stride_t = (size_t)H * N;
  size_t off = ((size_t)bidx * Tlen * H + h) * N;
  float p0 = to_float(src0[off + elem]);
  float p1 = second ? to_float(src1[off + elem]) : 0.f;
  for (int t = 0; t < Tlen; ++t) {
    const int buf = t & 1;
    sm[buf][dst0][elem] = (vec0 == 1) ? expf(-expf(p0)) : p0;
    if (second) sm[buf][dst1][elem] = p1;
    __syncthreads();
    const size_t cur = off;
    if (t + 1 < Tlen) {
      off += stride_t;
      p0 = to_float(src0[off + elem]);
      if (second) p1 = to_float(src1[off + elem]);
    }
    const float4* r4 = reinterpret_cast<const float4*>(sm[buf][0]);
    const float4* d4 = reinterpret_cast<const float4*>(sm[buf][1]);
    const float4* k4 = reinterpret_cast<const float4*>(sm[buf][2]);
    const float4* a4 = reinterpret_cast<const float4*>(sm[buf][3]);
    const float4* b4 = reinterpret_cast<const float4*>(sm[buf][4]);
    const float vi = sm[buf][5][i];
    float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const float4 aa = a4[q * 4 + p];
      sa0 += S[4 * q] * aa.x + S[4 * q + 2] * aa.z;
      sa1 += S[4 * q + 1] * aa.y + S[4 * q + 3] * aa.w;
    }
    const float sa = quad_sum(sa0 + sa1);
    float y0 = 0.f, y1 = 0.f;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const float4 dd = d4[q * 4 + p], bb = b4[q * 4 + p], kk = k4[q * 4 + p], rr = r4[q * 4 + p];
      S[4 * q] = S[4 * q] * dd.x + sa * bb.x + vi * kk.x;
      S[4 * q + 1] = S[4 * q + 1] * dd.y + sa * bb.y + vi * kk.y;
      S[4 * q + 2] = S[4 * q + 2] * dd.z + sa * bb.z + vi * kk.z;
      S[4 * q + 3] = S[4 * q + 3] * dd.w + sa * bb.w + vi * kk.w;
      y0 += S[4 * q] * rr.x + S[4 * q + 2] * rr.z;
      y1 += S[4 * q + 1] * rr.y + S[4 * q + 3] * rr.w;
    }
    const float yy = quad_sum(y0 + y1);
    if (p == 0) {
      y[cur + i] = from_float<T>(yy);
      if (SAVE) sa_out[cur + i] = sa;
    }
    if (SAVE && ((t + 1) % interval == 0 || t + 1 == Tlen)) {
      const int c = t / interval;
      float* dst = ckpt + (((size_t)c * BH + bh) * N + i) * N;
#pragma unroll
      for (int q = 0; q < NQ; ++q)
        *reinterpret_cast<float4*>(dst + pos_of<N>(q, p, 0)) =
            make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
    }
  }
  float* dst = sT + ((size_t)bh * N + i) * N;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
    *reinterpret_cast<float4*>(dst + pos_of<N>(q, p, 0)) = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
}

// vector ids inside the per-step shared buffer of the backward kernel
enum { VR = 0, VD, VK, VV, VA, VB, VSA, VDY, VEW, VCOUNT };

// 8N threads: the first 4N own rows of the state cotangent G (four threads per row), the other 4N own
// columns of both the state S and G (four threads per column).
template <typename T, int N>
__global__ void __launch_bounds__(8 * N) wkv7_bwd_kernel(
    const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k, const T* __restrict__ v,
    const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ dy, const float* __restrict__ sa,
    const float* __restrict__ ckpt, const float* __restrict__ s0, const float* __restrict__ dsT,
    T* __restrict__ dr, T* __restrict__ dw, T* __restrict__ dk, T* __restrict__ dv, T* __restrict__ da,
    T* __restrict__ db, float* __restrict__ ds0, int Tlen, int H, int interval) {
  constexpr int NQ = N / 16;
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const bool is_col = tid >= 4 * N;
  const int idx = (is_col ? tid - 4 * N : tid) >> 2;  // row i or column j
  const int p = tid & 3;
  const int BH = gridDim.x;
  __shared__ __align__(16) float sm[2][VCOUNT][N];
  __shared__ __align__(16) float sdsa[2][N];

  float G[4 * NQ];
  float S[4 * NQ];
#pragma unroll
  for (int e = 0; e < 4 * NQ; ++e) { G[e] = 0.f; S[e] = 0.f; }
  if (dsT != nullptr) {
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int o = pos_of<N>(q, p, x);
        G[4 * q + x] = is_col ? dsT[((size_t)bh * N + o) * N + idx] : dsT[((size_t)bh * N + idx) * N + o];
      }
  }
  const int nck = (Tlen + interval - 1) / interval;
  if (is_col) {
    const float* src = ckpt + ((size_t)(nck - 1) * BH + bh) * N * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int x = 0; x < 4; ++x) S[4 * q + x] = src[pos_of<N>(q, p, x) * N + idx];
  }

  // staging: 8 vectors of N values, one value per thread
  const int vec = tid / N, elem = tid % N;
  const size_t stride_t = (size_t)H * N;
  const size_t base = ((size_t)bidx * Tlen * H + h) * N;
  auto fetch = [&](int t) -> float {
    const size_t o = base + (size_t)t * stride_t + elem;
    switch (vec) {
      case 0: return to_float(r[o]);
      case 1: return to_float(w[o]);
      case 2: return to_float(k[o]);
      case 3: return to_float(v[o]);
      case 4: return to_float(a[o]);
      case 5: return to_float(b[o]);
      case 6: return sa[o];
      default: return to_float(dy[o]);
    }
  };
  float pre = fetch(Tlen - 1);
  for (int t = Tlen - 1; t >= 0; --t) {
    const int buf = t & 1;
    if (vec == 1) {
      const float ew = expf(pre);
      const float d = expf(-ew);
      sm[buf][VD][elem] = d;
      sm[buf][VEW][elem] = -ew * d;
    } else {
      const int dst = vec == 0 ? VR : (vec == 2 ? VK : (vec == 3 ? VV : (vec == 4 ? VA : (vec == 5 ? VB : (vec == 6 ? VSA : VDY)))));
      sm[buf][dst][elem] = pre;
    }
    __syncthreads();
    if (t > 0) pre = fetch(t - 1);
    const size_t o = base + (size_t)t * stride_t + idx;
    const float4* vr4 = reinterpret_cast<const float4*>(sm[buf][VR]);
    const float4* vd4 = reinterpret_cast<const float4*>(sm[buf][VD]);
    const float4* vk4 = reinterpret_cast<const float4*>(sm[buf][VK]);
    const float4* vv4 = reinterpret_cast<const float4*>(sm[buf][VV]);
    const float4* va4 = reinterpret_cast<const float4*>(sm[buf][VA]);
    const float4* vb4 = reinterpret_cast<const float4*>(sm[buf][VB]);
    const float4* vsa4 = reinterpret_cast<const float4*>(sm[buf][VSA]);
    const float4* vdy4 = reinterpret_cast<const float4*>(sm[buf][VDY]);
    if (!is_col) {
      const float dyi = sm[buf][VDY][idx];
      float dsa = 0.f, dvi = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 rr = vr4[q * 4 + p], bb = vb4[q * 4 + p], kk = vk4[q * 4 + p];
        G[4 * q] += dyi * rr.x; G[4 * q + 1] += dyi * rr.y; G[4 * q + 2] += dyi * rr.z; G[4 * q + 3] += dyi * rr.w;
        dsa += G[4 * q] * bb.x + G[4 * q + 1] * bb.y + G[4 * q + 2] * bb.z + G[4 * q + 3] * bb.w;
        dvi += G[4 * q] * kk.x + G[4 * q + 1] * kk.y + G[4 * q + 2] * kk.z + G[4 * q + 3] * kk.w;
      }
      dsa = quad_sum(dsa);
      dvi = quad_sum(dvi);
      if (p == 0) { sdsa[buf][idx] = dsa; dv[o] = from_float<T>(dvi); }
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 dd = vd4[q * 4 + p], aa = va4[q * 4 + p];
        G[4 * q] = G[4 * q] * dd.x + dsa * aa.x;
        G[4 * q + 1] = G[4 * q + 1] * dd.y + dsa * aa.y;
        G[4 * q + 2] = G[4 * q + 2] * dd.z + dsa * aa.z;
        G[4 * q + 3] = G[4 * q + 3] * dd.w + dsa * aa.w;
      }
    } else {
      const bool anchor = (t % interval) == 0;  // S_{t-1} is an exact checkpoint (or the initial state)
      const float rj = sm[buf][VR][idx], bj = sm[buf][VB][idx], kj = sm[buf][VK][idx], dj = sm[buf][VD][idx];
      const float inv_d = 1.0f / dj;
      const float* prev = nullptr;
      if (anchor)
        prev = (t == 0) ? (s0 + (size_t)bh * N * N) : (ckpt + ((size_t)(t / interval - 1) * BH + bh) * N * N);
      float drj = 0.f, ddj = 0.f, dbj = 0.f, dkj = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 dy4 = vdy4[q * 4 + p], sa4 = vsa4[q * 4 + p], v4 = vv4[q * 4 + p];
        const float dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        const float sav[4] = {sa4.x, sa4.y, sa4.z, sa4.w};
        const float vvv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int e = 4 * q + x;
          drj += S[e] * dyv[x];
          G[e] += dyv[x] * rj;
          const float sp = anchor ? prev[pos_of<N>(q, p, x) * N + idx] : (S[e] - sav[x] * bj - vvv[x] * kj) * inv_d;
          ddj += G[e] * sp;
          dbj += G[e] * sav[x];
          dkj += G[e] * vvv[x];
          S[e] = sp;
        }
      }
      drj = quad_sum(drj); ddj = quad_sum(ddj); dbj = quad_sum(dbj); dkj = quad_sum(dkj);
      if (p == 0) {
        dr[o] = from_float<T>(drj);
        dw[o] = from_float<T>(ddj * sm[buf][VEW][idx]);
        dk[o] = from_float<T>(dkj);
        db[o] = from_float<T>(dbj);
      }
    }
    __syncthreads();
    if (is_col) {
      const float aj = sm[buf][VA][idx], dj = sm[buf][VD][idx];
      const float4* ds4 = reinterpret_cast<const float4*>(sdsa[buf]);
      float daj = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 ds = ds4[q * 4 + p];
        daj += S[4 * q] * ds.x + S[4 * q + 1] * ds.y + S[4 * q + 2] * ds.z + S[4 * q + 3] * ds.w;
        G[4 * q] = G[4 * q] * dj + ds.x * aj;
        G[4 * q + 1] = G[4 * q + 1] * dj + ds.y * aj;
        G[4 * q + 2] = G[4 * q + 2] * dj + ds.z * aj;
        G[4 * q + 3] = G[4 * q + 3] * dj + ds.w * aj;
      }
      daj = quad_sum(daj);
      if (p == 0) da[o] = from_float<T>(daj);
    }
  }
  if (!is_col) {
    float* dst = ds0 + ((size_t)bh * N + idx) * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
      *reinterpret_cast<float4*>(dst + pos_of<N>(q, p, 0)) = make_float4(G[4 * q], G[4 * q + 1], G[4 * q + 2], G[4 * q + 3]);
  }
}

template <typename T>
static void launch_fwd(const WkvArgs& p, cudaStream_t st) {
  const T* r = (const T*)p.r; const T* w = (const T*)p.w; const T* k = (const T*)p.k;
  const T* v = (const T*)p.v; const T* a = (const T*)p.a; const T* b = (const T*)p.b;
  T* y = (T*)p.y;
  dim3 grid(p.B * p.H);
  const bool save = p.sa != nullptr;
#define RK_LAUNCH(NN)                                                                                        \
  if (save)                                                                                                  \
    wkv7_fwd_kernel<T, NN, true><<<grid, 4 * NN, 0, st>>>(r, w, k, v, a, b, p.s0, y, p.sT, p.sa, p.ckpt, p.T,    \
                                                      p.H, p.interval);                                      \
  else                                                                                                       \
    wkv7_fwd_kernel<T, NN, false><<<grid, 4 * NN, 0, st>>>(r, w, k, v, a, b, p.s0, y, p.sT, nullptr, nullptr,    \
                                                       p.T, p.H, p.interval);
  if (p.N == 64) { RK_LAUNCH(64) }
  else if (p.N == 32) { RK_LAUNCH(32) }
  else if (p.N == 16) { RK_LAUNCH(16) }
#undef RK_LAUNCH
}

template <typename T>
static void launch_bwd(const WkvArgs& p, cudaStream_t st) {
  const T* r = (const T*)p.r; const T* w = (const T*)p.w; const T* k = (const T*)p.k;
  const T* v = (const T*)p.v; const T* a = (const T*)p.a; const T* b = (const T*)p.b;
  dim3 grid(p.B * p.H);
#define RK_LAUNCH(NN)                                                                                        \
  wkv7_bwd_kernel<T, NN><<<grid, 8 * NN, 0, st>>>(r, w, k, v, a, b, (const T*)p.dy, p.sa, p.ckpt, p.s0,      \
                                                  p.dsT, (T*)p.dr, (T*)p.dw, (T*)p.dk, (T*)p.dv, (T*)p.da,   \
                                                  (T*)p.db, p.ds0, p.T, p.H, p.interval);
  if (p.N == 64) { RK_LAUNCH(64) }
  else if (p.N == 32) { RK_LAUNCH(32) }
  else if (p.N == 16) { RK_LAUNCH(16) }
#undef RK_LAUNCH
}

int wkv7_forward(const WkvArgs& p, cudaStream_t st) {
  if (p.N != 64 && p.N != 32 && p.N != 16) return 1;
  if (p.is_bf16) launch_fwd<__nv_bfloat16>(p, st); else launch_fwd<float>(p, st);
  return 0;
}

int wkv7_backward(const WkvArgs& p, cudaStream_t st) {
  if (p.N != 64 && p.N != 32 && p.N != 16) return 1;
  if (p.is_bf16) launch_bwd<__nv_bfloat16>(p, st); else launch_bwd<float>(p, st);
  return 0;
}

}  // namespace rk
