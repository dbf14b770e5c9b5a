// WKV7 generalised delta-rule recurrence, time-sequential form.
//
//   d_t  = exp(-exp(w_t))
//   sa_t = S_{t-1} a_t
//   S_t  = S_{t-1} diag(d_t) + sa_t b_t^T + v_t k_t^T        (S is [value row i, key column j])
//   y_t  = S_t r_t
//
// One CTA per (batch, head).  Forward: thread i owns row i of S in registers,
// so both mat-vec products are thread-local and the per-step vectors are
// broadcast from double-buffered shared memory (one barrier per step).
// Backward: 2N threads; the first N own rows of the state cotangent, the second
// N own columns of both the state and its cotangent, which makes every
// reduction thread-local as well.  The previous state is re-derived by undoing
// one step (division by the decay, which the soft clamp keeps above 0.545) and
// is re-anchored from an exact checkpoint at every chunk boundary.
//
// Reference semantics: src/rwkv7m/model/rwkv_core.py:54-86 and
// src/rwkv7m/kernels/wkv_pallas_gpu.py:66-282 (forward with aux, backward).
#include "common.cuh"
#include "kernels.h"

namespace rk {

template <typename T, int N, bool SAVE>
__global__ void __launch_bounds__(N) wkv7_fwd_kernel(const T* __restrict__ r, const T* __restrict__ w,
                                                     const T* __restrict__ k, const T* __restrict__ v,
                                                     const T* __restrict__ a, const T* __restrict__ b,
                                                     const float* __restrict__ s0, T* __restrict__ y,
                                                     float* __restrict__ sT, float* __restrict__ sa_out,
                                                     float* __restrict__ ckpt, int Tlen, int H, int interval) {
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int i = threadIdx.x;
  const int BH = gridDim.x;
  __shared__ __align__(16) float sm[2][5][N];  // r, d, k, a, b

  float S[N];
  {
    const float4* src = reinterpret_cast<const float4*>(s0 + ((size_t)bh * N + i) * N);
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
      float4 t4 = src[q];
      S[4 * q] = t4.x; S[4 * q + 1] = t4.y; S[4 * q + 2] = t4.z; S[4 * q + 3] = t4.w;
    }
  }
  const size_t stride_t = (size_t)H * N;
  size_t off = ((size_t)bidx * Tlen * H + h) * N + i;
  float pr = to_float(r[off]), pw = to_float(w[off]), pk = to_float(k[off]), pv = to_float(v[off]),
        pa = to_float(a[off]), pb = to_float(b[off]);
  for (int t = 0; t < Tlen; ++t) {
    const int buf = t & 1;
    sm[buf][0][i] = pr;
    sm[buf][1][i] = expf(-expf(pw));
    sm[buf][2][i] = pk;
    sm[buf][3][i] = pa;
    sm[buf][4][i] = pb;
    const float vi = pv;
    __syncthreads();
    const size_t cur = off;
    if (t + 1 < Tlen) {
      off += stride_t;
      pr = to_float(r[off]); pw = to_float(w[off]); pk = to_float(k[off]);
      pv = to_float(v[off]); pa = to_float(a[off]); pb = to_float(b[off]);
    }
    const float4* r4 = reinterpret_cast<const float4*>(sm[buf][0]);
    const float4* d4 = reinterpret_cast<const float4*>(sm[buf][1]);
    const float4* k4 = reinterpret_cast<const float4*>(sm[buf][2]);
    const float4* a4 = reinterpret_cast<const float4*>(sm[buf][3]);
    const float4* b4 = reinterpret_cast<const float4*>(sm[buf][4]);
    float sa = 0.f;
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
      float4 aa = a4[q];
      sa += S[4 * q] * aa.x + S[4 * q + 1] * aa.y + S[4 * q + 2] * aa.z + S[4 * q + 3] * aa.w;
    }
    float yy = 0.f;
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
      float4 dd = d4[q], bb = b4[q], kk = k4[q], rr = r4[q];
      S[4 * q] = S[4 * q] * dd.x + sa * bb.x + vi * kk.x;
      S[4 * q + 1] = S[4 * q + 1] * dd.y + sa * bb.y + vi * kk.y;
      S[4 * q + 2] = S[4 * q + 2] * dd.z + sa * bb.z + vi * kk.z;
      S[4 * q + 3] = S[4 * q + 3] * dd.w + sa * bb.w + vi * kk.w;
      yy += S[4 * q] * rr.x + S[4 * q + 1] * rr.y + S[4 * q + 2] * rr.z + S[4 * q + 3] * rr.w;
    }
    y[cur] = from_float<T>(yy);
    if (SAVE) {
      sa_out[cur] = sa;
      if ((t + 1) % interval == 0 || t + 1 == Tlen) {
        const int c = t / interval;
        float4* dst = reinterpret_cast<float4*>(ckpt + (((size_t)c * BH + bh) * N + i) * N);
#pragma unroll
        for (int q = 0; q < N / 4; ++q) dst[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
      }
    }
  }
  float4* dst = reinterpret_cast<float4*>(sT + ((size_t)bh * N + i) * N);
#pragma unroll
  for (int q = 0; q < N / 4; ++q) dst[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
}

// vector ids inside the per-step shared buffer of the backward kernel
enum { VR = 0, VD, VK, VV, VA, VB, VSA, VDY, VEW, VCOUNT };

template <typename T, int N>
__global__ void __launch_bounds__(2 * N) wkv7_bwd_kernel(
    const T* __restrict__ r, const T* __restrict__ w, const T* __restrict__ k, const T* __restrict__ v,
    const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ dy, const float* __restrict__ sa,
    const float* __restrict__ ckpt, const float* __restrict__ s0, const float* __restrict__ dsT,
    T* __restrict__ dr, T* __restrict__ dw, T* __restrict__ dk, T* __restrict__ dv, T* __restrict__ da,
    T* __restrict__ db, float* __restrict__ ds0, int Tlen, int H, int interval) {
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const int idx = tid % N;
  const bool is_col = tid >= N;
  const int BH = gridDim.x;
  __shared__ __align__(16) float sm[2][VCOUNT][N];
  __shared__ __align__(16) float sdsa[2][N];

  // row threads: G[j] = dS[idx][j];  col threads: G[i] = dS[i][idx], S[i] = S[i][idx]
  float G[N];
  float S[N];
  if (dsT != nullptr) {
    if (!is_col) {
#pragma unroll
      for (int j = 0; j < N; ++j) G[j] = dsT[((size_t)bh * N + idx) * N + j];
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) G[i] = dsT[((size_t)bh * N + i) * N + idx];
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) G[j] = 0.f;
  }
  const int nck = (Tlen + interval - 1) / interval;
  if (is_col) {
    const float* src = ckpt + ((size_t)(nck - 1) * BH + bh) * N * N;
#pragma unroll
    for (int i = 0; i < N; ++i) S[i] = src[i * N + idx];
  }

  const size_t stride_t = (size_t)H * N;
  const size_t base = ((size_t)bidx * Tlen * H + h) * N + idx;
  // Each thread stages 4 of the 8 per-step input vectors: rows load {r,k,a,sa}, columns load {w,v,b,dy}.
  float p0, p1, p2, p3;
  auto fetch = [&](int t) {
    const size_t o = base + (size_t)t * stride_t;
    if (!is_col) {
      p0 = to_float(r[o]); p1 = to_float(k[o]); p2 = to_float(a[o]); p3 = sa[o];
    } else {
      p0 = to_float(w[o]); p1 = to_float(v[o]); p2 = to_float(b[o]); p3 = to_float(dy[o]);
    }
  };
  fetch(Tlen - 1);
  for (int t = Tlen - 1; t >= 0; --t) {
    const int buf = t & 1;
    if (!is_col) {
      sm[buf][VR][idx] = p0; sm[buf][VK][idx] = p1; sm[buf][VA][idx] = p2; sm[buf][VSA][idx] = p3;
    } else {
      const float ew = expf(p0);
      const float d = expf(-ew);
      sm[buf][VD][idx] = d; sm[buf][VEW][idx] = -ew * d;
      sm[buf][VV][idx] = p1; sm[buf][VB][idx] = p2; sm[buf][VDY][idx] = p3;
    }
    __syncthreads();
    if (t > 0) fetch(t - 1);
    const size_t o = base + (size_t)t * stride_t;
    const float* vr = sm[buf][VR];
    const float* vd = sm[buf][VD];
    const float* vk = sm[buf][VK];
    const float* vv = sm[buf][VV];
    const float* va = sm[buf][VA];
    const float* vb = sm[buf][VB];
    const float* vsa = sm[buf][VSA];
    const float* vdy = sm[buf][VDY];
    const bool anchor = (t % interval) == 0;  // S_{t-1} is an exact checkpoint (or the initial state)
    float dk_j = 0.f, db_j = 0.f, dd_j = 0.f;
    if (!is_col) {
      const float dyi = vdy[idx];
      float dsa = 0.f, dvi = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        G[j] += dyi * vr[j];
        dsa += G[j] * vb[j];
        dvi += G[j] * vk[j];
      }
      sdsa[buf][idx] = dsa;
      dv[o] = from_float<T>(dvi);
#pragma unroll
      for (int j = 0; j < N; ++j) G[j] = G[j] * vd[j] + dsa * va[j];
    } else {
      const float rj = vr[idx], bj = vb[idx], kj = vk[idx], dj = vd[idx];
      const float inv_d = 1.0f / dj;
      float drj = 0.f;
      const float* prev = nullptr;
      if (anchor) prev = (t == 0) ? (s0 + (size_t)bh * N * N) : (ckpt + ((size_t)(t / interval - 1) * BH + bh) * N * N);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float dyi = vdy[i];
        drj += S[i] * dyi;
        G[i] += dyi * rj;
        float sp = anchor ? prev[i * N + idx] : (S[i] - vsa[i] * bj - vv[i] * kj) * inv_d;
        dd_j += G[i] * sp;
        db_j += G[i] * vsa[i];
        dk_j += G[i] * vv[i];
        S[i] = sp;
      }
      dr[o] = from_float<T>(drj);
      dw[o] = from_float<T>(dd_j * sm[buf][VEW][idx]);
      dk[o] = from_float<T>(dk_j);
      db[o] = from_float<T>(db_j);
    }
    __syncthreads();
    if (is_col) {
      const float aj = va[idx], dj = vd[idx];
      const float* ds = sdsa[buf];
      float daj = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        daj += S[i] * ds[i];
        G[i] = G[i] * dj + ds[i] * aj;
      }
      da[o] = from_float<T>(daj);
    }
  }
  if (!is_col) {
#pragma unroll
    for (int j = 0; j < N; ++j) ds0[((size_t)bh * N + idx) * N + j] = G[j];
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
    wkv7_fwd_kernel<T, NN, true><<<grid, NN, 0, st>>>(r, w, k, v, a, b, p.s0, y, p.sT, p.sa, p.ckpt, p.T,    \
                                                      p.H, p.interval);                                      \
  else                                                                                                       \
    wkv7_fwd_kernel<T, NN, false><<<grid, NN, 0, st>>>(r, w, k, v, a, b, p.s0, y, p.sT, nullptr, nullptr,    \
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
  wkv7_bwd_kernel<T, NN><<<grid, 2 * NN, 0, st>>>(r, w, k, v, a, b, (const T*)p.dy, p.sa, p.ckpt, p.s0,      \
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
