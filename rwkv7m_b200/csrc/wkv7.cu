// WKV7 generalised delta-rule recurrence, time-sequential form.
//
//   d_t  = exp(-exp(w_t))
//   sa_t = S_{t-1} a_t
//   S_t  = S_{t-1} diag(d_t) + sa_t b_t^T + v_t k_t^T        (S is [value row i, key column j])
//   y_t  = S_t r_t
//
// One CTA per (batch, head).  The per-step vectors are streamed through shared
// memory in chunks of 16 time steps with cp.async, double-buffered, so global
// latency is paid once per chunk and never inside the recurrence.  Forward: four
// threads share row i of S (16 columns each for N = 64); a mat-vec product is a
// short thread-local dot plus two shuffles and no block barrier is needed inside a
// chunk.  Backward: 8N threads; the first 4N own rows of the state cotangent, the
// other 4N own columns of both the state and its cotangent, exchanging one vector
// per step through shared memory.  The previous state is re-derived by undoing one
// step (division by the decay, which the soft clamp keeps above 0.545) and is
// re-anchored from an exact checkpoint at every chunk boundary.
//
// Reference semantics: src/rwkv7m/model/rwkv_core.py:54-86 and
// src/rwkv7m/kernels/wkv_pallas_gpu.py:66-282 (forward with aux, backward).
#include "common.cuh"
#include "kernels.h"

namespace rk {

constexpr int CH = 16;  // time steps per staged chunk == state checkpoint interval

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Element e = 4*q + x of a thread with part index p covers position 16*q + 4*p + x, so the four
// threads that share a row (or column) read consecutive 4-element groups of a broadcast vector.
__device__ __forceinline__ int pos_of(int q, int p, int x) { return 16 * q + 4 * p + x; }

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int NV>
struct VecPtrs {
  const T* p[NV];
};

// Stage chunk c of NV vectors ([CH][N] each) into tile; rows past the sequence end are zero-filled.
template <typename T, int N, int NV>
__device__ __forceinline__ void stage_chunk(T* tile, const VecPtrs<T, NV>& src, size_t base, size_t stride_t, int c,
                                            int Tlen, int tid, int nthreads) {
  constexpr int EPP = 16 / sizeof(T);  // elements per 16-byte piece
  constexpr int PPR = N / EPP;         // pieces per row
  constexpr int TOTAL = NV * CH * PPR;
  for (int pc = tid; pc < TOTAL; pc += nthreads) {
    const int vec = pc / (CH * PPR);
    const int rem = pc - vec * (CH * PPR);
    const int row = rem / PPR;
    const int col = (rem - row * PPR) * EPP;
    const int t = c * CH + row;
    T* dst = tile + ((size_t)vec * CH + row) * N + col;
    if (t < Tlen) cp_async16(dst, src.p[vec] + base + (size_t)t * stride_t + col);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <typename T, int N, bool SAVE>
__global__ void __launch_bounds__(4 * N) wkv7_fwd_kernel(VecPtrs<T, 6> src, const float* __restrict__ s0,
                                                         T* __restrict__ y, float* __restrict__ sT,
                                                         float* __restrict__ sa_out, float* __restrict__ ckpt,
                                                         int Tlen, int H) {
  constexpr int NQ = N / 16;
  constexpr int NT = 4 * N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tiles = reinterpret_cast<T*>(smem_raw);                                   // [2][6][CH][N]: r,w,k,v,a,b (raw)
  float* work = reinterpret_cast<float*>(smem_raw + 2 * 6 * CH * N * sizeof(T));  // [6][CH][N] fp32, slot 1 = decay
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const int i = tid >> 2, p = tid & 3;
  const int BH = gridDim.x;

  float S[4 * NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const float4 t4 = load4(s0 + ((size_t)bh * N + i) * N + pos_of(q, p, 0));
    S[4 * q] = t4.x; S[4 * q + 1] = t4.y; S[4 * q + 2] = t4.z; S[4 * q + 3] = t4.w;
  }
  const size_t stride_t = (size_t)H * N;
  const size_t base = ((size_t)bidx * Tlen * H + h) * N;
  const int nch = (Tlen + CH - 1) / CH;
  stage_chunk<T, N, 6>(tiles, src, base, stride_t, 0, Tlen, tid, NT);
  cp_async_commit();
  for (int c = 0; c < nch; ++c) {
    const int buf = c & 1;
    T* tile = tiles + (size_t)buf * 6 * CH * N;
    cp_async_wait_all();
    __syncthreads();  // chunk c landed; every thread is done with chunk c-1
    if (c + 1 < nch) {
      stage_chunk<T, N, 6>(tiles + (size_t)(buf ^ 1) * 6 * CH * N, src, base, stride_t, c + 1, Tlen, tid, NT);
      cp_async_commit();
    }
    // one conversion pass per chunk: fp32 copies of every vector, w replaced by the decay exp(-exp(w))
    for (int e = tid; e < 6 * CH * N; e += NT) {
      const float x = to_float(tile[e]);
      work[e] = (e >= CH * N && e < 2 * CH * N) ? expf(-expf(x)) : x;
    }
    __syncthreads();
    const int steps = min(CH, Tlen - c * CH);
    for (int s = 0; s < steps; ++s) {
      const float* vr = work + (0 * CH + s) * N;
      const float* vd = work + (1 * CH + s) * N;
      const float* vk = work + (2 * CH + s) * N;
      const float* vv = work + (3 * CH + s) * N;
      const float* va = work + (4 * CH + s) * N;
      const float* vb = work + (5 * CH + s) * N;
      const float vi = vv[i];
      float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 aa = load4(va + pos_of(q, p, 0));
        sa0 += S[4 * q] * aa.x + S[4 * q + 2] * aa.z;
        sa1 += S[4 * q + 1] * aa.y + S[4 * q + 3] * aa.w;
      }
      const float sa = quad_sum(sa0 + sa1);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const int o = pos_of(q, p, 0);
        const float4 dd = load4(vd + o), bb = load4(vb + o), kk = load4(vk + o), rr = load4(vr + o);
        S[4 * q] = S[4 * q] * dd.x + sa * bb.x + vi * kk.x;
        S[4 * q + 1] = S[4 * q + 1] * dd.y + sa * bb.y + vi * kk.y;
        S[4 * q + 2] = S[4 * q + 2] * dd.z + sa * bb.z + vi * kk.z;
        S[4 * q + 3] = S[4 * q + 3] * dd.w + sa * bb.w + vi * kk.w;
        y0 += S[4 * q] * rr.x + S[4 * q + 2] * rr.z;
        y1 += S[4 * q + 1] * rr.y + S[4 * q + 3] * rr.w;
      }
      const float yy = quad_sum(y0 + y1);
      if (p == 0) {
        const size_t o = base + (size_t)(c * CH + s) * stride_t + i;
        y[o] = from_float<T>(yy);
        if (SAVE) sa_out[o] = sa;
      }
    }
    if (SAVE) {
      float* dst = ckpt + (((size_t)c * BH + bh) * N + i) * N;
#pragma unroll
      for (int q = 0; q < NQ; ++q)
        *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
    }
  }
  float* dst = sT + ((size_t)bh * N + i) * N;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
    *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
}

template <typename T, int N>
constexpr size_t fwd_smem_bytes() { return 2 * 6 * CH * N * sizeof(T) + 6 * CH * N * sizeof(float); }

// Backward.  Tile vectors: r,w,k,v,a,b,dy (type T) and sa (fp32).
template <typename T, int N>
__global__ void __launch_bounds__(8 * N, (N == 64 ? 2 : 1)) wkv7_bwd_kernel(
    VecPtrs<T, 7> src, const float* __restrict__ sa, const float* __restrict__ ckpt, const float* __restrict__ s0,
    const float* __restrict__ dsT, T* __restrict__ dr, T* __restrict__ dw, T* __restrict__ dk, T* __restrict__ dv,
    T* __restrict__ da, T* __restrict__ db, float* __restrict__ ds0, int Tlen, int H) {
  constexpr int NQ = N / 16;
  constexpr int NT = 8 * N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tiles = reinterpret_cast<T*>(smem_raw);                                         // [2][7][CH][N]
  float* sa_tiles = reinterpret_cast<float*>(smem_raw + 2 * 7 * CH * N * sizeof(T));  // [2][CH][N]
  float* work = sa_tiles + 2 * CH * N;                                                // [7][CH][N] fp32, slot 1 = decay
  float* ewd = work + 7 * CH * N;                                                     // [CH][N]  -exp(w) * d
  float* sdsa = ewd + CH * N;                                                         // [2][N]
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const bool is_col = tid >= 4 * N;
  const int idx = (is_col ? tid - 4 * N : tid) >> 2;  // row i or column j
  const int p = tid & 3;
  const int BH = gridDim.x;

  float G[4 * NQ];
  float S[4 * NQ];
  float A[4 * NQ];  // prefetched anchor (exact S at the start of the chunk), column threads only
#pragma unroll
  for (int e = 0; e < 4 * NQ; ++e) { G[e] = 0.f; S[e] = 0.f; A[e] = 0.f; }
  if (dsT != nullptr) {
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int o = pos_of(q, p, x);
        G[4 * q + x] = is_col ? dsT[((size_t)bh * N + o) * N + idx] : dsT[((size_t)bh * N + idx) * N + o];
      }
  }
  const int nch = (Tlen + CH - 1) / CH;
  if (is_col) {
    const float* srcS = ckpt + ((size_t)(nch - 1) * BH + bh) * N * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int x = 0; x < 4; ++x) S[4 * q + x] = srcS[pos_of(q, p, x) * N + idx];
  }

  const size_t stride_t = (size_t)H * N;
  const size_t base = ((size_t)bidx * Tlen * H + h) * N;
  VecPtrs<float, 1> sa_src;
  sa_src.p[0] = sa;
  auto stage = [&](int c, int buf) {
    stage_chunk<T, N, 7>(tiles + (size_t)buf * 7 * CH * N, src, base, stride_t, c, Tlen, tid, NT);
    stage_chunk<float, N, 1>(sa_tiles + (size_t)buf * CH * N, sa_src, base, stride_t, c, Tlen, tid, NT);
    cp_async_commit();
  };
  stage(nch - 1, (nch - 1) & 1);
  for (int c = nch - 1; c >= 0; --c) {
    const int buf = c & 1;
    const T* tile = tiles + (size_t)buf * 7 * CH * N;
    const float* sat = sa_tiles + (size_t)buf * CH * N;
    cp_async_wait_all();
    __syncthreads();
    if (c > 0) stage(c - 1, buf ^ 1);
    for (int e = tid; e < 7 * CH * N; e += NT) {
      const float x = to_float(tile[e]);
      if (e >= CH * N && e < 2 * CH * N) {
        const float ew = expf(x);
        const float d = expf(-ew);
        work[e] = d;
        ewd[e - CH * N] = -ew * d;
      } else {
        work[e] = x;
      }
    }
    if (is_col) {
      // exact state before the first step of this chunk; its latency hides behind the chunk's steps
      const float* prev = (c == 0) ? (s0 + (size_t)bh * N * N) : (ckpt + ((size_t)(c - 1) * BH + bh) * N * N);
#pragma unroll
      for (int q = 0; q < NQ; ++q)
#pragma unroll
        for (int x = 0; x < 4; ++x) A[4 * q + x] = prev[pos_of(q, p, x) * N + idx];
    }
    __syncthreads();
    const int steps = min(CH, Tlen - c * CH);
    for (int s = steps - 1; s >= 0; --s) {
      const int t = c * CH + s;
      const int sb = t & 1;
      const size_t o = base + (size_t)t * stride_t + idx;
      const float* vr = work + (0 * CH + s) * N;
      const float* vd = work + (1 * CH + s) * N;
      const float* vk = work + (2 * CH + s) * N;
      const float* vv = work + (3 * CH + s) * N;
      const float* va = work + (4 * CH + s) * N;
      const float* vb = work + (5 * CH + s) * N;
      const float* vdy = work + (6 * CH + s) * N;
      const float* vsa = sat + s * N;
      if (!is_col) {
        const float dyi = vdy[idx];
        float dsa = 0.f, dvi = 0.f;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 rr = load4(vr + po), bb = load4(vb + po), kk = load4(vk + po);
          G[4 * q] += dyi * rr.x; G[4 * q + 1] += dyi * rr.y; G[4 * q + 2] += dyi * rr.z; G[4 * q + 3] += dyi * rr.w;
          dsa += G[4 * q] * bb.x + G[4 * q + 1] * bb.y + G[4 * q + 2] * bb.z + G[4 * q + 3] * bb.w;
          dvi += G[4 * q] * kk.x + G[4 * q + 1] * kk.y + G[4 * q + 2] * kk.z + G[4 * q + 3] * kk.w;
        }
        dsa = quad_sum(dsa);
        dvi = quad_sum(dvi);
        if (p == 0) { sdsa[sb * N + idx] = dsa; dv[o] = from_float<T>(dvi); }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 dd = load4(vd + po), aa = load4(va + po);
          G[4 * q] = G[4 * q] * dd.x + dsa * aa.x;
          G[4 * q + 1] = G[4 * q + 1] * dd.y + dsa * aa.y;
          G[4 * q + 2] = G[4 * q + 2] * dd.z + dsa * aa.z;
          G[4 * q + 3] = G[4 * q + 3] * dd.w + dsa * aa.w;
        }
      } else {
        const bool anchor = s == 0;
        const float rj = vr[idx], bj = vb[idx], kj = vk[idx], dj = vd[idx];
        const float inv_d = 1.0f / dj;
        float drj = 0.f, ddj = 0.f, dbj = 0.f, dkj = 0.f;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 dy4 = load4(vdy + po), sa4 = load4(vsa + po), v4 = load4(vv + po);
          const float dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
          const float sav[4] = {sa4.x, sa4.y, sa4.z, sa4.w};
          const float vvv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int e = 4 * q + x;
            drj += S[e] * dyv[x];
            G[e] += dyv[x] * rj;
            const float sp = anchor ? A[e] : (S[e] - sav[x] * bj - vvv[x] * kj) * inv_d;
            ddj += G[e] * sp;
            dbj += G[e] * sav[x];
            dkj += G[e] * vvv[x];
            S[e] = sp;
          }
        }
        drj = quad_sum(drj); ddj = quad_sum(ddj); dbj = quad_sum(dbj); dkj = quad_sum(dkj);
        if (p == 0) {
          dr[o] = from_float<T>(drj);
          dw[o] = from_float<T>(ddj * ewd[s * N + idx]);
          dk[o] = from_float<T>(dkj);
          db[o] = from_float<T>(dbj);
        }
      }
      __syncthreads();  // dsa of this step is visible; sdsa[sb] is rewritten two steps later
      if (is_col) {
        const float aj = va[idx], dj = vd[idx];
        const float* ds = sdsa + sb * N;
        float daj = 0.f;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const float4 d4 = load4(ds + pos_of(q, p, 0));
          daj += S[4 * q] * d4.x + S[4 * q + 1] * d4.y + S[4 * q + 2] * d4.z + S[4 * q + 3] * d4.w;
          G[4 * q] = G[4 * q] * dj + d4.x * aj;
          G[4 * q + 1] = G[4 * q + 1] * dj + d4.y * aj;
          G[4 * q + 2] = G[4 * q + 2] * dj + d4.z * aj;
          G[4 * q + 3] = G[4 * q + 3] * dj + d4.w * aj;
        }
        daj = quad_sum(daj);
        if (p == 0) da[o] = from_float<T>(daj);
      }
    }
  }
  if (!is_col) {
    float* dst = ds0 + ((size_t)bh * N + idx) * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
      *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) = make_float4(G[4 * q], G[4 * q + 1], G[4 * q + 2], G[4 * q + 3]);
  }
}

template <typename T, int N>
constexpr size_t bwd_smem_bytes() {
  return 2 * 7 * CH * N * sizeof(T) + (2 * CH * N + 7 * CH * N + CH * N + 2 * N) * sizeof(float);
}

template <typename T, int N>
static int launch_fwd_n(const WkvArgs& p, cudaStream_t st) {
  VecPtrs<T, 6> src;
  src.p[0] = (const T*)p.r; src.p[1] = (const T*)p.w; src.p[2] = (const T*)p.k;
  src.p[3] = (const T*)p.v; src.p[4] = (const T*)p.a; src.p[5] = (const T*)p.b;
  const size_t smem = fwd_smem_bytes<T, N>();
  dim3 grid(p.B * p.H);
  if (p.sa != nullptr) {
    auto kern = wkv7_fwd_kernel<T, N, true>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 4 * N, smem, st>>>(src, p.s0, (T*)p.y, p.sT, p.sa, p.ckpt, p.T, p.H);
  } else {
    auto kern = wkv7_fwd_kernel<T, N, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 4 * N, smem, st>>>(src, p.s0, (T*)p.y, p.sT, nullptr, nullptr, p.T, p.H);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <typename T, int N>
static int launch_bwd_n(const WkvArgs& p, cudaStream_t st) {
  VecPtrs<T, 7> src;
  src.p[0] = (const T*)p.r; src.p[1] = (const T*)p.w; src.p[2] = (const T*)p.k; src.p[3] = (const T*)p.v;
  src.p[4] = (const T*)p.a; src.p[5] = (const T*)p.b; src.p[6] = (const T*)p.dy;
  const size_t smem = bwd_smem_bytes<T, N>();
  auto kern = wkv7_bwd_kernel<T, N>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(p.B * p.H);
  kern<<<grid, 8 * N, smem, st>>>(src, p.sa, p.ckpt, p.s0, p.dsT, (T*)p.dr, (T*)p.dw, (T*)p.dk, (T*)p.dv, (T*)p.da,
                                 (T*)p.db, p.ds0, p.T, p.H);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <typename T>
static int dispatch(const WkvArgs& p, cudaStream_t st, bool backward) {
  switch (p.N) {
    case 64: return backward ? launch_bwd_n<T, 64>(p, st) : launch_fwd_n<T, 64>(p, st);
    case 32: return backward ? launch_bwd_n<T, 32>(p, st) : launch_fwd_n<T, 32>(p, st);
    case 16: return backward ? launch_bwd_n<T, 16>(p, st) : launch_fwd_n<T, 16>(p, st);
  }
  return 1;
}

int wkv7_forward(const WkvArgs& p, cudaStream_t st) {
  if (p.interval != CH) return 3;
  return p.is_bf16 ? dispatch<__nv_bfloat16>(p, st, false) : dispatch<float>(p, st, false);
}

int wkv7_backward(const WkvArgs& p, cudaStream_t st) {
  if (p.interval != CH) return 3;
  return p.is_bf16 ? dispatch<__nv_bfloat16>(p, st, true) : dispatch<float>(p, st, true);
}

}  // namespace rk
