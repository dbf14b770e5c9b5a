// WKV7 generalised delta-rule recurrence, time-sequential form.
//
//   d_t  = exp(-exp(w_t))
//   sa_t = S_{t-1} a_t
//   S_t  = S_{t-1} diag(d_t) + sa_t b_t^T + v_t k_t^T        (S is [value row i, key column j])
//   y_t  = S_t r_t
//
// One CTA per (batch, head).  The per-step vectors are streamed through shared
// memory in chunks of 16 time steps with cp.async, double-buffered, so global
// latency is paid once per chunk and never inside the recurrence.  Forward: each
// thread holds a 2 x 16 register tile of S (two rows, a quarter of the columns), so
// a mat-vec product is a short thread-local dot plus two shuffles, each broadcast
// value read from shared memory feeds two rows, and no block barrier is needed
// inside a chunk.  Backward: half of the threads own rows of the state cotangent,
// the other half own columns of both the state and its cotangent, exchanging one
// vector per step through shared memory.  The previous state is re-derived by undoing one
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

constexpr int RPT = 2;  // state rows (forward) / rows-or-columns (backward) held by one thread

// Forward: 2N threads.  Thread (g, p) holds rows 2g, 2g+1 of S restricted to the 16 columns of part p, so
// every broadcast vector value it loads from shared memory feeds two rows.
template <typename T, int N, bool SAVE>
__global__ void __launch_bounds__(4 * N / RPT) wkv7_fwd_kernel(VecPtrs<T, 6> src, const float* __restrict__ s0,
                                                               T* __restrict__ y, float* __restrict__ sT,
                                                               float* __restrict__ sa_out, float* __restrict__ ckpt,
                                                               int Tlen, int H) {
  constexpr int NQ = N / 16;
  constexpr int NT = 4 * N / RPT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tiles = reinterpret_cast<T*>(smem_raw);                                   // [2][6][CH][N]: r,w,k,v,a,b (raw)
  float* work = reinterpret_cast<float*>(smem_raw + 2 * 6 * CH * N * sizeof(T));  // [6][CH][N] fp32, slot 1 = decay
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const int i0 = (tid >> 2) * RPT, p = tid & 3;
  const int BH = gridDim.x;

  float S[RPT][4 * NQ];
#pragma unroll
  for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const float4 t4 = load4(s0 + ((size_t)bh * N + i0 + rr) * N + pos_of(q, p, 0));
      S[rr][4 * q] = t4.x; S[rr][4 * q + 1] = t4.y; S[rr][4 * q + 2] = t4.z; S[rr][4 * q + 3] = t4.w;
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
      float vi[RPT], sa[RPT], yy[RPT];
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) { vi[rr] = vv[i0 + rr]; sa[rr] = 0.f; yy[rr] = 0.f; }
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 aa = load4(va + pos_of(q, p, 0));
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr)
          sa[rr] += (S[rr][4 * q] * aa.x + S[rr][4 * q + 2] * aa.z) + (S[rr][4 * q + 1] * aa.y + S[rr][4 * q + 3] * aa.w);
      }
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) sa[rr] = quad_sum(sa[rr]);
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const int o = pos_of(q, p, 0);
        const float4 dd = load4(vd + o), bb = load4(vb + o), kk = load4(vk + o), rv = load4(vr + o);
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) {
          float* Sr = S[rr];
          Sr[4 * q] = Sr[4 * q] * dd.x + sa[rr] * bb.x + vi[rr] * kk.x;
          Sr[4 * q + 1] = Sr[4 * q + 1] * dd.y + sa[rr] * bb.y + vi[rr] * kk.y;
          Sr[4 * q + 2] = Sr[4 * q + 2] * dd.z + sa[rr] * bb.z + vi[rr] * kk.z;
          Sr[4 * q + 3] = Sr[4 * q + 3] * dd.w + sa[rr] * bb.w + vi[rr] * kk.w;
          yy[rr] += (Sr[4 * q] * rv.x + Sr[4 * q + 2] * rv.z) + (Sr[4 * q + 1] * rv.y + Sr[4 * q + 3] * rv.w);
        }
      }
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) yy[rr] = quad_sum(yy[rr]);
      if (p == 0) {
        const size_t o = base + (size_t)(c * CH + s) * stride_t + i0;
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) {
          y[o + rr] = from_float<T>(yy[rr]);
          if (SAVE) sa_out[o + rr] = sa[rr];
        }
      }
    }
    if (SAVE) {
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) {
        float* dst = ckpt + (((size_t)c * BH + bh) * N + i0 + rr) * N;
#pragma unroll
        for (int q = 0; q < NQ; ++q)
          *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) =
              make_float4(S[rr][4 * q], S[rr][4 * q + 1], S[rr][4 * q + 2], S[rr][4 * q + 3]);
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < RPT; ++rr) {
    float* dst = sT + ((size_t)bh * N + i0 + rr) * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
      *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) =
          make_float4(S[rr][4 * q], S[rr][4 * q + 1], S[rr][4 * q + 2], S[rr][4 * q + 3]);
  }
}

template <typename T, int N>
constexpr size_t fwd_smem_bytes() { return 2 * 6 * CH * N * sizeof(T) + 6 * CH * N * sizeof(float); }

// Backward.  Tile vectors: r,w,k,v,a,b,dy (type T) and sa (fp32).  4N threads: the first 2N own two rows
// each of the state cotangent G (16 columns per thread), the other 2N own two columns each of both the
// state S and G (16 rows per thread).
template <typename T, int N>
__global__ void __launch_bounds__(8 * N / RPT, (N == 64 ? 2 : 1)) wkv7_bwd_kernel(
    VecPtrs<T, 7> src, const float* __restrict__ sa, const float* __restrict__ ckpt, const float* __restrict__ s0,
    const float* __restrict__ dsT, T* __restrict__ dr, T* __restrict__ dw, T* __restrict__ dk, T* __restrict__ dv,
    T* __restrict__ da, T* __restrict__ db, float* __restrict__ ds0, int Tlen, int H) {
  constexpr int NQ = N / 16;
  constexpr int NE = 4 * NQ;
  constexpr int HALF = 4 * N / RPT;
  constexpr int NT = 2 * HALF;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tiles = reinterpret_cast<T*>(smem_raw);                                         // [2][7][CH][N]
  float* sa_tiles = reinterpret_cast<float*>(smem_raw + 2 * 7 * CH * N * sizeof(T));  // [2][CH][N]
  float* work = sa_tiles + 2 * CH * N;                                                // [7][CH][N] fp32, slot 1 = decay
  float* ewd = work + 7 * CH * N;                                                     // [CH][N]  -exp(w) * d
  float* sdsa = ewd + CH * N;                                                         // [2][N]
  float* anc = sdsa + 2 * N;                                                          // [2][N][N] exact chunk-start state
  const int bh = blockIdx.x;
  const int bidx = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const bool is_col = tid >= HALF;
  const int idx0 = ((is_col ? tid - HALF : tid) >> 2) * RPT;  // first row i (row threads) or column j (column threads)
  const int p = tid & 3;
  const int BH = gridDim.x;

  float G[RPT][NE];
  float S[RPT][NE];
#pragma unroll
  for (int u = 0; u < RPT; ++u)
#pragma unroll
    for (int e = 0; e < NE; ++e) { G[u][e] = 0.f; S[u][e] = 0.f; }
  if (dsT != nullptr) {
#pragma unroll
    for (int u = 0; u < RPT; ++u)
#pragma unroll
      for (int q = 0; q < NQ; ++q)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int o = pos_of(q, p, x);
          G[u][4 * q + x] = is_col ? dsT[((size_t)bh * N + o) * N + idx0 + u] : dsT[((size_t)bh * N + idx0 + u) * N + o];
        }
  }
  const int nch = (Tlen + CH - 1) / CH;
  if (is_col) {
    const float* srcS = ckpt + ((size_t)(nch - 1) * BH + bh) * N * N;
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float2 t2 = *reinterpret_cast<const float2*>(srcS + pos_of(q, p, x) * N + idx0);
        S[0][4 * q + x] = t2.x; S[1][4 * q + x] = t2.y;
      }
  }

  const size_t stride_t = (size_t)H * N;
  const size_t base = ((size_t)bidx * Tlen * H + h) * N;
  VecPtrs<float, 1> sa_src;
  sa_src.p[0] = sa;
  auto stage = [&](int c, int buf) {
    stage_chunk<T, N, 7>(tiles + (size_t)buf * 7 * CH * N, src, base, stride_t, c, Tlen, tid, NT);
    stage_chunk<float, N, 1>(sa_tiles + (size_t)buf * CH * N, sa_src, base, stride_t, c, Tlen, tid, NT);
    // exact state before the first step of chunk c (initial state for chunk 0)
    const float* prev = (c == 0) ? (s0 + (size_t)bh * N * N) : (ckpt + ((size_t)(c - 1) * BH + bh) * N * N);
    float* dst = anc + (size_t)buf * N * N;
    for (int pc = tid; pc < N * N / 4; pc += NT) cp_async16(dst + pc * 4, prev + pc * 4);
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
    const float* anchor_tile = anc + (size_t)buf * N * N;
    __syncthreads();
    const int steps = min(CH, Tlen - c * CH);
    for (int s = steps - 1; s >= 0; --s) {
      const int t = c * CH + s;
      const int sb = t & 1;
      const size_t o = base + (size_t)t * stride_t + idx0;
      const float* vr = work + (0 * CH + s) * N;
      const float* vd = work + (1 * CH + s) * N;
      const float* vk = work + (2 * CH + s) * N;
      const float* vv = work + (3 * CH + s) * N;
      const float* va = work + (4 * CH + s) * N;
      const float* vb = work + (5 * CH + s) * N;
      const float* vdy = work + (6 * CH + s) * N;
      const float* vsa = sat + s * N;
      if (!is_col) {
        float dyi[RPT], dsa[RPT], dvi[RPT];
#pragma unroll
        for (int u = 0; u < RPT; ++u) { dyi[u] = vdy[idx0 + u]; dsa[u] = 0.f; dvi[u] = 0.f; }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 rr = load4(vr + po), bb = load4(vb + po), kk = load4(vk + po);
#pragma unroll
          for (int u = 0; u < RPT; ++u) {
            float* g = G[u] + 4 * q;
            g[0] += dyi[u] * rr.x; g[1] += dyi[u] * rr.y; g[2] += dyi[u] * rr.z; g[3] += dyi[u] * rr.w;
            dsa[u] += (g[0] * bb.x + g[2] * bb.z) + (g[1] * bb.y + g[3] * bb.w);
            dvi[u] += (g[0] * kk.x + g[2] * kk.z) + (g[1] * kk.y + g[3] * kk.w);
          }
        }
#pragma unroll
        for (int u = 0; u < RPT; ++u) { dsa[u] = quad_sum(dsa[u]); dvi[u] = quad_sum(dvi[u]); }
        if (p == 0) {
#pragma unroll
          for (int u = 0; u < RPT; ++u) { sdsa[sb * N + idx0 + u] = dsa[u]; dv[o + u] = from_float<T>(dvi[u]); }
        }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 dd = load4(vd + po), aa = load4(va + po);
#pragma unroll
          for (int u = 0; u < RPT; ++u) {
            float* g = G[u] + 4 * q;
            g[0] = g[0] * dd.x + dsa[u] * aa.x;
            g[1] = g[1] * dd.y + dsa[u] * aa.y;
            g[2] = g[2] * dd.z + dsa[u] * aa.z;
            g[3] = g[3] * dd.w + dsa[u] * aa.w;
          }
        }
      } else {
        const bool anchor = s == 0;
        float rj[RPT], bj[RPT], kj[RPT], inv_d[RPT], drj[RPT], ddj[RPT], dbj[RPT], dkj[RPT];
#pragma unroll
        for (int u = 0; u < RPT; ++u) {
          rj[u] = vr[idx0 + u]; bj[u] = vb[idx0 + u]; kj[u] = vk[idx0 + u]; inv_d[u] = 1.0f / vd[idx0 + u];
          drj[u] = 0.f; ddj[u] = 0.f; dbj[u] = 0.f; dkj[u] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const int po = pos_of(q, p, 0);
          const float4 dy4 = load4(vdy + po), sa4 = load4(vsa + po), v4 = load4(vv + po);
          const float dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
          const float sav[4] = {sa4.x, sa4.y, sa4.z, sa4.w};
          const float vvv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
          for (int u = 0; u < RPT; ++u)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const int e = 4 * q + x;
              drj[u] += S[u][e] * dyv[x];
              G[u][e] += dyv[x] * rj[u];
              const float sp = anchor ? anchor_tile[pos_of(q, p, x) * N + idx0 + u]
                                      : (S[u][e] - sav[x] * bj[u] - vvv[x] * kj[u]) * inv_d[u];
              ddj[u] += G[u][e] * sp;
              dbj[u] += G[u][e] * sav[x];
              dkj[u] += G[u][e] * vvv[x];
              S[u][e] = sp;
            }
        }
#pragma unroll
        for (int u = 0; u < RPT; ++u) {
          drj[u] = quad_sum(drj[u]); ddj[u] = quad_sum(ddj[u]); dbj[u] = quad_sum(dbj[u]); dkj[u] = quad_sum(dkj[u]);
        }
        if (p == 0) {
#pragma unroll
          for (int u = 0; u < RPT; ++u) {
            dr[o + u] = from_float<T>(drj[u]);
            dw[o + u] = from_float<T>(ddj[u] * ewd[s * N + idx0 + u]);
            dk[o + u] = from_float<T>(dkj[u]);
            db[o + u] = from_float<T>(dbj[u]);
          }
        }
      }
      __syncthreads();  // dsa of this step is visible; sdsa[sb] is rewritten two steps later
      if (is_col) {
        const float* ds = sdsa + sb * N;
        float aj[RPT], dj[RPT], daj[RPT];
#pragma unroll
        for (int u = 0; u < RPT; ++u) { aj[u] = va[idx0 + u]; dj[u] = vd[idx0 + u]; daj[u] = 0.f; }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const float4 d4 = load4(ds + pos_of(q, p, 0));
#pragma unroll
          for (int u = 0; u < RPT; ++u) {
            float* g = G[u] + 4 * q;
            const float* sv = S[u] + 4 * q;
            daj[u] += (sv[0] * d4.x + sv[2] * d4.z) + (sv[1] * d4.y + sv[3] * d4.w);
            g[0] = g[0] * dj[u] + d4.x * aj[u];
            g[1] = g[1] * dj[u] + d4.y * aj[u];
            g[2] = g[2] * dj[u] + d4.z * aj[u];
            g[3] = g[3] * dj[u] + d4.w * aj[u];
          }
        }
#pragma unroll
        for (int u = 0; u < RPT; ++u) daj[u] = quad_sum(daj[u]);
        if (p == 0) {
#pragma unroll
          for (int u = 0; u < RPT; ++u) da[o + u] = from_float<T>(daj[u]);
        }
      }
    }
  }
  if (!is_col) {
#pragma unroll
    for (int u = 0; u < RPT; ++u) {
      float* dst = ds0 + ((size_t)bh * N + idx0 + u) * N;
#pragma unroll
      for (int q = 0; q < NQ; ++q)
        *reinterpret_cast<float4*>(dst + pos_of(q, p, 0)) =
            make_float4(G[u][4 * q], G[u][4 * q + 1], G[u][4 * q + 2], G[u][4 * q + 3]);
    }
  }
}

template <typename T, int N>
constexpr size_t bwd_smem_bytes() {
  return 2 * 7 * CH * N * sizeof(T) + (2 * CH * N + 7 * CH * N + CH * N + 2 * N + 2 * N * N) * sizeof(float);
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
    kern<<<grid, 4 * N / RPT, smem, st>>>(src, p.s0, (T*)p.y, p.sT, (float*)p.sa, p.ckpt, p.T, p.H);
  } else {
    auto kern = wkv7_fwd_kernel<T, N, false>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 4 * N / RPT, smem, st>>>(src, p.s0, (T*)p.y, p.sT, nullptr, nullptr, p.T, p.H);
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
  kern<<<grid, 8 * N / RPT, smem, st>>>(src, (const float*)p.sa, p.ckpt, p.s0, p.dsT, (T*)p.dr, (T*)p.dw, (T*)p.dk, (T*)p.dv, (T*)p.da,
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
