// State-level screening memory: the slot-dependent part of the layer, sequential over time, as one kernel per
// direction.  One CTA (256 threads) owns one batch row and walks the T steps; the slot bank S [M, ds] lives in
// shared memory (transposed, [ds][16]).
//
// Per step t (names follow src/rwkv7m/model/nnx_model.py:1024-1159 and src/rwkv7m/model/screening.py:11-88):
//   k_r[m] = unit(S[m] Wk^T)   val[m] = unit(S[m] Wv^T)   k_w[m] = unit((S[m] + E[m]) Wkw^T)
//   rel_r[m] = trim_square(q_r[t] . k_r[m], tau_r) (* age mask)      rel_w[m] = trim_square(q_w[t] . k_w[m], tau_w)
//   u[t]    = tanh_norm(sum_m rel_r[m] val[m])                       (output; the out-projection is a GEMM outside)
//   S[m]   += mu[m] * max(rel_w[m], floor) * (tanh(dxh[t] + dslot[m]) - S[m])     (rate mu[m] alone without write screening)
// The raw projections P[m] = S[m] W^T (+ E[m] Wkw^T for the write keys; W^T [ds][J], J = dk + dv + dk) are never
// recomputed inside the loop.  The slot update is an interpolation towards a vector that does not depend on the state,
//   S_{t+1}[m] = S_t[m] + s_m (D_t[m] - S_t[m]),   D_t[m] = tanh(dxh[t] + dslot[m]),
// and the projections are linear, so they obey the same recurrence:
//   P_{t+1}[m] = P_t[m] + s_m (PD_t[m] - P_t[m]),  PD_t[m] = D_t[m] W^T (+ E[m] Wkw^T),
// where PD for all steps is one GEMM done by the caller before the scan.  A step therefore costs O(M (ds + J)) instead
// of O(M ds J).  The backward kernel walks the steps in reverse from the saved per-step S and P, carries the cotangents
// of both, and returns the gradients of q_r, q_w, dxh, dslot (direct part), PD, the initial S and P, and the scalars;
// the caller turns d PD into weight / dxh / dslot gradients with GEMMs over all steps at once.
#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

constexpr int kMp = 16;      // slots are padded to 16
constexpr int kJp = 256;     // row stride of the raw projections
constexpr int kThreads = 256;
constexpr int kSc = 12;     // per-slot scalars: nk, nv, nw, simr, simw, relr, relw, strength, relr / nv

__device__ __forceinline__ float trim_sq(float sim, float tau, float eps, float& x_out) {
  const float x = fmaxf((sim - tau) / (1.f - tau + eps), 0.f);
  x_out = x;
  return x * x;
}

struct ScanSmem {
  float* St;     // [ds][16]   slots, transposed
  float* DSt;    // [ds][16]   delta_slot, transposed
  float* P;      // [16][256]  raw projections of the current step
  float* PD;     // [16][256]  projections of the step's write target
  float* EW;     // [16][dk]   slot_embed Wkw^T
  float* qr;     // [dk]
  float* qw;     // [dk]
  float* dxh;    // [ds]
  float* z;      // [dv]
  float* sc;     // [16][kSc]  per-slot scalars
  float* ages;   // [16]
  float* usage;  // [16]
  float* upd;    // [16]       squared update norm of the step
};

__device__ __forceinline__ ScanSmem carve(float* base, int ds, int dk, int dv) {
  ScanSmem s;
  s.St = base; base += ds * kMp;
  s.DSt = base; base += ds * kMp;
  s.P = base; base += kMp * kJp;
  s.PD = base; base += kMp * kJp;
  s.EW = base; base += kMp * dk;
  s.qr = base; base += dk;
  s.qw = base; base += dk;
  s.dxh = base; base += ds;
  s.z = base; base += dv;
  s.sc = base; base += kMp * kSc;
  s.ages = base; base += kMp;
  s.usage = base; base += kMp;
  s.upd = base; base += kMp;
  return s;
}

__host__ __device__ inline int scan_smem_floats(int ds, int dk, int dv) {
  return 2 * ds * kMp + 2 * kMp * kJp + kMp * dk + 2 * dk + ds + dv + kMp * kSc + 3 * kMp + 8 * kMp /*per-warp update norms*/;
}

// raw projections of all slots: P[m][j] = sum_d St[d][m] * WT[d][j]  (+ EW for the write keys)
template <bool SMEM_W>
__device__ __forceinline__ void project(const ScanSmem& s, const float* __restrict__ WT, int wstride, int ds, int J, int dk,
                                        int dv, int tid, bool add_ew) {
  if (tid < J) {
    float acc[kMp];
#pragma unroll
    for (int m = 0; m < kMp; ++m) acc[m] = 0.f;
#pragma unroll 4
    for (int d = 0; d < ds; ++d) {
      const float w = SMEM_W ? WT[d * wstride + tid] : __ldg(WT + (size_t)d * wstride + tid);
      const float4* sp = reinterpret_cast<const float4*>(s.St + d * kMp);
      const float4 a = sp[0], b = sp[1], c = sp[2], e = sp[3];
      acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]); acc[2] = fmaf(w, a.z, acc[2]); acc[3] = fmaf(w, a.w, acc[3]);
      acc[4] = fmaf(w, b.x, acc[4]); acc[5] = fmaf(w, b.y, acc[5]); acc[6] = fmaf(w, b.z, acc[6]); acc[7] = fmaf(w, b.w, acc[7]);
      acc[8] = fmaf(w, c.x, acc[8]); acc[9] = fmaf(w, c.y, acc[9]); acc[10] = fmaf(w, c.z, acc[10]); acc[11] = fmaf(w, c.w, acc[11]);
      acc[12] = fmaf(w, e.x, acc[12]); acc[13] = fmaf(w, e.y, acc[13]); acc[14] = fmaf(w, e.z, acc[14]); acc[15] = fmaf(w, e.w, acc[15]);
    }
    const bool is_kw = tid >= dk + dv;
#pragma unroll
    for (int m = 0; m < kMp; ++m) s.P[m * kJp + tid] = acc[m] + ((add_ew && is_kw) ? s.EW[m * dk + tid - dk - dv] : 0.f);
  }
}

// per-slot norms, similarities, relevances and the write strength; half-warp h (16 lanes) handles slot h
__device__ __forceinline__ float half_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void slot_scalars(const ScanSmem& s, const ScreenScanArgs& a, int warp, int lane) {
  const int m = warp * 2 + (lane >> 4), hl = lane & 15;
  const float* Pm = s.P + m * kJp;
  float sk = 0.f, dkq = 0.f, sv = 0.f, sw = 0.f, dwq = 0.f;
  for (int j = hl; j < a.dk; j += 16) { const float x = Pm[j]; sk = fmaf(x, x, sk); dkq = fmaf(x, s.qr[j], dkq); }
  for (int j = hl; j < a.dv; j += 16) { const float x = Pm[a.dk + j]; sv = fmaf(x, x, sv); }
  if (a.write_enabled)
    for (int j = hl; j < a.dk; j += 16) { const float x = Pm[a.dk + a.dv + j]; sw = fmaf(x, x, sw); dwq = fmaf(x, s.qw[j], dwq); }
  sk = half_sum(sk); dkq = half_sum(dkq); sv = half_sum(sv); sw = half_sum(sw); dwq = half_sum(dwq);
  if (hl == 0) {
    float* c = s.sc + m * kSc;
    const float e2 = a.eps * a.eps;
    const float nk = sqrtf(sk + e2), nv = a.value_unit_norm ? sqrtf(sv + e2) : 1.f, nw = sqrtf(sw + e2);
    const float simr = dkq / nk, simw = dwq / nw;
    float xr, xw;
    float relr = trim_sq(simr, a.tau_r, a.eps, xr);
    if (a.age_mask) relr *= 1.f / (1.f + __expf(-(a.age_ref - s.ages[m]) / (a.age_sigma + a.eps)));
    const bool live = m < a.M;
    if (!live) relr = 0.f;
    float relw = 0.f, strength = live ? a.mu[m] : 0.f;
    if (a.write_enabled && live) {
      relw = trim_sq(simw, a.tau_w, a.eps, xw);
      strength *= fmaxf(relw, a.write_rel_floor);
    }
    c[0] = nk; c[1] = nv; c[2] = nw; c[3] = simr; c[4] = simw; c[5] = relr; c[6] = relw; c[7] = strength;
    c[8] = relr / nv;
  }
}

template <bool SMEM_W>
__global__ void __launch_bounds__(kThreads) screen_scan_fwd_kernel(ScreenScanArgs a) {
  extern __shared__ float smem_f[];
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const ScanSmem s = carve(smem_f, a.ds, a.dk, a.dv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  const int J = 2 * a.dk + a.dv;
  const int nel = a.ds * kMp;
  // the projection weights are only needed for the initial bank: they stream through L1 / L2 once
  const float* WTp = a.WT;
  const int wstride = J;

  // ---- load the bank, delta_slot and the slot embedding (all transposed to [d][16]) ----------------------------------
  for (int e = tid; e < nel; e += kThreads) {
    const int d = e / kMp, m = e % kMp;
    const bool live = m < a.M;
    s.St[e] = live ? a.slot_embed[m * a.ds + d] : 0.f;
    s.DSt[e] = live ? a.delta_slot[m * a.ds + d] : 0.f;
  }
  if (tid < kMp) {
    s.ages[tid] = tid < a.M ? a.ages0[b * a.M + tid] : 0.f;
    s.usage[tid] = tid < a.M ? a.usage0[b * a.M + tid] : 0.f;
  }
  float* updw = s.upd + kMp;   // [8 warps][16] partial squared update norms of the current step
  __syncthreads();
  project<SMEM_W>(s, WTp, wstride, a.ds, J, a.dk, a.dv, tid, false);   // E Wkw^T (only the write-key columns are kept)
  __syncthreads();
  for (int e = tid; e < kMp * a.dk; e += kThreads) s.EW[e] = s.P[(e / a.dk) * kJp + a.dk + a.dv + e % a.dk];
  __syncthreads();
  for (int e = tid; e < nel; e += kThreads) {
    const int d = e / kMp, m = e % kMp;
    s.St[e] = m < a.M ? a.slots0[((size_t)b * a.M + m) * a.ds + d] : 0.f;
  }
  float st_acc[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) st_acc[i] = 0.f;
  __syncthreads();

  // projections of the initial bank (the only pass over the weights); afterwards they follow the slot recurrence
  project<SMEM_W>(s, WTp, wstride, a.ds, J, a.dk, a.dv, tid, true);

  // the step's vectors are fetched one step ahead into registers (thread tid: q_r / q_w element tid, delta_xh element tid,
  // column tid of the write target's projections for all 16 slots)
  float n_qr = 0.f, n_qw = 0.f, n_dx = 0.f;
  float n_pd[kMp];
#pragma unroll
  for (int m = 0; m < kMp; ++m) n_pd[m] = 0.f;
  auto fetch = [&](int t) {
    const size_t bt = (size_t)b * a.T + t;
    if (tid < a.dk) { n_qr = a.q_r[bt * a.dk + tid]; n_qw = a.write_enabled ? a.q_w[bt * a.dk + tid] : 0.f; }
    if (tid < a.ds) n_dx = a.delta_xh[bt * a.ds + tid];
    if (tid < J) {
      const float* src = a.PD + bt * kMp * J + tid;
#pragma unroll
      for (int m = 0; m < kMp; ++m) n_pd[m] = src[m * J];
    }
  };
  fetch(0);
  for (int t = 0; t < a.T; ++t) {
    const size_t bt = (size_t)b * a.T + t;
    // ---- stage the step's vectors; save the bank and its projections for the backward pass -------------------------------
    if (tid < a.dk) { s.qr[tid] = n_qr; s.qw[tid] = n_qw; }
    if (tid < a.ds) s.dxh[tid] = n_dx;
    float pd[kMp];
#pragma unroll
    for (int m = 0; m < kMp; ++m) pd[m] = n_pd[m];
    if (t + 1 < a.T) fetch(t + 1);
    __syncthreads();   // s.P and s.St of this step are complete (written at the end of the previous iteration)
    if (a.saved_slots != nullptr) {
      float* dst = a.saved_slots + bt * nel;
      for (int e = tid; e < nel; e += kThreads) dst[e] = s.St[e];
      if (tid < kMp) a.saved_ages[bt * kMp + tid] = s.ages[tid];
      if (tid < J) {
        float* dp = a.saved_P + bt * kMp * J + tid;
#pragma unroll
        for (int m = 0; m < kMp; ++m) dp[m * J] = s.P[m * kJp + tid];
      }
    }
    slot_scalars(s, a, warp, lane);
    __syncthreads();
    // ---- read-out ----------------------------------------------------------------------------------------------------------
    if (tid < a.dv) {
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) acc = fmaf(s.sc[m * kSc + 8], s.P[m * kJp + a.dk + tid], acc);
      s.z[tid] = acc;
    }
    __syncthreads();
    float zn2 = 0.f;
    for (int v = lane; v < a.dv; v += 32) zn2 = fmaf(s.z[v], s.z[v], zn2);
    zn2 = warp_sum(zn2);
    const float zn = sqrtf(zn2 + a.eps * a.eps);
    const float f = a.cap * tanhf(zn / a.cap) / zn;
    if (tid < a.dv) a.u_out[bt * a.dv + tid] = f * s.z[tid];
    // ---- slot update ---------------------------------------------------------------------------------------------------------
    {
      const int m = tid % kMp;   // every element this thread touches belongs to the same slot (= lane & 15)
      const float strength = s.sc[m * kSc + 7];
      float un = 0.f;
      for (int e = tid; e < nel; e += kThreads) {
        const int d = e / kMp;
        const float old = s.St[e];
        const float delta = tanhf(s.dxh[d] + s.DSt[e]);
        const float nw = old + strength * (delta - old);
        s.St[e] = nw;
        un = fmaf(nw - old, nw - old, un);
      }
      un += __shfl_xor_sync(0xffffffffu, un, 16);
      if (lane < kMp) updw[warp * kMp + m] = un;   // per-warp partial of the squared update norm (no atomics)
    }
    if (tid < J) {   // the projections follow the same interpolation
#pragma unroll
      for (int mm = 0; mm < kMp; ++mm) {
        const float old = s.P[mm * kJp + tid];
        s.P[mm * kJp + tid] = fmaf(s.sc[mm * kSc + 7], pd[mm] - old, old);
      }
    }
    __syncthreads();
    // ---- ages, usage and the logged statistics: lane m of warp 0 keeps slot m's running sums in registers -------------------
    if (warp == 0) {
      const int m = lane & 15;
      const bool live = lane < kMp && m < a.M;
      const float relr = live ? s.sc[m * kSc + 5] : 0.f, relw = live ? s.sc[m * kSc + 6] : 0.f;
      float rx = relr;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) rx = fmaxf(rx, __shfl_xor_sync(0xffffffffu, rx, o));
      if (live) {
        if (a.write_enabled) s.ages[m] = relw > 1e-3f ? 0.f : s.ages[m] + 1.f;
        const float act = a.write_enabled ? fmaxf(relr, relw) : relr;
        const float us = a.usage_decay * s.usage[m] + (1.f - a.usage_decay) * act;
        s.usage[m] = us;
        float un = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) un += updw[w * kMp + m];
        st_acc[0] += relr; st_acc[2] += relr > 1e-3f ? 1.f : 0.f;
        st_acc[5] += relw; st_acc[6] += a.write_enabled ? fmaxf(relw, a.write_rel_floor) : relw;
        st_acc[7] += sqrtf(un); st_acc[8] += us;
      }
      if (lane == 0) { st_acc[1] += rx; st_acc[3] += zn; st_acc[4] += f * zn; }
    }
  }
  for (int e = tid; e < nel; e += kThreads) {
    const int d = e / kMp, m = e % kMp;
    if (m < a.M) a.slots_out[((size_t)b * a.M + m) * a.ds + d] = s.St[e];
  }
  if (tid < a.M) { a.ages_out[b * a.M + tid] = s.ages[tid]; a.usage_out[b * a.M + tid] = s.usage[tid]; }
  if (warp == 0) {   // per-slot sums -> means over slots (sums over steps and batch rows stay sums; the host divides)
    const float im = 1.f / a.M;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      float v = lane < kMp ? st_acc[i] : 0.f;
      v = half_sum(v);
      const bool per_slot_mean = i == 0 || i == 5 || i == 6 || i == 7 || i == 8;
      if (lane == 0) atomicAdd(a.stats + i, per_slot_mean ? v * im : v);
    }
  }
}

}  // namespace

namespace {

__host__ __device__ inline int scan_bwd_smem_floats(int ds, int dk, int dv) {
  return scan_smem_floats(ds, dk, dv) + ds * kMp /*dSt*/ + kJp * kMp /*dPc*/ + 2 * dv /*du, dz*/ + kMp * 4 /*dstr, dsimr, dsimw, pad*/;
}

template <bool SMEM_W>
__global__ void __launch_bounds__(kThreads) screen_scan_bwd_kernel(ScreenScanArgs a) {
  extern __shared__ float smem_f[];
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const ScanSmem s = carve(smem_f, a.ds, a.dk, a.dv);
  float* extra = smem_f + scan_smem_floats(a.ds, a.dk, a.dv);
  float* dSt = extra; extra += a.ds * kMp;      // [ds][16] cotangent of the bank after the current step
  float* dPc = extra; extra += kJp * kMp;       // [16][256] cotangent of the carried raw projections
  float* du = extra; extra += a.dv;
  float* dz = extra; extra += a.dv;
  float* dstr = extra; extra += kMp;            // cotangent of the write strength
  float* dsimr = extra; extra += kMp;
  float* dsimw = extra; extra += kMp;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  const int J = 2 * a.dk + a.dv;
  const int nel = a.ds * kMp;
  const float e2 = a.eps * a.eps;

  for (int e = tid; e < nel; e += kThreads) {
    const int d = e / kMp, m = e % kMp;
    const bool live = m < a.M;
    s.DSt[e] = live ? a.delta_slot[m * a.ds + d] : 0.f;
    dSt[e] = (live && a.dslots_out != nullptr) ? a.dslots_out[((size_t)b * a.M + m) * a.ds + d] : 0.f;
  }
  for (int e = tid; e < kMp * kJp; e += kThreads) dPc[e] = 0.f;   // the projections after the last step feed nothing
  float dslot_acc[16];          // this thread's elements of d(delta_slot): e = tid + 256 i
#pragma unroll
  for (int i = 0; i < 16; ++i) dslot_acc[i] = 0.f;
  float dmu_acc = 0.f, dtaur_acc = 0.f, dtauw_acc = 0.f;   // lane 0 of warp w: slots 2w, 2w+1 (dmu kept per slot below)
  float dmu_acc2 = 0.f;
  __syncthreads();

  // everything a step reads from global memory is fetched one step ahead into registers: the step vectors, the saved
  // bank (elements tid + 256 i), and column tid of the saved projections and of the write target's projections
  float n_qr = 0.f, n_qw = 0.f, n_dx = 0.f, n_du = 0.f, n_age = 0.f;
  float n_S[16], n_P[kMp], n_PD[kMp];
#pragma unroll
  for (int i = 0; i < 16; ++i) n_S[i] = 0.f;
#pragma unroll
  for (int m = 0; m < kMp; ++m) { n_P[m] = 0.f; n_PD[m] = 0.f; }
  auto fetch = [&](int t) {
    const size_t bt = (size_t)b * a.T + t;
    if (tid < a.dk) { n_qr = a.q_r[bt * a.dk + tid]; n_qw = a.write_enabled ? a.q_w[bt * a.dk + tid] : 0.f; }
    if (tid < a.ds) n_dx = a.delta_xh[bt * a.ds + tid];
    if (tid < a.dv) n_du = a.du[bt * a.dv + tid];
    if (tid < kMp) n_age = a.saved_ages[bt * kMp + tid];
    const float* src = a.saved_slots + bt * nel;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = tid + i * kThreads;
      if (e < nel) n_S[i] = src[e];
    }
    if (tid < J) {
      const float* sp = a.saved_P + bt * kMp * J + tid;
      const float* pp = a.PD + bt * kMp * J + tid;
#pragma unroll
      for (int m = 0; m < kMp; ++m) { n_P[m] = sp[m * J]; n_PD[m] = pp[m * J]; }
    }
  };
  fetch(a.T - 1);
  for (int t = a.T - 1; t >= 0; --t) {
    const size_t bt = (size_t)b * a.T + t;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = tid + i * kThreads;
      if (e < nel) s.St[e] = n_S[i];
    }
    if (tid < J) {
#pragma unroll
      for (int m = 0; m < kMp; ++m) { s.P[m * kJp + tid] = n_P[m]; s.PD[m * kJp + tid] = n_PD[m]; }
    }
    if (tid < kMp) { s.ages[tid] = n_age; dstr[tid] = 0.f; }
    if (tid < a.dk) { s.qr[tid] = n_qr; s.qw[tid] = n_qw; }
    if (tid < a.ds) s.dxh[tid] = n_dx;
    if (tid < a.dv) du[tid] = n_du;
    if (t > 0) fetch(t - 1);
    __syncthreads();
    slot_scalars(s, a, warp, lane);
    __syncthreads();
    if (tid < a.dv) {
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) acc = fmaf(s.sc[m * kSc + 8], s.P[m * kJp + a.dk + tid], acc);
      s.z[tid] = acc;
    }
    // ---- backward of the slot update (uses the cotangent carried from step t+1) -----------------------------------------
    {
      const int m = tid % kMp;
      const float strength = s.sc[m * kSc + 7];
      float dsp = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {   // constant trip count keeps dslot_acc in registers; nel is a multiple of 256
        const int e = tid + i * kThreads;
        if (e >= nel) break;
        const int d = e / kMp;
        const float old = s.St[e];
        const float delta = tanhf(s.dxh[d] + s.DSt[e]);
        const float g = dSt[e];
        dsp = fmaf(g, delta - old, dsp);
        const float dpre = strength * g * (1.f - delta * delta);
        dSt[e] = (1.f - strength) * g;
        dslot_acc[i] += dpre;
        // sum of dpre over the 16 slots of this d: the 16 lanes of a half-warp share d
        float r = dpre;
        r += __shfl_xor_sync(0xffffffffu, r, 1); r += __shfl_xor_sync(0xffffffffu, r, 2);
        r += __shfl_xor_sync(0xffffffffu, r, 4); r += __shfl_xor_sync(0xffffffffu, r, 8);
        if (m == 0) a.d_delta_xh[bt * a.ds + d] = r;
      }
      atomicAdd(&dstr[m], dsp);
    }
    // ---- backward of the projection update P' = P + s (PD - P): warp w owns slots 2w and 2w+1 -------------------------------
    for (int mm = 0; mm < 2; ++mm) {
      const int m = warp * 2 + mm;
      const float strength = s.sc[m * kSc + 7];
      float* gp = dPc + m * kJp;
      float* out = a.d_PD + (bt * kMp + m) * J;
      float dsp = 0.f;
      for (int j = lane; j < J; j += 32) {
        const float g = gp[j];
        dsp = fmaf(g, s.PD[m * kJp + j] - s.P[m * kJp + j], dsp);
        out[j] = strength * g;
        gp[j] = (1.f - strength) * g;
      }
      dsp = warp_sum(dsp);
      if (lane == 0) atomicAdd(&dstr[m], dsp);
    }
    __syncthreads();
    // ---- cotangent of z from the cotangent of u = f(n) z ---------------------------------------------------------------------
    float zn2 = 0.f, zdu = 0.f;
    for (int v = lane; v < a.dv; v += 32) { zn2 = fmaf(s.z[v], s.z[v], zn2); zdu = fmaf(s.z[v], du[v], zdu); }
    zn2 = warp_sum(zn2); zdu = warp_sum(zdu);
    const float n2 = zn2 + e2, zn = sqrtf(n2);
    const float th = tanhf(zn / a.cap);
    const float f = a.cap * th / zn;
    const float coef = zdu * ((1.f - th * th) - f) / n2;
    if (tid < a.dv) dz[tid] = f * du[tid] + coef * s.z[tid];
    __syncthreads();
    // ---- per-slot scalars backward; cotangent of the raw projections (transposed into dPt[j][m]) ------------------------------
    for (int mm = 0; mm < 2; ++mm) {
      const int m = warp * 2 + mm;
      const float* c = s.sc + m * kSc;
      const float nk = c[0], nv = c[1], nw = c[2], simr = c[3], simw = c[4], relr = c[5], relw = c[6];
      const float* Pm = s.P + m * kJp;
      const bool live = m < a.M;
      float drelr = 0.f;
      for (int v = lane; v < a.dv; v += 32) drelr = fmaf(dz[v], Pm[a.dk + v] / nv, drelr);
      drelr = warp_sum(drelr);
      float mask = 1.f;
      if (a.age_mask) mask = 1.f / (1.f + __expf(-(a.age_ref - s.ages[m]) / (a.age_sigma + a.eps)));
      const float den_r = 1.f - a.tau_r + a.eps;
      const float xr = fmaxf((simr - a.tau_r) / den_r, 0.f);
      const float dtrim = live ? drelr * mask : 0.f;
      const float dsr = dtrim * 2.f * xr / den_r;
      float dsw = 0.f, gate_w = 1.f;
      const float ds_m = dstr[m];
      if (a.write_enabled && live) {
        gate_w = fmaxf(relw, a.write_rel_floor);
        const float drelw = relw > a.write_rel_floor ? ds_m * a.mu[m] : 0.f;
        const float den_w = 1.f - a.tau_w + a.eps;
        const float xw = fmaxf((simw - a.tau_w) / den_w, 0.f);
        dsw = drelw * 2.f * xw / den_w;
        if (lane == 0) dtauw_acc += drelw * 2.f * xw * (simw - 1.f - a.eps) / (den_w * den_w);
      }
      if (lane == 0 && live) {
        dtaur_acc += dtrim * 2.f * xr * (simr - 1.f - a.eps) / (den_r * den_r);
        if (mm == 0) dmu_acc += ds_m * gate_w; else dmu_acc2 += ds_m * gate_w;
        dsimr[m] = dsr; dsimw[m] = dsw;
      } else if (lane == 0) {
        dsimr[m] = 0.f; dsimw[m] = 0.f;
      }
      float* gp = dPc + m * kJp;   // same warp and lanes as the scaling above: no barrier needed in between
      for (int j = lane; j < a.dk; j += 32) {   // read keys: k = x / nk, sim = q . k
        if (live) gp[j] += dsr * (s.qr[j] - Pm[j] / nk * simr) / nk;
      }
      for (int v = lane; v < a.dv; v += 32) {   // values
        const float val = Pm[a.dk + v] / nv;
        if (live) gp[a.dk + v] += a.value_unit_norm ? relr * (dz[v] - val * drelr) / nv : relr * dz[v];
      }
      for (int j = lane; j < a.dk; j += 32) {   // write keys
        if (live && a.write_enabled) gp[a.dk + a.dv + j] += dsw * (s.qw[j] - Pm[a.dk + a.dv + j] / nw * simw) / nw;
      }
    }
    __syncthreads();
    // ---- cotangents of the queries --------------------------------------------------------------------------------------------
    if (tid < a.dk) {
      float gr = 0.f, gw = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) {
        gr = fmaf(dsimr[m], s.P[m * kJp + tid] / s.sc[m * kSc + 0], gr);
        gw = fmaf(dsimw[m], s.P[m * kJp + a.dk + a.dv + tid] / s.sc[m * kSc + 2], gw);
      }
      a.d_q_r[bt * a.dk + tid] = gr;
      if (a.write_enabled) a.d_q_w[bt * a.dk + tid] = gw;
    }
    __syncthreads();
  }
  // cotangent of the initial projections: the caller folds it into d slots0, d W and d slot_embed
  if (tid < J) {
#pragma unroll
    for (int m = 0; m < kMp; ++m) a.d_P0[((size_t)b * kMp + m) * J + tid] = dPc[m * kJp + tid];
  }
  for (int e = tid; e < nel; e += kThreads) {
    const int d = e / kMp, m = e % kMp;
    if (m < a.M) a.d_slots0[((size_t)b * a.M + m) * a.ds + d] = dSt[e];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int e = tid + i * kThreads;
    if (e < nel) {
      const int d = e / kMp, m = e % kMp;
      if (m < a.M) atomicAdd(a.d_delta_slot + m * a.ds + d, dslot_acc[i]);
    }
  }
  if (lane == 0) {
    atomicAdd(a.d_scalars + 0, dtaur_acc);
    atomicAdd(a.d_scalars + 1, dtauw_acc);
    if (warp * 2 < a.M) atomicAdd(a.d_mu + warp * 2, dmu_acc);
    if (warp * 2 + 1 < a.M) atomicAdd(a.d_mu + warp * 2 + 1, dmu_acc2);
  }
}

}  // namespace

bool screen_scan_supported(const ScreenScanArgs& a) {
  return a.M >= 1 && a.M <= kMp && a.ds % 4 == 0 && a.ds >= 16 && a.ds <= 256 && kThreads % a.ds == 0 && a.dk >= 1 &&
         a.dv >= 1 && 2 * a.dk + a.dv <= kJp && a.dk <= kThreads && a.dv <= kThreads;
}

int screen_scan_forward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr) return 1;
  const size_t bytes = (size_t)scan_smem_floats(a.ds, a.dk, a.dv) * sizeof(float);
  cudaFuncSetAttribute(screen_scan_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  screen_scan_fwd_kernel<false><<<a.B, kThreads, bytes, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int screen_scan_backward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr || a.saved_P == nullptr) return 1;
  const size_t bytes = (size_t)(scan_bwd_smem_floats(a.ds, a.dk, a.dv) + kMp) * sizeof(float);
  cudaFuncSetAttribute(screen_scan_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  screen_scan_bwd_kernel<false><<<a.B, kThreads, bytes, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace rk
