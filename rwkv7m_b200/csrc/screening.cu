// State-level screening memory: the slot-dependent part of the layer as kernels.
//
// Per step t (names follow src/rwkv7m/model/nnx_model.py:1024-1159 and src/rwkv7m/model/screening.py:11-88):
//   k_r[m] = unit(S[m] Wk^T)   val[m] = unit(S[m] Wv^T)   k_w[m] = unit((S[m] + E[m]) Wkw^T)
//   rel_r[m] = trim_square(q_r[t] . k_r[m], tau_r) (* age mask)      rel_w[m] = trim_square(q_w[t] . k_w[m], tau_w)
//   u[t]    = tanh_norm(sum_m rel_r[m] val[m])                       (output; the out-projection is a GEMM outside)
//   S[m]   += s_t[m] (tanh(dxh[t] + dslot[m]) - S[m]),   s_t[m] = mu[m] * max(rel_w[m], floor)   (mu[m] alone without
//                                                                                                  write screening)
// Two observations split the work into one sequential kernel of width J = dk + dv + dk and a few parallel ones of
// width ds (the slot width, up to 1024):
//  (1) The update interpolates towards a target D_t[m] = tanh(dxh[t] + dslot[m]) that does not depend on the state, and
//      the raw projections P[m] = S[m] W^T (+ E[m] Wkw^T on the write keys) are linear in S, so they obey
//        P_{t+1}[m] = P_t[m] + s_t[m] (PD_t[m] - P_t[m]),   PD_t[m] = D_t[m] W^T (+ E[m] Wkw^T),
//      where PD for all steps is one GEMM done by the caller.  Everything a step decides (norms, similarities,
//      relevances, the read-out, the write strengths) follows from P alone: the sequential kernel carries only P.
//  (2) Given the strengths s_t[m] the bank itself is an independent scalar recurrence per element: a parallel kernel
//      over (batch, slot, d) produces the final bank and the update-norm statistic.  In backward the bank's cotangent is
//      dS_{t+1}[m] = c_{t+1}[m] dS_T[m] with c the suffix products of (1 - s), so the strength cotangent that comes
//      through the bank is c_{t+1}[m] (h_t[m] - e_t[m]) with h_t[m] = <dS_T[m], D_t[m]> (parallel over all steps) and
//      e_t[m] = <dS_T[m], S_t[m]>, which follows the same scalar recurrence as the bank.  The sequential backward
//      kernel receives that number per (step, slot) and never touches a ds-wide vector; the dxh / dslot / initial-bank
//      gradients of the bank path are one more parallel kernel.
// The sequential kernels run one CTA of 16 warps per batch row: warp m owns slot m in the per-slot phases, thread j owns
// columns j and j + 512 of the projections in the per-column phases.
#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

constexpr int kMp = 16;            // slots are padded to 16
constexpr int kSeqThreads = 512;   // 16 warps
constexpr int kSc = 12;            // per-slot scalars: nk, nv, nw, simr, simw, relr, relw, strength, relr / nv
constexpr int kTileD = 64;         // rows of the bank staged at a time for the initial projections

__device__ __forceinline__ float trim_sq(float sim, float tau, float eps) {
  const float x = fmaxf((sim - tau) / (1.f - tau + eps), 0.f);
  return x * x;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// read relevance before the age mask, and its derivatives with respect to the similarity and the threshold
__device__ __forceinline__ float read_relevance(float sim, const ScreenScanArgs& a) {
  if (!a.leaky) return trim_sq(sim, a.tau_r, a.eps);
  return (1.f - a.leaky_alpha) * trim_sq(sim, a.tau_r, 1e-6f) + a.leaky_alpha * sigmoidf_(a.leaky_gamma * (sim - a.tau_r));
}

__device__ __forceinline__ void read_relevance_grad(float sim, const ScreenScanArgs& a, float& d_sim, float& d_tau) {
  const float e = a.leaky ? 1e-6f : a.eps;
  const float den = 1.f - a.tau_r + e;
  const float x = fmaxf((sim - a.tau_r) / den, 0.f);
  d_sim = 2.f * x / den;
  d_tau = 2.f * x * (sim - 1.f - e) / (den * den);
  if (a.leaky) {
    const float sg = sigmoidf_(a.leaky_gamma * (sim - a.tau_r));
    const float ds = a.leaky_gamma * sg * (1.f - sg);
    d_sim = (1.f - a.leaky_alpha) * d_sim + a.leaky_alpha * ds;
    d_tau = (1.f - a.leaky_alpha) * d_tau - a.leaky_alpha * ds;
  }
}

__host__ __device__ inline int padded_J(int J) { return (J + 3) & ~3; }

struct SeqSmem {
  float* P;      // [16][Jp]  raw projections of the current step (backward: two copies, alternating by step parity)
  float* PD;     // [16][Jp]  backward: projections of the step's write target
  float* dP;     // [16][Jp]  backward: cotangent of the carried projections
  float* EW;     // [16][dk]  forward: slot_embed Wkw^T
  float* tile;   // [64][16]  forward: rows of the bank staged for the initial projections
  float* qr;     // [dk]
  float* qw;     // [dk]
  float* z;      // [dv]
  float* du;     // [dv]      backward
  float* dz;     // [dv]      backward
  float* sc;     // [16][kSc] per-slot scalars
  float* ages;   // [16]
  float* usage;  // [16]
  float* dstr;   // [16]      backward: cotangent of the write strength
  float* dsimr;  // [16]
  float* dsimw;  // [16]
};

__host__ __device__ inline int seq_smem_floats(int J, int dk, int dv, bool backward) {
  const int Jp = padded_J(J);
  int n = kMp * Jp * (backward ? 4 : 1) + 2 * dk + dv + kMp * kSc + 2 * kMp;
  n += backward ? 2 * dv + 3 * kMp : kMp * dk + kTileD * kMp;
  return n + 8;
}

__device__ __forceinline__ SeqSmem carve(float* base, int J, int dk, int dv, bool backward) {
  const int Jp = padded_J(J);
  SeqSmem s{};
  s.P = base; base += kMp * Jp * (backward ? 2 : 1);
  if (backward) {
    s.PD = base; base += kMp * Jp;
    s.dP = base; base += kMp * Jp;
    s.du = base; base += dv;
    s.dz = base; base += dv;
    s.dstr = base; base += kMp;
    s.dsimr = base; base += kMp;
    s.dsimw = base; base += kMp;
  } else {
    s.EW = base; base += kMp * dk;
    s.tile = base; base += kTileD * kMp;
  }
  s.qr = base; base += dk;
  s.qw = base; base += dk;
  s.z = base; base += dv;
  s.sc = base; base += kMp * kSc;
  s.ages = base; base += kMp;
  s.usage = base; base += kMp;
  return s;
}

// acc[c][m] = sum_d src[m][d] * WT[d][j], j = tid + c * 512: the [M, ds] source is staged 64 rows of d at a time
template <int CPT>
__device__ __forceinline__ void project_rows(const float* __restrict__ src, const ScreenScanArgs& a, float* tile, int J,
                                             int tid, float (&acc)[CPT][kMp]) {
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < kMp; ++m) acc[c][m] = 0.f;
  for (int d0 = 0; d0 < a.ds; d0 += kTileD) {
    __syncthreads();
    for (int e = tid; e < kTileD * kMp; e += kSeqThreads) {
      const int dd = e / kMp, m = e % kMp;
      tile[e] = (m < a.M && d0 + dd < a.ds) ? __ldg(src + (size_t)m * a.ds + d0 + dd) : 0.f;
    }
    __syncthreads();
    const int nd = min(kTileD, a.ds - d0);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j >= J) continue;
      for (int dd = 0; dd < nd; ++dd) {
        const float w = __ldg(a.WT + (size_t)(d0 + dd) * J + j);
        const float4* sp = reinterpret_cast<const float4*>(tile + dd * kMp);
        const float4 p = sp[0], q = sp[1], r = sp[2], t = sp[3];
        acc[c][0] = fmaf(w, p.x, acc[c][0]); acc[c][1] = fmaf(w, p.y, acc[c][1]); acc[c][2] = fmaf(w, p.z, acc[c][2]);
        acc[c][3] = fmaf(w, p.w, acc[c][3]); acc[c][4] = fmaf(w, q.x, acc[c][4]); acc[c][5] = fmaf(w, q.y, acc[c][5]);
        acc[c][6] = fmaf(w, q.z, acc[c][6]); acc[c][7] = fmaf(w, q.w, acc[c][7]); acc[c][8] = fmaf(w, r.x, acc[c][8]);
        acc[c][9] = fmaf(w, r.y, acc[c][9]); acc[c][10] = fmaf(w, r.z, acc[c][10]); acc[c][11] = fmaf(w, r.w, acc[c][11]);
        acc[c][12] = fmaf(w, t.x, acc[c][12]); acc[c][13] = fmaf(w, t.y, acc[c][13]); acc[c][14] = fmaf(w, t.z, acc[c][14]);
        acc[c][15] = fmaf(w, t.w, acc[c][15]);
      }
    }
  }
}

// norms, similarities, relevances and the write strength of slot m from its row of raw projections (one warp)
__device__ __forceinline__ void slot_scalars(const float* __restrict__ Pm, const SeqSmem& s, const ScreenScanArgs& a, int m,
                                             int lane) {
  float sk = 0.f, dkq = 0.f, sv = 0.f, sw = 0.f, dwq = 0.f;
  for (int j = lane; j < a.dk; j += 32) { const float x = Pm[j]; sk = fmaf(x, x, sk); dkq = fmaf(x, s.qr[j], dkq); }
  for (int j = lane; j < a.dv; j += 32) { const float x = Pm[a.dk + j]; sv = fmaf(x, x, sv); }
  if (a.write_enabled)
    for (int j = lane; j < a.dk; j += 32) { const float x = Pm[a.dk + a.dv + j]; sw = fmaf(x, x, sw); dwq = fmaf(x, s.qw[j], dwq); }
  sk = warp_sum(sk); dkq = warp_sum(dkq); sv = warp_sum(sv);
  if (a.write_enabled) { sw = warp_sum(sw); dwq = warp_sum(dwq); }
  if (lane == 0) {
    float* c = s.sc + m * kSc;
    const float e2 = a.eps * a.eps;
    const float nk = sqrtf(sk + e2), nv = a.value_unit_norm ? sqrtf(sv + e2) : 1.f, nw = sqrtf(sw + e2);
    const float simr = dkq / nk, simw = dwq / nw;
    float relr = read_relevance(simr, a);
    if (a.age_mask) relr *= sigmoidf_((a.age_ref - s.ages[m]) / (a.age_sigma + a.eps));
    const bool live = m < a.M;
    if (!live) relr = 0.f;
    float relw = 0.f, strength = live ? a.mu[m] : 0.f;
    if (a.write_enabled && live) {
      relw = trim_sq(simw, a.tau_w, a.eps);
      strength *= fmaxf(relw, a.write_rel_floor);
    }
    c[0] = nk; c[1] = nv; c[2] = nw; c[3] = simr; c[4] = simw; c[5] = relr; c[6] = relw; c[7] = strength;
    c[8] = relr / nv;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Sequential forward: u, the write strengths, ages, usage and the logged statistics; saves P and the ages per step.
// ------------------------------------------------------------------------------------------------------------------
template <int CPT>
__global__ void __launch_bounds__(kSeqThreads) screen_seq_fwd_kernel(ScreenScanArgs a) {
  extern __shared__ float smem_f[];
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const int J = 2 * a.dk + a.dv, Jp = padded_J(J);
  const SeqSmem s = carve(smem_f, J, a.dk, a.dv, false);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;

  if (tid < kMp) {
    s.ages[tid] = tid < a.M ? a.ages0[b * a.M + tid] : 0.f;
    s.usage[tid] = tid < a.M ? a.usage0[b * a.M + tid] : 0.f;
  }
  {
    float acc[CPT][kMp];
    // E Wkw^T: only the write-key columns are kept
    project_rows<CPT>(a.slot_embed, a, s.tile, J, tid, acc);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j >= a.dk + a.dv && j < J) {
#pragma unroll
        for (int m = 0; m < kMp; ++m) s.EW[m * a.dk + j - a.dk - a.dv] = acc[c][m];
      }
    }
    // projections of the initial bank (the only pass over the weights); afterwards they follow the slot recurrence
    project_rows<CPT>(a.slots0 + (size_t)b * a.M * a.ds, a, s.tile, J, tid, acc);
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j < J) {
        const bool is_kw = j >= a.dk + a.dv;   // this thread wrote these EW entries itself
#pragma unroll
        for (int m = 0; m < kMp; ++m) s.P[m * Jp + j] = acc[c][m] + (is_kw ? s.EW[m * a.dk + j - a.dk - a.dv] : 0.f);
      }
    }
  }
  float st_acc[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) st_acc[i] = 0.f;

  // the step's vectors are fetched one step ahead into registers
  float n_qr = 0.f, n_qw = 0.f;
  float n_pd[CPT][kMp];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < kMp; ++m) n_pd[c][m] = 0.f;
  auto fetch = [&](int t) {
    const size_t bt = (size_t)b * a.T + t;
    if (tid < a.dk) { n_qr = a.q_r[bt * a.dk + tid]; n_qw = a.write_enabled ? a.q_w[bt * a.dk + tid] : 0.f; }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j < J) {
        const float* src = a.PD + bt * kMp * J + j;
#pragma unroll
        for (int m = 0; m < kMp; ++m) n_pd[c][m] = src[m * J];
      }
    }
  };
  fetch(0);
  for (int t = 0; t < a.T; ++t) {
    const size_t bt = (size_t)b * a.T + t;
    if (tid < a.dk) { s.qr[tid] = n_qr; s.qw[tid] = n_qw; }
    float pd[CPT][kMp];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
      for (int m = 0; m < kMp; ++m) pd[c][m] = n_pd[c][m];
    if (t + 1 < a.T) fetch(t + 1);
    __syncthreads();   // P of this step is complete (written at the end of the previous iteration); q staged
    if (a.saved_P != nullptr) {
      if (tid < kMp) a.saved_ages[bt * kMp + tid] = s.ages[tid];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const int j = tid + c * kSeqThreads;
        if (j < J) {
          float* dp = a.saved_P + bt * kMp * J + j;
#pragma unroll
          for (int m = 0; m < kMp; ++m) dp[m * J] = s.P[m * Jp + j];
        }
      }
    }
    slot_scalars(s.P + warp * Jp, s, a, warp, lane);
    __syncthreads();
    // ---- read-out -------------------------------------------------------------------------------------------------
    if (tid < a.dv) {
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) acc = fmaf(s.sc[m * kSc + 8], s.P[m * Jp + a.dk + tid], acc);
      s.z[tid] = acc;
    }
    if (tid < kMp) a.strength[bt * kMp + tid] = s.sc[tid * kSc + 7];
    __syncthreads();
    float zn2 = 0.f;
    for (int v = lane; v < a.dv; v += 32) zn2 = fmaf(s.z[v], s.z[v], zn2);
    zn2 = warp_sum(zn2);
    const float zn = sqrtf(zn2 + a.eps * a.eps);
    const float f = a.cap * tanhf(zn / a.cap) / zn;
    if (tid < a.dv) a.u_out[bt * a.dv + tid] = f * s.z[tid];
    // ---- the projections follow the slot interpolation ----------------------------------------------------------------
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j < J) {
#pragma unroll
        for (int m = 0; m < kMp; ++m) {
          const float old = s.P[m * Jp + j];
          s.P[m * Jp + j] = fmaf(s.sc[m * kSc + 7], pd[c][m] - old, old);
        }
      }
    }
    // ---- ages, usage and the logged statistics: lane m of warp 0 keeps slot m's running sums in registers ------------
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
        st_acc[0] += relr; st_acc[2] += relr > 1e-3f ? 1.f : 0.f;
        st_acc[5] += relw; st_acc[6] += a.write_enabled ? fmaxf(relw, a.write_rel_floor) : relw;
        st_acc[8] += us;
      }
      if (lane == 0) { st_acc[1] += rx; st_acc[3] += zn; st_acc[4] += f * zn; }
    }
  }
  __syncthreads();
  if (tid < a.M) { a.ages_out[b * a.M + tid] = s.ages[tid]; a.usage_out[b * a.M + tid] = s.usage[tid]; }
  if (warp == 0) {   // per-slot sums -> means over slots (sums over steps and batch rows stay sums; the host divides)
    const float im = 1.f / a.M;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      if (i == 7) continue;   // the update norm comes from the bank kernel
      float v = lane < kMp ? st_acc[i] : 0.f;
      v = warp_sum(v);
      const bool per_slot_mean = i == 0 || i == 5 || i == 6 || i == 8;
      if (lane == 0) atomicAdd(a.stats + i, per_slot_mean ? v * im : v);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Bank recurrence given the strengths: block (slot m, batch row b), thread d.  Writes the final bank and adds the
// update-norm statistic sum_t |S_{t+1}[m] - S_t[m]| / M to stats[7].
// ------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) screen_bank_fwd_kernel(ScreenScanArgs a) {
  __shared__ float part[32][33];   // [warp][step within a group of 32]
  const int m = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int warp = d >> 5, lane = d & 31, nw = blockDim.x >> 5;
  const bool on = d < a.ds;
  float S = on ? a.slots0[((size_t)b * a.M + m) * a.ds + d] : 0.f;
  const float dsl = on ? a.delta_slot[(size_t)m * a.ds + d] : 0.f;
  const float* str = a.strength + (size_t)b * a.T * kMp + m;
  const float* xh = a.delta_xh + (size_t)b * a.T * a.ds + d;
  float norm_acc = 0.f;
  for (int t0 = 0; t0 < a.T; t0 += 32) {
    const int n = min(32, a.T - t0);
    // the 32 steps' inputs are requested together: nothing in the recurrence decides an address
    float xv[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) xv[i] = (on && i < n) ? __ldg(xh + (size_t)(t0 + i) * a.ds) : 0.f;
    const float sv = lane < n ? __ldg(str + (size_t)(t0 + lane) * kMp) : 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float sg = __shfl_sync(0xffffffffu, sv, i);   // 0 beyond the last step: the bank stays put
      float diff = 0.f;
      if (on) {
        const float target = tanhf(xv[i] + dsl);
        diff = sg * (target - S);
        S += diff;
      }
      const float q = warp_sum(diff * diff);
      if (lane == 0) part[warp][i] = q;
    }
    __syncthreads();
    if (warp == 0 && lane < n) {
      float tot = 0.f;
      for (int w = 0; w < nw; ++w) tot += part[w][lane];
      norm_acc += sqrtf(tot);
    }
    __syncthreads();
  }
  if (on) a.slots_out[((size_t)b * a.M + m) * a.ds + d] = S;
  if (warp == 0) {
    norm_acc = warp_sum(norm_acc);
    if (lane == 0) atomicAdd(a.stats + 7, norm_acc / a.M);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Backward, bank path.  (1) h[b,t,m] = <dS_T[b,m], tanh(dxh[b,t] + dslot[m])>: block (step tile, slot, batch row), a warp
// per step, lanes over d.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kDotTile = 256;   // steps per block
constexpr int kDotMaxPerLane = 32;   // ds <= 1024

__global__ void __launch_bounds__(256) screen_target_dot_kernel(ScreenScanArgs a) {
  const int m = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float g[kDotMaxPerLane], dsl[kDotMaxPerLane];
#pragma unroll
  for (int i = 0; i < kDotMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    const bool on = d < a.ds;
    g[i] = on ? a.dslots_out[((size_t)b * a.M + m) * a.ds + d] : 0.f;
    dsl[i] = on ? a.delta_slot[(size_t)m * a.ds + d] : 0.f;
  }
  const int t_end = min(a.T, (int)(blockIdx.x + 1) * kDotTile);
  for (int t = blockIdx.x * kDotTile + warp; t < t_end; t += 8) {
    const float* xh = a.delta_xh + ((size_t)b * a.T + t) * a.ds;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kDotMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < a.ds) acc = fmaf(g[i], tanhf(__ldg(xh + d) + dsl[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) a.ws_h[((size_t)b * a.T + t) * kMp + m] = acc;
  }
}

// (2) Scalar recurrences per (batch row, slot), one warp each: e_{t+1} = e_t + s_t (h_t - e_t) forwards from
// e_0 = <dS_T, S_0>, the suffix products c backwards.  Writes G[t] = c_{t+1} (h_t - e_t) (the strength cotangent that
// arrives through the bank), coef[t] = s_t c_{t+1} (the factor of dS_T in the target's cotangent) and c_0.
__global__ void __launch_bounds__(32) screen_bank_scalars_kernel(ScreenScanArgs a) {
  const int m = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  float e = 0.f;
  for (int d = lane; d < a.ds; d += 32) {
    const size_t o = ((size_t)b * a.M + m) * a.ds + d;
    e = fmaf(a.dslots_out[o], a.slots0[o], e);
  }
  e = warp_sum(e);
  const size_t base = (size_t)b * a.T * kMp + m;
  for (int t0 = 0; t0 < a.T; t0 += 32) {   // forwards: G <- h_t - e_t
    const int t = t0 + lane;
    const bool on = t < a.T;
    const float h = on ? a.ws_h[base + (size_t)t * kMp] : 0.f;
    const float sg = on ? a.strength[base + (size_t)t * kMp] : 0.f;
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float hi = __shfl_sync(0xffffffffu, h, i), si = __shfl_sync(0xffffffffu, sg, i);
      const float diff = hi - e;
      if (lane == i) mine = diff;
      e = fmaf(si, diff, e);   // lanes beyond T carry s = 0
    }
    if (on) a.ws_G[base + (size_t)t * kMp] = mine;
  }
  float c = 1.f;   // c_T
  for (int t0 = ((a.T - 1) / 32) * 32; t0 >= 0; t0 -= 32) {   // backwards
    const int t = t0 + lane;
    const bool on = t < a.T;
    const float sg = on ? a.strength[base + (size_t)t * kMp] : 0.f;
    const float diff = on ? a.ws_G[base + (size_t)t * kMp] : 0.f;
    float c_next = 0.f;   // c_{t+1} of this lane's step
#pragma unroll
    for (int i = 31; i >= 0; --i) {
      const float si = __shfl_sync(0xffffffffu, sg, i);
      if (lane == i) c_next = c;
      c *= 1.f - si;
    }
    if (on) {
      a.ws_G[base + (size_t)t * kMp] = c_next * diff;
      a.ws_coef[base + (size_t)t * kMp] = sg * c_next;
    }
  }
  if (lane == 0) a.ws_c0[b * kMp + m] = c;
}

// (3) d dxh[b,t,d] = sum_m coef[b,t,m] dS_T[b,m,d] (1 - D^2), d dslot[m,d] += the same term summed over (b, t), and the
// initial bank's direct cotangent c_0 dS_T.  Block (chunk of 256 d, step tile, batch row), thread d.
constexpr int kBankBwdTile = 128;

__global__ void __launch_bounds__(256) screen_bank_bwd_kernel(ScreenScanArgs a) {
  __shared__ float coef[kBankBwdTile][kMp];
  const int d = blockIdx.x * 256 + threadIdx.x, b = blockIdx.z;
  const int t0 = blockIdx.y * kBankBwdTile, n = min(kBankBwdTile, a.T - t0);
  for (int e = threadIdx.x; e < n * kMp; e += 256) coef[e / kMp][e % kMp] = a.ws_coef[((size_t)b * a.T + t0) * kMp + e];
  __syncthreads();
  if (d >= a.ds) return;
  float g[kMp], dsl[kMp], acc[kMp];
#pragma unroll
  for (int m = 0; m < kMp; ++m) {
    const bool live = m < a.M;
    g[m] = live ? a.dslots_out[((size_t)b * a.M + m) * a.ds + d] : 0.f;
    dsl[m] = live ? a.delta_slot[(size_t)m * a.ds + d] : 0.f;
    acc[m] = 0.f;
  }
  for (int i = 0; i < n; ++i) {
    const size_t o = ((size_t)b * a.T + t0 + i) * a.ds + d;
    const float x = __ldg(a.delta_xh + o);
    float sum = 0.f;
#pragma unroll
    for (int m = 0; m < kMp; ++m) {
      const float D = tanhf(x + dsl[m]);
      const float term = coef[i][m] * g[m] * (1.f - D * D);
      acc[m] += term;
      sum += term;
    }
    a.d_delta_xh[o] = sum;
  }
#pragma unroll
  for (int m = 0; m < kMp; ++m)
    if (m < a.M) atomicAdd(a.d_delta_slot + (size_t)m * a.ds + d, acc[m]);
  if (blockIdx.y == 0) {
#pragma unroll
    for (int m = 0; m < kMp; ++m)
      if (m < a.M) a.d_slots0[((size_t)b * a.M + m) * a.ds + d] = a.ws_c0[b * kMp + m] * g[m];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Sequential backward over the saved projections: cotangents of q_r, q_w, PD, the initial projections, mu and the two
// thresholds.  ws_G (optional) is the strength cotangent that arrives through the bank.
// ------------------------------------------------------------------------------------------------------------------
template <int CPT>
__global__ void __launch_bounds__(kSeqThreads) screen_seq_bwd_kernel(ScreenScanArgs a) {
  extern __shared__ float smem_f[];
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const int J = 2 * a.dk + a.dv, Jp = padded_J(J);
  const SeqSmem s = carve(smem_f, J, a.dk, a.dv, true);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  const float e2 = a.eps * a.eps;

  for (int e = tid; e < kMp * Jp; e += kSeqThreads) s.dP[e] = 0.f;   // the projections after the last step feed nothing
  float dmu_acc = 0.f, dtaur_acc = 0.f, dtauw_acc = 0.f;   // lane 0 of warp m: slot m

  // everything a step reads from global memory is fetched one step ahead into registers
  float n_qr = 0.f, n_qw = 0.f, n_du = 0.f, n_age = 0.f, n_G = 0.f;
  float n_P[CPT][kMp], n_PD[CPT][kMp];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < kMp; ++m) { n_P[c][m] = 0.f; n_PD[c][m] = 0.f; }
  auto fetch = [&](int t) {
    const size_t bt = (size_t)b * a.T + t;
    if (tid < a.dk) { n_qr = a.q_r[bt * a.dk + tid]; n_qw = a.write_enabled ? a.q_w[bt * a.dk + tid] : 0.f; }
    if (tid < a.dv) n_du = a.du[bt * a.dv + tid];
    if (tid < kMp) {
      n_age = a.saved_ages[bt * kMp + tid];
      n_G = a.ws_G != nullptr ? a.ws_G[bt * kMp + tid] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j < J) {
        const float* sp = a.saved_P + bt * kMp * J + j;
        const float* pp = a.PD + bt * kMp * J + j;
#pragma unroll
        for (int m = 0; m < kMp; ++m) { n_P[c][m] = sp[m * J]; n_PD[c][m] = pp[m * J]; }
      }
    }
  };
  fetch(a.T - 1);
  for (int t = a.T - 1; t >= 0; --t) {
    const size_t bt = (size_t)b * a.T + t;
    // P alternates between two buffers: the query cotangents at the end of a step still read this step's copy while
    // the next step's staging writes the other one
    float* P = s.P + (t & 1) * kMp * Jp;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int j = tid + c * kSeqThreads;
      if (j < J) {
#pragma unroll
        for (int m = 0; m < kMp; ++m) { P[m * Jp + j] = n_P[c][m]; s.PD[m * Jp + j] = n_PD[c][m]; }
      }
    }
    if (tid < kMp) { s.ages[tid] = n_age; s.dstr[tid] = n_G; }
    if (tid < a.dk) { s.qr[tid] = n_qr; s.qw[tid] = n_qw; }
    if (tid < a.dv) s.du[tid] = n_du;
    if (t > 0) fetch(t - 1);
    __syncthreads();
    const float* Pm = P + warp * Jp;
    slot_scalars(Pm, s, a, warp, lane);
    __syncthreads();
    if (tid < a.dv) {
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) acc = fmaf(s.sc[m * kSc + 8], P[m * Jp + a.dk + tid], acc);
      s.z[tid] = acc;
    }
    // ---- backward of the projection update P' = P + s (PD - P): warp m owns slot m ------------------------------------
    {
      const int m = warp;
      const float strength = s.sc[m * kSc + 7];
      float* gp = s.dP + m * Jp;
      float* out = a.d_PD + (bt * kMp + m) * J;
      float dsp = 0.f;
      for (int j = lane; j < J; j += 32) {
        const float g = gp[j];
        dsp = fmaf(g, s.PD[m * Jp + j] - Pm[j], dsp);
        out[j] = strength * g;
        gp[j] = (1.f - strength) * g;
      }
      dsp = warp_sum(dsp);
      if (lane == 0) s.dstr[m] += dsp;   // this warp is the only writer of dstr[m] after the staging above
    }
    __syncthreads();
    // ---- cotangent of z from the cotangent of u = f(n) z -------------------------------------------------------------
    float zn2 = 0.f, zdu = 0.f;
    for (int v = lane; v < a.dv; v += 32) { zn2 = fmaf(s.z[v], s.z[v], zn2); zdu = fmaf(s.z[v], s.du[v], zdu); }
    zn2 = warp_sum(zn2); zdu = warp_sum(zdu);
    const float n2 = zn2 + e2, zn = sqrtf(n2);
    const float th = tanhf(zn / a.cap);
    const float f = a.cap * th / zn;
    const float coef = zdu * ((1.f - th * th) - f) / n2;
    if (tid < a.dv) s.dz[tid] = f * s.du[tid] + coef * s.z[tid];
    __syncthreads();
    // ---- per-slot scalars backward; cotangent of the raw projections ---------------------------------------------------
    {
      const int m = warp;
      const float* c = s.sc + m * kSc;
      const float nk = c[0], nv = c[1], nw = c[2], simr = c[3], simw = c[4], relr = c[5], relw = c[6];
      const bool live = m < a.M;
      float drelr = 0.f;
      for (int v = lane; v < a.dv; v += 32) drelr = fmaf(s.dz[v], Pm[a.dk + v] / nv, drelr);
      drelr = warp_sum(drelr);
      float mask = 1.f;
      if (a.age_mask) mask = sigmoidf_((a.age_ref - s.ages[m]) / (a.age_sigma + a.eps));
      float g_sim, g_tau;
      read_relevance_grad(simr, a, g_sim, g_tau);
      const float dtrim = live ? drelr * mask : 0.f;
      const float dsr = dtrim * g_sim;
      float dsw = 0.f, gate_w = 1.f;
      const float ds_m = s.dstr[m];
      if (a.write_enabled && live) {
        gate_w = fmaxf(relw, a.write_rel_floor);
        const float drelw = relw > a.write_rel_floor ? ds_m * a.mu[m] : 0.f;
        const float den_w = 1.f - a.tau_w + a.eps;
        const float xw = fmaxf((simw - a.tau_w) / den_w, 0.f);
        dsw = drelw * 2.f * xw / den_w;
        if (lane == 0) dtauw_acc += drelw * 2.f * xw * (simw - 1.f - a.eps) / (den_w * den_w);
      }
      if (lane == 0) {
        if (live) { dtaur_acc += dtrim * g_tau; dmu_acc += ds_m * gate_w; }
        s.dsimr[m] = live ? dsr : 0.f;
        s.dsimw[m] = live ? dsw : 0.f;
      }
      float* gp = s.dP + m * Jp;   // same warp and lanes as the scaling above: no barrier needed in between
      if (live) {
        for (int j = lane; j < a.dk; j += 32)   // read keys: k = x / nk, sim = q . k
          gp[j] += dsr * (s.qr[j] - Pm[j] / nk * simr) / nk;
        for (int v = lane; v < a.dv; v += 32) {   // values
          const float val = Pm[a.dk + v] / nv;
          gp[a.dk + v] += a.value_unit_norm ? relr * (s.dz[v] - val * drelr) / nv : relr * s.dz[v];
        }
        if (a.write_enabled)
          for (int j = lane; j < a.dk; j += 32)   // write keys
            gp[a.dk + a.dv + j] += dsw * (s.qw[j] - Pm[a.dk + a.dv + j] / nw * simw) / nw;
      }
    }
    __syncthreads();
    // ---- cotangents of the queries -------------------------------------------------------------------------------------
    if (tid < a.dk) {
      float gr = 0.f, gw = 0.f;
#pragma unroll
      for (int m = 0; m < kMp; ++m) {
        gr = fmaf(s.dsimr[m], P[m * Jp + tid] / s.sc[m * kSc + 0], gr);
        gw = fmaf(s.dsimw[m], P[m * Jp + a.dk + a.dv + tid] / s.sc[m * kSc + 2], gw);
      }
      a.d_q_r[bt * a.dk + tid] = gr;
      if (a.write_enabled) a.d_q_w[bt * a.dk + tid] = gw;
    }
    // no barrier here: the next step's staging touches the other P buffer, PD (last read two barriers ago) and the step
    // vectors, none of which the query cotangents read; sc, dsimr and dsimw are rewritten only after the next barrier
  }
  __syncthreads();
  // cotangent of the initial projections: the caller folds it into d slots0, d W and d slot_embed
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int j = tid + c * kSeqThreads;
    if (j < J) {
#pragma unroll
      for (int m = 0; m < kMp; ++m) a.d_P0[((size_t)b * kMp + m) * J + j] = s.dP[m * Jp + j];
    }
  }
  if (lane == 0) {
    atomicAdd(a.d_scalars + 0, dtaur_acc);
    atomicAdd(a.d_scalars + 1, dtauw_acc);
    if (warp < a.M) atomicAdd(a.d_mu + warp, dmu_acc);
  }
}

int columns_per_thread(int J) { return (J + kSeqThreads - 1) / kSeqThreads; }

}  // namespace

bool screen_scan_supported(const ScreenScanArgs& a) {
  const int J = 2 * a.dk + a.dv;
  return a.M >= 1 && a.M <= kMp && a.ds >= 1 && a.ds <= 32 * kDotMaxPerLane && a.dk >= 1 && a.dv >= 1 &&
         a.dk <= kSeqThreads && a.dv <= kSeqThreads && J <= 2 * kSeqThreads &&
         (size_t)seq_smem_floats(J, a.dk, a.dv, true) * sizeof(float) <= 227 * 1024 &&
         (size_t)seq_smem_floats(J, a.dk, a.dv, false) * sizeof(float) <= 227 * 1024;
}

int screen_scan_forward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr || a.strength == nullptr) return 1;
  const int J = 2 * a.dk + a.dv;
  const size_t bytes = (size_t)seq_smem_floats(J, a.dk, a.dv, false) * sizeof(float);
  if (columns_per_thread(J) == 1) {
    cudaFuncSetAttribute(screen_seq_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    screen_seq_fwd_kernel<1><<<a.B, kSeqThreads, bytes, st>>>(a);
  } else {
    cudaFuncSetAttribute(screen_seq_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    screen_seq_fwd_kernel<2><<<a.B, kSeqThreads, bytes, st>>>(a);
  }
  const int threads = ((a.ds + 31) / 32) * 32;
  screen_bank_fwd_kernel<<<dim3(a.M, a.B), threads, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int screen_scan_backward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr || a.saved_P == nullptr || a.strength == nullptr) return 1;
  const int J = 2 * a.dk + a.dv;
  const bool bank = a.dslots_out != nullptr;
  if (bank) {
    if (a.ws_h == nullptr || a.ws_G == nullptr || a.ws_coef == nullptr || a.ws_c0 == nullptr) return 1;
    screen_target_dot_kernel<<<dim3((a.T + kDotTile - 1) / kDotTile, a.M, a.B), 256, 0, st>>>(a);
    screen_bank_scalars_kernel<<<dim3(a.M, a.B), 32, 0, st>>>(a);
  }
  const size_t bytes = (size_t)seq_smem_floats(J, a.dk, a.dv, true) * sizeof(float);
  if (columns_per_thread(J) == 1) {
    cudaFuncSetAttribute(screen_seq_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    screen_seq_bwd_kernel<1><<<a.B, kSeqThreads, bytes, st>>>(a);
  } else {
    cudaFuncSetAttribute(screen_seq_bwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    screen_seq_bwd_kernel<2><<<a.B, kSeqThreads, bytes, st>>>(a);
  }
  if (bank)
    screen_bank_bwd_kernel<<<dim3((a.ds + 255) / 256, (a.T + kBankBwdTile - 1) / kBankBwdTile, a.B), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace rk
