// State-level screening memory: the slot-dependent part of the layer as kernels.
//
// Per step t (names follow src/rwkv7m/model/nnx_model.py:1024-1159 and src/rwkv7m/model/screening.py:11-88):
//   k_r[m] = unit(S[m] Wk^T)   val[m] = unit(S[m] Wv^T)   k_w[m] = unit((S[m] + E[m]) Wkw^T)
//   rel_r[m] = trim_square(q_r[t] . k_r[m], tau_r) (* age mask)      rel_w[m] = trim_square(q_w[t] . k_w[m], tau_w)
//   u[t]    = tanh_norm(sum_m rel_r[m] val[m])                       (output; the out-projection is a GEMM outside)
//   S[m]   += s_t[m] (tanh(dxh[t] + dslot[m]) - S[m]),   s_t[m] = mu[m] * max(rel_w[m], floor)   (mu[m] alone without
//                                                                                                  write screening)
// Three observations take the recurrence apart:
//  (1) The update interpolates towards a target D_t[m] = tanh(dxh[t] + dslot[m]) that does not depend on the state, and
//      the raw projections P[m] = S[m] W^T (+ E[m] Wkw^T on the write keys; J = dk + dv + dk columns) are linear in S,
//      so they obey P_{t+1}[m] = P_t[m] + s_t[m] (PD_t[m] - P_t[m]) with PD_t[m] = D_t[m] W^T (+ E[m] Wkw^T), where PD
//      for all steps is one GEMM done by the caller.  Everything a step decides follows from P alone.
//  (2) Slot m's strength depends only on slot m's own projections and on the step's queries: the slots do not interact
//      inside the recurrence.  The sequential kernels therefore run ONE WARP per (batch row, slot), the row of P in
//      registers (column j = lane + 32 i), no shared memory and no block barrier: a step is a few fused multiply-adds
//      per lane, one butterfly of shuffles for all the sums, and scalar arithmetic.  What couples the slots (the
//      read-out z = sum_m rel_r[m] val[m] and its tanh-norm, the per-step maximum for the statistics, the query
//      cotangents in backward) does not feed back into the recurrence, so parallel kernels over all (batch, step) pairs
//      compute it from the saved per-step rows of P and per-slot scalars.
//  (3) Given the strengths the bank itself is an independent scalar recurrence per element: a parallel kernel over
//      (batch, slot, d) produces the final bank and the update-norm statistic.  In backward the bank's cotangent is
//      dS_{t+1}[m] = c_{t+1}[m] dS_T[m] with c the suffix products of (1 - s), so the strength cotangent that comes
//      through the bank is c_{t+1}[m] (h_t[m] - e_t[m]) with h_t[m] = <dS_T[m], D_t[m]> (parallel over all steps) and
//      e_t[m] = <dS_T[m], S_t[m]>, which follows the same scalar recurrence as the bank.  The sequential backward
//      kernel receives that number per (step, slot) and never touches a ds-wide vector; the dxh / dslot / initial-bank
//      gradients of the bank path are one more parallel kernel.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

using bf16 = __nv_bfloat16;

constexpr int kMp = 16;   // slots are padded to 16 in the [B, T, 16, ...] tensors

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

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

constexpr int kAhead = 6;   // steps ahead of the register prefetch that a step's rows are pulled into L2

// Which of the three column groups register i of this lane belongs to (column j = lane + 32 i), as bit masks.
struct ColumnMasks { uint32_t key, val, wkey; };

template <int JPL>
__device__ __forceinline__ ColumnMasks column_masks(int lane, int dk, int dv, int J) {
  ColumnMasks c{0u, 0u, 0u};
#pragma unroll
  for (int i = 0; i < JPL; ++i) {
    const int j = lane + 32 * i;
    if (j < dk) c.key |= 1u << i;
    else if (j < dk + dv) c.val |= 1u << i;
    else if (j < J) c.wkey |= 1u << i;
  }
  return c;
}

// The per-slot scalars of a step from the five (already warp-reduced) sums.
struct SlotScalars { float nk, nv, nw, simr, simw, relr, relw, strength, mask; };

__device__ __forceinline__ SlotScalars slot_scalars(float sk, float dkq, float sv, float sw, float dwq, float age, float mu_m,
                                                    const ScreenScanArgs& a) {
  SlotScalars c;
  const float e2 = a.eps * a.eps;
  c.nk = sqrtf(sk + e2);
  c.nv = a.value_unit_norm ? sqrtf(sv + e2) : 1.f;
  c.nw = sqrtf(sw + e2);
  c.simr = dkq / c.nk;
  c.simw = dwq / c.nw;
  c.mask = a.age_mask ? sigmoidf_((a.age_ref - age) / (a.age_sigma + a.eps)) : 1.f;
  c.relr = read_relevance(c.simr, a) * c.mask;
  c.relw = 0.f;
  c.strength = mu_m;
  if (a.write_enabled) {
    c.relw = trim_sq(c.simw, a.tau_w, a.eps);
    c.strength *= fmaxf(c.relw, a.write_rel_floor);
  }
  return c;
}

// Packed per-step rows laid out like the columns of P: [q_r | 0 | q_w] (the value columns receive dz in backward).
__global__ void __launch_bounds__(256) screen_pack_rows_kernel(ScreenScanArgs a) {
  const int J = 2 * a.dk + a.dv;
  const size_t n = (size_t)a.B * a.T * J;
  for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < n; e += (size_t)gridDim.x * 256) {
    const size_t bt = e / J;
    const int j = (int)(e - bt * J);
    float v = 0.f;
    if (j < a.dk) v = a.q_r[bt * a.dk + j];
    else if (j >= a.dk + a.dv && a.write_enabled) v = a.q_w[bt * a.dk + j - a.dk - a.dv];
    a.ws_rows[e] = v;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Sequential forward, one warp per (slot, batch row): write strengths, read coefficients, ages, usage, the per-slot
// statistics, and the row of P before every step.
// ------------------------------------------------------------------------------------------------------------------
template <int JPL>
__global__ void __launch_bounds__(32) screen_slot_fwd_kernel(ScreenScanArgs a) {
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const int m = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const int J = 2 * a.dk + a.dv;
  const ColumnMasks cm = column_masks<JPL>(lane, a.dk, a.dv, J);
  const uint32_t any = cm.key | cm.val | cm.wkey;

  // projections of the initial bank (the only pass over the weights): P[j] = sum_d (S0[d] + [write key] E[d]) WT[d][j]
  float P[JPL];
#pragma unroll
  for (int i = 0; i < JPL; ++i) P[i] = 0.f;
  {
    const float* s0 = a.slots0 + ((size_t)b * a.M + m) * a.ds;
    const float* em = a.slot_embed + (size_t)m * a.ds;
#pragma unroll 4
    for (int d = 0; d < a.ds; ++d) {
      const float sv = __ldg(s0 + d), se = sv + __ldg(em + d);
      const float* w = a.WT + (size_t)d * J;
#pragma unroll
      for (int i = 0; i < JPL; ++i) P[i] = fmaf((cm.wkey >> i) & 1u ? se : sv, __ldg(w + min(lane + 32 * i, J - 1)), P[i]);
    }
  }
  float age = a.ages0[b * a.M + m], usage = a.usage0[b * a.M + m];
  const float mu_m = a.mu[m];
  float acc_relr = 0.f, acc_active = 0.f, acc_relw = 0.f, acc_eff = 0.f, acc_usage = 0.f;

  const size_t row0 = ((size_t)b * a.T * kMp + m) * J;   // row of step 0; a step advances by 16 J
  const size_t step = (size_t)kMp * J;
  // Loads are unconditional (a register past the last column re-reads column J - 1 and is ignored by every sum and
  // store): a select on a loaded value would make the warp wait for the load right where it is issued.  The queries
  // come as one packed row [q_r | 0 | q_w] laid out like the columns of P.
  float n_pd[JPL], n_q[JPL];
  auto fetch = [&](int t) {
    const float* pd = a.PD + row0 + (size_t)t * step;
    const float* rr = a.ws_rows + ((size_t)b * a.T + t) * J;
#pragma unroll
    for (int i = 0; i < JPL; ++i) {
      const int j = min(lane + 32 * i, J - 1);
      n_pd[i] = pd[j];
      n_q[i] = rr[j];
    }
  };
  auto pull = [&](int t) {   // towards L2, several steps ahead of the register prefetch
    if (t >= a.T) return;
    const float* pd = a.PD + row0 + (size_t)t * step + lane;
#pragma unroll
    for (int i = 0; i < JPL; ++i)
      if ((any >> i) & 1u) prefetch_l2(pd + 32 * i);
  };
  for (int t = 1; t < kAhead; ++t) pull(t);
  fetch(0);
  for (int t = 0; t < a.T; ++t) {
    const size_t bt = (size_t)b * a.T + t;
    float pd[JPL], q[JPL];
#pragma unroll
    for (int i = 0; i < JPL; ++i) { pd[i] = n_pd[i]; q[i] = n_q[i]; }
    if (t + 1 < a.T) fetch(t + 1);
    pull(t + kAhead);
    {
      float* dst = a.saved_P + row0 + (size_t)t * step + lane;
#pragma unroll
      for (int i = 0; i < JPL; ++i)
        if ((any >> i) & 1u) dst[32 * i] = P[i];
    }
    float sk = 0.f, dkq = 0.f, sv = 0.f, sw = 0.f, dwq = 0.f;
#pragma unroll
    for (int i = 0; i < JPL; ++i) {
      const float x = P[i], xx = x * x, xq = x * q[i];
      if ((cm.key >> i) & 1u) { sk += xx; dkq += xq; }
      if ((cm.val >> i) & 1u) sv += xx;
      if ((cm.wkey >> i) & 1u) { sw += xx; dwq += xq; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {   // one butterfly for all five sums: the shuffles of a stage overlap
      sk += __shfl_xor_sync(0xffffffffu, sk, o); dkq += __shfl_xor_sync(0xffffffffu, dkq, o);
      sv += __shfl_xor_sync(0xffffffffu, sv, o); sw += __shfl_xor_sync(0xffffffffu, sw, o);
      dwq += __shfl_xor_sync(0xffffffffu, dwq, o);
    }
    const SlotScalars c = slot_scalars(sk, dkq, sv, sw, dwq, age, mu_m, a);
    if (lane == 0) {
      a.strength[bt * kMp + m] = c.strength;
      a.rel_c[bt * kMp + m] = c.relr / c.nv;
      a.rel_r[bt * kMp + m] = c.relr;
      a.saved_ages[bt * kMp + m] = age;
    }
#pragma unroll
    for (int i = 0; i < JPL; ++i) P[i] = fmaf(c.strength, pd[i] - P[i], P[i]);
    if (a.write_enabled) age = c.relw > 1e-3f ? 0.f : age + 1.f;
    const float act = a.write_enabled ? fmaxf(c.relr, c.relw) : c.relr;
    usage = a.usage_decay * usage + (1.f - a.usage_decay) * act;
    acc_relr += c.relr; acc_active += c.relr > 1e-3f ? 1.f : 0.f;
    acc_relw += c.relw; acc_eff += a.write_enabled ? fmaxf(c.relw, a.write_rel_floor) : c.relw;
    acc_usage += usage;
  }
  if (lane == 0) {
    a.ages_out[b * a.M + m] = age;
    a.usage_out[b * a.M + m] = usage;
    const float im = 1.f / a.M;   // means over slots; sums over steps and batch rows stay sums (the host divides)
    atomicAdd(a.stats + 0, acc_relr * im);
    atomicAdd(a.stats + 2, acc_active);
    atomicAdd(a.stats + 5, acc_relw * im);
    atomicAdd(a.stats + 6, acc_eff * im);
    atomicAdd(a.stats + 8, acc_usage * im);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Read-out over all (batch row, step) pairs, a warp per step: z = sum_m (rel_r[m] / nv[m]) P_t[m][values],
// u = tanh_norm(z).  BWD = false writes u and the cross-slot statistics; BWD = true reads du and writes
// dz = f du + z <z, du> ((1 - th^2) - f) / n^2, the cotangent of z, into the value columns of the packed rows.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kReadTile = 64;   // steps per block of 8 warps
constexpr int kMaxVPL = 16;     // dv <= 512

template <bool BWD>
__global__ void __launch_bounds__(256) screen_readout_kernel(ScreenScanArgs a) {
  __shared__ float red[8][3];
  const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int J = 2 * a.dk + a.dv;
  const int t_end = min(a.T, (int)(blockIdx.x + 1) * kReadTile);
  float st_max = 0.f, st_zn = 0.f, st_un = 0.f;
  for (int t = blockIdx.x * kReadTile + warp; t < t_end; t += 8) {
    const size_t bt = (size_t)b * a.T + t;
    const float c_l = lane < a.M ? a.rel_c[bt * kMp + lane] : 0.f;
    float z[kMaxVPL];
#pragma unroll
    for (int i = 0; i < kMaxVPL; ++i) z[i] = 0.f;
    const float* Pt = a.saved_P + bt * kMp * J + a.dk + lane;
    for (int m = 0; m < a.M; ++m) {
      const float c = __shfl_sync(0xffffffffu, c_l, m);
#pragma unroll
      for (int i = 0; i < kMaxVPL; ++i)
        if (lane + 32 * i < a.dv) z[i] = fmaf(c, Pt[(size_t)m * J + 32 * i], z[i]);
    }
    float zn2 = 0.f, zdu = 0.f;
    float du[kMaxVPL];
#pragma unroll
    for (int i = 0; i < kMaxVPL; ++i) {
      du[i] = 0.f;
      if (BWD && lane + 32 * i < a.dv) du[i] = a.du[bt * a.dv + lane + 32 * i];
      zn2 = fmaf(z[i], z[i], zn2);
      zdu = fmaf(z[i], du[i], zdu);
    }
    zn2 = warp_sum(zn2);
    const float n2 = zn2 + a.eps * a.eps, zn = sqrtf(n2);
    const float th = tanhf(zn / a.cap);
    const float f = a.cap * th / zn;
    if (BWD) {
      zdu = warp_sum(zdu);
      const float coef = zdu * ((1.f - th * th) - f) / n2;
#pragma unroll
      for (int i = 0; i < kMaxVPL; ++i)
        if (lane + 32 * i < a.dv) a.ws_rows[bt * J + a.dk + lane + 32 * i] = f * du[i] + coef * z[i];
    } else {
#pragma unroll
      for (int i = 0; i < kMaxVPL; ++i)
        if (lane + 32 * i < a.dv) a.u_out[bt * a.dv + lane + 32 * i] = f * z[i];
      float rx = lane < a.M ? a.rel_r[bt * kMp + lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) rx = fmaxf(rx, __shfl_xor_sync(0xffffffffu, rx, o));
      st_max += rx; st_zn += zn; st_un += f * zn;
    }
  }
  if (!BWD) {
    if (lane == 0) { red[warp][0] = st_max; red[warp][1] = st_zn; red[warp][2] = st_un; }
    __syncthreads();
    if (threadIdx.x < 3) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += red[w][threadIdx.x];
      atomicAdd(a.stats + (threadIdx.x == 0 ? 1 : threadIdx.x == 1 ? 3 : 4), v);
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
      if (m < a.M) {   // rows of the workspaces beyond the live slots are never written
        const float D = tanhf(x + dsl[m]);
        const float term = coef[i][m] * g[m] * (1.f - D * D);
        acc[m] += term;
        sum += term;
      }
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
// Sequential backward, one warp per (slot, batch row), over the saved rows of P: cotangents of PD and of the initial
// projections, of mu and the two thresholds, and the per-step factors of the query cotangents.  ws_G (optional) is the
// strength cotangent that arrives through the bank; the value columns of the packed rows hold the cotangent of z.
// ------------------------------------------------------------------------------------------------------------------
template <int JPL>
__global__ void __launch_bounds__(32) screen_slot_bwd_kernel(ScreenScanArgs a) {
  if (a.tau_dev != nullptr) { a.tau_r = a.tau_dev[0]; a.tau_w = a.tau_dev[1]; }
  const int m = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const int J = 2 * a.dk + a.dv;
  const ColumnMasks cm = column_masks<JPL>(lane, a.dk, a.dv, J);
  const uint32_t any = cm.key | cm.val | cm.wkey;
  const float mu_m = a.mu[m];
  float g[JPL];   // cotangent of the carried row of P; the projections after the last step feed nothing
#pragma unroll
  for (int i = 0; i < JPL; ++i) g[i] = 0.f;
  float dmu_acc = 0.f, dtaur_acc = 0.f, dtauw_acc = 0.f;

  const size_t row0 = ((size_t)b * a.T * kMp + m) * J;
  const size_t step = (size_t)kMp * J;
  // per step: the saved row of P, the row of PD, and one row r = [q_r | dz | q_w] laid out like the columns of P
  float n_P[JPL], n_pd[JPL], n_r[JPL], n_age = 0.f, n_G = 0.f;
  const float* Gp = a.ws_G != nullptr ? a.ws_G : a.strength;   // without a bank cotangent: finite numbers, times zero
  const float g_on = a.ws_G != nullptr ? 1.f : 0.f;
  auto fetch = [&](int t) {   // unconditional loads, as in the forward kernel
    const size_t bt = (size_t)b * a.T + t;
    const float* sp = a.saved_P + row0 + (size_t)t * step;
    const float* pd = a.PD + row0 + (size_t)t * step;
    const float* rr = a.ws_rows + bt * J;
#pragma unroll
    for (int i = 0; i < JPL; ++i) {
      const int j = min(lane + 32 * i, J - 1);
      n_P[i] = sp[j];
      n_pd[i] = pd[j];
      n_r[i] = rr[j];
    }
    n_age = a.saved_ages[bt * kMp + m];
    n_G = Gp[bt * kMp + m];
  };
  auto pull = [&](int t) {
    if (t < 0) return;
    const float* sp = a.saved_P + row0 + (size_t)t * step + lane;
    const float* pd = a.PD + row0 + (size_t)t * step + lane;
#pragma unroll
    for (int i = 0; i < JPL; ++i)
      if ((any >> i) & 1u) { prefetch_l2(sp + 32 * i); prefetch_l2(pd + 32 * i); }
  };
  for (int t = a.T - 2; t > a.T - 1 - kAhead; --t) pull(t);
  fetch(a.T - 1);
  for (int t = a.T - 1; t >= 0; --t) {
    const size_t bt = (size_t)b * a.T + t;
    float P[JPL], pd[JPL], r[JPL];
#pragma unroll
    for (int i = 0; i < JPL; ++i) { P[i] = n_P[i]; pd[i] = n_pd[i]; r[i] = n_r[i]; }
    const float age = n_age, G = n_G * g_on;
    if (t > 0) fetch(t - 1);
    pull(t - kAhead);
    float sk = 0.f, dkq = 0.f, sv = 0.f, sw = 0.f, dwq = 0.f, sdz = 0.f, dsp = 0.f;
#pragma unroll
    for (int i = 0; i < JPL; ++i) {
      const float x = P[i], xx = x * x, xr = x * r[i];
      if ((cm.key >> i) & 1u) { sk += xx; dkq += xr; }
      if ((cm.val >> i) & 1u) { sv += xx; sdz += xr; }
      if ((cm.wkey >> i) & 1u) { sw += xx; dwq += xr; }
      dsp = fmaf(g[i], pd[i] - x, dsp);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sk += __shfl_xor_sync(0xffffffffu, sk, o); dkq += __shfl_xor_sync(0xffffffffu, dkq, o);
      sv += __shfl_xor_sync(0xffffffffu, sv, o); sw += __shfl_xor_sync(0xffffffffu, sw, o);
      dwq += __shfl_xor_sync(0xffffffffu, dwq, o); sdz += __shfl_xor_sync(0xffffffffu, sdz, o);
      dsp += __shfl_xor_sync(0xffffffffu, dsp, o);
    }
    const SlotScalars c = slot_scalars(sk, dkq, sv, sw, dwq, age, mu_m, a);
    // ---- backward of the projection update P' = P + s (PD - P) -------------------------------------------------------
    const float dstr = G + dsp;
    {
      if (a.d_PD_bf16 != nullptr) {   // as the operand of the tensor-core products that follow
        bf16* out = reinterpret_cast<bf16*>(a.d_PD_bf16) + row0 + (size_t)t * step + lane;
#pragma unroll
        for (int i = 0; i < JPL; ++i)
          if ((any >> i) & 1u) out[32 * i] = __float2bfloat16(c.strength * g[i]);
      } else {
        float* out = a.d_PD + row0 + (size_t)t * step + lane;
#pragma unroll
        for (int i = 0; i < JPL; ++i)
          if ((any >> i) & 1u) out[32 * i] = c.strength * g[i];
      }
#pragma unroll
      for (int i = 0; i < JPL; ++i) g[i] *= 1.f - c.strength;
    }
    // ---- per-slot scalars backward ----------------------------------------------------------------------------------------
    const float drelr = sdz / c.nv;   // cotangent of rel_r: sum_v dz[v] val[v]
    float g_sim, g_tau;
    read_relevance_grad(c.simr, a, g_sim, g_tau);
    const float dtrim = drelr * c.mask;
    const float dsr = dtrim * g_sim;
    dtaur_acc += dtrim * g_tau;
    float dsw = 0.f, gate_w = 1.f;
    if (a.write_enabled) {
      gate_w = fmaxf(c.relw, a.write_rel_floor);
      const float drelw = c.relw > a.write_rel_floor ? dstr * mu_m : 0.f;
      const float den_w = 1.f - a.tau_w + a.eps;
      const float xw = fmaxf((c.simw - a.tau_w) / den_w, 0.f);
      dsw = drelw * 2.f * xw / den_w;
      dtauw_acc += drelw * 2.f * xw * (c.simw - 1.f - a.eps) / (den_w * den_w);
    }
    dmu_acc += dstr * gate_w;
    if (lane == 0) {   // factors of the query cotangents: dq_r = sum_m (dsim_r / nk) P[m][keys], likewise for q_w
      a.ws_a[bt * kMp + m] = dsr / c.nk;
      a.ws_b[bt * kMp + m] = dsw / c.nw;
    }
    // ---- cotangent of this step's row of P ----------------------------------------------------------------------------------
    const float kr = dsr / c.nk, kr2 = kr * c.simr / c.nk;        // keys:   dsr (q - (P / nk) simr) / nk
    const float kw = dsw / c.nw, kw2 = kw * c.simw / c.nw;        // write keys
    const float relr_nv = c.relr / c.nv, vv = relr_nv * drelr / c.nv;   // values: relr (dz - (P / nv) drelr) / nv
#pragma unroll
    for (int i = 0; i < JPL; ++i) {
      if ((cm.key >> i) & 1u) g[i] += kr * r[i] - kr2 * P[i];
      if ((cm.val >> i) & 1u) g[i] += a.value_unit_norm ? relr_nv * r[i] - vv * P[i] : c.relr * r[i];
      if (((cm.wkey >> i) & 1u) && a.write_enabled) g[i] += kw * r[i] - kw2 * P[i];
    }
  }
  {   // cotangent of the initial projections: the caller folds it into d slots0, d W and d slot_embed
    float* out = a.d_P0 + ((size_t)b * kMp + m) * J + lane;
#pragma unroll
    for (int i = 0; i < JPL; ++i)
      if ((any >> i) & 1u) out[32 * i] = g[i];
  }
  if (lane == 0) {
    atomicAdd(a.d_scalars + 0, dtaur_acc);
    atomicAdd(a.d_scalars + 1, dtauw_acc);
    atomicAdd(a.d_mu + m, dmu_acc);
  }
}

// Query cotangents over all (batch row, step) pairs, a warp per step: dq_r[j] = sum_m ws_a[m] P_t[m][j],
// dq_w[j] = sum_m ws_b[m] P_t[m][dk + dv + j].
__global__ void __launch_bounds__(256) screen_query_grad_kernel(ScreenScanArgs a) {
  const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int J = 2 * a.dk + a.dv;
  const int t_end = min(a.T, (int)(blockIdx.x + 1) * kReadTile);
  for (int t = blockIdx.x * kReadTile + warp; t < t_end; t += 8) {
    const size_t bt = (size_t)b * a.T + t;
    const float a_l = lane < a.M ? a.ws_a[bt * kMp + lane] : 0.f;
    const float b_l = lane < a.M ? a.ws_b[bt * kMp + lane] : 0.f;
    const float* Pt = a.saved_P + bt * kMp * J;
    for (int j = lane; j < a.dk; j += 32) {
      float gr = 0.f, gw = 0.f;
      for (int m = 0; m < a.M; ++m) {
        gr = fmaf(__shfl_sync(0xffffffffu, a_l, m), Pt[(size_t)m * J + j], gr);
        if (a.write_enabled) gw = fmaf(__shfl_sync(0xffffffffu, b_l, m), Pt[(size_t)m * J + a.dk + a.dv + j], gw);
      }
      a.d_q_r[bt * a.dk + j] = gr;
      if (a.write_enabled) a.d_q_w[bt * a.dk + j] = gw;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Write targets for the tensor-core projections: D[b,t,m,d] = tanh(dxh[b,t,d] + dslot[m,d]) in bf16, rows m >= M zero.
// Block (chunk of 256 d, tile of 64 steps, batch row), thread d.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kTargetTile = 64;

__global__ void __launch_bounds__(256) screen_targets_fwd_kernel(const float* __restrict__ dxh, const float* __restrict__ dslot,
                                                                 bf16* __restrict__ D, int T, int M, int ds) {
  const int d = blockIdx.x * 256 + threadIdx.x, b = blockIdx.z;
  if (d >= ds) return;
  const int t0 = blockIdx.y * kTargetTile, n = min(kTargetTile, T - t0);
  float dsl[kMp];
#pragma unroll
  for (int m = 0; m < kMp; ++m) dsl[m] = m < M ? dslot[(size_t)m * ds + d] : 0.f;
  for (int i = 0; i < n; ++i) {
    const size_t bt = (size_t)b * T + t0 + i;
    const float x = __ldg(dxh + bt * ds + d);
    bf16* out = D + bt * kMp * ds + d;
#pragma unroll
    for (int m = 0; m < kMp; ++m) out[(size_t)m * ds] = __float2bfloat16(m < M ? tanhf(x + dsl[m]) : 0.f);
  }
}

// d dxh[b,t,d] += sum_m dD[b,t,m,d] (1 - D^2), d dslot[m,d] += the same term summed over (b, t); D is recomputed.
__global__ void __launch_bounds__(256) screen_targets_bwd_kernel(const bf16* __restrict__ dD, const float* __restrict__ dxh,
                                                                 const float* __restrict__ dslot, float* __restrict__ g_dxh,
                                                                 float* __restrict__ g_dslot, int T, int M, int ds) {
  const int d = blockIdx.x * 256 + threadIdx.x, b = blockIdx.z;
  if (d >= ds) return;
  const int t0 = blockIdx.y * kTargetTile, n = min(kTargetTile, T - t0);
  float dsl[kMp], acc[kMp];
#pragma unroll
  for (int m = 0; m < kMp; ++m) { dsl[m] = m < M ? dslot[(size_t)m * ds + d] : 0.f; acc[m] = 0.f; }
  for (int i = 0; i < n; ++i) {
    const size_t bt = (size_t)b * T + t0 + i;
    const float x = __ldg(dxh + bt * ds + d);
    const bf16* src = dD + bt * kMp * ds + d;
    float sum = 0.f;
#pragma unroll
    for (int m = 0; m < kMp; ++m) {
      if (m < M) {
        const float D = tanhf(x + dsl[m]);
        const float term = __bfloat162float(src[(size_t)m * ds]) * (1.f - D * D);
        acc[m] += term;
        sum += term;
      }
    }
    g_dxh[bt * ds + d] += sum;
  }
#pragma unroll
  for (int m = 0; m < kMp; ++m)
    if (m < M) atomicAdd(g_dslot + (size_t)m * ds + d, acc[m]);
}

template <template <int> class Launcher>
int dispatch_jpl(int J, const ScreenScanArgs& a, cudaStream_t st) {
  const int jpl = (J + 31) / 32;
  if (jpl <= 2) return Launcher<2>::run(a, st);
  if (jpl <= 4) return Launcher<4>::run(a, st);
  if (jpl <= 6) return Launcher<6>::run(a, st);
  if (jpl <= 8) return Launcher<8>::run(a, st);
  if (jpl <= 12) return Launcher<12>::run(a, st);
  if (jpl <= 18) return Launcher<18>::run(a, st);
  if (jpl <= 24) return Launcher<24>::run(a, st);
  if (jpl <= 32) return Launcher<32>::run(a, st);
  return 1;
}

template <int JPL> struct FwdLauncher {
  static int run(const ScreenScanArgs& a, cudaStream_t st) {
    screen_slot_fwd_kernel<JPL><<<dim3(a.M, a.B), 32, 0, st>>>(a);
    return 0;
  }
};
template <int JPL> struct BwdLauncher {
  static int run(const ScreenScanArgs& a, cudaStream_t st) {
    screen_slot_bwd_kernel<JPL><<<dim3(a.M, a.B), 32, 0, st>>>(a);
    return 0;
  }
};

}  // namespace

void screen_targets_forward(const float* dxh, const float* dslot, void* D, int B, int T, int M, int ds, cudaStream_t st) {
  screen_targets_fwd_kernel<<<dim3((ds + 255) / 256, (T + kTargetTile - 1) / kTargetTile, B), 256, 0, st>>>(
      dxh, dslot, (bf16*)D, T, M, ds);
}

void screen_targets_backward(const void* dD, const float* dxh, const float* dslot, float* g_dxh, float* g_dslot, int B, int T,
                             int M, int ds, cudaStream_t st) {
  screen_targets_bwd_kernel<<<dim3((ds + 255) / 256, (T + kTargetTile - 1) / kTargetTile, B), 256, 0, st>>>(
      (const bf16*)dD, dxh, dslot, g_dxh, g_dslot, T, M, ds);
}

bool screen_scan_supported(const ScreenScanArgs& a) {
  const int J = 2 * a.dk + a.dv;
  return a.M >= 1 && a.M <= kMp && a.ds >= 1 && a.ds <= 32 * kDotMaxPerLane && a.dk >= 1 && a.dv >= 1 &&
         a.dv <= 32 * kMaxVPL && J <= 1024;
}

int screen_scan_forward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr || a.strength == nullptr || a.saved_P == nullptr ||
      a.saved_ages == nullptr || a.rel_c == nullptr || a.rel_r == nullptr)
    return 1;
  const int J = 2 * a.dk + a.dv;
  if (a.ws_rows == nullptr) return 1;
  const int pack_blocks = (int)std::min<size_t>(148 * 8, ((size_t)a.B * a.T * J + 255) / 256);
  screen_pack_rows_kernel<<<pack_blocks, 256, 0, st>>>(a);
  if (dispatch_jpl<FwdLauncher>(J, a, st) != 0) return 1;
  screen_readout_kernel<false><<<dim3((a.T + kReadTile - 1) / kReadTile, a.B), 256, 0, st>>>(a);
  const int threads = ((a.ds + 31) / 32) * 32;
  screen_bank_fwd_kernel<<<dim3(a.M, a.B), threads, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int screen_scan_backward(const ScreenScanArgs& a, cudaStream_t st) {
  if (!screen_scan_supported(a) || a.PD == nullptr || a.saved_P == nullptr || a.strength == nullptr ||
      a.rel_c == nullptr || a.ws_rows == nullptr || a.ws_a == nullptr || a.ws_b == nullptr)
    return 1;
  const int J = 2 * a.dk + a.dv;
  const bool bank = a.dslots_out != nullptr;
  if (bank) {
    if (a.ws_h == nullptr || a.ws_G == nullptr || a.ws_coef == nullptr || a.ws_c0 == nullptr) return 1;
    screen_target_dot_kernel<<<dim3((a.T + kDotTile - 1) / kDotTile, a.M, a.B), 256, 0, st>>>(a);
    screen_bank_scalars_kernel<<<dim3(a.M, a.B), 32, 0, st>>>(a);
  }
  const int pack_blocks = (int)std::min<size_t>(148 * 8, ((size_t)a.B * a.T * J + 255) / 256);
  screen_pack_rows_kernel<<<pack_blocks, 256, 0, st>>>(a);
  screen_readout_kernel<true><<<dim3((a.T + kReadTile - 1) / kReadTile, a.B), 256, 0, st>>>(a);
  if (dispatch_jpl<BwdLauncher>(J, a, st) != 0) return 1;
  screen_query_grad_kernel<<<dim3((a.T + kReadTile - 1) / kReadTile, a.B), 256, 0, st>>>(a);
  if (bank)
    screen_bank_bwd_kernel<<<dim3((a.ds + 255) / 256, (a.T + kBankBwdTile - 1) / kBankBwdTile, a.B), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace rk
