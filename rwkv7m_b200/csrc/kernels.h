// Host-callable launchers of the sm_100a kernels.  Nothing here depends on
// PyTorch: arguments are raw device pointers plus a CUDA stream, so the same
// entry points serve the Python bindings and C callers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace rk {

// ---- WKV7 ---------------------------------------------------------------------
struct WkvArgs {
  int B, T, H, N;
  int interval;     // checkpoint interval in steps (training forward / backward)
  bool is_bf16;     // vector dtype: bf16 (true) or fp32 (false)
  const void *r, *w, *k, *v, *a, *b;   // [B,T,H,N]
  const float* s0;                      // [B,H,N,N]
  void* y;                              // [B,T,H,N]
  float* sT;                            // [B,H,N,N]
  void* sa;                             // [B,T,H,N]: fp32 for the scan kernels, bf16 for the chunked kernels (which only
                                        // ever use it as a bf16 tensor-core operand); nullptr = inference forward
  float* ckpt;                          // [ceil(T/interval), B*H, N, N]
  // backward only
  const void* dy;
  const float* dsT;                     // may be nullptr
  void *dr, *dw, *dk, *dv, *da, *db;
  float* ds0;
  // chunked backward only, all three or none: bf16 [B,T,H,N] gradients that reach r, k and v through another consumer of
  // the same tensors (the bonus term of the output normalisation); the kernel adds them to dr, dk, dv as it writes them
  const void *dr_add, *dk_add, *dv_add;
};
int wkv7_forward(const WkvArgs& p, cudaStream_t st);
int wkv7_backward(const WkvArgs& p, cudaStream_t st);
// Chunked tensor-core forward (head size 64, bf16, checkpoint interval 16 when aux is saved).
bool wkv7_chunk_supported(const WkvArgs& p);
int wkv7_chunk_forward(const WkvArgs& p, cudaStream_t st);
int wkv7_chunk_error(bool reset);   // non-zero after a bounded wait ran out inside the chunked forward kernel
// Chunked tensor-core backward: consumes the bf16 sa (= U) rows and the per-chunk states written by the chunked forward.
bool wkv7_chunk_bwd_supported(const WkvArgs& p);
int wkv7_chunk_backward(const WkvArgs& p, cudaStream_t st);
int wkv7_chunk_bwd_error(bool reset);
#ifdef RK_WKV_PROF
void wkv7_chunk_bwd_prof(long long* out, bool reset);
void wkv7_chunk_prof(long long* out, bool reset);   // per-phase clock counts of CTA 0 (profiling builds only)
#endif

// ---- optimizer ------------------------------------------------------------------
// out[0] += sum(g^2) over n elements (out must be zeroed by the caller).
void grad_norm_sq(const void* g, bool g_is_bf16, int64_t n, float* out, cudaStream_t st);

struct AdamWArgs {
  void* param; bool param_bf16;          // master parameters (fp32 or bf16)
  void* grad; bool grad_bf16;            // gradients; zeroed after use when zero_grad
  void* m; void* v; bool state_bf16;     // Adam moments
  void* shadow;                          // optional bf16 compute copy (nullptr = none)
  const float* norm_sq;                  // device scalar: global sum of squared grads
  int64_t begin, end;                    // element range to update
  int64_t n_decay, n_nodecay_end;        // group boundaries: [0,n_decay) decayed, [n_nodecay_end, ...) is w0 (x2)
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_norm, grad_scale;
  bool zero_grad;
};
void adamw_flat(const AdamWArgs& p, cudaStream_t st);

// ---- fused memory-bound kernels (bf16 activations, fp32 parameters) ---------------
void layernorm_fwd(const void* x, const float* w, const float* b, void* y, float* mean, float* rstd, int M, int C,
                   float eps, cudaStream_t st);
void layernorm_bwd(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                   float* dw_part, float* db_part, int parts, int M, int C, cudaStream_t st);
// Same with the gradient that arrives through the residual connection added to dx (dres: bf16 [M, C] or null).  Returns
// false, doing nothing, when dres is given but the width has no single-pass kernel.
bool layernorm_bwd_res(const void* dy, const void* x, const float* w, const float* mean, const float* rstd,
                       const void* dres, void* dx, float* dw_part, float* db_part, int parts, int M, int C,
                       cudaStream_t st);
int shift_mix_parts(int B, int T);
void shift_mix_fwd(const void* x, const float* prev, const float* mix, void* out, int K, int B, int T, int C,
                   cudaStream_t st);
// dout: K separate [B,T,C] gradient tensors
void shift_mix_bwd(const void* const* dout, const void* x, const float* prev, const float* mix, void* dx,
                   float* dprev, float* dmix_part, int K, int B, int T, int C, cudaStream_t st);
int row_parts(int M);
// out[g, c] = sum_p in[g * group_stride + p * row_stride + c]; cols and the strides are multiples of 4 floats
void partial_sum(const float* in, float* out, int groups, int parts, int cols, size_t row_stride, size_t group_stride,
                 cudaStream_t st);
// in: k_raw, v_raw, w_lora, a_lora, vg_lora, v_first (last two null on layer 0); par: w0, a0, v0, k_k, k_a;
// out: w, k_mod, v, neg_kk, kka
void tmix_pre_fwd(const void* const* in, const float* const* par, void* const* out, int M, int C, cudaStream_t st);
// gout: dw, dk_mod, dv, dneg_kk, dkka; gin: dk_raw, dv_raw, dw_lora, da_lora, dvg_lora, dv_first;
// gpar_part: dw0, da0, dv0, dk_k, dk_a as [row_parts(M), C]
void tmix_pre_bwd(const void* const* in, const float* const* par, const void* const* gout, void* const* gin,
                  float* const* gpar_part, int M, int C, cudaStream_t st);
// in: y, r, k, v, g; par: ln_w, ln_b, r_k
void gn_bonus_gate_fwd(const void* const* in, const float* const* par, void* out, int M, int C, float eps,
                       cudaStream_t st);
// gin: dy, dr, dk, dv, dg; gpar_part: dln_w, dln_b, dr_k as [row_parts(M), C]
void gn_bonus_gate_bwd(const void* const* in, const float* const* par, const void* dout, void* const* gin,
                       float* const* gpar_part, int M, int C, float eps, cudaStream_t st);
void relusq_bwd(const void* dh, const void* h, void* out, int64_t n, cudaStream_t st);
// Embedding row gather (bf16 output; table bf16 or fp32, C a multiple of 8) and the scatter-add of bf16 output-gradient
// rows into the fp32 table gradient.
void embedding_fwd(const int* ids, const void* table, bool table_bf16, void* out, int M, int C, int V, cudaStream_t st);
void embedding_bwd(const int* ids, const void* dout, float* grad, int M, int C, int V, cudaStream_t st);

// ---- loss ---------------------------------------------------------------------------
void ce_fwd(const void* logits, const int* targets, float* lse, float* maxv, int* argmax, float* nll, int rows, int V,
            cudaStream_t st);
// rows of per-tile statistics written by the kEpiCeStats GEMM epilogue -> lse, max, argmax, nll = lse - target logit
void ce_combine(const float* stats, int tiles, float* lse, float* maxv, int* argmax, float* nll, int rows, cudaStream_t st);
void ce_bwd(void* logits, const int* targets, const float* mask, const float* lse, const float* maxv,
            const int* argmax, const float* g_ce, const float* g_l2, int rows, int V, cudaStream_t st);

// ---- data-parallel optimizer step over symmetric memory -------------------------------
constexpr int kMaxRanks = 8;
struct DpPeers {
  void* grad[kMaxRanks];     // fp32 flat gradient buffer of every rank (peer-mapped)
  void* master[kMaxRanks];   // fp32 flat master parameters of every rank
  void* shadow[kMaxRanks];   // bf16 compute copy of every rank (entries may be null)
  void* aux[kMaxRanks];      // small scratch: barrier counters, norm partials, error word
  void* grad_mc;             // multicast addresses of the same buffers, or null without NVSwitch multicast
  void* master_mc;
  void* shadow_mc;
};
struct DpAdamW {
  int rank, world, parity;
  int64_t begin, end;              // owned element range in the flat buffers
  int64_t n_decay, n_nodecay_end;  // group boundaries
  int64_t master_bcast_from;       // new fp32 master values go to every rank from this index on; below it only the owner
                                   // keeps them (peers receive just the bf16 compute copy)
  float* m; float* v;              // Adam moments of the owned shard (local index = i - begin)
  float* norm_out;                 // receives the global gradient norm
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_norm;
};
// target = number of barriers issued so far on this buffer (same on every rank);
// publish_parity >= 0 also stores this rank's partial sum of squares to every peer first.
void dp_barrier(const DpPeers& peers, int rank, int world, uint32_t target, int publish_parity, cudaStream_t st);
void dp_reduce_shard(const DpPeers& peers, int rank, int world, int64_t begin, int64_t end, cudaStream_t st);
void dp_adamw_allgather(const DpPeers& peers, const DpAdamW& a, cudaStream_t st);
void dp_set_wait_limit_ms(double ms);   // limit of every device-side barrier wait (default 2000)
double dp_wait_limit_ms();
int dp_aux_error_word();
int dp_aux_words();

// ---- screening-memory slot scan -----------------------------------------------------------------------
struct ScreenScanArgs {
  int B, T, M, ds, dk, dv;
  // inputs (fp32)
  const float *q_r, *q_w;       // [B,T,dk]; q_w unused without write screening
  const float* delta_xh;        // [B,T,ds]
  const float* delta_slot;      // [M,ds]
  const float* slot_embed;      // [M,ds]
  const float* WT;              // [ds][J]  transposed concatenation of k_proj_r | v_proj | k_proj_w, J = dk + dv + dk
  const float* PD;              // [B,T,16,J] projections of every step's write target tanh(delta_xh + delta_slot)
                                //            (+ slot_embed Wkw^T on the write-key columns); rows >= M are zero
  const float* mu;              // [M] per-slot write rate
  const float *slots0, *ages0, *usage0;   // [B,M,ds], [B,M], [B,M]
  float tau_r, tau_w, eps, cap, write_rel_floor, usage_decay, age_ref, age_sigma;
  const float* tau_dev;         // [2] tau_r, tau_w on the device; when set it replaces the two host values above, so the
                                // learned thresholds never have to be read back to the host
  bool write_enabled, value_unit_norm, age_mask;
  bool leaky;                   // read relevance = (1 - alpha) trim_square + alpha sigmoid(gamma (sim - tau_r))
  float leaky_alpha, leaky_gamma;
  // forward outputs
  float* u_out;                 // [B,T,dv]
  float *slots_out, *ages_out, *usage_out;
  float* stats;                 // [9] running sums over batch rows and steps
  float* strength;              // [B,T,16] write strength of every step and slot (forward output, backward input)
  float* rel_c;                 // [B,T,16] read coefficient rel_r / |value| (forward output, backward input)
  float* rel_r;                 // [B,T,16] read relevance (forward only: statistics)
  float* saved_ages;            // [B,T,16]   ages before each step
  float* saved_P;               // [B,T,16,J] raw projections before each step (always written: the read-out kernel
                                //            forms u from it)
  // backward
  const float* du;              // [B,T,dv]
  const float* dslots_out;      // [B,M,ds] cotangent of the final bank, or nullptr (then d_delta_xh, d_delta_slot and
                                // d_slots0 are left untouched: the caller zeroes them)
  float *ws_h, *ws_G, *ws_coef; // [B,T,16] workspaces of the bank path (needed with dslots_out)
  float* ws_c0;                 // [B,16]
  float* ws_rows;               // [B,T,J] packed per-step rows [q_r | 0 or dz | q_w] (workspace of both directions)
  float *ws_a, *ws_b;           // [B,T,16] per-slot factors of the query cotangents (backward workspace)
  float *d_q_r, *d_q_w, *d_delta_xh;      // [B,T,dk], [B,T,dk], [B,T,ds]
  float* d_PD;                  // [B,T,16,J] cotangent of PD (rows of dead slots are not written)
  void* d_PD_bf16;              // when set, the same cotangent is written here in bf16 instead
  float* d_P0;                  // [B,16,J]   cotangent of the projections of the initial bank
  float* d_delta_slot;          // [M,ds]  accumulated with atomics (zeroed by the caller)
  float* d_slots0;              // [B,M,ds]
  float* d_mu;                  // [M]     atomics
  float* d_scalars;             // [2]     d tau_r, d tau_w (atomics)
};
bool screen_scan_supported(const ScreenScanArgs& a);
int screen_scan_forward(const ScreenScanArgs& a, cudaStream_t st);
int screen_scan_backward(const ScreenScanArgs& a, cudaStream_t st);
// D[b,t,m,d] = tanh(dxh[b,t,d] + dslot[m,d]) as bf16 [B,T,16,ds] (rows m >= M zero), and its backward: g_dxh[b,t,d] +=
// sum_m dD (1 - D^2), g_dslot[m,d] += the same term over (b, t) (atomics); D is recomputed
void screen_targets_forward(const float* dxh, const float* dslot, void* D, int B, int T, int M, int ds, cudaStream_t st);
void screen_targets_backward(const void* dD, const float* dxh, const float* dslot, float* g_dxh, float* g_dslot, int B, int T,
                             int M, int ds, cudaStream_t st);

// ---- tensor-parallel sequence collectives over symmetric memory ---------------------------
struct TpPeers {
  const void* buf[kMaxRanks];  // the same symmetric buffer on every rank (peer-mapped)
  const void* buf_mc;          // its multicast address, or null without NVSwitch multicast
  void* aux[kMaxRanks];        // scratch words: barrier counters and the error word
  int rank, world;
};
void tp_barrier(const TpPeers& peers, uint32_t target, cudaStream_t st);
// out[B, world*Tl, C] (local) <- buf_r[B, Tl, C] of every rank r
void tp_gather_seq(const TpPeers& peers, void* out, int B, int Tl, int C, cudaStream_t st);
// out[B, Tl, C] (local) <- residual + sum_r buf_r[B, world*Tl, C] restricted to this rank's time slice; residual may be null
void tp_reduce_scatter_add(const TpPeers& peers, const void* residual, void* out, int B, int Tl, int C, cudaStream_t st);
int tp_aux_error_word();
int tp_aux_words();

// ---- GEMM (tcgen05) -------------------------------------------------------------
enum GemmLayout { kGemmTN = 0, kGemmNN = 1, kGemmNT_wgrad = 2 };
enum GemmEpilogue {
  kEpiStoreBf16 = 0, kEpiReluSqBf16 = 1, kEpiStoreF32 = 2, kEpiAccumF32 = 3, kEpiScatterAddBf16 = 4,
  kEpiMulSqrt2Bf16 = 5,   // D = bf16(acc * 2 sqrt(aux)): backward of h = relu(.)^2 fused into the GEMM that produces dh
  kEpiAddBf16 = 6,        // D = bf16(acc + aux): residual add fused into the projection
  kEpiCeStats = 7         // no matrix output: per (row, 256-column tile) the cross-entropy statistics of the bf16-rounded
                          // result (maximum, sum of exp(x - maximum), arg-max column, logit of the row's target if it
                          // lies in the tile) as float4 into D [M, ceil(N / 256), 4]; aux = int32 targets [M].  Layout TN.
};
// Target of the kEpiScatterAddBf16 epilogue (GEMM -> reduce-scatter over time in one kernel): rows are [B, T] tokens,
// rank r owns tokens [r*Tl, (r+1)*Tl) of every batch row and receives them in out[r] laid out [B, Tl, N].
struct GemmScatter {
  void* out[kMaxRanks];
  int world, T, Tl, pad;
};
struct GemmArgs {
  // D[M,N] = A (M x K) * B (K x N) with fp32 accumulation.
  //  layout kGemmTN      : A stored [M,K] row-major, B stored [N,K] row-major      (y = x W^T)
  //  layout kGemmNN      : A stored [M,K] row-major, B stored [K,N] row-major      (dx = dy W)
  //  layout kGemmNT_wgrad: A stored [K,M] row-major, B stored [K,N] row-major      (dW = dy^T x)
  const void* A; const void* B; void* D;
  const void* aux;     // bf16 [M, N] second epilogue input (kEpiMulSqrt2Bf16, kEpiAddBf16), row pitch ldaux
  int ldaux;
  int act;             // kEpiStoreBf16: 0 = none, 1 = tanh, 2 = sigmoid applied to the result;
                       // kEpiMulSqrt2Bf16: factor 2 sqrt(aux) (0), 1 - aux^2 (1), aux (1 - aux) (2)
  int M, N, K;
  int lda, ldb, ldd;   // leading dimensions in elements of the stored matrices
  int layout, epilogue;
  int pair;            // non-zero: use the CTA-pair (cta_group::2) kernel when the shape allows
  int* error_flag;     // device int, set non-zero if a bounded wait ran out
  int decode_kernel;   // non-zero: shapes with M <= 64 (layout kGemmTN) take the swap-AB cluster split-K kernel
};
int gemm_bf16(const GemmArgs& p, cudaStream_t st);
// Up to four problems of layout kGemmTN with the bf16 store epilogue (each with its own activation) and the same M in one
// persistent launch; returns 1 when the set does not qualify (the caller then launches them one by one).
int gemm_bf16_group(const GemmArgs* ps, int count, cudaStream_t st);
// Tiled tensor map (128 bytes at `map`, 64-byte aligned) over a bf16 array of logical shape [d2][d1][d0], d0 contiguous,
// with byte strides stride1 / stride2 for the two outer dimensions; box = box0 x box1 x 1 elements, 128-byte swizzle,
// zero fill outside the array.  Used for operand tiles that land in shared memory in the tensor cores' canonical layout.
bool tma_encode_bf16_3d(void* map, const void* ptr, unsigned long long d0, unsigned long long d1, unsigned long long d2,
                        unsigned long long stride1, unsigned long long stride2, unsigned box0, unsigned box1);
bool gemm_decode_eligible(const GemmArgs& p);

}  // namespace rk
