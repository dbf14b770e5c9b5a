// PyTorch bindings: tensor checks, output allocation and stream plumbing around
// the launchers declared in kernels.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>

#include "kernels.h"

namespace {

using torch::Tensor;

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_vec(const Tensor& t, const Tensor& like, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(t.sizes() == like.sizes() && t.scalar_type() == like.scalar_type(), name, " shape/dtype mismatch");
}

rk::WkvArgs wkv_args(const Tensor& r, const Tensor& w, const Tensor& k, const Tensor& v, const Tensor& a,
                     const Tensor& b, const Tensor& s0, int64_t interval) {
  TORCH_CHECK(r.dim() == 4, "wkv7 vectors must be [B,T,H,N]");
  TORCH_CHECK(r.scalar_type() == at::kBFloat16 || r.scalar_type() == at::kFloat, "wkv7 vectors must be bf16 or fp32");
  check_vec(r, r, "r"); check_vec(w, r, "w"); check_vec(k, r, "k");
  check_vec(v, r, "v"); check_vec(a, r, "a"); check_vec(b, r, "b");
  const int64_t B = r.size(0), T = r.size(1), H = r.size(2), N = r.size(3);
  TORCH_CHECK(N == 16 || N == 32 || N == 64, "wkv7 head size must be 16, 32 or 64");
  TORCH_CHECK(T >= 1, "wkv7 needs at least one step");
  TORCH_CHECK(s0.is_cuda() && s0.is_contiguous() && s0.scalar_type() == at::kFloat, "initial state must be fp32");
  TORCH_CHECK(s0.dim() == 4 && s0.size(0) == B && s0.size(1) == H && s0.size(2) == N && s0.size(3) == N,
              "initial state must be [B,H,N,N]");
  rk::WkvArgs p{};
  p.B = (int)B; p.T = (int)T; p.H = (int)H; p.N = (int)N; p.interval = (int)interval;
  p.is_bf16 = r.scalar_type() == at::kBFloat16;
  p.r = r.data_ptr(); p.w = w.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.a = a.data_ptr(); p.b = b.data_ptr();
  p.s0 = s0.data_ptr<float>();
  return p;
}

std::vector<Tensor> wkv7_fwd(const Tensor& r, const Tensor& w, const Tensor& k, const Tensor& v, const Tensor& a,
                             const Tensor& b, const Tensor& s0, bool save, int64_t interval, bool chunked,
                             bool inplace_state) {
  c10::cuda::CUDAGuard guard(r.device());
  TORCH_CHECK(interval >= 1, "checkpoint interval must be positive");
  rk::WkvArgs p = wkv_args(r, w, k, v, a, b, s0, interval);
  Tensor y = torch::empty_like(r);
  // serving: the scan kernel holds a sequence's whole state in registers between its first load and its last store,
  // so the final state may overwrite the initial one (the returned state is then `s0` itself)
  const bool in_place = inplace_state && !save && !(chunked && rk::wkv7_chunk_supported(p));
  Tensor sT = in_place ? s0 : torch::empty_like(s0);
  Tensor sa, ckpt;
  p.y = y.data_ptr(); p.sT = sT.data_ptr<float>();
  if (save) p.sa = reinterpret_cast<void*>(1);   // placeholder: "training forward" for the support query below
  const bool use_chunk = chunked && rk::wkv7_chunk_supported(p);
  if (save) {
    auto f32 = r.options().dtype(at::kFloat);
    // the chunked kernels keep U only as a bf16 tensor-core operand, so they save it in bf16
    sa = torch::empty(r.sizes(), use_chunk ? r.options() : f32);
    const int64_t nck = (p.T + interval - 1) / interval;
    ckpt = torch::empty({nck, (int64_t)p.B * p.H, (int64_t)p.N, (int64_t)p.N}, f32);
    p.sa = sa.data_ptr(); p.ckpt = ckpt.data_ptr<float>();
  } else {
    sa = torch::empty({0}, r.options().dtype(at::kFloat));
    ckpt = sa;
  }
  if (use_chunk) {
    TORCH_CHECK(rk::wkv7_chunk_forward(p, stream()) == 0, "wkv7_chunk_forward: launch failed");
  } else {
    TORCH_CHECK(rk::wkv7_forward(p, stream()) == 0, "wkv7_forward: unsupported shape");
  }
  return {y, sT, sa, ckpt};
}

std::vector<Tensor> wkv7_bwd(const Tensor& r, const Tensor& w, const Tensor& k, const Tensor& v, const Tensor& a,
                             const Tensor& b, const Tensor& s0, const Tensor& sa, const Tensor& ckpt,
                             const Tensor& dy, const c10::optional<Tensor>& dsT, int64_t interval, bool chunked,
                             const c10::optional<std::vector<Tensor>>& add) {
  c10::cuda::CUDAGuard guard(r.device());
  rk::WkvArgs p = wkv_args(r, w, k, v, a, b, s0, interval);
  check_vec(dy, r, "dy");
  const bool use_chunk = chunked && rk::wkv7_chunk_bwd_supported(p);
  TORCH_CHECK(sa.is_contiguous() && sa.numel() == r.numel() &&
                  sa.scalar_type() == (use_chunk ? at::kBFloat16 : at::kFloat),
              "bad sa: the chunked backward takes the bf16 rows saved by the chunked forward, the scan backward fp32 rows");
  const int64_t nck = (p.T + interval - 1) / interval;
  TORCH_CHECK(ckpt.is_contiguous() && ckpt.scalar_type() == at::kFloat &&
                  ckpt.numel() == nck * p.B * p.H * p.N * p.N, "bad checkpoints");
  Tensor dr = torch::empty_like(r), dw = torch::empty_like(r), dk = torch::empty_like(r), dv = torch::empty_like(r),
         da = torch::empty_like(r), db = torch::empty_like(r);
  Tensor ds0 = torch::empty_like(s0);
  p.sa = sa.data_ptr(); p.ckpt = const_cast<float*>(ckpt.data_ptr<float>());
  p.dy = dy.data_ptr();
  Tensor dsT_c;
  if (dsT.has_value() && dsT->defined()) {
    dsT_c = dsT->contiguous().to(at::kFloat);
    TORCH_CHECK(dsT_c.sizes() == s0.sizes(), "dsT must match the state shape");
    p.dsT = dsT_c.data_ptr<float>();
  }
  p.dr = dr.data_ptr(); p.dw = dw.data_ptr(); p.dk = dk.data_ptr(); p.dv = dv.data_ptr();
  p.da = da.data_ptr(); p.db = db.data_ptr(); p.ds0 = ds0.data_ptr<float>();
  if (add.has_value() && !add->empty()) {
    TORCH_CHECK(use_chunk && add->size() == 3, "gradients to add go with the chunked backward, as (dr, dk, dv)");
    for (const Tensor& t : *add) check_vec(t, r, "add");
    p.dr_add = (*add)[0].data_ptr(); p.dk_add = (*add)[1].data_ptr(); p.dv_add = (*add)[2].data_ptr();
  }
  if (use_chunk) {
    TORCH_CHECK(rk::wkv7_chunk_backward(p, stream()) == 0, "wkv7_chunk_backward: launch failed");
  } else {
    TORCH_CHECK(rk::wkv7_backward(p, stream()) == 0, "wkv7_backward: unsupported shape");
  }
  return {dr, dw, dk, dv, da, db, ds0};
}

void grad_norm_sq(const Tensor& g, Tensor out) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_cuda() && g.is_contiguous() && out.is_cuda() && out.scalar_type() == at::kFloat);
  TORCH_CHECK(g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16);
  C10_CUDA_CHECK(cudaMemsetAsync(out.data_ptr<float>(), 0, sizeof(float), stream()));
  rk::grad_norm_sq(g.data_ptr(), g.scalar_type() == at::kBFloat16, g.numel(), out.data_ptr<float>(), stream());
}

void adamw_flat(Tensor param, Tensor grad, Tensor m, Tensor v, const c10::optional<Tensor>& shadow,
                const Tensor& norm_sq, int64_t n_decay, int64_t n_nodecay_end, int64_t begin, int64_t end,
                double lr, double beta1, double beta2, double eps, double weight_decay, double bc1, double bc2,
                double max_norm, double grad_scale, bool zero_grad) {
  c10::cuda::CUDAGuard guard(param.device());
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.is_contiguous() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16);
  };
  TORCH_CHECK(ok(param) && ok(grad) && ok(m) && ok(v), "adamw_flat: tensors must be contiguous CUDA fp32/bf16");
  TORCH_CHECK(m.scalar_type() == v.scalar_type(), "Adam moments must share a dtype");
  TORCH_CHECK(grad.numel() == param.numel() && m.numel() == param.numel() && v.numel() == param.numel());
  TORCH_CHECK(0 <= begin && begin <= end && end <= param.numel(), "adamw_flat: bad range");
  rk::AdamWArgs p{};
  p.param = param.data_ptr(); p.param_bf16 = param.scalar_type() == at::kBFloat16;
  p.grad = grad.data_ptr(); p.grad_bf16 = grad.scalar_type() == at::kBFloat16;
  p.m = m.data_ptr(); p.v = v.data_ptr(); p.state_bf16 = m.scalar_type() == at::kBFloat16;
  p.shadow = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    TORCH_CHECK(shadow->scalar_type() == at::kBFloat16 && shadow->numel() == param.numel() && shadow->is_contiguous());
    p.shadow = shadow->data_ptr();
  }
  p.norm_sq = norm_sq.data_ptr<float>();
  p.begin = begin; p.end = end; p.n_decay = n_decay; p.n_nodecay_end = n_nodecay_end;
  p.lr = (float)lr; p.beta1 = (float)beta1; p.beta2 = (float)beta2; p.eps = (float)eps;
  p.weight_decay = (float)weight_decay; p.bc1 = (float)bc1; p.bc2 = (float)bc2; p.max_norm = (float)max_norm;
  p.grad_scale = (float)grad_scale; p.zero_grad = zero_grad;
  rk::adamw_flat(p, stream());
}

Tensor& gemm_error_flag(const at::Device& dev) {
  static std::vector<Tensor> flags(64);
  Tensor& f = flags[dev.index() < 0 ? 0 : dev.index()];
  if (!f.defined()) f = torch::zeros({1}, torch::TensorOptions().dtype(at::kInt).device(dev));
  return f;
}

static bool g_decode_gemm = true;
void set_decode_gemm(bool on) { g_decode_gemm = on; }

// D = op(A) op(B); see kernels.h for the three layouts.  D must be preallocated.
void gemm(const Tensor& A, const Tensor& B, Tensor D, int64_t layout, int64_t epilogue, int64_t pair,
          const c10::optional<Tensor>& aux, int64_t act) {
  static const bool trace = [] { const char* e = getenv("RWKV7M_B200_TRACE"); return e != nullptr && e[0] == '1'; }();
  if (trace) { fprintf(stderr, "[gemm-bind] enter layout=%d epi=%d\n", (int)layout, (int)epilogue); fflush(stderr); }
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: A and B must be bf16");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2, "gemm: 2-D tensors required");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1, "gemm: rows must be contiguous");
  rk::GemmArgs p{};
  p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = D.data_ptr();
  p.lda = (int)A.stride(0); p.ldb = (int)B.stride(0); p.ldd = (int)D.stride(0);
  p.layout = (int)layout; p.epilogue = (int)epilogue; p.pair = (int)pair;
  TORCH_CHECK(act >= 0 && act <= 2 && (act == 0 || epilogue == rk::kEpiStoreBf16 || epilogue == rk::kEpiMulSqrt2Bf16),
              "gemm: an activation selector goes with the bf16 store or the derivative-factor epilogue only");
  p.act = (int)act;
  if (layout == rk::kGemmTN) {
    p.M = (int)A.size(0); p.K = (int)A.size(1); p.N = (int)B.size(0);
    TORCH_CHECK(B.size(1) == p.K, "gemm TN: K mismatch");
  } else if (layout == rk::kGemmNN) {
    p.M = (int)A.size(0); p.K = (int)A.size(1); p.N = (int)B.size(1);
    TORCH_CHECK(B.size(0) == p.K, "gemm NN: K mismatch");
  } else {
    p.K = (int)A.size(0); p.M = (int)A.size(1); p.N = (int)B.size(1);
    TORCH_CHECK(B.size(0) == p.K, "gemm wgrad: K mismatch");
  }
  TORCH_CHECK(D.size(0) == p.M && D.size(1) == p.N, "gemm: output shape mismatch");
  const bool two_input = epilogue == rk::kEpiMulSqrt2Bf16 || epilogue == rk::kEpiAddBf16;
  if (two_input) {
    TORCH_CHECK(aux.has_value() && aux->defined(), "gemm: this epilogue needs a second input");
    TORCH_CHECK(aux->is_cuda() && aux->scalar_type() == at::kBFloat16 && aux->dim() == 2 && aux->stride(1) == 1 &&
                    aux->size(0) == D.size(0) && aux->size(1) == D.size(1),
                "gemm: the second epilogue input must be a bf16 matrix of the output's shape");
    p.aux = aux->data_ptr();
    p.ldaux = (int)aux->stride(0);
  }
  const bool out_bf16 = epilogue == rk::kEpiStoreBf16 || epilogue == rk::kEpiReluSqBf16 || two_input;
  TORCH_CHECK(D.scalar_type() == (out_bf16 ? at::kBFloat16 : at::kFloat), "gemm: output dtype mismatch");
  if (trace) { fprintf(stderr, "[gemm-bind] checks ok\n"); fflush(stderr); }
  p.error_flag = gemm_error_flag(A.device()).data_ptr<int>();
  if (trace) { fprintf(stderr, "[gemm-bind] flag ok\n"); fflush(stderr); }
  p.decode_kernel = g_decode_gemm ? 1 : 0;
  const int rc = rk::gemm_bf16(p, stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 launch failed with code ", rc);
}

// Head GEMM whose epilogue keeps only cross-entropy statistics: logits = A [M,K] B [V,K]^T are never written.  Returns
// lse, max, argmax, nll per row (the same four tensors as ce_fwd on stored bf16 logits).
std::vector<Tensor> gemm_ce_stats(const Tensor& A, const Tensor& B, const Tensor& targets, int64_t pair) {
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  A.dim() == 2 && B.dim() == 2 && A.stride(1) == 1 && B.stride(1) == 1 && A.size(1) == B.size(1),
              "gemm_ce_stats: bf16 row-major A [M,K] and B [V,K]");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kInt && targets.is_contiguous() && targets.numel() == A.size(0),
              "gemm_ce_stats: int32 targets, one per row");
  const int64_t M = A.size(0), V = B.size(0), tiles = (V + 255) / 256;
  auto f32 = A.options().dtype(at::kFloat);
  Tensor stats = torch::empty({M, tiles, 4}, f32);
  rk::GemmArgs p{};
  p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = stats.data_ptr(); p.aux = targets.data_ptr();
  p.lda = (int)A.stride(0); p.ldb = (int)B.stride(0); p.ldd = (int)(tiles * 4);
  p.M = (int)M; p.N = (int)V; p.K = (int)A.size(1);
  p.layout = rk::kGemmTN; p.epilogue = rk::kEpiCeStats; p.pair = (int)pair;
  p.error_flag = gemm_error_flag(A.device()).data_ptr<int>();
  const int rc = rk::gemm_bf16(p, stream());
  TORCH_CHECK(rc == 0, "gemm_ce_stats launch failed with code ", rc);
  Tensor lse = torch::empty({M}, f32), maxv = torch::empty({M}, f32), nll = torch::empty({M}, f32);
  Tensor argmax = torch::empty({M}, A.options().dtype(at::kInt));
  rk::ce_combine(stats.data_ptr<float>(), (int)tiles, lse.data_ptr<float>(), maxv.data_ptr<float>(), argmax.data_ptr<int>(),
                 nll.data_ptr<float>(), (int)M, stream());
  return {lse, maxv, argmax, nll};
}

// Up to four y_i = act_i(A_i B_i^T) with the same number of rows in one launch (bf16 in, bf16 out).  Returns false, having
// launched nothing, when the set does not qualify; the caller then issues the products one by one.
bool gemm_group(const std::vector<Tensor>& As, const std::vector<Tensor>& Bs, std::vector<Tensor> Ds,
                const std::vector<int64_t>& acts) {
  const size_t n = As.size();
  TORCH_CHECK(n >= 1 && n <= 4 && Bs.size() == n && Ds.size() == n && acts.size() == n, "gemm_group: 1 to 4 problems");
  c10::cuda::CUDAGuard guard(As[0].device());
  rk::GemmArgs ps[4];
  for (size_t i = 0; i < n; ++i) {
    const Tensor &A = As[i], &B = Bs[i];
    Tensor& D = Ds[i];
    TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm_group: CUDA tensors required");
    TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 && D.scalar_type() == at::kBFloat16,
                "gemm_group: bf16 tensors required");
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2 && A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1,
                "gemm_group: 2-D tensors with contiguous rows required");
    TORCH_CHECK(B.size(1) == A.size(1) && D.size(0) == A.size(0) && D.size(1) == B.size(0), "gemm_group: shape mismatch");
    TORCH_CHECK(acts[i] >= 0 && acts[i] <= 2, "gemm_group: activation selector out of range");
    rk::GemmArgs p{};
    p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = D.data_ptr();
    p.lda = (int)A.stride(0); p.ldb = (int)B.stride(0); p.ldd = (int)D.stride(0);
    p.M = (int)A.size(0); p.K = (int)A.size(1); p.N = (int)B.size(0);
    p.layout = rk::kGemmTN; p.epilogue = rk::kEpiStoreBf16; p.act = (int)acts[i];
    p.error_flag = gemm_error_flag(A.device()).data_ptr<int>();
    ps[i] = p;
  }
  const int rc = rk::gemm_bf16_group(ps, (int)n, stream());
  if (rc == 1) return false;
  TORCH_CHECK(rc == 0, "gemm_bf16_group launch failed with code ", rc);
  return true;
}

int64_t gemm_error(const Tensor& like) {
  return gemm_error_flag(like.device()).item<int>();
}

void gemm_error_reset(const Tensor& like) { gemm_error_flag(like.device()).zero_(); }

// ---- fused memory-bound kernels -------------------------------------------------------

void check_act(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kBFloat16, name,
              " must be a contiguous bf16 CUDA tensor");
}
void check_par(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kFloat && t.numel() == n, name,
              " must be a contiguous fp32 CUDA tensor with ", n, " elements");
}

std::vector<Tensor> layernorm_fwd(const Tensor& x, const Tensor& w, const Tensor& b, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  check_act(x, "x");
  const int64_t C = x.size(-1), M = x.numel() / C;
  TORCH_CHECK(C % 2 == 0, "layernorm: width must be even");
  check_par(w, C, "weight"); check_par(b, C, "bias");
  Tensor y = torch::empty_like(x);
  auto f32 = x.options().dtype(at::kFloat);
  Tensor mean = torch::empty({M}, f32), rstd = torch::empty({M}, f32);
  rk::layernorm_fwd(x.data_ptr(), w.data_ptr<float>(), b.data_ptr<float>(), y.data_ptr(), mean.data_ptr<float>(),
                    rstd.data_ptr<float>(), (int)M, (int)C, (float)eps, stream());
  return {y, mean, rstd};
}

// Sum over the partial-row axis of a contiguous fp32 [groups, parts, cols] tensor with this extension's fixed-order kernel.
static Tensor sum_parts(const Tensor& t) {
  TORCH_CHECK(t.dim() == 3 && t.is_contiguous() && t.scalar_type() == at::kFloat);
  const int64_t G = t.size(0), P = t.size(1), C = t.size(2);
  if (C % 4 != 0) return t.sum(1);
  Tensor out = torch::empty({G, C}, t.options());
  rk::partial_sum(t.data_ptr<float>(), out.data_ptr<float>(), (int)G, (int)P, (int)C, (size_t)C, (size_t)(P * C), stream());
  return out;
}

std::vector<Tensor> layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& mean,
                                  const Tensor& rstd, const c10::optional<Tensor>& dres) {
  c10::cuda::CUDAGuard guard(x.device());
  check_act(dy, "dy"); check_act(x, "x");
  const int64_t C = x.size(-1), M = x.numel() / C;
  check_par(w, C, "weight"); check_par(mean, M, "mean"); check_par(rstd, M, "rstd");
  TORCH_CHECK(dy.numel() == x.numel());
  Tensor dx = torch::empty_like(x);
  // blocks of the backward grid (one row of partial weight / bias gradients each): several resident blocks per SM keep
  // enough 16-byte loads in flight for the one-pass kernel
  int parts = (int)std::min<int64_t>(148 * 6, std::max<int64_t>(1, M / 16));
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dwb = torch::empty({2, parts, C}, f32);
  Tensor dwp = dwb[0], dbp = dwb[1];
  const bool has_res = dres.has_value() && dres->defined();
  if (has_res) { check_act(*dres, "dres"); TORCH_CHECK(dres->numel() == x.numel()); }
  const bool fused = rk::layernorm_bwd_res(dy.data_ptr(), x.data_ptr(), w.data_ptr<float>(), mean.data_ptr<float>(),
                                           rstd.data_ptr<float>(), has_res ? dres->data_ptr() : nullptr, dx.data_ptr(),
                                           dwp.data_ptr<float>(), dbp.data_ptr<float>(), parts, (int)M, (int)C, stream());
  if (!fused) {   // width without a single-pass kernel: plain backward, then add
    rk::layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                      dx.data_ptr(), dwp.data_ptr<float>(), dbp.data_ptr<float>(), parts, (int)M, (int)C, stream());
    dx.add_(*dres);
  }
  Tensor sums = sum_parts(dwb);
  return {dx, sums[0], sums[1]};
}

Tensor shift_mix_fwd(const Tensor& x, const Tensor& prev, const Tensor& mix) {
  c10::cuda::CUDAGuard guard(x.device());
  check_act(x, "x");
  TORCH_CHECK(x.dim() == 3, "shift_mix: x must be [B,T,C]");
  const int64_t B = x.size(0), T = x.size(1), C = x.size(2), K = mix.size(0);
  TORCH_CHECK(K == 1 || K == 6, "shift_mix supports 1 or 6 mixes");
  TORCH_CHECK(C % 2 == 0);
  check_par(prev, B * C, "prev"); check_par(mix, K * C, "mix");
  Tensor out = torch::empty({K, B, T, C}, x.options());
  rk::shift_mix_fwd(x.data_ptr(), prev.data_ptr<float>(), mix.data_ptr<float>(), out.data_ptr(), (int)K, (int)B,
                    (int)T, (int)C, stream());
  return out;
}

std::vector<Tensor> shift_mix_bwd(const std::vector<Tensor>& dout, const Tensor& x, const Tensor& prev,
                                  const Tensor& mix) {
  c10::cuda::CUDAGuard guard(x.device());
  check_act(x, "x");
  const int64_t B = x.size(0), T = x.size(1), C = x.size(2), K = mix.size(0);
  TORCH_CHECK((int64_t)dout.size() == K, "shift_mix_bwd: one gradient per mix");
  const void* gp[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int64_t z = 0; z < K; ++z) {
    check_act(dout[z], "dout");
    TORCH_CHECK(dout[z].numel() == x.numel(), "shift_mix_bwd: gradient shape mismatch");
    gp[z] = dout[z].data_ptr();
  }
  check_par(prev, B * C, "prev"); check_par(mix, K * C, "mix");
  Tensor dx = torch::empty_like(x);
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dprev = torch::empty({B, C}, f32);
  const int parts = rk::shift_mix_parts((int)B, (int)T);
  Tensor dmp = torch::empty({parts, K, C}, f32);
  rk::shift_mix_bwd(gp, x.data_ptr(), prev.data_ptr<float>(), mix.data_ptr<float>(), dx.data_ptr(),
                    dprev.data_ptr<float>(), dmp.data_ptr<float>(), (int)K, (int)B, (int)T, (int)C, stream());
  return {dx, dprev, sum_parts(dmp.view({1, parts, K * C})).view({K, C})};
}

// tmix_pre: acts = [k_raw, v_raw, w_lora, a_lora] (+ [vg_lora, v_first] past layer 0); pars = [w0, a0, k_k, k_a] (+ [v0])
Tensor tmix_pre_fwd(const std::vector<Tensor>& acts, const std::vector<Tensor>& pars) {
  TORCH_CHECK(acts.size() == 4 || acts.size() == 6, "tmix_pre: 4 or 6 activations");
  const bool has_v = acts.size() == 6;
  TORCH_CHECK(pars.size() == (has_v ? 5u : 4u), "tmix_pre: parameter count mismatch");
  c10::cuda::CUDAGuard guard(acts[0].device());
  const int64_t C = acts[0].size(-1), M = acts[0].numel() / C;
  TORCH_CHECK(C % 64 == 0, "tmix_pre needs head size 64");
  for (auto& t : acts) { check_act(t, "activation"); TORCH_CHECK(t.numel() == M * C); }
  for (auto& t : pars) check_par(t, C, "parameter");
  Tensor out = torch::empty({5, M, C}, acts[0].options());
  const void* in[6] = {acts[0].data_ptr(), acts[1].data_ptr(), acts[2].data_ptr(), acts[3].data_ptr(),
                       has_v ? acts[4].data_ptr() : nullptr, has_v ? acts[5].data_ptr() : nullptr};
  const float* par[5] = {pars[0].data_ptr<float>(), pars[1].data_ptr<float>(),
                         has_v ? pars[4].data_ptr<float>() : nullptr, pars[2].data_ptr<float>(),
                         pars[3].data_ptr<float>()};
  char* o = (char*)out.data_ptr();
  const size_t plane = (size_t)M * C * 2;
  void* outs[5] = {o, o + plane, o + 2 * plane, o + 3 * plane, o + 4 * plane};
  rk::tmix_pre_fwd(in, par, outs, (int)M, (int)C, stream());
  return out;
}

// gouts = five [M,C] gradients (dw, dk_mod, dv, dneg_kk, dkka).
// Returns {gin [6 or 4 planes: dk_raw, dv_raw, dw_lora, da_lora, (dvg_lora, dv_first)], dw0, da0, dk_k, dk_a, (dv0)}
std::vector<Tensor> tmix_pre_bwd(const std::vector<Tensor>& acts, const std::vector<Tensor>& pars,
                                 const std::vector<Tensor>& gouts) {
  const bool has_v = acts.size() == 6;
  c10::cuda::CUDAGuard guard(acts[0].device());
  const int64_t C = acts[0].size(-1), M = acts[0].numel() / C;
  for (auto& t : acts) check_act(t, "activation");
  for (auto& t : pars) check_par(t, C, "parameter");
  TORCH_CHECK(gouts.size() == 5, "tmix_pre_bwd: five output gradients");
  for (auto& t : gouts) { check_act(t, "grad output"); TORCH_CHECK(t.numel() == M * C); }
  const int nplanes = has_v ? 6 : 4;
  Tensor gin = torch::empty({nplanes, M, C}, acts[0].options());
  const int parts = rk::row_parts((int)M);
  auto f32 = acts[0].options().dtype(at::kFloat);
  Tensor gp = torch::empty({5, parts, C}, f32);
  const void* in[6] = {acts[0].data_ptr(), acts[1].data_ptr(), acts[2].data_ptr(), acts[3].data_ptr(),
                       has_v ? acts[4].data_ptr() : nullptr, has_v ? acts[5].data_ptr() : nullptr};
  const float* par[5] = {pars[0].data_ptr<float>(), pars[1].data_ptr<float>(),
                         has_v ? pars[4].data_ptr<float>() : nullptr, pars[2].data_ptr<float>(),
                         pars[3].data_ptr<float>()};
  const size_t plane = (size_t)M * C * 2;
  const void* gout[5] = {gouts[0].data_ptr(), gouts[1].data_ptr(), gouts[2].data_ptr(), gouts[3].data_ptr(),
                         gouts[4].data_ptr()};
  char* gi = (char*)gin.data_ptr();
  void* gins[6] = {gi, gi + plane, gi + 2 * plane, gi + 3 * plane, has_v ? gi + 4 * plane : nullptr,
                   has_v ? gi + 5 * plane : nullptr};
  float* gpp = gp.data_ptr<float>();
  const size_t pp = (size_t)parts * C;
  // kernel order: dw0, da0, dv0, dk_k, dk_a
  float* gpar[5] = {gpp, gpp + pp, gpp + 4 * pp, gpp + 2 * pp, gpp + 3 * pp};
  rk::tmix_pre_bwd(in, par, gout, gins, gpar, (int)M, (int)C, stream());
  Tensor sums = sum_parts(gp);  // [5, C]: dw0, da0, dk_k, dk_a, dv0
  std::vector<Tensor> out = {gin, sums[0], sums[1], sums[2], sums[3]};
  if (has_v) out.push_back(sums[4]);
  return out;
}

Tensor gn_bonus_gate_fwd(const std::vector<Tensor>& acts, const std::vector<Tensor>& pars, double eps) {
  TORCH_CHECK(acts.size() == 5 && pars.size() == 3);
  c10::cuda::CUDAGuard guard(acts[0].device());
  const int64_t C = acts[0].size(-1), M = acts[0].numel() / C;
  TORCH_CHECK(C % 64 == 0, "gn_bonus_gate needs head size 64");
  for (auto& t : acts) { check_act(t, "activation"); TORCH_CHECK(t.numel() == M * C); }
  for (auto& t : pars) check_par(t, C, "parameter");
  Tensor out = torch::empty_like(acts[0]);
  const void* in[5] = {acts[0].data_ptr(), acts[1].data_ptr(), acts[2].data_ptr(), acts[3].data_ptr(), acts[4].data_ptr()};
  const float* par[3] = {pars[0].data_ptr<float>(), pars[1].data_ptr<float>(), pars[2].data_ptr<float>()};
  rk::gn_bonus_gate_fwd(in, par, out.data_ptr(), (int)M, (int)C, (float)eps, stream());
  return out;
}

// Returns {gin [5,M,C]: dy, dr, dk, dv, dg; dln_w, dln_b, dr_k}
std::vector<Tensor> gn_bonus_gate_bwd(const std::vector<Tensor>& acts, const std::vector<Tensor>& pars,
                                      const Tensor& dout, double eps) {
  c10::cuda::CUDAGuard guard(acts[0].device());
  const int64_t C = acts[0].size(-1), M = acts[0].numel() / C;
  for (auto& t : acts) check_act(t, "activation");
  for (auto& t : pars) check_par(t, C, "parameter");
  check_act(dout, "dout");
  TORCH_CHECK(dout.numel() == M * C);
  Tensor gin = torch::empty({5, M, C}, acts[0].options());
  const int parts = rk::row_parts((int)M);
  Tensor gp = torch::empty({3, parts, C}, acts[0].options().dtype(at::kFloat));
  const void* in[5] = {acts[0].data_ptr(), acts[1].data_ptr(), acts[2].data_ptr(), acts[3].data_ptr(), acts[4].data_ptr()};
  const float* par[3] = {pars[0].data_ptr<float>(), pars[1].data_ptr<float>(), pars[2].data_ptr<float>()};
  const size_t plane = (size_t)M * C * 2;
  char* gi = (char*)gin.data_ptr();
  void* gins[5] = {gi, gi + plane, gi + 2 * plane, gi + 3 * plane, gi + 4 * plane};
  float* gpp = gp.data_ptr<float>();
  const size_t pp = (size_t)parts * C;
  float* gpar[3] = {gpp, gpp + pp, gpp + 2 * pp};
  rk::gn_bonus_gate_bwd(in, par, dout.data_ptr(), gins, gpar, (int)M, (int)C, (float)eps, stream());
  Tensor sums = sum_parts(gp);
  return {gin, sums[0], sums[1], sums[2]};
}

Tensor relusq_bwd(const Tensor& dh, const Tensor& h) {
  c10::cuda::CUDAGuard guard(dh.device());
  check_act(dh, "dh"); check_act(h, "h");
  TORCH_CHECK(dh.numel() == h.numel() && dh.numel() % 8 == 0);
  Tensor out = torch::empty_like(dh);
  rk::relusq_bwd(dh.data_ptr(), h.data_ptr(), out.data_ptr(), dh.numel(), stream());
  return out;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(ids.is_cuda() && ids.is_contiguous() && ids.scalar_type() == at::kInt, "ids must be contiguous int32 CUDA");
  TORCH_CHECK(table.is_cuda() && table.is_contiguous() && table.dim() == 2 &&
                  (table.scalar_type() == at::kBFloat16 || table.scalar_type() == at::kFloat),
              "embedding table must be a contiguous bf16 or fp32 matrix");
  const int64_t M = ids.numel(), V = table.size(0), C = table.size(1);
  TORCH_CHECK(C % 8 == 0 && M < ((int64_t)1 << 31), "embedding width must be a multiple of 8");
  auto shape = ids.sizes().vec();
  shape.push_back(C);
  Tensor out = torch::empty(shape, table.options().dtype(at::kBFloat16));
  if (M > 0)
    rk::embedding_fwd(ids.data_ptr<int>(), table.data_ptr(), table.scalar_type() == at::kBFloat16, out.data_ptr(), (int)M,
                      (int)C, (int)V, stream());
  return out;
}

void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor grad) {
  c10::cuda::CUDAGuard guard(grad.device());
  TORCH_CHECK(ids.is_cuda() && ids.is_contiguous() && ids.scalar_type() == at::kInt, "ids must be contiguous int32 CUDA");
  check_act(dout, "dout");
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.scalar_type() == at::kFloat && grad.dim() == 2,
              "table gradient must be a contiguous fp32 matrix");
  const int64_t M = ids.numel(), V = grad.size(0), C = grad.size(1);
  TORCH_CHECK(C % 8 == 0 && dout.numel() == M * C, "gradient rows do not match the ids");
  if (M > 0) rk::embedding_bwd(ids.data_ptr<int>(), dout.data_ptr(), grad.data_ptr<float>(), (int)M, (int)C, (int)V, stream());
}

std::vector<Tensor> ce_fwd(const Tensor& logits, const Tensor& targets) {
  c10::cuda::CUDAGuard guard(logits.device());
  check_act(logits, "logits");
  TORCH_CHECK(logits.dim() == 2);
  const int64_t M = logits.size(0), V = logits.size(1);
  TORCH_CHECK(V % 8 == 0, "vocabulary must be a multiple of 8");
  TORCH_CHECK(targets.is_cuda() && targets.is_contiguous() && targets.scalar_type() == at::kInt && targets.numel() == M);
  auto f32 = logits.options().dtype(at::kFloat);
  Tensor lse = torch::empty({M}, f32), maxv = torch::empty({M}, f32), nll = torch::empty({M}, f32);
  Tensor am = torch::empty({M}, logits.options().dtype(at::kInt));
  rk::ce_fwd(logits.data_ptr(), targets.data_ptr<int>(), lse.data_ptr<float>(), maxv.data_ptr<float>(),
             am.data_ptr<int>(), nll.data_ptr<float>(), (int)M, (int)V, stream());
  return {lse, maxv, am, nll};
}

void ce_bwd(Tensor logits, const Tensor& targets, const c10::optional<Tensor>& mask, const Tensor& lse,
            const Tensor& maxv, const Tensor& am, const Tensor& g_ce, const Tensor& g_l2) {
  c10::cuda::CUDAGuard guard(logits.device());
  check_act(logits, "logits");
  const int64_t M = logits.size(0), V = logits.size(1);
  check_par(lse, M, "lse"); check_par(maxv, M, "max"); check_par(g_ce, 1, "g_ce"); check_par(g_l2, 1, "g_l2");
  TORCH_CHECK(targets.scalar_type() == at::kInt && targets.numel() == M && am.scalar_type() == at::kInt);
  const float* mp = nullptr;
  if (mask.has_value() && mask->defined()) { check_par(*mask, M, "mask"); mp = mask->data_ptr<float>(); }
  rk::ce_bwd(logits.data_ptr(), targets.data_ptr<int>(), mp, lse.data_ptr<float>(), maxv.data_ptr<float>(),
             am.data_ptr<int>(), g_ce.data_ptr<float>(), g_l2.data_ptr<float>(), (int)M, (int)V, stream());
}

// ---- data-parallel optimizer step -------------------------------------------------------

rk::DpPeers make_peers(const std::vector<int64_t>& grad, const std::vector<int64_t>& master,
                       const std::vector<int64_t>& shadow, const std::vector<int64_t>& aux, int64_t grad_mc,
                       int64_t master_mc, int64_t shadow_mc) {
  const size_t world = grad.size();
  TORCH_CHECK(world >= 1 && world <= (size_t)rk::kMaxRanks, "data-parallel world size must be 1..", rk::kMaxRanks);
  TORCH_CHECK(master.size() == world && aux.size() == world && (shadow.empty() || shadow.size() == world));
  rk::DpPeers p{};
  for (size_t i = 0; i < world; ++i) {
    p.grad[i] = reinterpret_cast<void*>(grad[i]);
    p.master[i] = reinterpret_cast<void*>(master[i]);
    p.shadow[i] = shadow.empty() ? nullptr : reinterpret_cast<void*>(shadow[i]);
    p.aux[i] = reinterpret_cast<void*>(aux[i]);
  }
  p.grad_mc = reinterpret_cast<void*>(grad_mc);
  p.master_mc = reinterpret_cast<void*>(master_mc);
  p.shadow_mc = reinterpret_cast<void*>(shadow_mc);
  return p;
}

// One optimizer step.  Pointer lists are raw device addresses of the symmetric buffers of every rank.
// Returns the number of barriers issued so far.
// Optional per-kernel timing of the fused data-parallel step (RWKV7M_B200_DP_TIMING=1): CUDA events around the five
// launches of the most recent step, read back with dp_step_timings().
struct DpTiming {
  bool on = false, init = false, valid = false;
  cudaEvent_t ev[6];
};
static DpTiming& dp_timing() {
  static DpTiming t;
  if (!t.init) {
    t.init = true;
    const char* e = getenv("RWKV7M_B200_DP_TIMING");
    t.on = e != nullptr && e[0] == '1';
    if (t.on) for (auto& ev : t.ev) cudaEventCreate(&ev);
  }
  return t;
}
std::vector<double> dp_step_timings() {
  DpTiming& t = dp_timing();
  std::vector<double> out;
  if (!t.on || !t.valid) return out;
  cudaEventSynchronize(t.ev[5]);
  for (int i = 0; i < 5; ++i) { float ms = 0.f; cudaEventElapsedTime(&ms, t.ev[i], t.ev[i + 1]); out.push_back(ms); }
  return out;
}

int64_t dp_step(const std::vector<int64_t>& grad, const std::vector<int64_t>& master, const std::vector<int64_t>& shadow,
                const std::vector<int64_t>& aux, int64_t grad_mc, int64_t master_mc, int64_t shadow_mc, Tensor m,
                Tensor v, Tensor norm_out, int64_t rank, int64_t begin, int64_t end, int64_t n_decay,
                int64_t n_nodecay_end, int64_t master_bcast_from, int64_t barriers_done, int64_t step_index, double lr, double beta1, double beta2,
                double eps, double weight_decay, double bc1, double bc2, double max_norm) {
  c10::cuda::CUDAGuard guard(m.device());
  const int world = (int)grad.size();
  TORCH_CHECK(m.is_cuda() && m.is_contiguous() && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(m.numel() == end - begin && v.numel() == end - begin, "moment shards must match the owned range");
  TORCH_CHECK(begin % 4 == 0 && end % 4 == 0, "shard bounds must be multiples of 4 elements");
  const bool has_mc = grad_mc != 0 && master_mc != 0;
  rk::DpPeers peers = make_peers(grad, master, shadow, aux, has_mc ? grad_mc : 0, has_mc ? master_mc : 0,
                                 has_mc ? shadow_mc : 0);
  cudaStream_t st = stream();
  uint32_t b = (uint32_t)barriers_done;
  const int parity = (int)(step_index & 1);
  DpTiming& tm = dp_timing();
  auto mark = [&](int i) { if (tm.on) cudaEventRecord(tm.ev[i], st); };
  mark(0);
  rk::dp_barrier(peers, (int)rank, world, ++b, -1, st);
  mark(1);
  rk::dp_reduce_shard(peers, (int)rank, world, begin, end, st);
  mark(2);
  rk::dp_barrier(peers, (int)rank, world, ++b, parity, st);
  mark(3);
  rk::DpAdamW a{};
  a.rank = (int)rank; a.world = world; a.parity = parity; a.begin = begin; a.end = end;
  a.n_decay = n_decay; a.n_nodecay_end = n_nodecay_end;
  // without a bf16 compute copy the forward reads the master values, so every rank needs all of them
  a.master_bcast_from = shadow.empty() ? 0 : master_bcast_from;
  TORCH_CHECK(a.master_bcast_from % 4 == 0, "master_bcast_from must be a multiple of 4 elements");
  a.m = m.data_ptr<float>(); a.v = v.data_ptr<float>(); a.norm_out = norm_out.data_ptr<float>();
  a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2; a.eps = (float)eps;
  a.weight_decay = (float)weight_decay; a.bc1 = (float)bc1; a.bc2 = (float)bc2; a.max_norm = (float)max_norm;
  rk::dp_adamw_allgather(peers, a, st);
  mark(4);
  rk::dp_barrier(peers, (int)rank, world, ++b, -1, st);
  mark(5);
  tm.valid = tm.on;
  return (int64_t)b;
}

// ---- ZeRO-3 building blocks: the same kernels as the fused data-parallel step, launched unit by unit ----------------------
static rk::DpPeers aux_only_peers(const std::vector<int64_t>& aux) {
  TORCH_CHECK(aux.size() >= 1 && aux.size() <= (size_t)rk::kMaxRanks, "bad peer list");
  rk::DpPeers p{};
  for (size_t i = 0; i < aux.size(); ++i) p.aux[i] = reinterpret_cast<void*>(aux[i]);
  return p;
}

// Device barrier over the symmetric scratch words; target = number of barriers issued so far + 1 (same on every rank).
void dp_barrier_only(const std::vector<int64_t>& aux, int64_t rank, int64_t target, const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  rk::DpPeers p = aux_only_peers(aux);
  rk::dp_barrier(p, (int)rank, (int)aux.size(), (uint32_t)target, -1, stream());
}

// out[r * n + i] = src[r][i] for every rank r (bf16, n a multiple of 8): all-gather of parameter pieces by peer loads.
void zero_gather(const std::vector<int64_t>& src, Tensor out, int64_t n) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 && n % 8 == 0 && n > 0);
  TORCH_CHECK(out.numel() >= n * (int64_t)src.size() && n < (int64_t)1 << 31, "gather output too small");
  TORCH_CHECK(src.size() >= 1 && src.size() <= (size_t)rk::kMaxRanks, "bad peer list");
  rk::TpPeers p{};
  for (size_t i = 0; i < src.size(); ++i) p.buf[i] = reinterpret_cast<const void*>(src[i]);
  p.world = (int)src.size();
  rk::tp_gather_seq(p, out.data_ptr(), 1, 1, (int)n, stream());
}

// Sum elements [begin, end) of every rank's fp32 gradient buffer into this rank's own buffer (multimem.ld_reduce when a
// multicast address is given, else peer loads).  The caller frames it with barriers.
void zero_reduce(const std::vector<int64_t>& grad, const std::vector<int64_t>& aux, int64_t grad_mc, int64_t rank,
                 int64_t begin, int64_t end, const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  TORCH_CHECK(grad.size() == aux.size() && begin % 4 == 0 && end % 4 == 0 && begin <= end);
  rk::DpPeers p = aux_only_peers(aux);
  for (size_t i = 0; i < grad.size(); ++i) p.grad[i] = reinterpret_cast<void*>(grad[i]);
  p.grad_mc = reinterpret_cast<void*>(grad_mc);
  rk::dp_reduce_shard(p, (int)rank, (int)grad.size(), begin, end, stream());
}

static const float* fptr(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kFloat, "screening scan tensors must be contiguous fp32 CUDA tensors");
  return t.data_ptr<float>();
}

rk::ScreenScanArgs screen_args(const Tensor& q_r, const Tensor& q_w, const Tensor& delta_xh, const Tensor& delta_slot,
                               const Tensor& slot_embed, const Tensor& WT, const Tensor& PD, const Tensor& mu,
                               const Tensor& slots0, const Tensor& ages0, const Tensor& usage0,
                               const std::vector<double>& f, bool write_enabled, bool value_unit_norm, bool age_mask) {
  rk::ScreenScanArgs a{};
  a.B = (int)q_r.size(0); a.T = (int)q_r.size(1); a.dk = (int)q_r.size(2);
  a.M = (int)slots0.size(1); a.ds = (int)slots0.size(2);
  a.dv = (int)WT.size(1) - 2 * a.dk;
  const int J = (int)WT.size(1);
  TORCH_CHECK(f.size() == 8 || f.size() == 11, "expected 8 scalar settings (+ leaky flag, alpha, gamma)");
  TORCH_CHECK(WT.size(0) == a.ds && a.dv >= 1, "weight shapes");
  TORCH_CHECK(PD.dim() == 4 && PD.size(0) == a.B && PD.size(1) == a.T && PD.size(2) == 16 && PD.size(3) == J,
              "PD must be [B, T, 16, J]");
  a.q_r = fptr(q_r); a.q_w = fptr(q_w); a.delta_xh = fptr(delta_xh); a.delta_slot = fptr(delta_slot);
  a.slot_embed = fptr(slot_embed); a.WT = fptr(WT); a.PD = fptr(PD); a.mu = fptr(mu);
  a.slots0 = fptr(slots0); a.ages0 = fptr(ages0); a.usage0 = fptr(usage0);
  a.tau_r = (float)f[0]; a.tau_w = (float)f[1]; a.eps = (float)f[2]; a.cap = (float)f[3]; a.write_rel_floor = (float)f[4];
  a.usage_decay = (float)f[5]; a.age_ref = (float)f[6]; a.age_sigma = (float)f[7];
  a.write_enabled = write_enabled; a.value_unit_norm = value_unit_norm; a.age_mask = age_mask;
  if (f.size() == 11) { a.leaky = f[8] != 0.0; a.leaky_alpha = (float)f[9]; a.leaky_gamma = (float)f[10]; }
  TORCH_CHECK(rk::screen_scan_supported(a), "screening scan: unsupported sizes");
  return a;
}

// returns u, slots_out, ages_out, usage_out, stats[9], strength [B,T,16], saved_ages, saved_P, rel_c [B,T,16]
std::vector<Tensor> screen_scan_fwd(const Tensor& q_r, const Tensor& q_w, const Tensor& delta_xh, const Tensor& delta_slot,
                                    const Tensor& slot_embed, const Tensor& WT, const Tensor& PD, const Tensor& mu,
                                    const Tensor& slots0, const Tensor& ages0, const Tensor& usage0,
                                    const std::vector<double>& f, bool write_enabled, bool value_unit_norm, bool age_mask,
                                    bool save, const c10::optional<Tensor>& tau_dev) {
  c10::cuda::CUDAGuard guard(q_r.device());
  rk::ScreenScanArgs a = screen_args(q_r, q_w, delta_xh, delta_slot, slot_embed, WT, PD, mu, slots0, ages0, usage0, f,
                                     write_enabled, value_unit_norm, age_mask);
  if (tau_dev.has_value() && tau_dev->defined()) { TORCH_CHECK(tau_dev->numel() == 2); a.tau_dev = fptr(*tau_dev); }
  auto o = q_r.options();
  const int J = 2 * a.dk + a.dv;
  Tensor u = torch::empty({a.B, a.T, a.dv}, o);
  Tensor so = torch::empty_like(slots0), ao = torch::empty_like(ages0), uo = torch::empty_like(usage0);
  Tensor stats = torch::zeros({9}, o);
  Tensor strength = torch::empty({a.B, a.T, 16}, o), rel_c = torch::empty({a.B, a.T, 16}, o);
  Tensor rel_r = torch::empty({a.B, a.T, 16}, o);
  // the rows of P are written in inference too: the read-out kernel forms u from them
  Tensor saved_ages = torch::empty({a.B, a.T, 16}, o);
  Tensor saved_P = torch::empty({a.B, a.T, 16, J}, o);
  a.u_out = u.data_ptr<float>(); a.slots_out = so.data_ptr<float>(); a.ages_out = ao.data_ptr<float>();
  a.usage_out = uo.data_ptr<float>(); a.stats = stats.data_ptr<float>();
  a.strength = strength.data_ptr<float>(); a.rel_c = rel_c.data_ptr<float>(); a.rel_r = rel_r.data_ptr<float>();
  a.saved_ages = saved_ages.data_ptr<float>();
  a.saved_P = saved_P.data_ptr<float>();
  Tensor rows = torch::empty({a.B, a.T, J}, o);
  a.ws_rows = rows.data_ptr<float>();
  TORCH_CHECK(rk::screen_scan_forward(a, stream()) == 0, "screen_scan_forward failed");
  if (!save) return {u, so, ao, uo, stats, torch::empty({0}, o), torch::empty({0}, o), torch::empty({0}, o), torch::empty({0}, o)};
  return {u, so, ao, uo, stats, strength, saved_ages, saved_P, rel_c};
}

// returns d q_r, d q_w, d delta_xh (direct part), d delta_slot (direct part), d slots0 (direct part), d mu,
// d (tau_r, tau_w), d PD [B,T,16,J], d P0 [B,16,J]
std::vector<Tensor> screen_scan_bwd(const Tensor& q_r, const Tensor& q_w, const Tensor& delta_xh, const Tensor& delta_slot,
                                    const Tensor& slot_embed, const Tensor& WT, const Tensor& PD, const Tensor& mu,
                                    const Tensor& slots0, const Tensor& ages0, const Tensor& usage0,
                                    const std::vector<double>& f, bool write_enabled, bool value_unit_norm, bool age_mask,
                                    const Tensor& strength, const Tensor& saved_ages, const Tensor& saved_P,
                                    const Tensor& rel_c, const Tensor& du,
                                    const c10::optional<Tensor>& dslots_out, const c10::optional<Tensor>& tau_dev,
                                    bool dpd_bf16) {
  c10::cuda::CUDAGuard guard(q_r.device());
  rk::ScreenScanArgs a = screen_args(q_r, q_w, delta_xh, delta_slot, slot_embed, WT, PD, mu, slots0, ages0, usage0, f,
                                     write_enabled, value_unit_norm, age_mask);
  if (tau_dev.has_value() && tau_dev->defined()) { TORCH_CHECK(tau_dev->numel() == 2); a.tau_dev = fptr(*tau_dev); }
  auto o = q_r.options();
  const int J = 2 * a.dk + a.dv;
  TORCH_CHECK(saved_P.numel() == (int64_t)a.B * a.T * 16 * J && strength.numel() == (int64_t)a.B * a.T * 16 &&
                  saved_ages.numel() == (int64_t)a.B * a.T * 16, "saved tensors do not match the problem size");
  const bool bank = dslots_out.has_value() && dslots_out->defined();
  Tensor dqr = torch::empty_like(q_r), dqw = torch::zeros_like(q_r);
  // without a cotangent for the final bank nothing reaches delta_xh, delta_slot or the initial bank directly
  Tensor dxh = bank ? torch::empty_like(delta_xh) : torch::zeros_like(delta_xh);
  Tensor ds0 = bank ? torch::empty_like(slots0) : torch::zeros_like(slots0);
  Tensor dds = torch::zeros_like(delta_slot), dmu = torch::zeros_like(mu);
  Tensor dsc = torch::zeros({2}, o);
  // rows of dead slots are not written by the kernel: zero them when the tensor feeds a GEMM over all 16 rows
  auto od = dpd_bf16 ? o.dtype(at::kBFloat16) : o;
  Tensor dPD = (dpd_bf16 && a.M < 16) ? torch::zeros({a.B, a.T, 16, J}, od) : torch::empty({a.B, a.T, 16, J}, od);
  Tensor dP0 = torch::empty({a.B, 16, J}, o);
  TORCH_CHECK(rel_c.numel() == (int64_t)a.B * a.T * 16 && du.numel() == (int64_t)a.B * a.T * a.dv, "saved tensors do not match");
  a.strength = const_cast<float*>(fptr(strength)); a.saved_ages = const_cast<float*>(fptr(saved_ages));
  a.rel_c = const_cast<float*>(fptr(rel_c));
  Tensor ws2 = torch::empty({(int64_t)a.B * a.T * (J + 32)}, o);
  a.ws_rows = ws2.data_ptr<float>(); a.ws_a = a.ws_rows + (int64_t)a.B * a.T * J; a.ws_b = a.ws_a + (int64_t)a.B * a.T * 16;
  a.saved_P = const_cast<float*>(fptr(saved_P));
  a.du = fptr(du);
  Tensor dso, ws;
  if (bank) {
    dso = dslots_out->contiguous().to(at::kFloat);
    TORCH_CHECK(dso.numel() == slots0.numel(), "final-bank cotangent must match the bank");
    a.dslots_out = dso.data_ptr<float>();
    ws = torch::empty({3 * (int64_t)a.B * a.T * 16 + (int64_t)a.B * 16}, o);
    const int64_t n = (int64_t)a.B * a.T * 16;
    a.ws_h = ws.data_ptr<float>(); a.ws_G = a.ws_h + n; a.ws_coef = a.ws_G + n; a.ws_c0 = a.ws_coef + n;
  }
  a.d_q_r = dqr.data_ptr<float>(); a.d_q_w = dqw.data_ptr<float>(); a.d_delta_xh = dxh.data_ptr<float>();
  if (dpd_bf16) a.d_PD_bf16 = dPD.data_ptr(); else a.d_PD = dPD.data_ptr<float>();
  a.d_P0 = dP0.data_ptr<float>();
  a.d_delta_slot = dds.data_ptr<float>(); a.d_slots0 = ds0.data_ptr<float>();
  a.d_mu = dmu.data_ptr<float>(); a.d_scalars = dsc.data_ptr<float>();
  TORCH_CHECK(rk::screen_scan_backward(a, stream()) == 0, "screen_scan_backward failed");
  return {dqr, dqw, dxh, dds, ds0, dmu, dsc, dPD, dP0};
}

// D = tanh(delta_xh[:, :, None] + delta_slot[None, None]) as bf16 [B, T, 16, ds]; rows of slots >= M are zero
Tensor screen_targets_fwd(const Tensor& delta_xh, const Tensor& delta_slot) {
  c10::cuda::CUDAGuard guard(delta_xh.device());
  const int64_t B = delta_xh.size(0), T = delta_xh.size(1), ds = delta_xh.size(2), M = delta_slot.size(0);
  TORCH_CHECK(M <= 16 && delta_slot.size(1) == ds);
  Tensor D = torch::empty({B, T, 16, ds}, delta_xh.options().dtype(at::kBFloat16));
  rk::screen_targets_forward(fptr(delta_xh), fptr(delta_slot), D.data_ptr(), (int)B, (int)T, (int)M, (int)ds, stream());
  return D;
}

// g_dxh += sum_m dD (1 - D^2), g_dslot += the same over (batch, step); both fp32, updated in place
void screen_targets_bwd(const Tensor& dD, const Tensor& delta_xh, const Tensor& delta_slot, Tensor& g_dxh, Tensor& g_dslot) {
  c10::cuda::CUDAGuard guard(delta_xh.device());
  const int64_t B = delta_xh.size(0), T = delta_xh.size(1), ds = delta_xh.size(2), M = delta_slot.size(0);
  TORCH_CHECK(dD.scalar_type() == at::kBFloat16 && dD.is_contiguous() && dD.numel() == B * T * 16 * ds);
  TORCH_CHECK(g_dxh.numel() == delta_xh.numel() && g_dslot.numel() == delta_slot.numel());
  rk::screen_targets_backward(dD.data_ptr(), fptr(delta_xh), fptr(delta_slot), const_cast<float*>(fptr(g_dxh)),
                              const_cast<float*>(fptr(g_dslot)), (int)B, (int)T, (int)M, (int)ds, stream());
}

rk::TpPeers make_tp_peers(const std::vector<int64_t>& buf, int64_t buf_mc, const std::vector<int64_t>& aux, int64_t rank) {
  rk::TpPeers p{};
  TORCH_CHECK(buf.size() == aux.size() && buf.size() >= 1 && buf.size() <= (size_t)rk::kMaxRanks, "bad peer lists");
  for (size_t i = 0; i < buf.size(); ++i) {
    p.buf[i] = reinterpret_cast<const void*>(buf[i]);
    p.aux[i] = reinterpret_cast<void*>(aux[i]);
  }
  p.buf_mc = reinterpret_cast<const void*>(buf_mc);
  p.rank = (int)rank; p.world = (int)buf.size();
  return p;
}

// barrier (target = barriers issued so far on this aux buffer + 1), then all-gather over time into `out`
void tp_gather_seq(const std::vector<int64_t>& buf, const std::vector<int64_t>& aux, int64_t rank, int64_t target, Tensor out,
                   int64_t B, int64_t Tl, int64_t C) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 && C % 8 == 0);
  TORCH_CHECK(out.numel() == B * Tl * C * (int64_t)buf.size(), "gather output must be [B, world*Tl, C]");
  rk::TpPeers p = make_tp_peers(buf, 0, aux, rank);
  rk::tp_barrier(p, (uint32_t)target, stream());
  rk::tp_gather_seq(p, out.data_ptr(), (int)B, (int)Tl, (int)C, stream());
}

// barrier, then out = residual + sum over ranks of this rank's time slice of the partial buffers
void tp_reduce_scatter_add(const std::vector<int64_t>& buf, int64_t buf_mc, const std::vector<int64_t>& aux, int64_t rank,
                           int64_t target, const c10::optional<Tensor>& residual, Tensor out, int64_t B, int64_t Tl, int64_t C) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kBFloat16 && C % 8 == 0);
  TORCH_CHECK(out.numel() == B * Tl * C, "reduce-scatter output must be [B, Tl, C]");
  const void* res = nullptr;
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == at::kBFloat16 && residual->numel() == out.numel());
    res = residual->data_ptr();
  }
  rk::TpPeers p = make_tp_peers(buf, buf_mc, aux, rank);
  rk::tp_barrier(p, (uint32_t)target, stream());
  rk::tp_reduce_scatter_add(p, res, out.data_ptr(), (int)B, (int)Tl, (int)C, stream());
}

// Row-parallel GEMM fused with the reduce-scatter over time: barrier (every owner initialised its output buffer),
// y = x W^T with the scatter-add epilogue pushing each tile into its owner's buffer over NVLink, barrier (all pushes
// landed).  `scatter` is a device-resident rk::GemmScatter (int64 words: 8 pointers, world | T << 32, Tl).
void tp_gemm_reduce_scatter(const Tensor& x2, const Tensor& w, const Tensor& scatter, int64_t ldd,
                            const std::vector<int64_t>& buf, const std::vector<int64_t>& aux, int64_t rank,
                            int64_t target_before, int64_t pair) {
  c10::cuda::CUDAGuard guard(x2.device());
  TORCH_CHECK(x2.is_cuda() && x2.is_contiguous() && x2.scalar_type() == at::kBFloat16 && x2.dim() == 2);
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 && w.size(1) == x2.size(1));
  TORCH_CHECK(scatter.is_cuda() && scatter.scalar_type() == at::kLong && scatter.numel() >= 10);
  rk::TpPeers peers = make_tp_peers(buf, 0, aux, rank);
  rk::tp_barrier(peers, (uint32_t)target_before, stream());
  rk::GemmArgs p{};
  p.A = x2.data_ptr(); p.B = w.data_ptr(); p.D = scatter.data_ptr();
  p.M = (int)x2.size(0); p.K = (int)x2.size(1); p.N = (int)w.size(0);
  p.lda = (int)x2.stride(0); p.ldb = (int)w.stride(0); p.ldd = (int)ldd;
  p.layout = rk::kGemmTN; p.epilogue = rk::kEpiScatterAddBf16; p.pair = (int)pair;
  p.error_flag = gemm_error_flag(x2.device()).data_ptr<int>();
  const int rc = rk::gemm_bf16(p, stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 (scatter epilogue) launch failed with code ", rc);
  rk::tp_barrier(peers, (uint32_t)target_before + 1, stream());
}

int64_t dp_aux_error_word() { return rk::dp_aux_error_word(); }
void dp_set_wait_limit_ms(double ms) { rk::dp_set_wait_limit_ms(ms); }
double dp_wait_limit_ms() { return rk::dp_wait_limit_ms(); }
int64_t dp_aux_words() { return rk::dp_aux_words(); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("wkv7_fwd", &wkv7_fwd, py::arg("r"), py::arg("w"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"),
        py::arg("s0"), py::arg("save"), py::arg("interval"), py::arg("chunked"), py::arg("inplace_state") = false);
  m.def("wkv7_bwd", &wkv7_bwd, py::arg("r"), py::arg("w"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"),
        py::arg("s0"), py::arg("sa"), py::arg("ckpt"), py::arg("dy"), py::arg("dsT"), py::arg("interval"), py::arg("chunked"),
        py::arg("add") = py::none());
  m.def("wkv7_chunk_error", [](bool reset) { return rk::wkv7_chunk_error(reset) | rk::wkv7_chunk_bwd_error(reset); });
#ifdef RK_WKV_PROF
  m.def("wkv7_chunk_bwd_prof", [](bool reset) {
    std::vector<int64_t> v(16);
    long long raw[16];
    rk::wkv7_chunk_bwd_prof(raw, reset);
    for (int i = 0; i < 16; ++i) v[i] = raw[i];
    return v;
  });
  m.def("wkv7_chunk_prof", [](bool reset) {
    std::vector<int64_t> v(16);
    long long raw[16];
    rk::wkv7_chunk_prof(raw, reset);
    for (int i = 0; i < 16; ++i) v[i] = raw[i];
    return v;
  });
#endif
  m.def("grad_norm_sq", &grad_norm_sq);
  m.def("adamw_flat", &adamw_flat);
  m.def("gemm", &gemm, py::arg("A"), py::arg("B"), py::arg("D"), py::arg("layout"), py::arg("epilogue"), py::arg("pair"),
        py::arg("aux") = py::none(), py::arg("act") = 0);
  m.def("gemm_group", &gemm_group);
  m.def("gemm_error", &gemm_error);
  m.def("gemm_error_reset", &gemm_error_reset);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("shift_mix_fwd", &shift_mix_fwd);
  m.def("shift_mix_bwd", &shift_mix_bwd);
  m.def("tmix_pre_fwd", &tmix_pre_fwd);
  m.def("tmix_pre_bwd", &tmix_pre_bwd);
  m.def("gn_bonus_gate_fwd", &gn_bonus_gate_fwd);
  m.def("gn_bonus_gate_bwd", &gn_bonus_gate_bwd);
  m.def("set_decode_gemm", &set_decode_gemm);
  m.def("relusq_bwd", &relusq_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("gemm_ce_stats", &gemm_ce_stats);
  m.def("ce_bwd", &ce_bwd);
  m.def("dp_step", &dp_step);
  m.def("dp_step_timings", &dp_step_timings);
  m.def("dp_barrier_only", &dp_barrier_only);
  m.def("zero_gather", &zero_gather);
  m.def("zero_reduce", &zero_reduce);
  m.def("screen_scan_fwd", &screen_scan_fwd);
  m.def("screen_scan_bwd", &screen_scan_bwd);
  m.def("screen_targets_fwd", &screen_targets_fwd);
  m.def("screen_targets_bwd", &screen_targets_bwd);
  m.def("tp_gather_seq", &tp_gather_seq);
  m.def("tp_gemm_reduce_scatter", &tp_gemm_reduce_scatter);
  m.def("tp_reduce_scatter_add", &tp_reduce_scatter_add);
  m.def("tp_aux_error_word", []() { return (int64_t)rk::tp_aux_error_word(); });
  m.def("tp_aux_words", []() { return (int64_t)rk::tp_aux_words(); });
  m.def("dp_aux_error_word", &dp_aux_error_word);
  m.def("dp_set_wait_limit_ms", &dp_set_wait_limit_ms);
  m.def("dp_wait_limit_ms", &dp_wait_limit_ms);
  m.def("dp_aux_words", &dp_aux_words);
}
