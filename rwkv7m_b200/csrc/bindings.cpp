// PyTorch bindings: tensor checks, output allocation and stream plumbing around
// the launchers declared in kernels.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

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
                             const Tensor& b, const Tensor& s0, bool save, int64_t interval) {
  c10::cuda::CUDAGuard guard(r.device());
  TORCH_CHECK(interval >= 1, "checkpoint interval must be positive");
  rk::WkvArgs p = wkv_args(r, w, k, v, a, b, s0, interval);
  Tensor y = torch::empty_like(r);
  Tensor sT = torch::empty_like(s0);
  Tensor sa, ckpt;
  p.y = y.data_ptr(); p.sT = sT.data_ptr<float>();
  if (save) {
    auto f32 = r.options().dtype(at::kFloat);
    sa = torch::empty(r.sizes(), f32);
    const int64_t nck = (p.T + interval - 1) / interval;
    ckpt = torch::empty({nck, (int64_t)p.B * p.H, (int64_t)p.N, (int64_t)p.N}, f32);
    p.sa = sa.data_ptr<float>(); p.ckpt = ckpt.data_ptr<float>();
  } else {
    sa = torch::empty({0}, r.options().dtype(at::kFloat));
    ckpt = sa;
  }
  TORCH_CHECK(rk::wkv7_forward(p, stream()) == 0, "wkv7_forward: unsupported shape");
  return {y, sT, sa, ckpt};
}

std::vector<Tensor> wkv7_bwd(const Tensor& r, const Tensor& w, const Tensor& k, const Tensor& v, const Tensor& a,
                             const Tensor& b, const Tensor& s0, const Tensor& sa, const Tensor& ckpt,
                             const Tensor& dy, const c10::optional<Tensor>& dsT, int64_t interval) {
  c10::cuda::CUDAGuard guard(r.device());
  rk::WkvArgs p = wkv_args(r, w, k, v, a, b, s0, interval);
  check_vec(dy, r, "dy");
  TORCH_CHECK(sa.is_contiguous() && sa.scalar_type() == at::kFloat && sa.numel() == r.numel(), "bad sa");
  const int64_t nck = (p.T + interval - 1) / interval;
  TORCH_CHECK(ckpt.is_contiguous() && ckpt.scalar_type() == at::kFloat &&
                  ckpt.numel() == nck * p.B * p.H * p.N * p.N, "bad checkpoints");
  Tensor dr = torch::empty_like(r), dw = torch::empty_like(r), dk = torch::empty_like(r), dv = torch::empty_like(r),
         da = torch::empty_like(r), db = torch::empty_like(r);
  Tensor ds0 = torch::empty_like(s0);
  p.sa = const_cast<float*>(sa.data_ptr<float>()); p.ckpt = const_cast<float*>(ckpt.data_ptr<float>());
  p.dy = dy.data_ptr();
  Tensor dsT_c;
  if (dsT.has_value() && dsT->defined()) {
    dsT_c = dsT->contiguous().to(at::kFloat);
    TORCH_CHECK(dsT_c.sizes() == s0.sizes(), "dsT must match the state shape");
    p.dsT = dsT_c.data_ptr<float>();
  }
  p.dr = dr.data_ptr(); p.dw = dw.data_ptr(); p.dk = dk.data_ptr(); p.dv = dv.data_ptr();
  p.da = da.data_ptr(); p.db = db.data_ptr(); p.ds0 = ds0.data_ptr<float>();
  TORCH_CHECK(rk::wkv7_backward(p, stream()) == 0, "wkv7_backward: unsupported shape");
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

// D = op(A) op(B); see kernels.h for the three layouts.  D must be preallocated.
void gemm(const Tensor& A, const Tensor& B, Tensor D, int64_t layout, int64_t epilogue) {
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: A and B must be bf16");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2, "gemm: 2-D tensors required");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1, "gemm: rows must be contiguous");
  rk::GemmArgs p{};
  p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = D.data_ptr();
  p.lda = (int)A.stride(0); p.ldb = (int)B.stride(0); p.ldd = (int)D.stride(0);
  p.layout = (int)layout; p.epilogue = (int)epilogue;
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
  const bool out_bf16 = epilogue == rk::kEpiStoreBf16 || epilogue == rk::kEpiReluSqBf16;
  TORCH_CHECK(D.scalar_type() == (out_bf16 ? at::kBFloat16 : at::kFloat), "gemm: output dtype mismatch");
  p.error_flag = gemm_error_flag(A.device()).data_ptr<int>();
  const int rc = rk::gemm_bf16(p, stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 launch failed with code ", rc);
}

int64_t gemm_error(const Tensor& like) {
  return gemm_error_flag(like.device()).item<int>();
}

void gemm_error_reset(const Tensor& like) { gemm_error_flag(like.device()).zero_(); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("wkv7_fwd", &wkv7_fwd);
  m.def("wkv7_bwd", &wkv7_bwd);
  m.def("grad_norm_sq", &grad_norm_sq);
  m.def("adamw_flat", &adamw_flat);
  m.def("gemm", &gemm);
  m.def("gemm_error", &gemm_error);
  m.def("gemm_error_reset", &gemm_error_reset);
}
