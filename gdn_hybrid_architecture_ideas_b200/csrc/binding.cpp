// Python bindings of the sm_100a kernels: tensors in, raw pointers + the current CUDA stream out.
// Shape and dtype checks live here so that no kernel ever receives a pointer it was not written for.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels.h"

namespace {

using torch::Tensor;

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }
void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, ": launch refused (code ", rc, ")"); }
bool is_bf16(const Tensor& t) { return t.scalar_type() == torch::kBFloat16; }
bool is_f32(const Tensor& t) { return t.scalar_type() == torch::kFloat32; }
const float* fptr(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }

// D = A B^T (+ D). a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn), 2-D with unit inner stride.
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, bool accumulate, Tensor& err) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda() && is_bf16(a) && is_bf16(b), "gemm: bf16 CUDA operands");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm: 2-D, unit inner stride");
  const c10::cuda::CUDAGuard guard(a.device());
  const int M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm: shape mismatch");
  int mode;
  if (is_bf16(out)) { TORCH_CHECK(!accumulate, "gemm: accumulation needs an fp32 output"); mode = 0; }
  else { TORCH_CHECK(is_f32(out), "gemm: output bf16 or fp32"); mode = accumulate ? 2 : 1; }
  const int rc = ghb::gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), a_mn, b_mn, mode,
                                err.data_ptr<int>(), sm_count(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 refused (code ", rc, "): M=", M, " N=", N, " K=", K, " lda=", a.stride(0), " ldb=", b.stride(0), " ldc=",
              out.stride(0), " a_mn=", a_mn, " b_mn=", b_mn, " cuerr=", ghb::last_encode_error(), " ptrs%16=", reinterpret_cast<uintptr_t>(a.data_ptr()) % 16, ",",
              reinterpret_cast<uintptr_t>(b.data_ptr()) % 16, ",", reinterpret_cast<uintptr_t>(out.data_ptr()) % 16);
}

void rmsnorm_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& z, int64_t gate, const c10::optional<Tensor>& resid,
                 Tensor& y, const c10::optional<Tensor>& rstd, double eps, double scale) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && is_f32(w), "rmsnorm_fwd: contiguous inputs, fp32 gain");
  const int d = x.size(-1);
  const long rows = x.numel() / d;
  TORCH_CHECK(w.numel() == d || w.numel() == 1, "rmsnorm_fwd: gain of size d or 1");
  if (gate) TORCH_CHECK(z.has_value() && is_bf16(*z) && z->is_contiguous() && z->numel() == x.numel(), "rmsnorm_fwd: bf16 gate input");
  if (resid.has_value()) TORCH_CHECK(is_f32(*resid) && is_f32(y) && resid->is_contiguous() && resid->numel() == x.numel(), "rmsnorm_fwd: fp32 residual");
  check(ghb::rmsnorm_fwd(x.data_ptr(), is_bf16(x), w.data_ptr<float>(), w.numel() == 1, gate ? z->data_ptr() : nullptr, gate, fptr(resid),
                         y.data_ptr(), is_bf16(y), rstd.has_value() ? rstd->data_ptr<float>() : nullptr, rows, d, eps, scale, stream()),
        "rmsnorm_fwd");
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const c10::optional<Tensor>& z, int64_t gate, const Tensor& rstd,
                 const c10::optional<Tensor>& dres, Tensor& dx, const c10::optional<Tensor>& dz, Tensor& dw, double scale) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous() && is_f32(dw) && dx.scalar_type() == x.scalar_type(), "rmsnorm_bwd: layout");
  const int d = x.size(-1);
  const long rows = x.numel() / d;
  if (gate) TORCH_CHECK(z.has_value() && dz.has_value() && is_bf16(*dz), "rmsnorm_bwd: gate tensors");
  check(ghb::rmsnorm_bwd(dy.data_ptr(), is_bf16(dy), x.data_ptr(), is_bf16(x), w.data_ptr<float>(), w.numel() == 1, gate ? z->data_ptr() : nullptr,
                         gate, rstd.data_ptr<float>(), fptr(dres), dx.data_ptr(), gate ? dz->data_ptr() : nullptr, dw.data_ptr<float>(), rows, d,
                         scale, sm_count(), stream()), "rmsnorm_bwd");
}

void silu_mul_fwd(const Tensor& gu, Tensor& h) {
  const c10::cuda::CUDAGuard guard(gu.device());
  const int f = h.size(-1);
  TORCH_CHECK(is_bf16(gu) && is_bf16(h) && gu.size(-1) == 2 * f && gu.is_contiguous() && h.is_contiguous(), "silu_mul_fwd: gu [rows, 2f] bf16");
  const long rows = h.numel() / f;
  auto* p = static_cast<const __nv_bfloat16*>(gu.data_ptr());
  check(ghb::silu_mul_fwd(p, p + f, 2L * f, h.data_ptr(), rows, f, sm_count(), stream()), "silu_mul_fwd");
}
void silu_mul_bwd(const Tensor& dh, const Tensor& gu, Tensor& dgu) {
  const c10::cuda::CUDAGuard guard(gu.device());
  const int f = dh.size(-1);
  TORCH_CHECK(is_bf16(gu) && is_bf16(dh) && is_bf16(dgu) && gu.is_contiguous() && dh.is_contiguous() && dgu.is_contiguous(), "silu_mul_bwd: bf16 contiguous");
  const long rows = dh.numel() / f;
  auto* p = static_cast<const __nv_bfloat16*>(gu.data_ptr());
  auto* q = static_cast<__nv_bfloat16*>(dgu.data_ptr());
  check(ghb::silu_mul_bwd(dh.data_ptr(), p, p + f, 2L * f, q, q + f, rows, f, sm_count(), stream()), "silu_mul_bwd");
}

void adamw(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const c10::optional<Tensor>& lp, double lr, double b1, double b2, double eps,
           double wd, double c1, double c2, const c10::optional<Tensor>& grad_scale, double scale_host) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(is_f32(p) && is_f32(g) && is_f32(m) && is_f32(v) && p.is_contiguous() && g.is_contiguous(), "adamw: fp32 flat buffers");
  check(ghb::adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), lp.has_value() ? lp->data_ptr() : nullptr,
                   p.numel(), lr, b1, b2, eps, wd, c1, c2, fptr(grad_scale), scale_host, sm_count(), stream()), "adamw");
}
Tensor sumsq(const Tensor& x) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_f32(x) && x.is_contiguous(), "sumsq: fp32 contiguous");
  const int blocks = 1024;
  Tensor part = torch::empty({blocks}, x.options());
  check(ghb::sumsq_partials(x.data_ptr<float>(), x.numel(), part.data_ptr<float>(), blocks, stream()), "sumsq");
  return part.sum();
}
void cast_bf16(const Tensor& x, Tensor& y) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_f32(x) && is_bf16(y) && x.numel() == y.numel(), "cast_bf16");
  check(ghb::cast_bf16(x.data_ptr<float>(), y.data_ptr(), x.numel(), sm_count(), stream()), "cast_bf16");
}

void gdn_prep_fwd(const Tensor& u, const c10::optional<Tensor>& doc, const Tensor& w, Tensor& out, int64_t L, int64_t nq, double qscale) {
  const c10::cuda::CUDAGuard guard(u.device());
  const int C = u.size(-1);
  TORCH_CHECK(is_bf16(u) && is_bf16(out) && u.is_contiguous() && out.is_contiguous() && is_f32(w) && w.is_contiguous() && w.size(0) == C && w.size(1) == 4,
              "gdn_prep_fwd: bf16 [rows, C], conv weight fp32 [C, 4]");
  if (doc.has_value()) TORCH_CHECK(doc->scalar_type() == torch::kInt32 && doc->is_contiguous() && doc->numel() * C == u.numel(), "gdn_prep_fwd: int32 doc ids");
  check(ghb::gdn_prep_fwd(u.data_ptr(), doc.has_value() ? doc->data_ptr<int>() : nullptr, w.data_ptr<float>(), out.data_ptr(), u.numel() / C, L, C, nq,
                          qscale, stream()), "gdn_prep_fwd");
}
void gdn_prep_bwd(const Tensor& u, const c10::optional<Tensor>& doc, const Tensor& w, const Tensor& dout, Tensor& du, Tensor& dw,
                  int64_t L, int64_t nq, double qscale) {
  const c10::cuda::CUDAGuard guard(u.device());
  const int C = u.size(-1);
  TORCH_CHECK(is_bf16(dout) && dout.is_contiguous() && is_bf16(du) && du.is_contiguous() && is_f32(dw) && dw.is_contiguous(), "gdn_prep_bwd: layout");
  check(ghb::gdn_prep_bwd(u.data_ptr(), doc.has_value() ? doc->data_ptr<int>() : nullptr, w.data_ptr<float>(), dout.data_ptr(),
                          du.data_ptr(), dw.data_ptr<float>(), u.numel() / C, L, C, nq, qscale, stream()), "gdn_prep_bwd");
}

void depth_mix_fwd(const std::vector<Tensor>& src, const Tensor& ueff, Tensor& out, Tensor& alpha, Tensor& rnorm, double eps) {
  const c10::cuda::CUDAGuard guard(out.device());
  const int d = out.size(-1);
  std::vector<const float*> p;
  for (auto& s : src) { TORCH_CHECK(is_f32(s) && s.is_contiguous() && s.numel() == out.numel(), "depth_mix_fwd: fp32 contiguous sources"); p.push_back(s.data_ptr<float>()); }
  check(ghb::depth_mix_fwd(p.data(), p.size(), ueff.data_ptr<float>(), out.data_ptr<float>(), alpha.data_ptr<float>(), rnorm.data_ptr<float>(),
                           out.numel() / d, d, eps, stream()), "depth_mix_fwd");
}
void depth_mix_bwd(const std::vector<Tensor>& src, std::vector<Tensor>& dsrc, const Tensor& ueff, const Tensor& dh, const Tensor& alpha,
                   const Tensor& rnorm, Tensor& du) {
  const c10::cuda::CUDAGuard guard(dh.device());
  const int d = dh.size(-1);
  TORCH_CHECK(is_f32(dh) && dh.is_contiguous() && is_f32(du), "depth_mix_bwd: fp32");
  std::vector<const float*> p; std::vector<float*> q;
  for (auto& s : src) p.push_back(s.data_ptr<float>());
  for (auto& s : dsrc) { TORCH_CHECK(is_f32(s) && s.is_contiguous(), "depth_mix_bwd: fp32 outputs"); q.push_back(s.data_ptr<float>()); }
  check(ghb::depth_mix_bwd(p.data(), q.data(), p.size(), ueff.data_ptr<float>(), dh.data_ptr<float>(), alpha.data_ptr<float>(), rnorm.data_ptr<float>(),
                           du.data_ptr<float>(), dh.numel() / d, d, sm_count(), stream()), "depth_mix_bwd");
}

// Q readers over the same n sources: ueff [Q, d]; outs: Q tensors like a source; alpha, vu [rows, Q, n]; rnorm [rows, n].
void depth_mix_multi_fwd(const std::vector<Tensor>& src, const Tensor& ueff, std::vector<Tensor>& outs, Tensor& alpha, Tensor& rnorm, Tensor& vu, double eps) {
  const c10::cuda::CUDAGuard guard(ueff.device());
  const int d = ueff.size(-1);
  std::vector<const float*> p; std::vector<float*> o;
  for (auto& s : src) { TORCH_CHECK(is_f32(s) && s.is_contiguous() && s.numel() == src[0].numel(), "depth_mix_multi_fwd: fp32 contiguous sources"); p.push_back(s.data_ptr<float>()); }
  for (auto& t : outs) { TORCH_CHECK(is_f32(t) && t.is_contiguous() && t.numel() == src[0].numel(), "depth_mix_multi_fwd: fp32 outputs"); o.push_back(t.data_ptr<float>()); }
  TORCH_CHECK(is_f32(ueff) && ueff.is_contiguous() && ueff.size(0) == static_cast<long>(outs.size()) && is_f32(alpha) && is_f32(rnorm) && is_f32(vu), "depth_mix_multi_fwd: layout");
  check(ghb::depth_mix_multi_fwd(p.data(), p.size(), o.data(), o.size(), ueff.data_ptr<float>(), alpha.data_ptr<float>(), rnorm.data_ptr<float>(),
                                 vu.data_ptr<float>(), src[0].numel() / d, d, eps, stream()), "depth_mix_multi_fwd");
}
void depth_mix_multi_bwd(const std::vector<Tensor>& src, std::vector<Tensor>& dsrc, const Tensor& ueff, const std::vector<c10::optional<Tensor>>& dhs,
                         const Tensor& alpha, const Tensor& rnorm, const Tensor& vu, Tensor& du) {
  const c10::cuda::CUDAGuard guard(ueff.device());
  const int d = ueff.size(-1);
  std::vector<const float*> p, g; std::vector<float*> q;
  for (auto& s : src) p.push_back(s.data_ptr<float>());
  for (auto& s : dsrc) { TORCH_CHECK(is_f32(s) && s.is_contiguous() && s.numel() == src[0].numel(), "depth_mix_multi_bwd: fp32 outputs"); q.push_back(s.data_ptr<float>()); }
  for (auto& t : dhs) {
    if (t.has_value()) { TORCH_CHECK(is_f32(*t) && t->is_contiguous() && t->numel() == src[0].numel(), "depth_mix_multi_bwd: fp32 gradients"); g.push_back(t->data_ptr<float>()); }
    else g.push_back(nullptr);
  }
  TORCH_CHECK(ueff.size(0) == static_cast<long>(g.size()) && is_f32(du) && du.is_contiguous() && du.numel() == ueff.numel() && p.size() == q.size(), "depth_mix_multi_bwd: layout");
  check(ghb::depth_mix_multi_bwd(p.data(), q.data(), p.size(), g.data(), g.size(), ueff.data_ptr<float>(), alpha.data_ptr<float>(), rnorm.data_ptr<float>(),
                                 vu.data_ptr<float>(), du.data_ptr<float>(), src[0].numel() / d, d, sm_count(), stream()), "depth_mix_multi_bwd");
}

// One decode token of the gated delta rule, in place on S [B, Hv, 128, dv] fp32. q, k [B, Hk, 128]; v, o [B, Hv, dv]; g, beta [B, Hv]
// (all fp32, contiguous); start: optional bool [B] (document start: the state is dropped first).
void gdn_step(Tensor& S, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, const c10::optional<Tensor>& start, Tensor& o) {
  const c10::cuda::CUDAGuard guard(S.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&S, &q, &k, &v, &g, &beta, &o}) TORCH_CHECK(is_f32(*t) && t->is_contiguous(), "gdn_step: fp32 contiguous tensors");
  TORCH_CHECK(S.dim() == 4 && q.dim() == 3 && v.dim() == 3 && q.sizes() == k.sizes() && o.sizes() == v.sizes() && S.size(0) == q.size(0) && S.size(1) == v.size(1) &&
              S.size(2) == q.size(2) && S.size(3) == v.size(2) && g.numel() == S.size(0) * S.size(1) && beta.numel() == g.numel(), "gdn_step: shapes");
  const unsigned char* sp = nullptr;
  if (start.has_value()) { TORCH_CHECK(start->scalar_type() == at::kBool && start->is_contiguous() && start->numel() == S.size(0), "gdn_step: start"); sp = reinterpret_cast<const unsigned char*>(start->data_ptr<bool>()); }
  check(ghb::gdn_step(S.data_ptr<float>(), q.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), beta.data_ptr<float>(), sp,
                      o.data_ptr<float>(), S.size(0), q.size(1), S.size(1), S.size(2), S.size(3), stream()), "gdn_step");
}

// x: [rows, n] fp32 or bf16 contiguous; out: bf16 like x; blocks of 32 along the last dimension, or along rows.
// x [R, C] -> (q_row [R, C], sf_row) and / or (q_col [C, R], sf_col): uint8 tensors; a pair is skipped when its q is undefined.
void mx_quantize(const Tensor& x, const c10::optional<Tensor>& q_row, const c10::optional<Tensor>& sf_row, const c10::optional<Tensor>& q_col,
                 const c10::optional<Tensor>& sf_col) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && (is_f32(x) || is_bf16(x)), "mx_quantize: 2-D fp32 / bf16 input with unit inner stride");
  const long R = x.size(0), C = x.size(1);
  auto ok = [&](const c10::optional<Tensor>& q, const c10::optional<Tensor>& sf, long rows, long k) {
    if (!q.has_value()) return true;
    return sf.has_value() && q->is_contiguous() && q->numel() == rows * k && q->element_size() == 1 && sf->is_contiguous() &&
           sf->element_size() == 1 && sf->numel() >= ghb::mx_scale_bytes(rows, k);
  };
  TORCH_CHECK(ok(q_row, sf_row, R, C) && ok(q_col, sf_col, C, R), "mx_quantize: output sizes");
  check(ghb::mx_quantize(x.data_ptr(), is_bf16(x), R, C, x.stride(0), q_row.has_value() ? q_row->data_ptr() : nullptr,
                         sf_row.has_value() ? sf_row->data_ptr() : nullptr, q_col.has_value() ? q_col->data_ptr() : nullptr,
                         sf_col.has_value() ? sf_col->data_ptr() : nullptr, sm_count(), stream()), "mx_quantize");
}
int64_t mx_scale_bytes(int64_t rows, int64_t k) { return ghb::mx_scale_bytes(rows, k); }
// out [M, N] (+)= a [M, K] b [N, K]^T over E4M3 bytes with scale cells.
void gemm_mx(const Tensor& a, const Tensor& sfa, const Tensor& b, const Tensor& sfb, Tensor& out, bool accumulate, Tensor& err) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.is_contiguous() && b.is_contiguous() && out.stride(1) == 1 &&
              a.element_size() == 1 && b.element_size() == 1, "gemm_mx: contiguous 1-byte operands");
  const int M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K && out.size(0) == M && out.size(1) == N, "gemm_mx: shape mismatch");
  TORCH_CHECK(sfa.numel() >= ghb::mx_scale_bytes(M, K) && sfb.numel() >= ghb::mx_scale_bytes(N, K), "gemm_mx: scale cells too small");
  int mode;
  if (is_bf16(out)) { TORCH_CHECK(!accumulate, "gemm_mx: accumulation needs an fp32 output"); mode = 0; }
  else { TORCH_CHECK(is_f32(out), "gemm_mx: output bf16 or fp32"); mode = accumulate ? 2 : 1; }
  const int rc = ghb::gemm_mxfp8(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), M, N, K, out.stride(0), mode,
                                 err.data_ptr<int>(), sm_count(), stream());
  TORCH_CHECK(rc == 0, "gemm_mxfp8 refused (code ", rc, "): M=", M, " N=", N, " K=", K, " ldc=", out.stride(0), " cuerr=", ghb::last_encode_error());
}
void mx_fake(const Tensor& x, Tensor& out, bool along_rows) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && (is_f32(x) || is_bf16(x)) && is_bf16(out) && out.is_contiguous() && out.sizes() == x.sizes(), "mx_fake: layout");
  check(ghb::mx_fake(x.data_ptr(), is_bf16(x), out.data_ptr(), x.size(0), x.size(1), along_rows, sm_count(), stream()), "mx_fake");
}

// ids: int64 [n, s] contiguous (all inside the table); table / grad: fp32 [V, d]; rows: fp32 [n, d].
void embedding_fwd(const Tensor& ids, const Tensor& table, Tensor& out) {
  const c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.dim() == 2 && is_f32(table) && table.is_contiguous() && is_f32(out) && out.is_contiguous() &&
              out.numel() == ids.size(0) * table.size(1), "embedding_fwd: layout");
  check(ghb::embedding_fwd(reinterpret_cast<const long*>(ids.data_ptr<int64_t>()), table.data_ptr<float>(), out.data_ptr<float>(), ids.size(0), ids.size(1),
                           table.size(1), sm_count(), stream()), "embedding_fwd");
}
void embedding_bwd(const Tensor& ids, const Tensor& g, Tensor& table_grad) {
  const c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.dim() == 2 && is_f32(g) && g.is_contiguous() && is_f32(table_grad) &&
              table_grad.is_contiguous() && g.numel() == ids.size(0) * table_grad.size(1), "embedding_bwd: layout");
  check(ghb::embedding_bwd(reinterpret_cast<const long*>(ids.data_ptr<int64_t>()), g.data_ptr<float>(), table_grad.data_ptr<float>(), ids.size(0), ids.size(1),
                           table_grad.size(1), sm_count(), stream()), "embedding_bwd");
}

void ce_grad(const Tensor& logits, const Tensor& targets, const Tensor& a, const Tensor& b, Tensor& grad, Tensor& ce, Tensor& lse, bool fixed) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(is_f32(logits) && logits.is_contiguous() && is_bf16(grad) && grad.is_contiguous() && targets.scalar_type() == torch::kInt64 &&
              targets.is_contiguous() && is_f32(a) && a.is_contiguous() && is_f32(b) && b.is_contiguous(), "ce_grad: layout");
  const long rows = logits.size(0);
  const int V = logits.size(1), s = targets.numel() / rows;
  check(ghb::ce_grad(logits.data_ptr<float>(), reinterpret_cast<const long*>(targets.data_ptr<int64_t>()), a.data_ptr<float>(), b.data_ptr<float>(),
                     grad.data_ptr(), ce.data_ptr<float>(), lse.data_ptr<float>(), rows, V, s, fixed, stream()), "ce_grad");
}

const void* optr(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
void check_heads(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.is_contiguous() && t.dim() == 4 && t.size(3) == 64, name, ": bf16 contiguous [B, L, H, 64]");
}

void attention_fwd(const Tensor& q, const c10::optional<Tensor>& qf, const Tensor& k, const c10::optional<Tensor>& kf, const Tensor& v, Tensor& o,
                   Tensor& lse, const c10::optional<Tensor>& doc, const c10::optional<Tensor>& pos, int64_t cap, double scale, Tensor& err) {
  const c10::cuda::CUDAGuard guard(q.device());
  check_heads(q, "q"); check_heads(k, "k"); check_heads(v, "v"); check_heads(o, "o");
  if (cap >= 0) { TORCH_CHECK(qf.has_value() && kf.has_value(), "attention_fwd: the cap needs q_far and k_far"); check_heads(*qf, "q_far"); check_heads(*kf, "k_far"); }
  if (doc.has_value()) TORCH_CHECK(pos.has_value() && doc->scalar_type() == torch::kInt32 && pos->scalar_type() == torch::kInt32 && doc->is_contiguous() && pos->is_contiguous(), "attention_fwd: int32 doc / pos");
  TORCH_CHECK(is_f32(lse) && lse.is_contiguous(), "attention_fwd: fp32 lse");
  check(ghb::attention_fwd(q.data_ptr(), optr(qf), k.data_ptr(), optr(kf), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                           doc.has_value() ? doc->data_ptr<int>() : nullptr, pos.has_value() ? pos->data_ptr<int>() : nullptr, q.size(0), q.size(1),
                           q.size(2), k.size(2), cap, scale, err.data_ptr<int>(), stream()), "attention_fwd");
}

void attention_bwd(const Tensor& q, const c10::optional<Tensor>& qf, const Tensor& k, const c10::optional<Tensor>& kf, const Tensor& v, const Tensor& o,
                   const Tensor& dO, const Tensor& lse, Tensor& dsum, Tensor& dq, const c10::optional<Tensor>& dqf, Tensor& dk,
                   const c10::optional<Tensor>& dkf, Tensor& dv, const c10::optional<Tensor>& pos, int64_t cap, double scale, Tensor& err) {
  const c10::cuda::CUDAGuard guard(q.device());
  check_heads(q, "q"); check_heads(k, "k"); check_heads(v, "v"); check_heads(o, "o"); check_heads(dO, "dO"); check_heads(dk, "dk"); check_heads(dv, "dv");
  TORCH_CHECK(is_f32(dq) && dq.is_contiguous() && is_f32(dsum) && is_f32(lse), "attention_bwd: fp32 dq / dsum / lse");
  if (cap >= 0) TORCH_CHECK(qf.has_value() && kf.has_value() && dqf.has_value() && dkf.has_value() && is_f32(*dqf), "attention_bwd: far tensors");
  if (pos.has_value()) TORCH_CHECK(pos->scalar_type() == torch::kInt32 && pos->is_contiguous(), "attention_bwd: int32 pos");
  check(ghb::attention_bwd(q.data_ptr(), optr(qf), k.data_ptr(), optr(kf), v.data_ptr(), o.data_ptr(), dO.data_ptr(), lse.data_ptr<float>(),
                           dsum.data_ptr<float>(), dq.data_ptr<float>(), dqf.has_value() ? dqf->data_ptr<float>() : nullptr, dk.data_ptr(),
                           dkf.has_value() ? dkf->data_ptr() : nullptr, dv.data_ptr(), pos.has_value() ? pos->data_ptr<int>() : nullptr, q.size(0),
                           q.size(1), q.size(2), k.size(2), cap, scale, err.data_ptr<int>(), stream()), "attention_bwd");
}

void check_rows(const Tensor& t, int64_t cols, const char* name) {
  TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.is_contiguous() && t.size(-1) == cols, name, ": bf16 contiguous [..., ", cols, "]");
}
float* fmut(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }
void* vmut(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

void dual_lerp_fwd(const Tensor& x, const Tensor& ya, const c10::optional<Tensor>& yb, const Tensor& la, const c10::optional<Tensor>& lb, Tensor& oa,
                   const c10::optional<Tensor>& ob) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_bf16(x) && is_bf16(ya) && is_bf16(oa) && x.is_contiguous() && ya.is_contiguous() && oa.is_contiguous() && is_f32(la) && ya.numel() == x.numel(),
              "dual_lerp_fwd: bf16 contiguous tensors, fp32 scalar weights");
  if (yb.has_value()) TORCH_CHECK(is_bf16(*yb) && yb->is_contiguous() && yb->numel() == x.numel() && lb.has_value() && is_f32(*lb) && ob.has_value() && is_bf16(*ob) && ob->is_contiguous(), "dual_lerp_fwd: second mix");
  check(ghb::dual_lerp_fwd(x.data_ptr(), ya.data_ptr(), optr(yb), la.data_ptr<float>(), fptr(lb), oa.data_ptr(), vmut(ob), x.numel(), sm_count(), stream()),
        "dual_lerp_fwd");
}
void dual_lerp_bwd(const Tensor& ga, const c10::optional<Tensor>& gb, const Tensor& x, const Tensor& ya, const c10::optional<Tensor>& yb, const Tensor& la,
                   const c10::optional<Tensor>& lb, Tensor& dx, Tensor& dya, const c10::optional<Tensor>& dyb, Tensor& dl) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_bf16(ga) && ga.is_contiguous() && is_bf16(dx) && dx.is_contiguous() && is_bf16(dya) && dya.is_contiguous() && is_f32(dl) && dl.numel() >= 2,
              "dual_lerp_bwd: layout");
  if (yb.has_value()) TORCH_CHECK(gb.has_value() && is_bf16(*gb) && gb->is_contiguous() && dyb.has_value() && is_bf16(*dyb) && dyb->is_contiguous(), "dual_lerp_bwd: second mix");
  check(ghb::dual_lerp_bwd(ga.data_ptr(), optr(gb), x.data_ptr(), ya.data_ptr(), optr(yb), la.data_ptr<float>(), fptr(lb), dx.data_ptr(), dya.data_ptr(),
                           vmut(dyb), dl.data_ptr<float>(), x.numel(), sm_count(), stream()), "dual_lerp_bwd");
}

// All operands laid out [B, H, L, *] with L a multiple of 64 (chunks never straddle rows).
void gdn_scan_fwd(const Tensor& W, const Tensor& Qin, const Tensor& Kout, const Tensor& Aqk, const Tensor& U, const Tensor& carry,
                  const c10::optional<Tensor>& S0, Tensor& O, const c10::optional<Tensor>& Sfinal, const c10::optional<Tensor>& Hsave,
                  const c10::optional<Tensor>& Vnew, Tensor& err) {
  const c10::cuda::CUDAGuard guard(W.device());
  const int B = U.size(0), H = U.size(1), L = U.size(2), dv = U.size(3);
  check_rows(W, 128, "W"); check_rows(Qin, 128, "q_in"); check_rows(Kout, 128, "k_out"); check_rows(Aqk, 64, "Aqk"); check_rows(U, dv, "U"); check_rows(O, dv, "O");
  TORCH_CHECK(O.dim() == 4 && O.size(1) == L && O.size(2) == H, "gdn_scan_fwd: O is token-major [B, L, H, dv]");
  TORCH_CHECK(is_f32(carry) && carry.is_contiguous() && carry.numel() == static_cast<int64_t>(B) * H * (L / 64), "gdn_scan_fwd: carry [B, H, L/64] fp32");
  if (S0.has_value()) TORCH_CHECK(is_f32(*S0) && S0->is_contiguous(), "gdn_scan_fwd: S0 fp32");
  check(ghb::gdn_scan_fwd(W.data_ptr(), Qin.data_ptr(), Kout.data_ptr(), Aqk.data_ptr(), U.data_ptr(), carry.data_ptr<float>(), fptr(S0), O.data_ptr(),
                          fmut(Sfinal), vmut(Hsave), vmut(Vnew), B, H, L, dv, err.data_ptr<int>(), stream()), "gdn_scan_fwd");
}

void gdn_scan_bwd(const Tensor& W, const Tensor& Qin, const Tensor& Kout, const Tensor& Aqk, const Tensor& Hsave, const Tensor& Vnew, const Tensor& dO,
                  const Tensor& carry, const c10::optional<Tensor>& dSfinal, Tensor& dU, Tensor& dWp, Tensor& dQp, Tensor& dKp, Tensor& dcarry,
                  const c10::optional<Tensor>& dS0, Tensor& err) {
  const c10::cuda::CUDAGuard guard(W.device());
  const int B = Vnew.size(0), H = Vnew.size(1), L = Vnew.size(2), dv = Vnew.size(3);
  check_rows(W, 128, "W"); check_rows(Qin, 128, "q_in"); check_rows(Kout, 128, "k_out"); check_rows(Aqk, 64, "Aqk"); check_rows(Vnew, dv, "v_new");
  check_rows(dO, dv, "dO"); check_rows(dU, dv, "dU"); check_rows(Hsave, 128, "h_save");
  TORCH_CHECK(dO.dim() == 4 && dO.size(1) == L && dO.size(2) == H, "gdn_scan_bwd: dO is token-major [B, L, H, dv]");
  TORCH_CHECK(is_f32(dWp) && is_f32(dQp) && is_f32(dKp) && is_f32(dcarry) && dWp.is_contiguous() && dQp.is_contiguous() && dKp.is_contiguous(), "gdn_scan_bwd: fp32 partials");
  check(ghb::gdn_scan_bwd(W.data_ptr(), Qin.data_ptr(), Kout.data_ptr(), Aqk.data_ptr(), Hsave.data_ptr(), Vnew.data_ptr(), dO.data_ptr(),
                          carry.data_ptr<float>(), fptr(dSfinal), dU.data_ptr(), dWp.data_ptr<float>(), dQp.data_ptr<float>(), dKp.data_ptr<float>(),
                          dcarry.data_ptr<float>(), fmut(dS0), B, H, L, dv, err.data_ptr<int>(), stream()), "gdn_scan_bwd");
}

void check_tok_major(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(0) == t.stride(1) * t.size(1),
              name, ": bf16 [B, L, H, d] with contiguous heads and a constant token stride");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && t.stride(1) % 8 == 0, name, ": 16-byte aligned rows");
}

// q, k: [B, L, Hk, 128]; v: [B, L, Hv, dv]; g, beta: [B, L, Hv] fp32; start: [B, L] uint8. Outputs are [B, Hv, L, *].
void gdn_local_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, const Tensor& start, Tensor& U, Tensor& W,
                   Tensor& Aqk, Tensor& Qin, Tensor& Kout, Tensor& carry) {
  const c10::cuda::CUDAGuard guard(q.device());
  check_tok_major(q, "q"); check_tok_major(k, "k"); check_tok_major(v, "v");
  TORCH_CHECK(is_f32(g) && g.is_contiguous() && is_f32(beta) && beta.is_contiguous() && start.scalar_type() == torch::kUInt8 && start.is_contiguous(), "gdn_local_fwd: gates fp32, starts uint8");
  const int B = v.size(0), L = v.size(1), Hv = v.size(2), dv = v.size(3), Hk = q.size(2);
  TORCH_CHECK(q.size(3) == 128 && k.size(3) == 128, "gdn_local_fwd: key dimension 128");
  check(ghb::gdn_local_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), k.stride(1), v.stride(1), g.data_ptr<float>(), beta.data_ptr<float>(),
                           start.data_ptr<uint8_t>(), B, L, Hv, Hk, dv, U.data_ptr(), W.data_ptr(), Aqk.data_ptr(), Qin.data_ptr(), Kout.data_ptr(),
                           carry.data_ptr<float>(), stream()), "gdn_local_fwd");
}
void gdn_local_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, const Tensor& start, const Tensor& U,
                   const Tensor& W, const Tensor& dU, const Tensor& parts, const Tensor& dO, const Tensor& Vnew, const Tensor& dcarry, Tensor& dq,
                   Tensor& dk, Tensor& dv_, Tensor& dg, Tensor& dbeta) {
  // parts: [3, n_part, B, H, L, 128] fp32 = per value-slice partial sums of (dW, dq_in, dk_out) from the state pass.
  // dq, dk: fp32 [B, L, Hv, 128] (per value head), or bf16 token-major views [B, L, Hk, 128] (Hv == Hk) written in place;
  // dv: bf16 token-major view [B, L, Hv, dv]. The views may be column ranges of one packed gradient buffer.
  const c10::cuda::CUDAGuard guard(q.device());
  check_tok_major(q, "q"); check_tok_major(k, "k"); check_tok_major(v, "v"); check_tok_major(dv_, "dv");
  const int B = v.size(0), L = v.size(1), Hv = v.size(2), dv = v.size(3), Hk = q.size(2);
  for (const Tensor* t : {&U, &W, &dU, &dO, &Vnew}) TORCH_CHECK(is_bf16(*t) && t->is_contiguous(), "gdn_local_bwd: bf16 contiguous operands");
  TORCH_CHECK(is_f32(parts) && parts.is_contiguous() && parts.dim() == 6 && parts.size(0) == 3, "gdn_local_bwd: parts [3, n, B, H, L, 128] fp32");
  TORCH_CHECK(dO.dim() == 4 && dO.size(1) == L && dO.size(2) == Hv, "gdn_local_bwd: dO token-major [B, L, H, dv]");
  TORCH_CHECK(is_f32(dg) && is_f32(dbeta) && is_f32(dcarry), "gdn_local_bwd: fp32 gate gradients");
  const bool half = is_bf16(dq);
  if (half) { check_tok_major(dq, "dq"); check_tok_major(dk, "dk"); TORCH_CHECK(dq.stride(1) == dk.stride(1) && Hv == Hk, "gdn_local_bwd: bf16 dq / dk need Hv == Hk"); }
  else TORCH_CHECK(is_f32(dq) && is_f32(dk) && dq.is_contiguous() && dk.is_contiguous(), "gdn_local_bwd: fp32 dq / dk contiguous");
  const int n_part = parts.size(1);
  const long each = parts.stride(0);
  const float* p = parts.data_ptr<float>();
  check(ghb::gdn_local_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), k.stride(1), v.stride(1), g.data_ptr<float>(), beta.data_ptr<float>(),
                           start.data_ptr<uint8_t>(), B, L, Hv, Hk, dv, U.data_ptr(), W.data_ptr(), dU.data_ptr(), p, p + each, p + 2 * each, n_part,
                           dO.data_ptr(), Vnew.data_ptr(), dcarry.data_ptr<float>(), half ? nullptr : dq.data_ptr<float>(), half ? nullptr : dk.data_ptr<float>(),
                           half ? dq.data_ptr() : nullptr, half ? dk.data_ptr() : nullptr, half ? dq.stride(1) : 0, dv_.data_ptr(), dv_.stride(1),
                           dg.data_ptr<float>(), dbeta.data_ptr<float>(), stream()), "gdn_local_bwd");
}

void decode_attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& lens, const c10::optional<Tensor>& doc_start, const Tensor& cos_t,
                      const Tensor& sin_t, Tensor& out, Tensor& part_o, Tensor& part_ml, int64_t rot, int64_t cap, int64_t splits, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(is_f32(q) && q.is_contiguous() && q.dim() == 3 && q.size(2) == 64, "decode_attention: q fp32 [B, Hq, 64]");
  check_heads(k, "k cache"); check_heads(v, "v cache");
  TORCH_CHECK(lens.scalar_type() == torch::kInt32 && is_bf16(out) && out.is_contiguous() && is_f32(part_o) && is_f32(part_ml) && is_f32(cos_t) && is_f32(sin_t),
              "decode_attention: dtypes");
  const int B = q.size(0), Hq = q.size(1), T = k.size(1), Hkv = k.size(2);
  TORCH_CHECK(part_o.numel() >= static_cast<int64_t>(B) * Hq * splits * 64 && part_ml.numel() >= static_cast<int64_t>(B) * Hq * splits * 2, "decode_attention: scratch too small");
  check(ghb::decode_attention(q.data_ptr<float>(), k.data_ptr(), v.data_ptr(), lens.data_ptr<int>(), doc_start.has_value() ? doc_start->data_ptr<int>() : nullptr,
                              cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), out.data_ptr(), part_o.data_ptr<float>(), part_ml.data_ptr<float>(), B, T, Hq,
                              Hkv, rot, cap, rot ? cos_t.size(0) : 1, splits, scale, stream()), "decode_attention");
}

// q [B, 16, 64] fp32; k, v [B, T, 256] bf16 raw grid components; gain: the key norm's [64] fp32 gain, or none.
void decode_attention_grid(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& lens, const c10::optional<Tensor>& doc_start,
                           const Tensor& cos_t, const Tensor& sin_t, const c10::optional<Tensor>& gain, Tensor& out, Tensor& part_o, Tensor& part_ml,
                           int64_t rot, int64_t cap, int64_t splits, double scale, double eps) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(is_f32(q) && q.is_contiguous() && q.dim() == 3 && q.size(1) == 16 && q.size(2) == 64, "decode_attention_grid: q fp32 [B, 16, 64]");
  TORCH_CHECK(is_bf16(k) && is_bf16(v) && k.is_contiguous() && v.is_contiguous() && k.dim() == 3 && k.size(2) == 256 && v.sizes() == k.sizes(),
              "decode_attention_grid: k, v bf16 [B, T, 256]");
  TORCH_CHECK(lens.scalar_type() == torch::kInt32 && is_bf16(out) && out.is_contiguous() && is_f32(part_o) && is_f32(part_ml) && is_f32(cos_t) && is_f32(sin_t),
              "decode_attention_grid: dtypes");
  TORCH_CHECK(!gain.has_value() || (is_f32(*gain) && gain->numel() == 64), "decode_attention_grid: gain fp32 [64]");
  const int B = q.size(0), T = k.size(1);
  TORCH_CHECK(part_o.numel() >= static_cast<int64_t>(B) * 16 * splits * 64 && part_ml.numel() >= static_cast<int64_t>(B) * 16 * splits * 2,
              "decode_attention_grid: scratch too small");
  check(ghb::decode_attention_grid(q.data_ptr<float>(), k.data_ptr(), v.data_ptr(), lens.data_ptr<int>(), doc_start.has_value() ? doc_start->data_ptr<int>() : nullptr,
                                   cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), fptr(gain), out.data_ptr(), part_o.data_ptr<float>(),
                                   part_ml.data_ptr<float>(), B, T, rot, cap, rot ? cos_t.size(0) : 1, splits, scale, eps, stream()), "decode_attention_grid");
}

// ---- fused data-parallel step over peer memory. `peers` is a CPU uint8 tensor holding the pointer table.
void comm_reduce(const Tensor& peers, int64_t rank, int64_t world, int64_t lo, int64_t n, Tensor& shard, int64_t ticket, int64_t publish_seq,
                 Tensor& acc, Tensor& counter, Tensor& err, int64_t ctas) {
  const c10::cuda::CUDAGuard guard(shard.device());
  TORCH_CHECK(!peers.is_cuda() && peers.numel() == static_cast<int64_t>(ghb::comm_peers_bytes()), "comm_reduce: peer table of ", ghb::comm_peers_bytes(), " bytes");
  TORCH_CHECK(is_f32(shard) && shard.numel() >= n, "comm_reduce: fp32 shard");
  check(ghb::comm_reduce(peers.data_ptr(), rank, world, lo, n, shard.data_ptr<float>(), static_cast<unsigned int>(ticket),
                         static_cast<unsigned int>(publish_seq), acc.data_ptr<float>(), reinterpret_cast<unsigned int*>(counter.data_ptr<int>()),
                         err.data_ptr<int>(), ctas > 0 ? static_cast<int>(ctas) : 2 * sm_count(), stream()), "comm_reduce");
}
void comm_update(const Tensor& peers, int64_t rank, int64_t world, int64_t lo, int64_t n, const Tensor& shard, Tensor& m, Tensor& v,
                 const std::vector<int64_t>& group_start, const std::vector<double>& group_wd, const std::vector<double>& group_lr, double b1, double b2,
                 double eps, double c1, double c2, double max_norm, int64_t seq, bool first, Tensor& coef_buf, const c10::optional<Tensor>& fp32_map,
                 int64_t ticket, Tensor& counter, Tensor& err, int64_t ctas) {
  const c10::cuda::CUDAGuard guard(shard.device());
  TORCH_CHECK(!peers.is_cuda() && peers.numel() == static_cast<int64_t>(ghb::comm_peers_bytes()), "comm_update: peer table");
  TORCH_CHECK(is_f32(shard) && shard.numel() >= n && m.numel() >= n && v.numel() >= n && coef_buf.numel() >= 2, "comm_update: shard / moment sizes");
  std::vector<long> gs(group_start.begin(), group_start.end());
  std::vector<float> wd(group_wd.begin(), group_wd.end()), lr(group_lr.begin(), group_lr.end());
  check(ghb::comm_update(peers.data_ptr(), rank, world, lo, n, shard.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), gs.size(), gs.data(),
                         wd.data(), lr.data(), b1, b2, eps, c1, c2, max_norm, static_cast<unsigned int>(seq), first ? 1 : 0, coef_buf.data_ptr<float>(),
                         fp32_map.has_value() ? reinterpret_cast<const unsigned int*>(fp32_map->data_ptr<int>()) : nullptr,
                         static_cast<unsigned int>(ticket), reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), err.data_ptr<int>(),
                         ctas > 0 ? static_cast<int>(ctas) : 2 * sm_count(), stream()), "comm_update");
}
void comm_wait_probe(const Tensor& flag, int64_t seq, int64_t limit_ns, Tensor& err) {
  const c10::cuda::CUDAGuard guard(flag.device());
  check(ghb::comm_wait_probe(reinterpret_cast<const unsigned int*>(flag.data_ptr<int>()), static_cast<unsigned int>(seq), limit_ns, err.data_ptr<int>(), stream()),
        "comm_wait_probe");
}
int64_t comm_peers_bytes() { return ghb::comm_peers_bytes(); }

}  // namespace

// ---- attention q / k preparation. q: [B, L, Hq, 64] view of the query projection (head stride 64 or 128 with the gate
// interleaved), k: [B, L, Hkv, 64]; cos / sin: [B * L, R2] fp32 (R2 may be 0); cos_c / sin_c: [R2] or none.
void attn_prep_fwd(const Tensor& q, const Tensor& k, const Tensor& wq, const Tensor& wk, const Tensor& cos, const Tensor& sin,
                   const c10::optional<Tensor>& cos_c, const c10::optional<Tensor>& sin_c, double eps, Tensor& qr, const c10::optional<Tensor>& qf,
                   Tensor& kr, const c10::optional<Tensor>& kf) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(is_bf16(q) && is_bf16(k) && q.dim() == 4 && k.dim() == 4 && q.size(3) == 64 && k.size(3) == 64 && q.stride(3) == 1 && k.stride(3) == 1 &&
              k.stride(2) == 64 && q.stride(0) == q.stride(1) * q.size(1) && k.stride(0) == k.stride(1) * k.size(1), "attn_prep_fwd: q / k layout");
  TORCH_CHECK(is_f32(wq) && is_f32(wk) && is_f32(cos) && is_f32(sin) && cos.is_contiguous() && sin.is_contiguous(), "attn_prep_fwd: fp32 gains and tables");
  const long tokens = q.size(0) * q.size(1);
  const int R2 = cos.numel() / std::max<long>(tokens, 1);
  check(ghb::attn_prep_fwd(q.data_ptr(), q.stride(1), q.stride(2), k.data_ptr(), k.stride(1), wq.data_ptr<float>(), wk.data_ptr<float>(), cos.data_ptr<float>(),
                           sin.data_ptr<float>(), fptr(cos_c), fptr(sin_c), q.size(2), k.size(2), R2, eps, tokens, qr.data_ptr(), vmut(qf), kr.data_ptr(), vmut(kf),
                           sm_count(), stream()), "attn_prep_fwd");
}
void attn_prep_bwd(const Tensor& q, const Tensor& k, const Tensor& wq, const Tensor& wk, const Tensor& cos, const Tensor& sin,
                   const c10::optional<Tensor>& cos_c, const c10::optional<Tensor>& sin_c, double eps, const Tensor& dqr, const c10::optional<Tensor>& dqf,
                   const Tensor& dkr, const c10::optional<Tensor>& dkf, Tensor& dqraw, Tensor& dkraw, Tensor& dw) {
  const c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(is_bf16(dqr) && dqr.is_contiguous() && is_bf16(dkr) && dkr.is_contiguous() && is_bf16(dqraw) && is_bf16(dkraw) && is_f32(dw) && dw.numel() == 128,
              "attn_prep_bwd: layout");
  TORCH_CHECK(dqraw.strides() == q.strides() && dkraw.strides() == k.strides(), "attn_prep_bwd: gradients laid out like the raw q / k");
  const long tokens = q.size(0) * q.size(1);
  const int R2 = cos.numel() / std::max<long>(tokens, 1);
  check(ghb::attn_prep_bwd(q.data_ptr(), q.stride(1), q.stride(2), k.data_ptr(), k.stride(1), wq.data_ptr<float>(), wk.data_ptr<float>(), cos.data_ptr<float>(),
                           sin.data_ptr<float>(), fptr(cos_c), fptr(sin_c), q.size(2), k.size(2), R2, eps, tokens, dqr.data_ptr(), optr(dqf), dkr.data_ptr(), optr(dkf),
                           dqraw.data_ptr(), dkraw.data_ptr(), dw.data_ptr<float>(), sm_count(), stream()), "attn_prep_bwd");
}

// o, y: [B, L, Hq, 64] contiguous; qg: [B, L, Hq * 128] contiguous (per head [q | gate]).
void gate_out_fwd(const Tensor& o, const Tensor& qg, Tensor& y) {
  const c10::cuda::CUDAGuard guard(o.device());
  TORCH_CHECK(is_bf16(o) && is_bf16(qg) && is_bf16(y) && o.is_contiguous() && qg.is_contiguous() && y.is_contiguous() && qg.numel() == 2 * o.numel(), "gate_out_fwd: layout");
  check(ghb::gate_out_fwd(o.data_ptr(), qg.data_ptr(), y.data_ptr(), o.numel() / 64, sm_count(), stream()), "gate_out_fwd");
}
void gate_out_bwd(const Tensor& dy, const Tensor& o, const Tensor& qg, Tensor& dO, Tensor& dqg) {
  const c10::cuda::CUDAGuard guard(o.device());
  TORCH_CHECK(is_bf16(dy) && dy.is_contiguous() && is_bf16(dO) && dO.is_contiguous() && is_bf16(dqg) && dqg.is_contiguous() && dqg.numel() == qg.numel(), "gate_out_bwd: layout");
  check(ghb::gate_out_bwd(dy.data_ptr(), o.data_ptr(), qg.data_ptr(), dO.data_ptr(), dqg.data_ptr(), o.numel() / 64, sm_count(), stream()), "gate_out_bwd");
}

// ---- tensor-parallel fused GEMMs. args: CPU uint8 tensor holding the kernel's argument table.
void gemm_tp(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& out, bool a_mn, bool b_mn, bool accumulate, const Tensor& args, Tensor& err) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && is_bf16(a) && is_bf16(b) && a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_tp: bf16 2-D operands");
  TORCH_CHECK(!args.is_cuda() && args.numel() == static_cast<int64_t>(ghb::tp_args_bytes()), "gemm_tp: argument table size");
  const c10::cuda::CUDAGuard guard(a.device());
  const int M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm_tp: reduction sizes differ");
  int mode = 0; long ldc = 8; void* c = nullptr;
  if (out.has_value()) {
    TORCH_CHECK(out->dim() == 2 && out->size(0) == M && out->size(1) == N && out->stride(1) == 1, "gemm_tp: output shape");
    mode = is_bf16(*out) ? 0 : (accumulate ? 2 : 1);
    TORCH_CHECK(mode == 0 || is_f32(*out), "gemm_tp: output bf16 or fp32");
    ldc = out->stride(0); c = out->data_ptr();
  }
  const int rc = ghb::gemm_tp(a.data_ptr(), b.data_ptr(), c, M, N, K, a.stride(0), b.stride(0), ldc, a_mn, b_mn, mode, args.data_ptr(),
                              err.data_ptr<int>(), sm_count(), stream());
  TORCH_CHECK(rc == 0, "gemm_tp refused (code ", rc, "): M=", M, " N=", N, " K=", K, " cuerr=", ghb::last_encode_error());
}
void tp_signal(const Tensor& args, int64_t word, const Tensor& like, int64_t wait_word, const c10::optional<Tensor>& err) {
  const c10::cuda::CUDAGuard guard(like.device());
  TORCH_CHECK(wait_word < 0 || (err.has_value() && err->is_cuda()), "tp_signal: a wait needs the status word");
  check(ghb::tp_signal(args.data_ptr(), word, wait_word, err.has_value() ? err->data_ptr<int>() : nullptr, stream()), "tp_signal");
}
// Sum of a scatter's partial rows delivered into this rank's staging slot (bounded wait for the peers' flags inside).
void tp_reduce(const Tensor& args, int64_t N, Tensor& err) {
  TORCH_CHECK(!args.is_cuda() && args.numel() == static_cast<int64_t>(ghb::tp_args_bytes()), "tp_reduce: argument table size");
  const c10::cuda::CUDAGuard guard(err.device());
  const int rc = ghb::tp_reduce(args.data_ptr(), static_cast<int>(N), err.data_ptr<int>(), sm_count(), stream());
  TORCH_CHECK(rc == 0, "tp_reduce refused (code ", rc, ")");
}
// Copy-engine delivery into (possibly a peer's) memory by address, with a flag word behind it, on a side stream.
void tp_copy_flagged(int64_t dst, const Tensor& src, int64_t bytes, int64_t flag_dst, const Tensor& flag_src, int64_t stream_handle) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && bytes <= static_cast<int64_t>(src.numel() * src.element_size()), "tp_copy_flagged: source");
  TORCH_CHECK(flag_src.is_cuda() && flag_src.scalar_type() == at::kInt && flag_src.numel() >= 1, "tp_copy_flagged: flag source");
  const c10::cuda::CUDAGuard guard(src.device());
  const int rc = ghb::tp_copy_flagged(reinterpret_cast<void*>(dst), src.data_ptr(), static_cast<size_t>(bytes), reinterpret_cast<void*>(flag_dst),
                                      flag_src.data_ptr(), reinterpret_cast<cudaStream_t>(stream_handle));
  TORCH_CHECK(rc == 0, "tp_copy_flagged refused (code ", rc, ")");
}
// Queues the copy-engine push of a gather on the caller's side streams (handles; one per peer).
void tp_push_copies(const Tensor& args, const Tensor& seq_src, int64_t pieces, const std::vector<int64_t>& stream_handles) {
  TORCH_CHECK(!args.is_cuda() && args.numel() == static_cast<int64_t>(ghb::tp_args_bytes()), "tp_push_copies: argument table size");
  TORCH_CHECK(seq_src.is_cuda() && seq_src.scalar_type() == at::kInt && seq_src.is_contiguous(), "tp_push_copies: int32 device words");
  const c10::cuda::CUDAGuard guard(seq_src.device());
  std::vector<cudaStream_t> streams;
  for (int64_t h : stream_handles) streams.push_back(reinterpret_cast<cudaStream_t>(h));
  const int rc = ghb::tp_push_copies(args.data_ptr(), seq_src.data_ptr(), pieces, streams.data(), static_cast<int>(streams.size()));
  TORCH_CHECK(rc == 0, "tp_push_copies refused (code ", rc, ")");
}
int64_t tp_args_bytes() { return ghb::tp_args_bytes(); }
int64_t tp_pad_words() { return ghb::tp_pad_words(); }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("silu_mul_fwd", &silu_mul_fwd);
  m.def("silu_mul_bwd", &silu_mul_bwd);
  m.def("adamw", &adamw);
  m.def("sumsq", &sumsq);
  m.def("cast_bf16", &cast_bf16);
  m.def("gdn_prep_fwd", &gdn_prep_fwd);
  m.def("gdn_prep_bwd", &gdn_prep_bwd);
  m.def("dual_lerp_fwd", &dual_lerp_fwd);
  m.def("dual_lerp_bwd", &dual_lerp_bwd);
  m.def("depth_mix_fwd", &depth_mix_fwd);
  m.def("depth_mix_bwd", &depth_mix_bwd);
  m.def("depth_mix_multi_fwd", &depth_mix_multi_fwd);
  m.def("depth_mix_multi_bwd", &depth_mix_multi_bwd);
  m.def("ce_grad", &ce_grad);
  m.def("gdn_step", &gdn_step);
  m.def("mx_fake", &mx_fake);
  m.def("mx_quantize", &mx_quantize);
  m.def("mx_scale_bytes", &mx_scale_bytes);
  m.def("gemm_mx", &gemm_mx);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("decode_attention", &decode_attention);
  m.def("decode_attention_grid", &decode_attention_grid);
  m.def("comm_reduce", &comm_reduce);
  m.def("comm_update", &comm_update);
  m.def("comm_wait_probe", &comm_wait_probe);
  m.def("comm_peers_bytes", &comm_peers_bytes);
  m.def("gdn_local_fwd", &gdn_local_fwd);
  m.def("gdn_local_bwd", &gdn_local_bwd);
  m.def("gdn_scan_fwd", &gdn_scan_fwd);
  m.def("gdn_scan_bwd", &gdn_scan_bwd);
  m.def("gate_out_fwd", &gate_out_fwd);
  m.def("gate_out_bwd", &gate_out_bwd);
  m.def("attn_prep_fwd", &attn_prep_fwd);
  m.def("attn_prep_bwd", &attn_prep_bwd);
  m.def("gemm_tp", &gemm_tp);
  m.def("tp_signal", &tp_signal, py::arg("args"), py::arg("word"), py::arg("like"), py::arg("wait_word") = -1, py::arg("err") = py::none());
  m.def("tp_push_copies", &tp_push_copies);
  m.def("tp_reduce", &tp_reduce);
  m.def("tp_copy_flagged", &tp_copy_flagged);
  m.def("tp_args_bytes", &tp_args_bytes);
  m.def("tp_pad_words", &tp_pad_words);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
}
