// Python bindings: thin checks + raw-pointer calls into the C entry points of fmb_api.h. Every
// function enqueues on the current CUDA stream of the tensor's device and never synchronises.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <atomic>

#include "fmb_api.h"


namespace {

using torch::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dt(const Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return FMB_BF16;
  if (t.scalar_type() == at::kFloat) return FMB_F32;
  TORCH_CHECK(false, "forgeminds_b200: unsupported dtype ", t.scalar_type());
}

// Number of kernels of this library enqueued so far by this process (reported by the benchmarks).
std::atomic<long long> g_launches{0};

void ok(int rc, const char* what, int kernels = 1) {
  TORCH_CHECK(rc == 0, "forgeminds_b200 native call '", what, "' failed with code ", rc);
  g_launches.fetch_add(kernels, std::memory_order_relaxed);
}

long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

void cuda_contig(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

const void* cptr(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// D = alpha * op(A) op(B)^T + beta * C.  A is [M,K] (a_mn=false) or [K,M] (a_mn=true); B is [N,K]
// or [K,N]. Rows may be strided (last dim contiguous).
void gemm(const Tensor& A, const Tensor& B, Tensor& D, const c10::optional<Tensor>& C, bool a_mn, bool b_mn,
          double alpha, double beta, const c10::optional<Tensor>& alpha_dev, bool allow_split,
          const c10::optional<Tensor>& status, int64_t force_bn) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && D.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: bf16 operands required");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2, "gemm: 2-D tensors required");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1, "gemm: innermost dimension must be contiguous");
  const int64_t M = a_mn ? A.size(1) : A.size(0);
  const int64_t K = a_mn ? A.size(0) : A.size(1);
  const int64_t N = b_mn ? B.size(1) : B.size(0);
  const int64_t Kb = b_mn ? B.size(0) : B.size(1);
  TORCH_CHECK(K == Kb, "gemm: inner dimensions differ: ", K, " vs ", Kb);
  TORCH_CHECK(D.size(0) == M && D.size(1) == N, "gemm: output shape mismatch");
  const bool d_f32 = D.scalar_type() == at::kFloat;
  TORCH_CHECK(d_f32 || D.scalar_type() == at::kBFloat16, "gemm: output must be bf16 or fp32");
  const void* c = nullptr;
  int64_t ldc = 0;
  int c_f32 = 0;
  if (C.has_value() && C->defined()) {
    TORCH_CHECK(C->dim() == 2 && C->size(0) == M && C->size(1) == N && C->stride(1) == 1, "gemm: C shape mismatch");
    c = C->data_ptr();
    ldc = C->stride(0);
    c_f32 = C->scalar_type() == at::kFloat;
    TORCH_CHECK(c_f32 || C->scalar_type() == at::kBFloat16, "gemm: C must be bf16 or fp32");
  }
  c10::cuda::CUDAGuard guard(A.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  int rc = fmb_gemm_bf16(A.data_ptr(), B.data_ptr(), D.data_ptr(), c, static_cast<int>(M), static_cast<int>(N),
                         static_cast<int>(K), a_mn, b_mn, A.stride(0), B.stride(0), D.stride(0), ldc, d_f32, c_f32,
                         static_cast<float>(alpha), static_cast<float>(beta), static_cast<const float*>(cptr(alpha_dev)), allow_split, st,
                         static_cast<int>(force_bn), cur_stream());
  ok(rc, "gemm_bf16");
}

// ---- products with fused epilogues (fmb_gemm_bf16_epi)
void check_bf16_rows(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.scalar_type() == at::kBFloat16 && t.stride(1) == 1, name,
              ": 2-D bf16 CUDA tensor with contiguous rows required");
}

// gu[M, 2h] = x[M, K] @ w13[2h, K].T (gate | up) and act[M, h] = silu(gate) * up in one kernel
void gemm_swiglu_fwd(const Tensor& x, const Tensor& w13, Tensor& gu, Tensor& act, Tensor& status) {
  check_bf16_rows(x, "x"); check_bf16_rows(w13, "w13"); check_bf16_rows(gu, "gu"); check_bf16_rows(act, "act");
  const int64_t M = x.size(0), K = x.size(1), h = w13.size(0) / 2;
  TORCH_CHECK(w13.size(1) == K && gu.size(0) == M && gu.size(1) == 2 * h && act.size(0) == M && act.size(1) == h);
  c10::cuda::CUDAGuard guard(x.device());
  ok(fmb_gemm_bf16_epi(x.data_ptr(), w13.data_ptr(), gu.data_ptr(), static_cast<int>(M), static_cast<int>(2 * h),
                       static_cast<int>(K), 0, 0, x.stride(0), w13.stride(0), gu.stride(0), 0, 1.f, 1,
                       static_cast<int>(h), 0, nullptr, 0, act.data_ptr(), act.stride(0), status.data_ptr<int>(),
                       cur_stream()), "gemm_swiglu_fwd");
}

// dgu[M, 2h] = SwiGLU backward of (dy[M, d] @ w2[d, h]) through gu[M, 2h]; d(act) is never stored
void gemm_swiglu_bwd(const Tensor& dy, const Tensor& w2, const Tensor& gu, Tensor& dgu, Tensor& status) {
  check_bf16_rows(dy, "dy"); check_bf16_rows(w2, "w2"); check_bf16_rows(gu, "gu"); check_bf16_rows(dgu, "dgu");
  const int64_t M = dy.size(0), K = dy.size(1), h = w2.size(1);
  TORCH_CHECK(w2.size(0) == K && gu.size(0) == M && gu.size(1) == 2 * h && dgu.sizes() == gu.sizes());
  c10::cuda::CUDAGuard guard(dy.device());
  ok(fmb_gemm_bf16_epi(dy.data_ptr(), w2.data_ptr(), dgu.data_ptr(), static_cast<int>(M), static_cast<int>(h),
                       static_cast<int>(K), 0, 1, dy.stride(0), w2.stride(0), dgu.stride(0), 0, 1.f, 2,
                       static_cast<int>(h), 0, gu.data_ptr(), gu.stride(0), nullptr, 0, status.data_ptr<int>(),
                       cur_stream()), "gemm_swiglu_bwd");
}

// out[M, N] = a @ op(b) and rowdot[M, N / seg] = sums of out * src over seg-wide column groups
// `seq` > 0: rows are (batch, t) pairs with t < seq and rowdot is stored as [batch, N / seg, seq]
void gemm_rowdot(const Tensor& a, const Tensor& b, bool b_mn, Tensor& out, const Tensor& src, Tensor& rowdot,
                 int64_t seg, int64_t seq, Tensor& status) {
  check_bf16_rows(a, "a"); check_bf16_rows(b, "b"); check_bf16_rows(out, "out"); check_bf16_rows(src, "src");
  const int64_t M = a.size(0), K = a.size(1), N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K && out.size(0) == M && out.size(1) == N && src.sizes() == out.sizes());
  TORCH_CHECK(rowdot.scalar_type() == at::kFloat && rowdot.is_contiguous() && rowdot.numel() == M * (N / seg));
  c10::cuda::CUDAGuard guard(a.device());
  ok(fmb_gemm_bf16_epi(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(M), static_cast<int>(N),
                       static_cast<int>(K), 0, b_mn, a.stride(0), b.stride(0), out.stride(0), 0, 1.f, 3,
                       static_cast<int>(seq), static_cast<int>(seg), src.data_ptr(), src.stride(0), rowdot.data_ptr(), N / seg,
                       status.data_ptr<int>(), cur_stream()), "gemm_rowdot");
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  cuda_contig(x, "x"); cuda_contig(w, "w");
  const int64_t d = x.size(-1);
  const int64_t rows = x.numel() / d;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(at::kFloat));
  ok(fmb_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, static_cast<int>(d),
                     static_cast<float>(eps), dt(x), dt(w), cur_stream()), "rmsnorm_fwd");
  return {y, rstd};
}

std::vector<Tensor> add_rmsnorm_fwd(const Tensor& x, const Tensor& delta, const Tensor& w, double eps) {
  cuda_contig(x, "x"); cuda_contig(delta, "delta"); cuda_contig(w, "w");
  const int64_t d = x.size(-1);
  const int64_t rows = x.numel() / d;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor xn = torch::empty_like(x), y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(at::kFloat));
  ok(fmb_add_rmsnorm_fwd(x.data_ptr(), delta.data_ptr(), w.data_ptr(), xn.data_ptr(), y.data_ptr(),
                         rstd.data_ptr<float>(), rows, static_cast<int>(d), static_cast<float>(eps), dt(x), dt(w),
                         cur_stream()), "add_rmsnorm_fwd");
  return {xn, y, rstd};
}

// returns (dx, dw fp32)
// dw_acc (optional, fp32 [d]): the weight gradient is ADDED to it by the column-sum kernel (a flat gradient store
// owns the parameter) and the second result is undefined.
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                const c10::optional<Tensor>& dres, bool need_dw, const c10::optional<Tensor>& dw_acc) {
  cuda_contig(dy, "dy"); cuda_contig(x, "x"); cuda_contig(w, "w");
  const int64_t d = x.size(-1);
  const int64_t rows = x.numel() / d;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  const int nb = fmb_rmsnorm_bwd_blocks(rows, static_cast<int>(d));
  const bool into = need_dw && dw_acc.has_value() && dw_acc->defined();
  if (into) TORCH_CHECK(dw_acc->is_cuda() && dw_acc->scalar_type() == at::kFloat && dw_acc->is_contiguous() &&
                        dw_acc->numel() == d, "rmsnorm_bwd: dw_acc must be a contiguous fp32 vector of the row width");
  Tensor dwp, dw;
  if (need_dw) {
    dwp = torch::empty({nb, d}, x.options().dtype(at::kFloat));
    if (!into) dw = torch::empty({d}, x.options().dtype(at::kFloat));
  }
  if (dres.has_value() && dres->defined()) cuda_contig(*dres, "dres");
  float* dw_ptr = !need_dw ? nullptr : into ? dw_acc->data_ptr<float>() : dw.data_ptr<float>();
  ok(fmb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), cptr(dres), dx.data_ptr(),
                     need_dw ? dwp.data_ptr<float>() : nullptr, dw_ptr, into ? 1 : 0, rows,
                     static_cast<int>(d), dt(x), dt(w), nb, cur_stream()), "rmsnorm_bwd", need_dw ? 2 : 1);
  return {dx, dw};
}

const int* limit_ptr(const c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->numel() >= 1, "row limit: CUDA int32 tensor required");
  return t->data_ptr<int>();
}

Tensor swiglu_fwd(const Tensor& gate, const Tensor& up, const c10::optional<Tensor>& row_limit) {
  TORCH_CHECK(gate.is_cuda() && gate.stride(-1) == 1 && up.stride(-1) == 1 && gate.dim() == 2 && up.dim() == 2);
  TORCH_CHECK(gate.stride(0) == up.stride(0), "swiglu: gate and up must share a row pitch");
  c10::cuda::CUDAGuard guard(gate.device());
  Tensor out = torch::empty({gate.size(0), gate.size(1)}, gate.options());
  ok(fmb_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.size(0), static_cast<int>(gate.size(1)),
                    gate.stride(0), dt(gate), limit_ptr(row_limit), cur_stream()), "swiglu_fwd");
  return out;
}

void swiglu_bwd(const Tensor& gate, const Tensor& up, const Tensor& dy, Tensor& dgate, Tensor& dup,
                const c10::optional<Tensor>& row_limit) {
  TORCH_CHECK(gate.dim() == 2 && gate.stride(0) == up.stride(0) && dgate.stride(0) == gate.stride(0) &&
              dup.stride(0) == gate.stride(0), "swiglu_bwd: all gate/up views must share one row pitch");
  cuda_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(gate.device());
  ok(fmb_swiglu_bwd(gate.data_ptr(), up.data_ptr(), dy.data_ptr(), dgate.data_ptr(), dup.data_ptr(), gate.size(0),
                    static_cast<int>(gate.size(1)), gate.stride(0), dt(gate), limit_ptr(row_limit), cur_stream()),
     "swiglu_bwd");
}

// q32 (optional, fp32 [rows, n_q, hd] packed): source of the first n_q heads instead of x
void rope(const Tensor& x, Tensor& out, const Tensor& cos, const Tensor& sin, int64_t T, int64_t n_rot,
          int64_t heads_total, int64_t hd, double sign, const c10::optional<Tensor>& q32) {
  cuda_contig(x, "x"); cuda_contig(out, "out"); cuda_contig(cos, "cos"); cuda_contig(sin, "sin");
  TORCH_CHECK(out.numel() == x.numel() && out.scalar_type() == x.scalar_type(), "rope: out must match x");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat, "rope tables must be fp32");
  TORCH_CHECK(cos.numel() >= T * hd / 2, "rope table shorter than the sequence");
  const int64_t rows = x.numel() / (heads_total * hd);
  const float* q32_ptr = nullptr;
  int n_q32 = 0;
  if (q32.has_value() && q32->defined()) {
    cuda_contig(*q32, "q32");
    TORCH_CHECK(q32->scalar_type() == at::kFloat && q32->numel() % (rows * hd) == 0, "rope: q32 must be fp32 [rows, n_q, hd]");
    n_q32 = static_cast<int>(q32->numel() / (rows * hd));
    TORCH_CHECK(n_q32 >= 1 && n_q32 <= n_rot, "rope: q32 holds more heads than are rotated");
    q32_ptr = q32->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  ok(fmb_rope(x.data_ptr(), out.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), rows, static_cast<int>(T),
              static_cast<int>(n_rot), static_cast<int>(heads_total), static_cast<int>(hd), static_cast<float>(sign),
              dt(x), q32_ptr, n_q32, cur_stream()), "rope");
}

std::vector<Tensor> qk_norm_rope_fwd(const Tensor& x, const Tensor& w, const Tensor& cos, const Tensor& sin, double eps) {
  cuda_contig(x, "x"); cuda_contig(w, "w"); cuda_contig(cos, "cos"); cuda_contig(sin, "sin");
  TORCH_CHECK(x.dim() == 4, "qk_norm_rope expects [B,T,H,D]");
  const int64_t T = x.size(1), H = x.size(2), hd = x.size(3);
  const int64_t rows = x.size(0) * T;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows * H}, x.options().dtype(at::kFloat));
  ok(fmb_qk_norm_rope_fwd(x.data_ptr(), w.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), y.data_ptr(),
                          rstd.data_ptr<float>(), rows, static_cast<int>(T), static_cast<int>(H), static_cast<int>(hd),
                          static_cast<float>(eps), dt(x), dt(w), cur_stream()), "qk_norm_rope_fwd");
  return {y, rstd};
}

std::vector<Tensor> qk_norm_rope_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& cos,
                                     const Tensor& sin, const Tensor& rstd) {
  cuda_contig(dy, "dy"); cuda_contig(x, "x");
  const int64_t T = x.size(1), H = x.size(2), hd = x.size(3);
  const int64_t rows = x.size(0) * T;
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  const int nb = 296;
  Tensor dwp = torch::zeros({nb, hd}, x.options().dtype(at::kFloat));
  Tensor dw = torch::empty({hd}, x.options().dtype(at::kFloat));
  ok(fmb_qk_norm_rope_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(),
                          rstd.data_ptr<float>(), dx.data_ptr(), dwp.data_ptr<float>(), dw.data_ptr<float>(), rows,
                          static_cast<int>(T), static_cast<int>(H), static_cast<int>(hd), dt(x), dt(w), nb,
                          cur_stream()), "qk_norm_rope_bwd", 2);
  return {dx, dw};
}

Tensor softmax_fwd(const Tensor& x) {
  cuda_contig(x, "x");
  const int64_t n = x.size(-1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  ok(fmb_softmax_fwd(x.data_ptr(), y.data_ptr(), x.numel() / n, static_cast<int>(n), dt(x), cur_stream()), "softmax_fwd");
  return y;
}

Tensor softmax_bwd(const Tensor& y, const Tensor& dy) {
  cuda_contig(y, "y"); cuda_contig(dy, "dy");
  const int64_t n = y.size(-1);
  c10::cuda::CUDAGuard guard(y.device());
  Tensor dx = torch::empty_like(y);
  ok(fmb_softmax_bwd(y.data_ptr(), dy.data_ptr(), dx.data_ptr(), y.numel() / n, static_cast<int>(n), dt(y),
                     cur_stream()), "softmax_bwd");
  return dx;
}

std::vector<Tensor> topk(const Tensor& x, int64_t k) {
  cuda_contig(x, "x");
  const int64_t n = x.size(-1);
  c10::cuda::CUDAGuard guard(x.device());
  auto shape = x.sizes().vec();
  shape.back() = k;
  Tensor values = torch::empty(shape, x.options());
  Tensor indices = torch::empty(shape, x.options().dtype(at::kLong));
  ok(fmb_topk(x.data_ptr(), values.data_ptr(), reinterpret_cast<long long*>(indices.data_ptr<int64_t>()),
              x.numel() / n, static_cast<int>(n), static_cast<int>(k), dt(x), cur_stream()), "topk");
  return {values, indices};
}

// logits [rows, V] bf16 are overwritten with their gradient (scaled); returns per-row losses
Tensor ce_fwd_bwd(Tensor& logits, const Tensor& labels, double grad_scale, const c10::optional<Tensor>& scale_dev,
                  int64_t ignore_index, bool write_grad) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == at::kBFloat16);
  cuda_contig(labels, "labels");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor row_loss = torch::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  ok(fmb_ce_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                    row_loss.data_ptr<float>(), logits.size(0), static_cast<int>(logits.size(1)), logits.stride(0),
                    static_cast<float>(grad_scale), static_cast<const float*>(cptr(scale_dev)), ignore_index, write_grad,
                    cur_stream()), "ce_fwd_bwd");
  return row_loss;
}

std::vector<Tensor> kl_fwd_bwd(const Tensor& student, const Tensor& teacher, double grad_scale, bool write_grad,
                               bool reuse_student) {
  cuda_contig(student, "student"); cuda_contig(teacher, "teacher");
  const int64_t V = student.size(-1);
  const int64_t rows = student.numel() / V;
  c10::cuda::CUDAGuard guard(student.device());
  Tensor row_loss = torch::empty({rows}, student.options().dtype(at::kFloat));
  Tensor grad;
  if (write_grad) grad = reuse_student ? student : torch::empty_like(student);
  ok(fmb_kl_fwd_bwd(student.data_ptr(), teacher.data_ptr(), row_loss.data_ptr<float>(),
                    write_grad ? grad.data_ptr() : nullptr, rows, static_cast<int>(V), static_cast<float>(grad_scale),
                    dt(student), write_grad, cur_stream()), "kl_fwd_bwd");
  return {row_loss, grad};
}

void sum_f32(const Tensor& x, Tensor& out, double scale, bool accumulate) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(x.device());
  ok(fmb_sum_f32(x.data_ptr<float>(), out.data_ptr<float>(), x.numel(), static_cast<float>(scale), accumulate,
                 cur_stream()), "sum_f32");
}

void adamw_flat(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const c10::optional<Tensor>& shadow, double lr,
                double beta1, double beta2, double eps, double wd, double bc1, double bc2,
                const c10::optional<Tensor>& ctl) {
  cuda_contig(p, "p"); cuda_contig(g, "g"); cuda_contig(m, "m"); cuda_contig(v, "v");
  TORCH_CHECK(p.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
              v.scalar_type() == at::kFloat, "adamw_flat: fp32 state required");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel());
  void* sh = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    TORCH_CHECK(shadow->scalar_type() == at::kBFloat16 && shadow->numel() == p.numel() && shadow->is_contiguous());
    sh = shadow->data_ptr();
  }
  c10::cuda::CUDAGuard guard(p.device());
  ok(fmb_adamw_flat(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), sh, p.numel(),
                    static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
                    static_cast<float>(eps), static_cast<float>(wd), static_cast<float>(bc1), static_cast<float>(bc2),
                    static_cast<const float*>(cptr(ctl)), cur_stream()), "adamw_flat");
}

void sqnorm(const Tensor& x, Tensor& scratch, Tensor& out, bool accumulate) {
  cuda_contig(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kFloat && scratch.numel() >= 1024 && scratch.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(x.device());
  ok(fmb_sqnorm_f32_scratch(x.data_ptr<float>(), scratch.data_ptr<float>(), out.data_ptr<float>(), x.numel(),
                            accumulate, cur_stream()), "sqnorm", 2);
}

void scale_cast(const Tensor& src, Tensor& dst, double scale) {
  cuda_contig(src, "src"); cuda_contig(dst, "dst");
  TORCH_CHECK(src.numel() == dst.numel());
  c10::cuda::CUDAGuard guard(src.device());
  ok(fmb_scale_cast(src.data_ptr(), dst.data_ptr(), src.numel(), static_cast<float>(scale), dt(src), dt(dst),
                    cur_stream()), "scale_cast");
}

void ns_axpby(const Tensor& x, const Tensor& y, Tensor& out, double a, double b) {
  cuda_contig(x, "x"); cuda_contig(y, "y"); cuda_contig(out, "out");
  c10::cuda::CUDAGuard guard(x.device());
  ok(fmb_ns_axpby(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), static_cast<float>(a), static_cast<float>(b),
                  dt(x), cur_stream()), "ns_axpby");
}

// ---- expert parallelism over peer memory
const unsigned* uflags(const Tensor& flags) {
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_cuda());
  return reinterpret_cast<const unsigned*>(flags.data_ptr<int>());
}

void ep_collect_idx(const std::vector<int64_t>& idx_ptrs, Tensor& out, int64_t n, int64_t rank, int64_t e_local,
                    const Tensor& flags, int64_t slot, int64_t epoch, double timeout_ms, Tensor& status);
void ep_gather(const std::vector<int64_t>& x_ptrs, const Tensor& token_of_slot, const Tensor& limit, Tensor& out,
               int64_t tokens_per_rank, const Tensor& flags, int64_t slot, int64_t epoch, double timeout_ms,
               Tensor& status);
void ep_combine(const std::vector<int64_t>& ys_ptrs, const std::vector<int64_t>& slot_ptrs, const Tensor& idx,
                const c10::optional<Tensor>& w, Tensor& out, int64_t e_local, int64_t rank, const Tensor& flags,
                int64_t slot, int64_t epoch, double timeout_ms, Tensor& status);
void ep_combine_bwd(const std::vector<int64_t>& dout_ptrs, const std::vector<int64_t>& w_ptrs,
                    const std::vector<int64_t>& drw_ptrs, const Tensor& ys, const Tensor& entry_of_slot,
                    const Tensor& limit, Tensor& dys, int64_t n, int64_t k, const Tensor& flags, int64_t slot,
                    int64_t epoch, double timeout_ms, Tensor& status);

// ---- 8-bit products. kind: 0 = int8, 1 = fp8 e4m3. Quantised tensors travel as uint8.
std::vector<Tensor> quant_rows(const Tensor& x, int64_t kind, int64_t block) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "quant_rows: 2-D CUDA tensor with contiguous rows");
  const int64_t rows = x.size(0), cols = x.size(1);
  TORCH_CHECK(cols % 16 == 0, "quant_rows: the row length must be a multiple of 16");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({rows, cols}, x.options().dtype(at::kByte));
  const int64_t nb = block > 0 ? (cols + block - 1) / block : 1;
  Tensor scale = block > 0 ? torch::empty({rows, nb}, x.options().dtype(at::kFloat))
                           : torch::empty({rows}, x.options().dtype(at::kFloat));
  ok(fmb_quant_rows(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), rows, static_cast<int>(cols), x.stride(0),
                    dt(x), static_cast<int>(kind), static_cast<int>(block), cur_stream()), "quant_rows");
  return {q, scale};
}

std::vector<Tensor> quant_tiles_fp8(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "quant_tiles_fp8: 2-D CUDA tensor with contiguous rows");
  const int64_t rows = x.size(0), cols = x.size(1);
  TORCH_CHECK(cols % 16 == 0, "quant_tiles_fp8: the row length must be a multiple of 16");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({rows, cols}, x.options().dtype(at::kByte));
  Tensor scale = torch::empty({(rows + 127) / 128, (cols + 127) / 128}, x.options().dtype(at::kFloat));
  ok(fmb_quant_tiles_fp8(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), static_cast<int>(rows),
                         static_cast<int>(cols), x.stride(0), dt(x), cur_stream()), "quant_tiles_fp8");
  return {q, scale};
}

// out[M, N] = (a_q[M, K] * sa) @ (b_q[N, K] * sb).T ; row scales when sa is 1-D, block scales (fp8) when 2-D.
Tensor gemm8(const Tensor& a_q, const Tensor& b_q, const Tensor& sa, const Tensor& sb, int64_t kind, bool out_f32,
             Tensor& status) {
  TORCH_CHECK(a_q.is_cuda() && b_q.is_cuda() && a_q.scalar_type() == at::kByte && b_q.scalar_type() == at::kByte);
  TORCH_CHECK(a_q.dim() == 2 && b_q.dim() == 2 && a_q.size(1) == b_q.size(1) && a_q.stride(1) == 1 && b_q.stride(1) == 1);
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat && sa.is_contiguous() && sb.is_contiguous());
  const int64_t M = a_q.size(0), N = b_q.size(0), K = a_q.size(1);
  const bool blocked = sa.dim() == 2;
  if (blocked) {
    TORCH_CHECK(sb.dim() == 2 && sa.size(0) == M && sb.size(0) == (N + 127) / 128, "gemm8: block scale shapes");
  } else {
    TORCH_CHECK(sa.numel() == M && sb.numel() == N, "gemm8: row scale shapes");
  }
  c10::cuda::CUDAGuard guard(a_q.device());
  Tensor out = torch::empty({M, N}, a_q.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  ok(fmb_gemm8(a_q.data_ptr(), b_q.data_ptr(), out.data_ptr(), static_cast<int>(M), static_cast<int>(N),
               static_cast<int>(K), a_q.stride(0), b_q.stride(0), out.stride(0), out_f32 ? 1 : 0,
               static_cast<int>(kind), sa.data_ptr<float>(), sb.data_ptr<float>(),
               blocked ? static_cast<int>(sa.size(1)) : 0, blocked ? static_cast<int>(sb.size(1)) : 0,
               status.data_ptr<int>(), cur_stream()), "gemm8");
  return out;
}

// ---- collectives over peer memory. Pointer tables are Python lists of ints (one device address per rank).
struct PtrTable {
  const void* p[FMB_MAX_PEERS];
  int world;
  explicit PtrTable(const std::vector<int64_t>& v) : world(static_cast<int>(v.size())) {
    TORCH_CHECK(world >= 1 && world <= FMB_MAX_PEERS, "peer table: 1..", FMB_MAX_PEERS, " ranks, got ", v.size());
    for (int r = 0; r < FMB_MAX_PEERS; ++r) p[r] = r < world ? reinterpret_cast<const void*>(v[r]) : nullptr;
  }
};

unsigned long long to_ns(double ms) { return static_cast<unsigned long long>(ms * 1e6); }

void comm_rs_reduce(const std::vector<int64_t>& grad_ptrs, int64_t lo, int64_t n, double scale, Tensor& partial,
                    const std::vector<int64_t>& flag_ptrs, int64_t slot, int64_t epoch, int64_t rank, double timeout_ms,
                    Tensor& status, const c10::optional<Tensor>& dst) {
  PtrTable g(grad_ptrs), f(flag_ptrs);
  TORCH_CHECK(g.world == f.world && partial.is_cuda() && partial.scalar_type() == at::kFloat);
  float* out = nullptr;
  if (dst.has_value() && dst->defined()) {
    TORCH_CHECK(dst->is_cuda() && dst->scalar_type() == at::kFloat && dst->is_contiguous() && dst->numel() >= n,
                "rs_reduce: dst must be a contiguous fp32 CUDA tensor of at least n elements");
    out = dst->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(partial.device());
  ok(fmb_comm_rs_reduce(g.p, lo, n, static_cast<float>(scale), out, partial.data_ptr<float>(),
                        static_cast<int>(partial.numel()), f.p, static_cast<int>(slot), static_cast<unsigned>(epoch),
                        static_cast<int>(rank), g.world, to_ns(timeout_ms), status.data_ptr<int>(), cur_stream()),
     "comm_rs_reduce");
}

void comm_step_reduce(const Tensor& partial, const c10::optional<Tensor>& extra_sq, const c10::optional<Tensor>& loss,
                      const std::vector<int64_t>& xchg_ptrs, const std::vector<int64_t>& flag_ptrs, int64_t slot,
                      int64_t epoch, int64_t rank, double max_norm, bool skip_nonfinite, Tensor& stats, Tensor& ctl,
                      double timeout_ms, Tensor& status) {
  PtrTable x(xchg_ptrs), f(flag_ptrs);
  TORCH_CHECK(x.world == f.world && partial.is_cuda() && partial.scalar_type() == at::kFloat);
  TORCH_CHECK(stats.scalar_type() == at::kFloat && stats.numel() >= 3 && ctl.scalar_type() == at::kFloat &&
              ctl.numel() >= 2);
  if (loss.has_value() && loss->defined()) TORCH_CHECK(loss->scalar_type() == at::kFloat && loss->is_cuda());
  c10::cuda::CUDAGuard guard(partial.device());
  ok(fmb_comm_step_reduce(partial.data_ptr<float>(), static_cast<int>(partial.numel()),
                          static_cast<const float*>(cptr(extra_sq)), static_cast<const float*>(cptr(loss)), x.p, f.p,
                          static_cast<int>(slot), static_cast<unsigned>(epoch), static_cast<int>(rank), x.world,
                          static_cast<float>(max_norm), skip_nonfinite ? 1 : 0, stats.data_ptr<float>(),
                          ctl.data_ptr<float>(), to_ns(timeout_ms), status.data_ptr<int>(), cur_stream()),
     "comm_step_reduce");
}

void comm_adamw_push(Tensor& master, const Tensor& grad, Tensor& m, Tensor& v, const std::vector<int64_t>& shadow_ptrs,
                     const Tensor& off, const Tensor& soff, const Tensor& len, const Tensor& wd, double lr,
                     double beta1, double beta2, double eps, double bc1, double bc2, const Tensor& ctl,
                     bool grad_compact) {
  PtrTable s(shadow_ptrs);
  TORCH_CHECK(master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
              v.scalar_type() == at::kFloat, "adamw_push: fp32 state required");
  TORCH_CHECK(off.scalar_type() == at::kLong && soff.scalar_type() == at::kLong && len.scalar_type() == at::kInt &&
              wd.scalar_type() == at::kFloat && off.is_cuda() && soff.is_cuda() && len.is_cuda() && wd.is_cuda());
  TORCH_CHECK(soff.numel() == off.numel() && len.numel() == off.numel() && wd.numel() == off.numel());
  c10::cuda::CUDAGuard guard(master.device());
  ok(fmb_comm_adamw_push(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                         s.p, s.world, reinterpret_cast<const long long*>(off.data_ptr<int64_t>()),
                         reinterpret_cast<const long long*>(soff.data_ptr<int64_t>()), len.data_ptr<int>(),
                         wd.data_ptr<float>(), static_cast<int>(off.numel()), static_cast<float>(lr),
                         static_cast<float>(beta1), static_cast<float>(beta2), static_cast<float>(eps),
                         static_cast<float>(bc1), static_cast<float>(bc2), ctl.data_ptr<float>(),
                         grad_compact ? 1 : 0, cur_stream()),
     "comm_adamw_push");
}

void comm_push_cast(const Tensor& master, const std::vector<int64_t>& shadow_ptrs, const Tensor& off, const Tensor& len) {
  PtrTable s(shadow_ptrs);
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && off.is_cuda() && len.is_cuda() &&
              off.scalar_type() == at::kLong && len.scalar_type() == at::kInt && off.numel() == len.numel(),
              "push_cast: fp32 master, int64 offsets and int32 lengths on the device");
  c10::cuda::CUDAGuard guard(master.device());
  ok(fmb_comm_push_cast(master.data_ptr<float>(), s.p, s.world, reinterpret_cast<const long long*>(off.data_ptr<int64_t>()),
                        len.data_ptr<int>(), static_cast<int>(off.numel()), cur_stream()), "comm_push_cast");
}

// Product with operands / output spread over the ranks (see fmb_gemm_bf16_peer). `gather` = 1 / 2: `a` / `b` is this
// rank's full-size symmetric buffer of the gathered operand and `gather_ptrs` every rank's; `ready` holds one int
// per 128 rows of it. With `d_ptrs`, `d` is this rank's bf16 staging buffer [world * rows_per_rank, N].
void gemm_peer(const Tensor& a, const Tensor& b, Tensor& d, bool a_mn, bool b_mn, double alpha, bool accumulate,
               int64_t rank, int64_t world, int64_t gather, const std::vector<int64_t>& gather_ptrs,
               const c10::optional<Tensor>& ready, const std::vector<int64_t>& d_ptrs, const Tensor& flags,
               int64_t slot, int64_t epoch, double timeout_ms, Tensor& status) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda() && a.dim() == 2 && b.dim() == 2 && d.dim() == 2);
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm_peer: bf16 operands required");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm_peer: innermost dimension must be contiguous");
  TORCH_CHECK(world >= 1 && world <= FMB_MAX_PEERS && gather >= 0 && gather <= 2);
  const bool d_sh = !d_ptrs.empty();
  TORCH_CHECK((gather == 0 || static_cast<int64_t>(gather_ptrs.size()) == world) &&
              (!d_sh || static_cast<int64_t>(d_ptrs.size()) == world), "gemm_peer: one pointer per rank");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "gemm_peer: inner dimensions differ");
  TORCH_CHECK(d.size(1) == N && d.size(0) == M, "gemm_peer: output shape mismatch");
  const bool d_f32 = d.scalar_type() == at::kFloat;
  TORCH_CHECK(d_f32 || d.scalar_type() == at::kBFloat16);
  int* ready_ptr = nullptr;
  if (gather) {
    TORCH_CHECK(ready.has_value() && ready->scalar_type() == at::kInt && ready->is_cuda() &&
                ready->numel() >= ((gather == 1 ? (a_mn ? K : M) : K) + 127) / 128, "gemm_peer: ready counters");
    ready_ptr = ready->data_ptr<int>();
  }
  const void* gp[FMB_MAX_PEERS];
  void* dp[FMB_MAX_PEERS];
  for (int r = 0; r < FMB_MAX_PEERS; ++r) {
    gp[r] = gather && r < world ? reinterpret_cast<const void*>(gather_ptrs[r]) : nullptr;
    dp[r] = d_sh && r < world ? reinterpret_cast<void*>(d_ptrs[r]) : nullptr;
  }
  c10::cuda::CUDAGuard guard(a.device());
  ok(fmb_gemm_bf16_peer(a.data_ptr(), b.data_ptr(), d.data_ptr(), static_cast<int>(M), static_cast<int>(N),
                        static_cast<int>(K), a_mn, b_mn, a.stride(0), b.stride(0), d.stride(0), d_f32,
                        static_cast<float>(alpha), accumulate ? 1 : 0, static_cast<int>(rank), static_cast<int>(world),
                        static_cast<int>(gather), gather ? gp : nullptr, ready_ptr, d_sh ? dp : nullptr,
                        uflags(flags), static_cast<int>(slot), static_cast<unsigned>(epoch), to_ns(timeout_ms),
                        status.data_ptr<int>(), cur_stream()), "gemm_bf16_peer", gather ? 2 : 1);
}

// out[rows, cols] = sum of the slices of staging[world, rows, cols] (+ residual), all bf16
void comm_sum_partials(const Tensor& staging, const c10::optional<Tensor>& residual, Tensor& out, int64_t world) {
  TORCH_CHECK(staging.is_cuda() && staging.is_contiguous() && staging.scalar_type() == at::kBFloat16 &&
              out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 &&
              staging.numel() == out.numel() * world);
  if (residual.has_value() && residual->defined())
    TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == at::kBFloat16 && residual->numel() == out.numel());
  c10::cuda::CUDAGuard guard(out.device());
  ok(fmb_comm_sum_partials(staging.data_ptr(), cptr(residual), out.data_ptr(), out.size(0), static_cast<int>(out.size(1)),
                           static_cast<int>(world), cur_stream()), "comm_sum_partials");
}

// Post this rank's epoch on a flag slot of every rank (no wait): "my shard is ready".
void comm_signal(const std::vector<int64_t>& flag_ptrs, int64_t slot, int64_t epoch, int64_t rank, Tensor& status) {
  PtrTable f(flag_ptrs);
  c10::cuda::CUDAGuard guard(status.device());
  ok(fmb_comm_signal(f.p, static_cast<int>(slot), static_cast<unsigned>(epoch), static_cast<int>(rank), f.world,
                     cur_stream()), "comm_signal");
}

void comm_barrier(const std::vector<int64_t>& flag_ptrs, int64_t slot, int64_t epoch, int64_t rank, double timeout_ms,
                  Tensor& status) {
  PtrTable f(flag_ptrs);
  c10::cuda::CUDAGuard guard(status.device());
  ok(fmb_comm_barrier(f.p, static_cast<int>(slot), static_cast<unsigned>(epoch), static_cast<int>(rank), f.world,
                      to_ns(timeout_ms), status.data_ptr<int>(), cur_stream()), "comm_barrier");
}

void ep_collect_idx(const std::vector<int64_t>& idx_ptrs, Tensor& out, int64_t n, int64_t rank, int64_t e_local,
                    const Tensor& flags, int64_t slot, int64_t epoch, double timeout_ms, Tensor& status) {
  PtrTable p(idx_ptrs);
  TORCH_CHECK(out.scalar_type() == at::kInt && out.is_cuda() && out.numel() == n * p.world);
  c10::cuda::CUDAGuard guard(out.device());
  ok(fmb_ep_collect_idx(p.p, out.data_ptr<int>(), n, p.world, static_cast<int>(rank), static_cast<int>(e_local),
                        uflags(flags), static_cast<int>(slot), static_cast<unsigned>(epoch), to_ns(timeout_ms),
                        status.data_ptr<int>(), cur_stream()), "ep_collect_idx");
}

void ep_clamp_plan(Tensor& region, int64_t rows, Tensor& status, int64_t code) {
  TORCH_CHECK(region.is_cuda() && region.scalar_type() == at::kInt && region.is_contiguous() && region.numel() % 3 == 0);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(region.device());
  ok(fmb_ep_clamp_plan(region.data_ptr<int>(), static_cast<int>(region.numel() / 3), static_cast<int>(rows),
                       status.data_ptr<int>(), static_cast<int>(code), cur_stream()), "ep_clamp_plan");
}

void ep_gather(const std::vector<int64_t>& x_ptrs, const Tensor& token_of_slot, const Tensor& limit, Tensor& out,
               int64_t tokens_per_rank, const Tensor& flags, int64_t slot, int64_t epoch, double timeout_ms,
               Tensor& status) {
  PtrTable p(x_ptrs);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.is_contiguous());
  TORCH_CHECK(token_of_slot.scalar_type() == at::kInt && token_of_slot.numel() >= out.size(0) && limit.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(out.device());
  ok(fmb_ep_gather(p.p, token_of_slot.data_ptr<int>(), limit.data_ptr<int>(), out.data_ptr(), out.size(0),
                   static_cast<int>(out.size(1)), tokens_per_rank, p.world, uflags(flags), static_cast<int>(slot),
                   static_cast<unsigned>(epoch), to_ns(timeout_ms), status.data_ptr<int>(), cur_stream()), "ep_gather");
}

void ep_combine(const std::vector<int64_t>& ys_ptrs, const std::vector<int64_t>& slot_ptrs, const Tensor& idx,
                const c10::optional<Tensor>& w, Tensor& out, int64_t e_local, int64_t rank, const Tensor& flags,
                int64_t slot, int64_t epoch, double timeout_ms, Tensor& status) {
  PtrTable y(ys_ptrs), s(slot_ptrs);
  TORCH_CHECK(y.world == s.world && idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous());
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.is_contiguous() && out.size(0) == idx.size(0));
  if (w.has_value() && w->defined()) TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == idx.numel());
  c10::cuda::CUDAGuard guard(out.device());
  ok(fmb_ep_combine(y.p, s.p, idx.data_ptr<int>(), static_cast<const float*>(cptr(w)), out.data_ptr(), idx.size(0),
                    static_cast<int>(idx.size(1)), static_cast<int>(out.size(1)), static_cast<int>(e_local),
                    static_cast<int>(rank), y.world, uflags(flags), static_cast<int>(slot),
                    static_cast<unsigned>(epoch), to_ns(timeout_ms), status.data_ptr<int>(), cur_stream()), "ep_combine");
}

void ep_combine_bwd(const std::vector<int64_t>& dout_ptrs, const std::vector<int64_t>& w_ptrs,
                    const std::vector<int64_t>& drw_ptrs, const Tensor& ys, const Tensor& entry_of_slot,
                    const Tensor& limit, Tensor& dys, int64_t n, int64_t k, const Tensor& flags, int64_t slot,
                    int64_t epoch, double timeout_ms, Tensor& status) {
  PtrTable g(dout_ptrs), w(w_ptrs), dr(drw_ptrs);
  TORCH_CHECK(g.world == w.world && g.world == dr.world);
  TORCH_CHECK(ys.scalar_type() == at::kBFloat16 && ys.dim() == 2 && ys.is_contiguous() && dys.sizes() == ys.sizes() &&
              dys.is_contiguous() && entry_of_slot.scalar_type() == at::kInt && entry_of_slot.numel() >= ys.size(0));
  c10::cuda::CUDAGuard guard(ys.device());
  ok(fmb_ep_combine_bwd(g.p, w.p, dr.p, ys.data_ptr(), entry_of_slot.data_ptr<int>(), limit.data_ptr<int>(),
                        dys.data_ptr(), ys.size(0), n, static_cast<int>(k), static_cast<int>(ys.size(1)), g.world,
                        uflags(flags), static_cast<int>(slot), static_cast<unsigned>(epoch), to_ns(timeout_ms),
                        status.data_ptr<int>(), cur_stream()), "ep_combine_bwd");
}

// ---- router / MoE
std::vector<Tensor> router_fwd(const Tensor& logits, int64_t k) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  const int64_t rows = logits.size(0), E = logits.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  auto f32 = logits.options().dtype(at::kFloat);
  auto i32 = logits.options().dtype(at::kInt);
  const int nb = fmb_router_blocks(rows);
  Tensor probs = torch::empty({rows, E}, f32), weights = torch::empty({rows, k}, f32), idx = torch::empty({rows, k}, i32);
  Tensor lse = torch::empty({rows}, f32), partial = torch::empty({nb, E + 1}, f32), counts = torch::zeros({E}, i32);
  ok(fmb_router_fwd(logits.data_ptr(), logits.stride(0), dt(logits), probs.data_ptr<float>(), weights.data_ptr<float>(),
                    idx.data_ptr<int>(), lse.data_ptr<float>(), partial.data_ptr<float>(), counts.data_ptr<int>(), rows,
                    static_cast<int>(E), static_cast<int>(k), nb, cur_stream()), "router_fwd");
  return {probs, weights, idx, lse, partial, counts};
}

Tensor router_bwd(const Tensor& probs, const Tensor& idx, const Tensor& weights, const Tensor& lse,
                  const c10::optional<Tensor>& dweights, const c10::optional<Tensor>& aux_grad,
                  const c10::optional<Tensor>& zc, at::ScalarType out_dtype) {
  const int64_t rows = probs.size(0), E = probs.size(1), k = idx.size(1);
  c10::cuda::CUDAGuard guard(probs.device());
  Tensor dl = torch::empty({rows, E}, probs.options().dtype(out_dtype));
  if (dweights.has_value() && dweights->defined()) cuda_contig(*dweights, "dweights");
  ok(fmb_router_bwd(probs.data_ptr<float>(), idx.data_ptr<int>(), weights.data_ptr<float>(), lse.data_ptr<float>(),
                    static_cast<const float*>(cptr(dweights)), static_cast<const float*>(cptr(aux_grad)),
                    static_cast<const float*>(cptr(zc)), dl.data_ptr(), E, dt(dl), rows, static_cast<int>(E),
                    static_cast<int>(k), cur_stream()), "router_bwd");
  return dl;
}

// returns (slot_of_entry [N*k], token_of_slot [max_slots], region [E,3], meta [1])
std::vector<Tensor> moe_plan(const Tensor& idx, int64_t E, int64_t align, int64_t cap, int64_t mode, int64_t max_slots) {
  cuda_contig(idx, "idx");
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.dim() == 2);
  const int64_t entries = idx.numel(), k = idx.size(1);
  c10::cuda::CUDAGuard guard(idx.device());
  auto i32 = idx.options();
  const int64_t nchunks = (entries + 1023) / 1024;
  Tensor chunk = torch::empty({nchunks, E}, i32), region = torch::empty({E, 3}, i32), meta = torch::empty({1}, i32);
  Tensor slot_of = torch::empty({entries}, i32), token_of = torch::full({max_slots}, -1, i32);
  ok(fmb_moe_plan(idx.data_ptr<int>(), chunk.data_ptr<int>(), region.data_ptr<int>(), meta.data_ptr<int>(),
                  slot_of.data_ptr<int>(), token_of.data_ptr<int>(), entries, static_cast<int>(E), static_cast<int>(k),
                  static_cast<int>(align), static_cast<int>(cap), static_cast<int>(mode), cur_stream()), "moe_plan", 3);
  return {slot_of, token_of, region, meta};
}

Tensor moe_gather(const Tensor& x, const Tensor& token_of_slot) {
  cuda_contig(x, "x"); cuda_contig(token_of_slot, "token_of_slot");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({token_of_slot.numel(), x.size(1)}, x.options());
  ok(fmb_moe_gather(x.data_ptr(), token_of_slot.data_ptr<int>(), out.data_ptr(), token_of_slot.numel(),
                    static_cast<int>(x.size(1)), cur_stream()), "moe_gather");
  return out;
}

Tensor moe_combine(const Tensor& ys, const Tensor& slot_of_entry, const c10::optional<Tensor>& w, int64_t tokens, int64_t k) {
  cuda_contig(ys, "ys"); cuda_contig(slot_of_entry, "slot_of_entry");
  TORCH_CHECK(ys.scalar_type() == at::kBFloat16 && ys.dim() == 2);
  c10::cuda::CUDAGuard guard(ys.device());
  Tensor out = torch::empty({tokens, ys.size(1)}, ys.options());
  ok(fmb_moe_combine(ys.data_ptr(), slot_of_entry.data_ptr<int>(), static_cast<const float*>(cptr(w)), out.data_ptr(),
                     tokens, static_cast<int>(k), static_cast<int>(ys.size(1)), cur_stream()), "moe_combine");
  return out;
}

std::vector<Tensor> moe_combine_bwd(const Tensor& dout, const Tensor& ys, const Tensor& slot_of_entry, const Tensor& w,
                                    int64_t k) {
  cuda_contig(dout, "dout"); cuda_contig(ys, "ys");
  c10::cuda::CUDAGuard guard(ys.device());
  Tensor dys = torch::zeros_like(ys);
  Tensor dw = torch::empty({slot_of_entry.numel()}, ys.options().dtype(at::kFloat));
  ok(fmb_moe_combine_bwd(dout.data_ptr(), ys.data_ptr(), slot_of_entry.data_ptr<int>(), w.data_ptr<float>(),
                         dys.data_ptr(), dw.data_ptr<float>(), slot_of_entry.numel(), static_cast<int>(k),
                         static_cast<int>(ys.size(1)), cur_stream()), "moe_combine_bwd");
  return {dys, dw};
}

// Row-grouped product: out[rows, N] = a[rows, K] @ B[group(row)]^T where `b` is [G, N, K] (b_mn=false)
// or [G, K, N] (b_mn=true) and `tile_group[rows / 128]` names the group of each 128-row tile (-1: skip).
// pair_aligned: every group starts on a multiple of 256 rows (and the row count is one), so 256-row tiles on CTA
// pairs may serve the product
void gemm_grouped_rows(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& tile_group, bool b_mn,
                       bool accumulate, const c10::optional<Tensor>& status, bool pair_aligned) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && b.dim() == 3 && out.dim() == 2 && a.stride(1) == 1 && b.is_contiguous() &&
              out.stride(1) == 1 && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  const int64_t M = a.size(0), K = a.size(1), G = b.size(0);
  const int64_t N = b_mn ? b.size(2) : b.size(1);
  TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == K && out.size(0) == M && out.size(1) == N && M % 128 == 0);
  TORCH_CHECK(tile_group.numel() >= M / 128 && tile_group.scalar_type() == at::kInt);
  TORCH_CHECK(!pair_aligned || M % 256 == 0, "pair-aligned groups need a row count that is a multiple of 256");
  c10::cuda::CUDAGuard guard(a.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  const bool f32 = out.scalar_type() == at::kFloat;
  ok(fmb_gemm_bf16_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), accumulate ? out.data_ptr() : nullptr,
                           static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), 0, b_mn, a.stride(0),
                           b.stride(1), out.stride(0), out.stride(0), f32, f32, 1.f, accumulate ? 1.f : 0.f,
                           pair_aligned ? 3 : 1, static_cast<int>(G),
                           tile_group.data_ptr<int>(), nullptr, b.stride(0), 0, st, cur_stream()), "gemm_grouped_rows");
}

// Batched product out[g] = alpha * a[g] @ op(b[g]) + beta * c[g] in one launch: a [G, M, K] (M a multiple of
// 128), b [G, N, K] or, with b_mn, [G, K, N]; `tile_group[i]` = i / (M / 128) names the batch entry of row tile i.
void gemm_batched(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& c, bool b_mn, double alpha,
                  double beta, const Tensor& tile_group, const c10::optional<Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 3 && b.dim() == 3 && out.dim() == 3 && a.is_contiguous() && b.is_contiguous() &&
              out.is_contiguous() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  const int64_t G = a.size(0), M = a.size(1), K = a.size(2);
  const int64_t N = b_mn ? b.size(2) : b.size(1);
  TORCH_CHECK(b.size(0) == G && (b_mn ? b.size(1) : b.size(2)) == K && out.size(0) == G && out.size(1) == M &&
              out.size(2) == N && M % 128 == 0);
  TORCH_CHECK(tile_group.numel() >= G * M / 128 && tile_group.scalar_type() == at::kInt);
  const bool f32 = out.scalar_type() == at::kFloat;
  const void* cp = nullptr;
  bool c_f32 = false;
  if (c.has_value() && c->defined()) {
    TORCH_CHECK(c->is_contiguous() && c->sizes() == out.sizes());
    cp = c->data_ptr();
    c_f32 = c->scalar_type() == at::kFloat;
  }
  c10::cuda::CUDAGuard guard(a.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  ok(fmb_gemm_bf16_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), cp, static_cast<int>(G * M), static_cast<int>(N),
                           static_cast<int>(K), 0, b_mn, K, b.stride(1), N, N, f32, c_f32, static_cast<float>(alpha),
                           static_cast<float>(beta), M % 256 == 0 ? 3 : 1,      // entries start on multiples of 256 rows
                           static_cast<int>(G), tile_group.data_ptr<int>(), nullptr,
                           b.stride(0), 0, st, cur_stream()), "gemm_batched");
}

// Per-group weight gradient: out[g] [M, N] (+)= a[rows_g, M]^T @ b[rows_g, N]; `region` is [G, 3] int32
// {first row, used, padded rows}. `accumulate` adds to `out` (fp32) instead of overwriting it.
void gemm_grouped_wgrad(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& region, bool accumulate,
                        const c10::optional<Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && b.dim() == 2 && out.dim() == 3 && out.is_contiguous() && a.stride(1) == 1 &&
              b.stride(1) == 1 && a.size(0) == b.size(0) && a.scalar_type() == at::kBFloat16 &&
              b.scalar_type() == at::kBFloat16);
  const int64_t rows = a.size(0), M = a.size(1), N = b.size(1), G = out.size(0);
  TORCH_CHECK(out.size(1) == M && out.size(2) == N && region.numel() >= 3 * G && region.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(a.device());
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  const bool f32 = out.scalar_type() == at::kFloat;
  if (!accumulate) out.zero_();           // groups without rows are skipped by the kernel
  ok(fmb_gemm_bf16_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), accumulate ? out.data_ptr() : nullptr,
                           static_cast<int>(M), static_cast<int>(N), static_cast<int>(rows), 1, 1, a.stride(0),
                           b.stride(0), out.stride(1), out.stride(1), f32, f32, 1.f, accumulate ? 1.f : 0.f, 2,
                           static_cast<int>(G), nullptr, region.data_ptr<int>(), 0, out.stride(0), st, cur_stream()),
     "gemm_grouped_wgrad");
}

Tensor moe_tile_groups(const Tensor& region, int64_t n_tiles) {
  cuda_contig(region, "region");
  c10::cuda::CUDAGuard guard(region.device());
  Tensor tg = torch::empty({n_tiles}, region.options());
  ok(fmb_moe_tile_groups(region.data_ptr<int>(), tg.data_ptr<int>(), static_cast<int>(n_tiles),
                         static_cast<int>(region.numel() / 3), cur_stream()), "moe_tile_groups");
  return tg;
}

#ifdef FMB_WITH_ATTENTION
// q [B,T,Hq,hd], k/v [B,T,Hkv,hd] (rows may be views into one fused qkv buffer): returns (o, lse)
std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale, bool causal,
                             const c10::optional<Tensor>& status) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && q.scalar_type() == at::kBFloat16);
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && q.stride(2) == hd && k.stride(2) == hd &&
              v.stride(2) == hd, "attention: heads must be packed inside a token row");
  TORCH_CHECK(q.stride(0) == T * q.stride(1) && k.stride(0) == T * k.stride(1) && v.stride(0) == T * v.stride(1) &&
              k.stride(1) == v.stride(1), "attention: batch must be contiguous over tokens");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor o = torch::empty({B, T, Hq, hd}, q.options());
  Tensor lse = torch::empty({B, Hq, T}, q.options().dtype(at::kFloat));
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  ok(fmb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), static_cast<int>(B),
                  static_cast<int>(T), static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<int>(hd), q.stride(1),
                  k.stride(1), o.stride(1), static_cast<float>(scale), causal, st, cur_stream()), "attn_fwd");
  return {o, lse};
}

// writes dq/dk/dv into the given (possibly strided) views. Without dq the query gradient is only returned as
// the fp32 sum [B, T, Hq, hd] the kernel accumulates (the caller's next pass converts it).
Tensor attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o, const Tensor& lse,
                const c10::optional<Tensor>& dq_out, Tensor& dk, Tensor& dv, double scale, bool causal,
                const c10::optional<Tensor>& status, const c10::optional<Tensor>& delta_in) {
  const bool have_dq = dq_out.has_value() && dq_out->defined();
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2);
  TORCH_CHECK(d_o.is_contiguous() && o.is_contiguous(), "attention backward: o and d_o must be contiguous");
  TORCH_CHECK(dk.stride(1) == dv.stride(1), "attention backward: dk and dv must share a token pitch");
  c10::cuda::CUDAGuard guard(q.device());
  const bool have_delta = delta_in.has_value() && delta_in->defined();   // [B, Hq, T] fp32 computed elsewhere
  if (have_delta) TORCH_CHECK(delta_in->scalar_type() == at::kFloat && delta_in->is_contiguous() && delta_in->numel() == B * Hq * T);
  Tensor delta = have_delta ? *delta_in : torch::empty({B, Hq, T}, q.options().dtype(at::kFloat));
  Tensor dq_acc = torch::zeros({B, T, Hq, hd}, q.options().dtype(at::kFloat));
  int* st = status.has_value() && status->defined() ? status->data_ptr<int>() : nullptr;
  ok(fmb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                  have_dq ? dq_out->data_ptr() : nullptr, dk.data_ptr(), dv.data_ptr(), delta.data_ptr<float>(),
                  dq_acc.data_ptr<float>(),
                  static_cast<int>(B), static_cast<int>(T), static_cast<int>(Hq), static_cast<int>(Hkv),
                  static_cast<int>(hd), q.stride(1), k.stride(1), o.stride(1), have_dq ? dq_out->stride(1) : Hq * hd,
                  dk.stride(1), static_cast<float>(scale), causal, have_delta ? 1 : 0, st, cur_stream()), "attn_bwd",
     (have_delta ? 2 : 3) - (have_dq ? 0 : 1));
  return dq_acc;
}
#endif

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "forgeminds_b200 native kernels (sm_100a)";
  m.def("launch_count", &launch_count);
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("rstd"),
        pybind11::arg("dres"), pybind11::arg("need_dw"), pybind11::arg("dw_acc") = pybind11::none());
  m.def("swiglu_fwd", &swiglu_fwd, pybind11::arg("gate"), pybind11::arg("up"), pybind11::arg("row_limit") = pybind11::none());
  m.def("swiglu_bwd", &swiglu_bwd, pybind11::arg("gate"), pybind11::arg("up"), pybind11::arg("dy"), pybind11::arg("dgate"),
        pybind11::arg("dup"), pybind11::arg("row_limit") = pybind11::none());
  m.def("rope", &rope, pybind11::arg("x"), pybind11::arg("out"), pybind11::arg("cos"), pybind11::arg("sin"), pybind11::arg("T"),
        pybind11::arg("n_rot"), pybind11::arg("heads_total"), pybind11::arg("hd"), pybind11::arg("sign"),
        pybind11::arg("q32") = pybind11::none());
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("softmax_fwd", &softmax_fwd);
  m.def("softmax_bwd", &softmax_bwd);
  m.def("topk", &topk);
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("kl_fwd_bwd", &kl_fwd_bwd);
  m.def("sum_f32", &sum_f32);
  m.def("adamw_flat", &adamw_flat);
  m.def("sqnorm", &sqnorm);
  m.def("comm_rs_reduce", &comm_rs_reduce, py::arg("grad_ptrs"), py::arg("lo"), py::arg("n"), py::arg("scale"),
        py::arg("partial"), py::arg("flag_ptrs"), py::arg("slot"), py::arg("epoch"), py::arg("rank"),
        py::arg("timeout_ms"), py::arg("status"), py::arg("dst") = c10::optional<Tensor>());
  m.def("comm_step_reduce", &comm_step_reduce);
  m.def("comm_adamw_push", &comm_adamw_push, py::arg("master"), py::arg("grad"), py::arg("m"), py::arg("v"),
        py::arg("shadow_ptrs"), py::arg("off"), py::arg("soff"), py::arg("len"), py::arg("wd"), py::arg("lr"),
        py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("bc1"), py::arg("bc2"), py::arg("ctl"),
        py::arg("grad_compact") = false);
  m.def("comm_barrier", &comm_barrier);
  m.def("comm_push_cast", &comm_push_cast);
  m.def("debug_bounds", []() { return fmb_debug_bounds_enabled() != 0; });
  m.def("debug_register", [](int64_t base, int64_t bytes, Tensor& status) {
    c10::cuda::CUDAGuard guard(status.device());
    const int rc = fmb_debug_register_extent(reinterpret_cast<const void*>(base), static_cast<unsigned long long>(bytes),
                                             status.data_ptr<int>());
    TORCH_CHECK(rc == 0, "forgeminds_b200: debug_register failed with code ", rc);
  });
  m.def("gemm_swiglu_fwd", &gemm_swiglu_fwd);
  m.def("gemm_swiglu_bwd", &gemm_swiglu_bwd);
  m.def("gemm_rowdot", &gemm_rowdot);
  m.def("ep_collect_idx", &ep_collect_idx);
  m.def("ep_clamp_plan", &ep_clamp_plan);
  m.def("ep_gather", &ep_gather);
  m.def("ep_combine", &ep_combine);
  m.def("ep_combine_bwd", &ep_combine_bwd);
  m.def("quant_rows", &quant_rows);
  m.def("quant_tiles_fp8", &quant_tiles_fp8);
  m.def("gemm8", &gemm8);
  m.def("comm_signal", &comm_signal);
  m.def("gemm_peer", &gemm_peer);
  m.def("comm_sum_partials", &comm_sum_partials);
  m.def("comm_adam_chunk", []() { return fmb_comm_adam_chunk(); });
  m.attr("MAX_PEERS") = FMB_MAX_PEERS;
  m.def("scale_cast", &scale_cast);
  m.def("ns_axpby", &ns_axpby);
  m.def("router_fwd", &router_fwd);
  m.def("router_bwd", &router_bwd);
  m.def("moe_plan", &moe_plan);
  m.def("gemm_grouped_rows", &gemm_grouped_rows, pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("out"),
        pybind11::arg("tile_group"), pybind11::arg("b_mn"), pybind11::arg("accumulate"), pybind11::arg("status"),
        pybind11::arg("pair_aligned") = false);
  m.def("gemm_grouped_wgrad", &gemm_grouped_wgrad);
  m.def("gemm_batched", &gemm_batched);
  m.def("moe_tile_groups", &moe_tile_groups);
  m.def("moe_gather", &moe_gather);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
#ifdef FMB_WITH_ATTENTION
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
#endif
}
