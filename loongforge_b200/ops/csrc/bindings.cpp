// Torch bindings of the sm_100a kernels. Every function runs on the current CUDA
// stream, checks shapes/dtypes/alignment on the host, and counts the kernels it
// launches (`launch_count`) so that benchmarks can report how many of this
// library's kernels ran inside a timed region.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include "elementwise.h"
#include "gemm_sm100.h"
#include "wait_budget.h"
#ifdef LF_HAVE_ATTN
#include "attention_sm100.h"
#endif
#ifdef LF_HAVE_PEER
#include "peer_gemm.h"
#endif
#ifdef LF_HAVE_GROUPED
#include "grouped_gemm_sm100.h"
#endif
#ifdef LF_HAVE_MOE_PEER
#include "moe_peer.h"
#endif
#ifdef LF_HAVE_FP8
#include "fp8_sm100.h"
#endif
#ifdef LF_HAVE_PEER_OPTIM
#include "peer_optim.h"
#endif
#ifdef LF_HAVE_DSA
#include "dsa_sm100.h"
#endif

namespace {

int64_t g_launches = 0;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bf16");
}

// D = op(A) * op(B) [+ bias] [+ residual]; see gemm_sm100.h for operand layouts.
at::Tensor gemm(const at::Tensor& A, const at::Tensor& B, c10::optional<at::Tensor> D_, bool a_mn_major,
                bool b_mn_major, int64_t out_mode, c10::optional<at::Tensor> bias,
                c10::optional<at::Tensor> residual, double alpha, const at::Tensor& status, int64_t max_ctas) {
  check_bf16_cuda(A, "A");
  check_bf16_cuda(B, "B");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1, "gemm operands must be row-major (unit inner stride)");
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t M = a_mn_major ? A.size(1) : A.size(0);
  const int64_t K = a_mn_major ? A.size(0) : A.size(1);
  const int64_t N = b_mn_major ? B.size(1) : B.size(0);
  const int64_t Kb = b_mn_major ? B.size(0) : B.size(1);
  TORCH_CHECK(K == Kb, "gemm contraction mismatch: ", K, " vs ", Kb);
  TORCH_CHECK(N % 8 == 0, "gemm: the output width N = ", N, " must be a multiple of 8 (16-byte rows)");
  at::Tensor D;
  if (D_.has_value()) {
    D = *D_;
    TORCH_CHECK(D.dim() == 2 && D.size(0) == M && D.size(1) == N && D.stride(1) == 1, "bad output shape");
    TORCH_CHECK(D.scalar_type() == (out_mode == 0 ? at::kBFloat16 : at::kFloat), "bad output dtype");
  } else {
    TORCH_CHECK(out_mode != 2, "accumulate mode needs an output tensor");
    D = at::empty({M, N}, A.options().dtype(out_mode == 0 ? at::kBFloat16 : at::kFloat));
  }
  lf::GemmArgs g;
  g.A = A.data_ptr();
  g.B = B.data_ptr();
  g.D = D.data_ptr();
  g.lda = A.stride(0);
  g.ldb = B.stride(0);
  g.ldd = D.stride(0);
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.a_mn_major = a_mn_major;
  g.b_mn_major = b_mn_major;
  g.out_mode = static_cast<int>(out_mode);
  if (bias.has_value()) {
    check_bf16_cuda(*bias, "bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bad bias");
    g.bias = bias->data_ptr();
  }
  if (residual.has_value()) {
    check_bf16_cuda(*residual, "residual");
    TORCH_CHECK(out_mode == 0 && residual->dim() == 2 && residual->size(0) == M && residual->size(1) == N &&
                    residual->stride(1) == 1,
                "bad residual");
    g.residual = residual->data_ptr();
    g.ldr = residual->stride(0);
  }
  g.alpha = static_cast<float>(alpha);
  g.status = status.data_ptr<int>();
  g.max_ctas = static_cast<int>(max_ctas);
  const int rc = lf::gemm_bf16(g, cur_stream());
  TORCH_CHECK(rc == 0, "lf::gemm_bf16 failed with code ", rc, " (M=", M, " N=", N, " K=", K,
              "); leading dimensions must be multiples of 8 and bases 16-byte aligned");
  ++g_launches;
  return D;
}

std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps, double w_offset) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && w.numel() == H, "rmsnorm: H must be a multiple of 8");
  const int64_t T = x.numel() / H;
  at::Tensor y = at::empty_like(x);
  at::Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  lf::rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), T, static_cast<int>(H), H, H,
                  static_cast<float>(eps), static_cast<float>(w_offset), cur_stream());
  ++g_launches;
  return {y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w,
                                    const at::Tensor& rstd, c10::optional<at::Tensor> dres, double w_offset) {
  check_bf16_cuda(dy, "dy");
  check_bf16_cuda(x, "x");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && w.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t H = x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 8192, "rmsnorm_bwd: H must be a multiple of 8 and <= 8192");
  const int64_t T = x.numel() / H;
  TORCH_CHECK(T <= INT32_MAX, "rmsnorm_bwd: more than 2^31 - 1 rows");
  check_bf16_cuda(w, "w");
  TORCH_CHECK(w.numel() == H && w.device() == x.device(), "rmsnorm_bwd: w must hold H elements on x's device");
  TORCH_CHECK(rstd.is_cuda() && rstd.scalar_type() == at::kFloat && rstd.is_contiguous() && rstd.numel() == T &&
                  rstd.device() == x.device(),
              "rmsnorm_bwd: rstd must be fp32 [T] on x's device");
  TORCH_CHECK(dy.numel() == x.numel() && dy.device() == x.device(), "rmsnorm_bwd: dy must match x");
  at::Tensor dx = at::empty_like(x);
  const int grid = lf::rmsnorm_bwd_grid(T);
  at::Tensor partial = at::empty({grid, H}, x.options().dtype(at::kFloat));
  at::Tensor dw = at::empty({H}, x.options().dtype(at::kFloat));
  const void* dres_p = nullptr;
  if (dres.has_value()) {
    check_bf16_cuda(*dres, "dres");
    TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel());
    dres_p = dres->data_ptr();
  }
  lf::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dres_p, dx.data_ptr(),
                  partial.data_ptr<float>(), dw.data_ptr<float>(), nullptr, 0, T, static_cast<int>(H),
                  static_cast<float>(w_offset), cur_stream());
  g_launches += 2;
  return {dx, dw};
}

// In-place rotary embedding on a [T, heads, D] view (strides in elements).
void rope_(at::Tensor x, const at::Tensor& freqs, c10::optional<at::Tensor> pos_ids, int64_t T, int64_t heads,
           int64_t D, int64_t rot_dim, int64_t rot_offset, int64_t t_stride, int64_t h_stride, int64_t group,
           int64_t rope_in_group, bool interleaved, double mscale, double sign) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(freqs.is_cuda() && freqs.scalar_type() == at::kFloat && freqs.is_contiguous());
  TORCH_CHECK(freqs.size(-1) == rot_dim / 2, "freqs last dim must be rot_dim/2");
  TORCH_CHECK(rot_offset + rot_dim <= D);
  c10::cuda::CUDAGuard guard(x.device());
  const int* pid = nullptr;
  if (pos_ids.has_value()) {
    TORCH_CHECK(pos_ids->scalar_type() == at::kInt && pos_ids->is_contiguous() && pos_ids->numel() == T);
    pid = pos_ids->data_ptr<int>();
  } else {
    TORCH_CHECK(freqs.numel() / (rot_dim / 2) >= T, "freqs has fewer rows than tokens");
  }
  lf::rope_inplace(x.data_ptr(), freqs.data_ptr<float>(), pid, static_cast<int>(T), static_cast<int>(heads),
                   static_cast<int>(D), static_cast<int>(rot_dim), static_cast<int>(rot_offset), t_stride, h_stride,
                   static_cast<int>(group), static_cast<int>(rope_in_group), interleaved ? 1 : 0,
                   static_cast<float>(mscale), static_cast<float>(sign), cur_stream());
  ++g_launches;
}

at::Tensor hadamard128(const at::Tensor& x) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.is_contiguous() && x.dim() >= 1 && x.size(-1) == 128, "hadamard128 wants contiguous rows of 128");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  lf::hadamard128(x.data_ptr(), y.data_ptr(), x.numel() / 128, cur_stream());
  ++g_launches;
  return y;
}

at::Tensor swiglu_fwd(const at::Tensor& in) {
  check_bf16_cuda(in, "in");
  TORCH_CHECK(in.is_contiguous());
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t F2 = in.size(-1);
  TORCH_CHECK(F2 % 16 == 0, "swiglu: 2F must be a multiple of 16");
  const int64_t F = F2 / 2;
  const int64_t T = in.numel() / F2;
  auto sizes = in.sizes().vec();
  sizes.back() = F;
  at::Tensor out = at::empty(sizes, in.options());
  lf::swiglu_fwd(in.data_ptr(), out.data_ptr(), T, static_cast<int>(F), cur_stream());
  ++g_launches;
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& in) {
  check_bf16_cuda(dout, "dout");
  check_bf16_cuda(in, "in");
  TORCH_CHECK(in.is_contiguous() && dout.is_contiguous());
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t F2 = in.size(-1);
  const int64_t F = F2 / 2;
  const int64_t T = in.numel() / F2;
  TORCH_CHECK(dout.numel() == T * F);
  at::Tensor din = at::empty_like(in);
  lf::swiglu_bwd(dout.data_ptr(), in.data_ptr(), din.data_ptr(), T, static_cast<int>(F), cur_stream());
  ++g_launches;
  return din;
}

std::vector<at::Tensor> ce_stats(const at::Tensor& logits, const at::Tensor& labels, int64_t vocab_start,
                                 int64_t valid_v) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.size(1) % 8 == 0 && logits.stride(0) % 8 == 0);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0);
  auto fo = logits.options().dtype(at::kFloat);
  at::Tensor mx = at::empty({T}, fo), sm = at::empty({T}, fo), tg = at::empty({T}, fo);
  lf::ce_stats(logits.data_ptr(), labels.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()) : nullptr,
               mx.data_ptr<float>(), sm.data_ptr<float>(), tg.data_ptr<float>(), T, static_cast<int>(logits.size(1)),
               logits.stride(0), static_cast<int>(vocab_start), static_cast<int>(valid_v), cur_stream());
  ++g_launches;
  return {mx, sm, tg};
}

void ce_dlogits_(at::Tensor logits, const at::Tensor& labels, const at::Tensor& gmax, const at::Tensor& gsum,
                 const at::Tensor& row_scale, int64_t vocab_start, int64_t valid_v) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.size(1) % 8 == 0 && logits.stride(0) % 8 == 0);
  TORCH_CHECK(gmax.scalar_type() == at::kFloat && gsum.scalar_type() == at::kFloat &&
              row_scale.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0);
  lf::ce_dlogits(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                 gmax.data_ptr<float>(), gsum.data_ptr<float>(), row_scale.data_ptr<float>(), T,
                 static_cast<int>(logits.size(1)), logits.stride(0), static_cast<int>(vocab_start),
                 static_cast<int>(valid_v), cur_stream());
  ++g_launches;
}

void adam_step_(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                c10::optional<at::Tensor> model_out, double lr, double beta1, double beta2, double eps, double wd,
                int64_t step, double grad_scale) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  TORCH_CHECK(grad.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  const int64_t n = master.numel();
  TORCH_CHECK(grad.numel() == n && m.numel() == n && v.numel() == n);
  TORCH_CHECK(m.scalar_type() == v.scalar_type());
  c10::cuda::CUDAGuard guard(master.device());
  const bool gb = grad.scalar_type() == at::kBFloat16;
  TORCH_CHECK(gb || grad.scalar_type() == at::kFloat);
  const bool mb = m.scalar_type() == at::kBFloat16;
  TORCH_CHECK(mb || m.scalar_type() == at::kFloat);
  void* mo = nullptr;
  if (model_out.has_value()) {
    check_bf16_cuda(*model_out, "model_out");
    TORCH_CHECK(model_out->is_contiguous() && model_out->numel() == n);
    mo = model_out->data_ptr();
  }
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  lf::adam_step(master.data_ptr<float>(), grad.data_ptr(), gb, m.data_ptr(), v.data_ptr(), mb, mo, n,
                static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
                static_cast<float>(eps), static_cast<float>(wd), bc1, bc2, static_cast<float>(grad_scale),
                cur_stream());
  ++g_launches;
}

void adam_step_remainder_(at::Tensor w, at::Tensor lo, const at::Tensor& grad, at::Tensor m, at::Tensor v, double lr,
                          double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale) {
  check_bf16_cuda(w, "w");
  TORCH_CHECK(lo.is_cuda() && lo.scalar_type() == at::kShort && w.is_contiguous() && lo.is_contiguous());
  const int64_t n = w.numel();
  TORCH_CHECK(lo.numel() == n && grad.numel() == n && m.numel() == n && v.numel() == n);
  TORCH_CHECK(grad.is_contiguous() && m.is_contiguous() && v.is_contiguous() && m.scalar_type() == v.scalar_type());
  c10::cuda::CUDAGuard guard(w.device());
  const bool gb = grad.scalar_type() == at::kBFloat16;
  TORCH_CHECK(gb || grad.scalar_type() == at::kFloat);
  const bool mb = m.scalar_type() == at::kBFloat16;
  TORCH_CHECK(mb || m.scalar_type() == at::kFloat);
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  lf::adam_step_remainder(w.data_ptr(), lo.data_ptr(), grad.data_ptr(), gb, m.data_ptr(), v.data_ptr(), mb, n,
                          static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
                          static_cast<float>(eps), static_cast<float>(wd), bc1, bc2, static_cast<float>(grad_scale),
                          cur_stream());
  ++g_launches;
}

void master_split_(const at::Tensor& master, at::Tensor w, at::Tensor lo, bool write_w) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  check_bf16_cuda(w, "w");
  TORCH_CHECK(lo.scalar_type() == at::kShort && w.numel() == master.numel() && lo.numel() == master.numel());
  c10::cuda::CUDAGuard guard(w.device());
  lf::master_split(master.data_ptr<float>(), w.data_ptr(), lo.data_ptr(), master.numel(), write_w, cur_stream());
  ++g_launches;
}

at::Tensor master_join(const at::Tensor& w, const at::Tensor& lo) {
  check_bf16_cuda(w, "w");
  TORCH_CHECK(lo.scalar_type() == at::kShort && lo.numel() == w.numel() && w.is_contiguous() && lo.is_contiguous());
  c10::cuda::CUDAGuard guard(w.device());
  at::Tensor out = at::empty({w.numel()}, w.options().dtype(at::kFloat));
  lf::master_join(w.data_ptr(), lo.data_ptr(), out.data_ptr<float>(), w.numel(), cur_stream());
  ++g_launches;
  return out;
}

void sumsq_(const at::Tensor& x, at::Tensor out) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && out.scalar_type() == at::kFloat && out.numel() == 1);
  c10::cuda::CUDAGuard guard(x.device());
  const bool b = x.scalar_type() == at::kBFloat16;
  TORCH_CHECK(b || x.scalar_type() == at::kFloat);
  if (x.numel() == 0) return;
  at::Tensor partial = at::empty({lf::sumsq_partials(x.numel())}, out.options());
  lf::sumsq(x.data_ptr(), b, x.numel(), out.data_ptr<float>(), partial.data_ptr<float>(), cur_stream());
  g_launches += 2;
}

#ifdef LF_HAVE_ATTN
// ------------------------------------------------------------------ attention
// q: [Tq, G, R, D] (any token/group/head strides, e.g. a view into a packed QKV buffer),
// k, v: [Tk, G, D] views. Returns o [Tq, G*R, D] and lse [G*R, Tq].
void fill_attn_common(lf::AttnArgs& a, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                      const c10::optional<at::Tensor>& cu_q, const c10::optional<at::Tensor>& cu_k, double scale,
                      bool causal, const at::Tensor& status) {
  check_bf16_cuda(q, "q");
  check_bf16_cuda(k, "k");
  check_bf16_cuda(v, "v");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 3 && v.dim() == 3, "q must be [Tq,G,R,D], k/v [Tk,G,D]");
  const int64_t D = q.size(3);
  TORCH_CHECK(D >= 8 && D <= 128 && D % 8 == 0 && k.size(2) == D && v.size(2) == D,
              "head dim must be a multiple of 8, at most 128, and the same for q, k and v");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(2) == 1 && v.stride(2) == 1);
  TORCH_CHECK(k.size(1) == q.size(1) && v.size(1) == q.size(1) && v.size(0) == k.size(0));
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.Tq = static_cast<int>(q.size(0));
  a.Tk = static_cast<int>(k.size(0));
  a.D = static_cast<int>(D);
  a.Hkv = static_cast<int>(q.size(1));
  a.Hq = static_cast<int>(q.size(1) * q.size(2));
  a.q_ts = q.stride(0); a.q_gs = q.stride(1); a.q_hs = q.stride(2);
  a.k_ts = k.stride(0); a.k_hs = k.stride(1);
  a.v_ts = v.stride(0); a.v_hs = v.stride(1);
  a.scale = static_cast<float>(scale);
  a.causal = causal;
  a.status = status.data_ptr<int>();
  if (cu_q.has_value()) {
    TORCH_CHECK(cu_q->is_cuda() && cu_q->scalar_type() == at::kInt && cu_q->is_contiguous() && cu_q->numel() >= 2);
    a.cu_seqlens_q = cu_q->data_ptr<int>();
    a.num_seqs = static_cast<int>(cu_q->numel() - 1);
    if (cu_k.has_value()) {
      TORCH_CHECK(cu_k->is_cuda() && cu_k->scalar_type() == at::kInt && cu_k->is_contiguous() &&
                  cu_k->numel() == cu_q->numel());
      a.cu_seqlens_k = cu_k->data_ptr<int>();
    } else {
      TORCH_CHECK(a.Tq == a.Tk, "different query and key lengths with sequence boundaries need both boundary lists");
    }
  } else {
    TORCH_CHECK(!cu_k.has_value(), "key boundaries without query boundaries");
  }
}

std::vector<at::Tensor> attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                 c10::optional<at::Tensor> cu_q, c10::optional<at::Tensor> cu_k, double scale,
                                 bool causal, const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(q.device());
  lf::AttnArgs a;
  fill_attn_common(a, q, k, v, cu_q, cu_k, scale, causal, status);
  at::Tensor o = at::empty({a.Tq, a.Hq, a.D}, q.options());
  at::Tensor lse = at::empty({a.Hq, a.Tq}, q.options().dtype(at::kFloat));
  a.o = o.data_ptr();
  a.o_ts = o.stride(0); a.o_hs = o.stride(1);
  a.lse = lse.data_ptr<float>();
  const int rc = lf::attn_fwd(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::attn_fwd failed with code ", rc);
  ++g_launches;
  return {o, lse};
}

// dq/dk/dv are OUTPUT views (same shapes as q/k/v), typically into one packed gradient buffer.
void attn_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
              const at::Tensor& o, const at::Tensor& lse, at::Tensor dq, at::Tensor dk, at::Tensor dv,
              c10::optional<at::Tensor> cu_q, c10::optional<at::Tensor> cu_k, double scale, bool causal,
              const at::Tensor& status) {
  c10::cuda::CUDAGuard guard(q.device());
  lf::AttnArgs a;
  fill_attn_common(a, q, k, v, cu_q, cu_k, scale, causal, status);
  check_bf16_cuda(dout, "dout");
  check_bf16_cuda(o, "o");
  TORCH_CHECK(dout.dim() == 3 && dout.stride(2) == 1 && o.stride(2) == 1 && dout.size(1) == a.Hq &&
              dout.size(0) == a.Tq && dout.size(2) == a.D);
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes());
  TORCH_CHECK(dq.stride(3) == 1 && dk.stride(2) == 1 && dv.stride(2) == 1);
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == int64_t(a.Hq) * a.Tq);
  at::Tensor delta = at::empty({a.Hq, a.Tq}, q.options().dtype(at::kFloat));
  a.o = const_cast<void*>(o.data_ptr());
  a.o_ts = o.stride(0); a.o_hs = o.stride(1);
  a.lse = const_cast<float*>(lse.data_ptr<float>());
  a.dout = dout.data_ptr();
  a.do_ts = dout.stride(0); a.do_hs = dout.stride(1);
  a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  a.dq_ts = dq.stride(0); a.dq_gs = dq.stride(1); a.dq_hs = dq.stride(2);
  a.dk_ts = dk.stride(0); a.dk_hs = dk.stride(1);
  a.dv_ts = dv.stride(0); a.dv_hs = dv.stride(1);
  a.delta = delta.data_ptr<float>();
  const int rc = lf::attn_bwd(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::attn_bwd failed with code ", rc);
  g_launches += 3;
}

#endif  // LF_HAVE_ATTN

#ifdef LF_HAVE_PEER
// ------------------------------------------------------------------ fused TP GEMMs over peer memory
// Peer pointers are plain integers (device virtual addresses obtained from the symmetric-memory
// rendezvous); index r is rank r of the tensor-parallel group.
at::Tensor ag_gemm(std::vector<int64_t> peer_x, std::vector<int64_t> peer_sync, at::Tensor x_full,
                   at::Tensor chunk_flags, const at::Tensor& B, bool b_mn_major, c10::optional<at::Tensor> bias,
                   int64_t rank, int64_t rows_per_rank, int64_t epoch, int64_t copy_ctas, const at::Tensor& status) {
  check_bf16_cuda(B, "B");
  check_bf16_cuda(x_full, "x_full");
  TORCH_CHECK(B.dim() == 2 && B.stride(1) == 1 && x_full.dim() == 2 && x_full.is_contiguous());
  TORCH_CHECK(chunk_flags.scalar_type() == at::kInt && chunk_flags.is_contiguous());
  c10::cuda::CUDAGuard guard(B.device());
  const int64_t world = static_cast<int64_t>(peer_x.size());
  TORCH_CHECK(world >= 1 && world <= lf::kMaxPeers && static_cast<int64_t>(peer_sync.size()) == world);
  const int64_t K = x_full.size(1);
  const int64_t N = b_mn_major ? B.size(1) : B.size(0);
  TORCH_CHECK((b_mn_major ? B.size(0) : B.size(1)) == K, "contraction mismatch");
  TORCH_CHECK(x_full.size(0) == rows_per_rank * world && chunk_flags.numel() >= x_full.size(0) / 128);
  lf::AgGemmArgs a;
  for (int64_t r = 0; r < world; ++r) {
    a.peer_x[r] = reinterpret_cast<const void*>(peer_x[r]);
    a.peer_sync[r] = reinterpret_cast<int*>(peer_sync[r]);
  }
  a.x_full = x_full.data_ptr();
  a.chunk_flags = chunk_flags.data_ptr<int>();
  a.B = B.data_ptr();
  a.ldb = B.stride(0);
  a.b_mn_major = b_mn_major;
  at::Tensor out = at::empty({x_full.size(0), N}, B.options());
  a.out = out.data_ptr();
  a.ldo = N;
  if (bias.has_value()) {
    check_bf16_cuda(*bias, "bias");
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous());
    a.bias = bias->data_ptr();
  }
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(world);
  a.rows_per_rank = static_cast<int>(rows_per_rank);
  a.K = static_cast<int>(K);
  a.N = static_cast<int>(N);
  a.epoch = static_cast<int>(epoch);
  a.copy_ctas = static_cast<int>(copy_ctas);
  a.status = status.data_ptr<int>();
  const int rc = lf::ag_gemm(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::ag_gemm failed with code ", rc);
  ++g_launches;
  return out;
}

at::Tensor gemm_rs(const at::Tensor& A, const at::Tensor& B, bool b_mn_major, std::vector<int64_t> peer_recv,
                   std::vector<int64_t> peer_tile_flags, c10::optional<at::Tensor> residual, int64_t rank,
                   int64_t call_index, const at::Tensor& status) {
  check_bf16_cuda(A, "A");
  check_bf16_cuda(B, "B");
  TORCH_CHECK(A.dim() == 2 && A.stride(1) == 1 && B.dim() == 2 && B.stride(1) == 1);
  c10::cuda::CUDAGuard guard(B.device());
  const int64_t world = static_cast<int64_t>(peer_recv.size());
  TORCH_CHECK(world >= 1 && world <= lf::kMaxPeers && static_cast<int64_t>(peer_tile_flags.size()) == world);
  const int64_t T = A.size(0), K = A.size(1);
  const int64_t N = b_mn_major ? B.size(1) : B.size(0);
  TORCH_CHECK((b_mn_major ? B.size(0) : B.size(1)) == K, "contraction mismatch");
  lf::GemmRsArgs a;
  a.A = A.data_ptr();
  a.lda = A.stride(0);
  a.B = B.data_ptr();
  a.ldb = B.stride(0);
  a.b_mn_major = b_mn_major;
  for (int64_t r = 0; r < world; ++r) {
    a.peer_recv[r] = reinterpret_cast<void*>(peer_recv[r]);
    a.peer_tile_flags[r] = reinterpret_cast<int*>(peer_tile_flags[r]);
  }
  at::Tensor out = at::empty({T / world, N}, B.options());
  a.out = out.data_ptr();
  a.ldo = N;
  if (residual.has_value()) {
    check_bf16_cuda(*residual, "residual");
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == T / world && residual->size(1) == N &&
                residual->stride(1) == 1);
    a.residual = residual->data_ptr();
    a.ldr = residual->stride(0);
  }
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(world);
  a.T = static_cast<int>(T);
  a.K = static_cast<int>(K);
  a.N = static_cast<int>(N);
  a.call_index = static_cast<int>(call_index);
  a.status = status.data_ptr<int>();
  const int rc = lf::gemm_rs(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::gemm_rs failed with code ", rc);
  ++g_launches;
  return out;
}

#endif  // LF_HAVE_PEER

// ------------------------------------------------------------------ MoE router
// Returns (probs [T,E] f32, routing_map [T,E] bool, aux_scores [T,E] f32, topk_idx [T,k] i32, counts [E] i32).
std::vector<at::Tensor> router_fwd(const at::Tensor& logits, c10::optional<at::Tensor> bias, int64_t k, int64_t score,
                                   int64_t num_groups, int64_t group_topk, double scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(logits.scalar_type() == at::kFloat || logits.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  auto f32 = logits.options().dtype(at::kFloat);
  at::Tensor probs = at::empty({T, E}, f32), aux = at::empty({T, E}, f32);
  at::Tensor map = at::empty({T, E}, logits.options().dtype(at::kBool));
  at::Tensor idx = at::empty({T, k}, logits.options().dtype(at::kInt));
  at::Tensor counts = at::zeros({E}, logits.options().dtype(at::kInt));
  lf::RouterArgs a;
  a.logits = logits.data_ptr();
  a.logits_bf16 = logits.scalar_type() == at::kBFloat16;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->numel() == E);
    a.bias = bias->data_ptr<float>();
  }
  a.probs = probs.data_ptr<float>();
  a.map = reinterpret_cast<unsigned char*>(map.data_ptr());
  a.aux = aux.data_ptr<float>();
  a.topk_idx = idx.data_ptr<int>();
  a.counts = counts.data_ptr<int>();
  a.T = static_cast<int>(T); a.E = static_cast<int>(E); a.k = static_cast<int>(k); a.score = static_cast<int>(score);
  a.num_groups = static_cast<int>(num_groups); a.group_topk = static_cast<int>(group_topk);
  a.scale = static_cast<float>(scale);
  const int rc = lf::router_fwd(a, cur_stream());
  TORCH_CHECK(rc == 0, "router_fwd: unsupported shape (code ", rc, ")");
  ++g_launches;
  return {probs, map, aux, idx, counts};
}

at::Tensor router_bwd(const at::Tensor& logits, const at::Tensor& map, const at::Tensor& dprobs,
                      c10::optional<at::Tensor> daux, int64_t k, int64_t score, double scale) {
  TORCH_CHECK(logits.is_cuda() && logits.is_contiguous() && map.is_contiguous() && dprobs.is_contiguous());
  TORCH_CHECK(dprobs.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor dl = at::empty(logits.sizes(), logits.options().dtype(at::kFloat));
  lf::RouterArgs a;
  a.logits = logits.data_ptr();
  a.logits_bf16 = logits.scalar_type() == at::kBFloat16;
  a.map = reinterpret_cast<unsigned char*>(map.data_ptr());
  a.dprobs = dprobs.data_ptr<float>();
  if (daux.has_value()) {
    TORCH_CHECK(daux->scalar_type() == at::kFloat && daux->is_contiguous());
    a.daux = daux->data_ptr<float>();
  }
  a.dlogits = dl.data_ptr<float>();
  a.T = static_cast<int>(logits.size(0)); a.E = static_cast<int>(logits.size(1));
  a.k = static_cast<int>(k); a.score = static_cast<int>(score); a.scale = static_cast<float>(scale);
  const int rc = lf::router_bwd(a, cur_stream());
  TORCH_CHECK(rc == 0, "router_bwd: unsupported shape (code ", rc, ")");
  ++g_launches;
  return dl;
}

#ifdef LF_HAVE_GROUPED
// ------------------------------------------------------------------ grouped (per-expert) GEMM
// Rows of `A` (and `X`) are sorted by expert; expert e owns `tpe[e]` consecutive rows.
//   mode 0 forward: outs[0][rows_e, N] = A[rows_e, K] * weights[e][N, K]^T
//   mode 1 dgrad  : outs[0][rows_e, K] = A[rows_e, N] * weights[e][N, K]
//   mode 2 wgrad  : outs[e][N, K] (=|+=) A[rows_e, N]^T * X[rows_e, K]     (weights unused)
// One launch for all experts; descriptors are built on the host and copied with the stream.
void grouped_gemm(const at::Tensor& A, c10::optional<at::Tensor> X_, std::vector<at::Tensor> weights,
                  std::vector<at::Tensor> outs, std::vector<int64_t> tpe, int64_t mode, int64_t out_mode,
                  const at::Tensor& status) {
  check_bf16_cuda(A, "A");
  TORCH_CHECK(A.dim() == 2 && A.stride(1) == 1);
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t E = static_cast<int64_t>(tpe.size());
  TORCH_CHECK(E > 0);
  const bool a_mn = mode == 2, b_mn = mode != 0;
  const char* a_ptr = static_cast<const char*>(A.data_ptr());
  const int64_t lda = A.stride(0);
  at::Tensor X;
  if (mode == 2) {
    TORCH_CHECK(X_.has_value());
    X = *X_;
    check_bf16_cuda(X, "X");
    TORCH_CHECK(X.dim() == 2 && X.stride(1) == 1 && X.size(0) == A.size(0));
    TORCH_CHECK(static_cast<int64_t>(outs.size()) == E);
  } else {
    TORCH_CHECK(static_cast<int64_t>(weights.size()) == E && outs.size() == 1);
    TORCH_CHECK(outs[0].dim() == 2 && outs[0].stride(1) == 1 && outs[0].size(0) == A.size(0));
  }
  auto host_opts = at::TensorOptions().dtype(at::kByte).pinned_memory(true);
  at::Tensor desc_h = at::empty({E * static_cast<int64_t>(sizeof(lf::GroupDesc))}, host_opts);
  auto* descs = reinterpret_cast<lf::GroupDesc*>(desc_h.data_ptr());
  std::vector<int> order;
  int64_t num_tiles = 0, row = 0;
  std::vector<int> tiles_of(E, 0);
  for (int64_t e = 0; e < E; ++e) {
    const int64_t n = tpe[e];
    int rc = 0;
    if (mode == 0 || mode == 1) {
      const at::Tensor& w = weights[e];
      check_bf16_cuda(w, "weight");
      TORCH_CHECK(w.dim() == 2 && w.stride(1) == 1);
      const int64_t Nout = mode == 0 ? w.size(0) : w.size(1);
      const int64_t Kc = mode == 0 ? w.size(1) : w.size(0);
      TORCH_CHECK(A.size(1) == Kc && outs[0].size(1) == Nout, "grouped_gemm shape mismatch");
      char* d_ptr = static_cast<char*>(outs[0].data_ptr()) + row * outs[0].stride(0) * outs[0].element_size();
      rc = lf::grouped_gemm_fill_desc(&descs[e], a_ptr + row * lda * 2, lda, w.data_ptr(), w.stride(0), d_ptr,
                                      outs[0].stride(0), static_cast<int>(n), static_cast<int>(Nout),
                                      static_cast<int>(Kc), a_mn, b_mn, static_cast<int>(out_mode));
      tiles_of[e] = n > 0 ? lf::grouped_gemm_tiles_for(static_cast<int>(n), static_cast<int>(Nout)) : 0;
    } else {
      const at::Tensor& d = outs[e];
      TORCH_CHECK(d.is_cuda() && d.dim() == 2 && d.stride(1) == 1 && d.size(0) == A.size(1) && d.size(1) == X.size(1));
      TORCH_CHECK(out_mode == 0 ? d.scalar_type() == at::kBFloat16 : d.scalar_type() == at::kFloat);
      rc = lf::grouped_gemm_fill_desc(&descs[e], a_ptr + row * lda * 2, lda,
                                      static_cast<const char*>(X.data_ptr()) + row * X.stride(0) * 2, X.stride(0),
                                      d.data_ptr(), d.stride(0), static_cast<int>(A.size(1)),
                                      static_cast<int>(X.size(1)), static_cast<int>(n), a_mn, b_mn,
                                      static_cast<int>(out_mode));
      tiles_of[e] = n > 0 ? lf::grouped_gemm_tiles_for(static_cast<int>(A.size(1)), static_cast<int>(X.size(1))) : 0;
    }
    TORCH_CHECK(rc == 0, "grouped_gemm descriptor for expert ", e, " failed with code ", rc);
    num_tiles += tiles_of[e];
    order.push_back(static_cast<int>(e));
    row += n;
  }
  TORCH_CHECK(row == A.size(0), "tokens_per_expert sums to ", row, ", expected ", A.size(0));
  if (num_tiles == 0) return;
  // longest contraction first: with a static round-robin walk this keeps the tail short in wgrad
  if (mode == 2) std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tpe[a] > tpe[b]; });
  at::Tensor tiles_h = at::empty({num_tiles * 2}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
  int* tp = tiles_h.data_ptr<int>();
  for (int e : order)
    for (int t = 0; t < tiles_of[e]; ++t) {
      *tp++ = e;
      *tp++ = t;
    }
  at::Tensor desc_d = desc_h.to(A.device(), /*non_blocking=*/true);
  at::Tensor tiles_d = tiles_h.to(A.device(), /*non_blocking=*/true);
  const int rc = lf::grouped_gemm_launch(reinterpret_cast<const lf::GroupDesc*>(desc_d.data_ptr()), tiles_d.data_ptr(),
                                         static_cast<int>(num_tiles), a_mn, b_mn, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "grouped_gemm launch failed with code ", rc);
  ++g_launches;
}
#endif  // LF_HAVE_GROUPED

#ifdef LF_HAVE_MOE_PEER
// ------------------------------------------------------------------ expert-parallel exchange over peer memory
// Peer pointers are device virtual addresses from the symmetric-memory rendezvous (index = EP rank).
static lf::MoePeerBufs moe_bufs(const std::vector<int64_t>& buf, const std::vector<int64_t>& scal,
                                const std::vector<int64_t>& flags, int64_t rank, int64_t cap_rows) {
  const int64_t world = static_cast<int64_t>(buf.size());
  TORCH_CHECK(world >= 1 && world <= lf::kMoeMaxPeers && scal.size() == buf.size() && flags.size() == buf.size());
  lf::MoePeerBufs b;
  for (int64_t r = 0; r < world; ++r) {
    b.buf[r] = reinterpret_cast<void*>(buf[r]);
    b.scal[r] = reinterpret_cast<float*>(scal[r]);
    b.flags[r] = reinterpret_cast<int*>(flags[r]);
  }
  b.rank = static_cast<int>(rank);
  b.world = static_cast<int>(world);
  b.cap_rows = static_cast<int>(cap_rows);
  return b;
}

void moe_push(std::vector<int64_t> buf, std::vector<int64_t> scal, std::vector<int64_t> flags, int64_t rank,
              int64_t cap_rows, const at::Tensor& x, const at::Tensor& pair_token, const at::Tensor& pair_row,
              const at::Tensor& pair_dst, c10::optional<at::Tensor> pair_scal, const at::Tensor& done_counter,
              int64_t kind, int64_t epoch, const at::Tensor& status) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(pair_token.scalar_type() == at::kInt && pair_row.scalar_type() == at::kInt &&
              pair_dst.scalar_type() == at::kInt);
  TORCH_CHECK(pair_token.is_contiguous() && pair_row.is_contiguous() && pair_dst.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const float* ps = nullptr;
  if (pair_scal.has_value()) {
    TORCH_CHECK(pair_scal->scalar_type() == at::kFloat && pair_scal->is_contiguous() &&
                pair_scal->numel() == pair_token.numel());
    ps = pair_scal->data_ptr<float>();
  }
  const int rc = lf::moe_push(moe_bufs(buf, scal, flags, rank, cap_rows), x.data_ptr(), x.stride(0),
                              static_cast<int>(x.size(1)), pair_token.data_ptr<int>(), pair_row.data_ptr<int>(),
                              pair_dst.data_ptr<int>(), ps, static_cast<int>(pair_token.numel()),
                              done_counter.data_ptr<int>(), static_cast<int>(kind), static_cast<int>(epoch),
                              status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "moe_push failed with code ", rc);
  ++g_launches;
}

// Returns (out [T, H] bf16, slot_scal [T, k] f32 or empty).
std::vector<at::Tensor> moe_pull(std::vector<int64_t> buf, std::vector<int64_t> scal, std::vector<int64_t> flags,
                                 int64_t rank, int64_t cap_rows, int64_t T, int64_t k, int64_t H,
                                 const at::Tensor& slot_pair, const at::Tensor& pair_row, const at::Tensor& pair_dst,
                                 bool with_scal, const at::Tensor& status) {
  TORCH_CHECK(slot_pair.scalar_type() == at::kInt && slot_pair.is_contiguous() && slot_pair.numel() == T * k);
  TORCH_CHECK(pair_row.scalar_type() == at::kInt && pair_dst.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(slot_pair.device());
  at::Tensor out = at::empty({T, H}, slot_pair.options().dtype(at::kBFloat16));
  at::Tensor sc = with_scal ? at::empty({T, k}, slot_pair.options().dtype(at::kFloat))
                            : at::empty({0}, slot_pair.options().dtype(at::kFloat));
  const int rc = lf::moe_pull(moe_bufs(buf, scal, flags, rank, cap_rows), out.data_ptr(), H, static_cast<int>(H),
                              static_cast<int>(T), static_cast<int>(k), slot_pair.data_ptr<int>(),
                              pair_row.data_ptr<int>(), pair_dst.data_ptr<int>(),
                              with_scal ? sc.data_ptr<float>() : nullptr, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "moe_pull failed with code ", rc);
  ++g_launches;
  return {out, sc};
}

void moe_signal(std::vector<int64_t> buf, std::vector<int64_t> scal, std::vector<int64_t> flags, int64_t rank,
                int64_t kind, int64_t epoch) {
  TORCH_CHECK(lf::moe_signal(moe_bufs(buf, scal, flags, rank, 0), static_cast<int>(kind), static_cast<int>(epoch),
                             cur_stream()) == 0);
  ++g_launches;
}

void moe_wait(std::vector<int64_t> buf, std::vector<int64_t> scal, std::vector<int64_t> flags, int64_t rank,
              int64_t kind, int64_t epoch, const at::Tensor& status) {
  TORCH_CHECK(lf::moe_wait(moe_bufs(buf, scal, flags, rank, 0), static_cast<int>(kind), static_cast<int>(epoch),
                           status.data_ptr<int>(), cur_stream()) == 0);
  ++g_launches;
}
#endif  // LF_HAVE_MOE_PEER

#ifdef LF_HAVE_FP8
// ------------------------------------------------------------------ FP8 block quantisers + blockwise GEMM
std::vector<at::Tensor> quant_1x128(const at::Tensor& x, bool pow2) {
  check_bf16_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) % 128 == 0, "quant_1x128 wants contiguous [M, 128k]");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor q = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({x.size(0), x.size(1) / 128}, x.options().dtype(at::kFloat));
  TORCH_CHECK(lf::quant_1x128(x.data_ptr(), q.data_ptr(), s.data_ptr<float>(), x.size(0), static_cast<int>(x.size(1)),
                              pow2, cur_stream()) == 0);
  ++g_launches;
  return {q, s};
}

std::vector<at::Tensor> quant_128x128(const at::Tensor& w, bool pow2) {
  check_bf16_cuda(w, "w");
  TORCH_CHECK(w.dim() == 2 && w.is_contiguous() && w.size(0) % 128 == 0 && w.size(1) % 128 == 0);
  c10::cuda::CUDAGuard guard(w.device());
  at::Tensor q = at::empty(w.sizes(), w.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({w.size(0) / 128, w.size(1) / 128}, w.options().dtype(at::kFloat));
  TORCH_CHECK(lf::quant_128x128(w.data_ptr(), q.data_ptr(), s.data_ptr<float>(), static_cast<int>(w.size(0)),
                                static_cast<int>(w.size(1)), pow2, cur_stream()) == 0);
  ++g_launches;
  return {q, s};
}

at::Tensor gemm_fp8_blockwise(const at::Tensor& aq, const at::Tensor& sa, const at::Tensor& bq, const at::Tensor& sb,
                              const at::Tensor& status) {
  TORCH_CHECK(aq.is_cuda() && aq.scalar_type() == at::kFloat8_e4m3fn && bq.scalar_type() == at::kFloat8_e4m3fn);
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 2 && aq.is_contiguous() && bq.is_contiguous() && aq.size(1) == bq.size(1));
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat && sa.is_contiguous() && sb.is_contiguous());
  const int64_t M = aq.size(0), K = aq.size(1), N = bq.size(0);
  TORCH_CHECK(sa.size(0) == M && sa.size(1) == K / 128 && sb.size(0) == N / 128 && sb.size(1) == K / 128);
  c10::cuda::CUDAGuard guard(aq.device());
  at::Tensor d = at::empty({M, N}, aq.options().dtype(at::kBFloat16));
  const int rc = lf::gemm_fp8_blockwise(aq.data_ptr(), sa.data_ptr<float>(), bq.data_ptr(), sb.data_ptr<float>(),
                                        d.data_ptr(), N, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                                        status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_fp8_blockwise failed with code ", rc);
  ++g_launches;
  return d;
}
#endif  // LF_HAVE_FP8

#ifdef LF_HAVE_PEER_OPTIM
// ------------------------------------------------------------------ data-parallel optimizer over peer memory
static lf::PeerTable peer_table(const std::vector<int64_t>& ptrs, int64_t rank) {
  TORCH_CHECK(!ptrs.empty() && static_cast<int>(ptrs.size()) <= lf::kOptMaxPeers);
  lf::PeerTable t;
  for (size_t r = 0; r < ptrs.size(); ++r) t.ptr[r] = reinterpret_cast<void*>(ptrs[r]);
  t.world = static_cast<int>(ptrs.size());
  t.rank = static_cast<int>(rank);
  return t;
}

// grads: base pointers of the symmetric fp32 gradient buffer on every DP rank. The reduced shard replaces
// [start, start + n) of this rank's buffer; `sumsq` (fp32[1]) receives += its squared norm when given.
void grad_pull_reduce(std::vector<int64_t> grads, int64_t rank, int64_t start, int64_t n, double scale,
                      c10::optional<at::Tensor> sumsq) {
  float* ss = nullptr;
  if (sumsq.has_value()) {
    TORCH_CHECK(sumsq->is_cuda() && sumsq->scalar_type() == at::kFloat);
    ss = sumsq->data_ptr<float>();
  }
  // the kernel needs a valid accumulator address: without one the partial goes to a scratch word
  static thread_local at::Tensor scratch;
  if (ss == nullptr) {
    if (!scratch.defined()) scratch = at::zeros({1}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA));
    ss = scratch.data_ptr<float>();
  }
  TORCH_CHECK(lf::grad_pull_reduce(peer_table(grads, rank), start, n, static_cast<float>(scale), ss, cur_stream()) == 0,
              "grad_pull_reduce: start and n must be multiples of 4");
  ++g_launches;
}

void adam_push(std::vector<int64_t> params, int64_t rank, int64_t start, at::Tensor lo, const at::Tensor& grad,
               at::Tensor m, at::Tensor v, double lr, double beta1, double beta2, double eps, double wd, int64_t step,
               double grad_scale) {
  TORCH_CHECK(lo.is_cuda() && lo.scalar_type() == at::kShort && grad.scalar_type() == at::kFloat &&
              m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(lo.is_contiguous() && grad.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  const int64_t n = lo.numel();
  TORCH_CHECK(grad.numel() == n && m.numel() == n && v.numel() == n);
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  TORCH_CHECK(lf::adam_push(peer_table(params, rank), start, n, lo.data_ptr<int16_t>(), grad.data_ptr<float>(),
                            m.data_ptr<float>(), v.data_ptr<float>(), static_cast<float>(lr), static_cast<float>(beta1),
                            static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd), bc1, bc2,
                            static_cast<float>(grad_scale), cur_stream()) == 0,
              "adam_push: start and n must be even");
  ++g_launches;
}

void peer_signal(std::vector<int64_t> flags, int64_t rank, int64_t epoch) {
  TORCH_CHECK(lf::peer_signal(peer_table(flags, rank), static_cast<int>(epoch), cur_stream()) == 0);
  ++g_launches;
}

void peer_wait(std::vector<int64_t> flags, int64_t rank, int64_t epoch, const at::Tensor& status) {
  TORCH_CHECK(lf::peer_wait(peer_table(flags, rank), static_cast<int>(epoch), status.data_ptr<int>(), cur_stream()) == 0);
  ++g_launches;
}
#endif  // LF_HAVE_PEER_OPTIM

#ifdef LF_HAVE_DSA
// ------------------------------------------------------------------ DeepSeek sparse attention
// q [m, H, 576] bf16 (unit inner stride), kv [n, 576] bf16, idx [m, topk] int32 -> (o [m, H, 512] bf16, lse [m, H]).
std::vector<at::Tensor> sparse_mla_fwd(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& idx, double scale,
                                       const at::Tensor& status) {
  check_bf16_cuda(q, "q");
  check_bf16_cuda(kv, "kv");
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 576 && q.stride(2) == 1 && q.size(1) >= 1 && q.size(1) <= 128,
              "q must be [m, H <= 128, 576]");
  TORCH_CHECK(kv.dim() == 2 && kv.size(1) == 576 && kv.stride(1) == 1, "kv must be [n, 576]");
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous() &&
                  idx.size(0) == q.size(0),
              "idx must be int32 [m, topk]");
  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor o = at::empty({q.size(0), q.size(1), 512}, q.options());
  at::Tensor lse = at::empty({q.size(0), q.size(1)}, q.options().dtype(at::kFloat));
  lf::SparseMlaArgs a;
  a.q = q.data_ptr(); a.q_ts = q.stride(0); a.q_hs = q.stride(1);
  a.kv = kv.data_ptr(); a.kv_ts = kv.stride(0);
  a.idx = idx.data_ptr<int>();
  a.topk = static_cast<int>(idx.size(1));
  a.m = static_cast<int>(q.size(0));
  a.H = static_cast<int>(q.size(1));
  a.n_kv = static_cast<int>(kv.size(0));
  a.scale = static_cast<float>(scale);
  a.o = o.data_ptr(); a.o_ts = o.stride(0); a.o_hs = o.stride(1);
  a.lse = lse.data_ptr<float>();
  a.status = status.data_ptr<int>();
  const int rc = lf::sparse_mla_fwd(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::sparse_mla_fwd failed with code ", rc);
  ++g_launches;
  return {o, lse};
}

// Head-averaged attention probabilities of the selected slots, given the forward's lse [m, H] -> pmean [m, topk] fp32.
at::Tensor sparse_mla_probs(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& idx, const at::Tensor& lse,
                            double scale, const at::Tensor& status) {
  check_bf16_cuda(q, "q");
  check_bf16_cuda(kv, "kv");
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 576 && q.stride(2) == 1 && q.size(1) >= 1 && q.size(1) <= 128,
              "q must be [m, H <= 128, 576]");
  TORCH_CHECK(kv.dim() == 2 && kv.size(1) == 576 && kv.stride(1) == 1, "kv must be [n, 576]");
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous() &&
                  idx.size(0) == q.size(0),
              "idx must be int32 [m, topk]");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() &&
                  lse.numel() == q.size(0) * q.size(1),
              "lse must be fp32 [m, H]");
  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor pmean = at::zeros({q.size(0), idx.size(1)}, q.options().dtype(at::kFloat));
  lf::SparseMlaArgs a;
  a.q = q.data_ptr(); a.q_ts = q.stride(0); a.q_hs = q.stride(1);
  a.kv = kv.data_ptr(); a.kv_ts = kv.stride(0);
  a.idx = idx.data_ptr<int>();
  a.topk = static_cast<int>(idx.size(1));
  a.m = static_cast<int>(q.size(0));
  a.H = static_cast<int>(q.size(1));
  a.n_kv = static_cast<int>(kv.size(0));
  a.scale = static_cast<float>(scale);
  a.lse = lse.data_ptr<float>();
  a.pmean = pmean.data_ptr<float>();
  a.status = status.data_ptr<int>();
  const int rc = lf::sparse_mla_probs(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::sparse_mla_probs failed with code ", rc);
  ++g_launches;
  return pmean;
}

// Lightning-indexer logits for query rows [q0, q0 + rows) into `logits` [rows, ld] fp32 (entries outside each row's
// key range stay unwritten), then the top-k selection over those ranges into `out` [rows, topk] int32.
void indexer_topk(const at::Tensor& q, const at::Tensor& k, const at::Tensor& w, const at::Tensor& k_start,
                  const at::Tensor& k_end, at::Tensor logits, at::Tensor out, int64_t max_len, const at::Tensor& status) {
  check_bf16_cuda(q, "q");
  check_bf16_cuda(k, "k");
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.is_contiguous(), "q must be contiguous [m, Hi, 128]");
  TORCH_CHECK(k.dim() == 2 && k.size(1) == 128 && k.stride(1) == 1, "k must be [n, 128]");
  const int64_t m = q.size(0), Hi = q.size(1), n = k.size(0);
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == m * Hi);
  TORCH_CHECK(k_start.scalar_type() == at::kInt && k_end.scalar_type() == at::kInt && k_start.numel() == m &&
              k_end.numel() == m && k_start.is_contiguous() && k_end.is_contiguous());
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.size(0) >= m && logits.size(1) >= n &&
              logits.stride(1) == 1);
  TORCH_CHECK(out.scalar_type() == at::kInt && out.dim() == 2 && out.size(0) == m && out.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  lf::IndexerArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.k_ld = k.stride(0);
  a.w = w.data_ptr<float>();
  a.k_start = k_start.data_ptr<int>(); a.k_end = k_end.data_ptr<int>();
  a.logits = logits.data_ptr<float>(); a.ld = logits.stride(0);
  a.m = static_cast<int>(m); a.n = static_cast<int>(n); a.Hi = static_cast<int>(Hi);
  a.status = status.data_ptr<int>();
  int rc = lf::indexer_logits(a, cur_stream());
  TORCH_CHECK(rc == 0, "lf::indexer_logits failed with code ", rc);
  rc = lf::topk_range(a.logits, a.ld, a.k_start, a.k_end, out.data_ptr<int>(), a.m, static_cast<int>(out.size(1)),
                      static_cast<int>(max_len), cur_stream());
  TORCH_CHECK(rc == 0, "lf::topk_range failed with code ", rc);
  g_launches += 2;
}
#endif  // LF_HAVE_DSA

// Budget of the device-side waits on flags written by other GPUs, in milliseconds (see wait_budget.h).
void set_peer_wait_budget_ms(double ms) { lf::set_peer_wait_budget_ms(ms); }
double peer_wait_budget_ms() { return lf::peer_wait_budget_ms(); }

int64_t launch_count() { return g_launches; }
void reset_launch_count() { g_launches = 0; }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_", &rope_);
  m.def("hadamard128", &hadamard128);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_stats", &ce_stats);
  m.def("ce_dlogits_", &ce_dlogits_);
  m.def("adam_step_", &adam_step_);
  m.def("sumsq_", &sumsq_);
  m.def("adam_step_remainder_", &adam_step_remainder_);
  m.def("master_split_", &master_split_);
  m.def("master_join", &master_join);
#ifdef LF_HAVE_ATTN
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
#endif
#ifdef LF_HAVE_PEER
  m.def("ag_gemm", &ag_gemm);
  m.def("gemm_rs", &gemm_rs);
#endif
#ifdef LF_HAVE_GROUPED
  m.def("grouped_gemm", &grouped_gemm);
#endif
#ifdef LF_HAVE_MOE_PEER
  m.def("moe_push", &moe_push);
  m.def("moe_pull", &moe_pull);
  m.def("moe_signal", &moe_signal);
  m.def("moe_wait", &moe_wait);
#endif
#ifdef LF_HAVE_FP8
  m.def("quant_1x128", &quant_1x128);
  m.def("quant_128x128", &quant_128x128);
  m.def("gemm_fp8_blockwise", &gemm_fp8_blockwise);
#endif
#ifdef LF_HAVE_PEER_OPTIM
  m.def("grad_pull_reduce", &grad_pull_reduce);
  m.def("adam_push", &adam_push);
  m.def("peer_signal", &peer_signal);
  m.def("peer_wait", &peer_wait);
#endif
#ifdef LF_HAVE_DSA
  m.def("sparse_mla_fwd", &sparse_mla_fwd);
  m.def("sparse_mla_probs", &sparse_mla_probs);
  m.def("indexer_topk", &indexer_topk);
#endif
  m.def("router_fwd", &router_fwd);
  m.def("router_bwd", &router_bwd);
  m.def("set_peer_wait_budget_ms", &set_peer_wait_budget_ms);
  m.def("peer_wait_budget_ms", &peer_wait_budget_ms);
  m.def("launch_count", &launch_count);
  m.def("reset_launch_count", &reset_launch_count);
}
