// Host-side AdamW for optimizer-state offload: fp32 master weights and moments live in (pinned) host memory, the
// update runs on the CPU cores while the GPU computes, and the refreshed low-precision weights are written to a
// staging buffer for the copy back (the role DeepSpeed's CPU-Adam plays for the reference's optimizer CPU offload).
// Plain loops written so that the compiler vectorises them; at::parallel_for splits the range over the torch
// intra-op thread pool.
#include <torch/extension.h>
#include <ATen/Parallel.h>

#include <cmath>
#include <cstdint>

namespace {

inline uint16_t float_to_bf16_rn(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

template <typename G>
inline float load_grad(const G* g, int64_t i);
template <>
inline float load_grad<float>(const float* g, int64_t i) { return g[i]; }
template <>
inline float load_grad<uint16_t>(const uint16_t* g, int64_t i) {
  uint32_t u = static_cast<uint32_t>(g[i]) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

template <typename G>
void adam_loop(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
               uint16_t* __restrict__ out_bf16, int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1,
               float bc2, float grad_scale) {
  const float inv_bc1 = 1.0f / bc1, inv_sqrt_bc2 = 1.0f / std::sqrt(bc2);
  at::parallel_for(0, n, 1 << 15, [&](int64_t lo, int64_t hi) {
  for (int64_t i = lo; i < hi; ++i) {
    const float gi = load_grad<G>(g, i) * grad_scale;
    const float mi = b1 * m[i] + (1.0f - b1) * gi;
    const float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    float pi = p[i] * (1.0f - lr * wd);  // decoupled weight decay
    pi -= lr * (mi * inv_bc1) / (std::sqrt(vi) * inv_sqrt_bc2 + eps);
    p[i] = pi;
    if (out_bf16 != nullptr) out_bf16[i] = float_to_bf16_rn(pi);
  }
  });
}

}  // namespace

// master, exp_avg, exp_avg_sq: fp32 CPU tensors; grad: fp32 or bf16 CPU tensor; out: optional bf16 CPU tensor.
void cpu_adam_step(at::Tensor master, at::Tensor grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
                   c10::optional<at::Tensor> out_bf16, double lr, double beta1, double beta2, double eps,
                   double weight_decay, int64_t step, double grad_scale) {
  TORCH_CHECK(!master.is_cuda() && !grad.is_cuda(), "cpu_adam_step works on host tensors");
  TORCH_CHECK(master.scalar_type() == at::kFloat && exp_avg.scalar_type() == at::kFloat &&
              exp_avg_sq.scalar_type() == at::kFloat);
  TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && exp_avg.is_contiguous() && exp_avg_sq.is_contiguous());
  const int64_t n = master.numel();
  TORCH_CHECK(grad.numel() == n && exp_avg.numel() == n && exp_avg_sq.numel() == n);
  uint16_t* out = nullptr;
  if (out_bf16.has_value()) {
    TORCH_CHECK(out_bf16->scalar_type() == at::kBFloat16 && out_bf16->numel() == n && out_bf16->is_contiguous());
    out = reinterpret_cast<uint16_t*>(out_bf16->data_ptr());
  }
  const float bc1 = 1.0f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.0f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  if (grad.scalar_type() == at::kFloat) {
    adam_loop<float>(master.data_ptr<float>(), grad.data_ptr<float>(), exp_avg.data_ptr<float>(),
                     exp_avg_sq.data_ptr<float>(), out, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
  } else {
    TORCH_CHECK(grad.scalar_type() == at::kBFloat16, "grad must be fp32 or bf16");
    adam_loop<uint16_t>(master.data_ptr<float>(), reinterpret_cast<const uint16_t*>(grad.data_ptr()),
                        exp_avg.data_ptr<float>(), exp_avg_sq.data_ptr<float>(), out, n, lr, beta1, beta2, eps,
                        weight_decay, bc1, bc2, grad_scale);
  }
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def("cpu_adam_step", &cpu_adam_step); }
