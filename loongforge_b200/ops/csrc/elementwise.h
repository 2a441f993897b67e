// Host launchers of the bandwidth-bound kernels in elementwise.cu (raw pointers + stream).
#pragma once
#include <cuda_runtime.h>

namespace lf {

void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long T, int H, long long x_stride,
                 long long y_stride, float eps, float w_offset, cudaStream_t s);
// Number of CTAs (= rows of the fp32 `dw_partial[grid, H]` scratch) the backward uses for T rows.
int rmsnorm_bwd_grid(long long T);
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                 float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, long long T, int H, float w_offset,
                 cudaStream_t s);
void rope_inplace(void* x, const float* freqs, const int* pos_ids, int T, int heads, int D, int rot_dim,
                  int rot_offset, long long t_stride, long long h_stride, int group, int rope_in_group,
                  int interleaved, float mscale, float sign, cudaStream_t s);
// y = x H_128 / sqrt(128) on `rows` contiguous rows of 128 bf16 (x and y may alias).
void hadamard128(const void* x, void* y, long long rows, cudaStream_t s);
void swiglu_fwd(const void* in, void* out, long long T, int F, cudaStream_t s);
void swiglu_bwd(const void* dout, const void* in, void* din, long long T, int F, cudaStream_t s);
void ce_stats(const void* logits, const long long* labels, float* row_max, float* row_sum, float* tgt, long long T,
              int V, long long ld, int vocab_start, int valid_v, cudaStream_t s);
void ce_dlogits(void* logits, const long long* labels, const float* gmax, const float* gsum, const float* row_scale,
                long long T, int V, long long ld, int vocab_start, int valid_v, cudaStream_t s);
void adam_step(float* master, const void* grad, int grad_is_bf16, void* m, void* v, int moments_bf16,
               void* model_out, long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
               float bc2, float grad_scale, cudaStream_t s);
void adam_step_remainder(void* w, void* lo, const void* grad, int grad_is_bf16, void* m, void* v, int moments_bf16,
                         long long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                         float grad_scale, cudaStream_t s);
void master_split(const float* master, void* w, void* lo, long long n, int write_w, cudaStream_t s);
void master_join(const void* w, const void* lo, float* master, long long n, cudaStream_t s);
// out[0] += sum x^2, deterministic: per-CTA partial sums go to `partial` (at least sumsq_partials(n) floats of
// scratch) and are added in a fixed order.
int sumsq_partials(long long n);
void sumsq(const void* x, int is_bf16, long long n, float* out, float* partial, cudaStream_t s);

// MoE router (router.cu). score: 0 softmax over the selected k, 1 softmax over all experts then top-k, 2 sigmoid.
struct RouterArgs {
  const void* logits = nullptr;  // [T, E] fp32 or bf16
  int logits_bf16 = 0;
  const float* bias = nullptr;   // [E], selection only
  float* probs = nullptr;        // [T, E], zero off the top-k
  unsigned char* map = nullptr;  // [T, E] 0/1
  float* aux = nullptr;          // [T, E] scores for the load-balancing loss
  int* topk_idx = nullptr;       // [T, k]
  int* counts = nullptr;         // [E] += tokens routed to each expert (optional)
  const float* dprobs = nullptr; // backward inputs / output
  const float* daux = nullptr;
  float* dlogits = nullptr;
  int T = 0, E = 0, k = 0, score = 0, num_groups = 0, group_topk = 0;
  float scale = 1.f;
};
// 0 on success; negative when E > 512, k > 32, or the group shape is unsupported (callers fall back).
int router_fwd(const RouterArgs& a, cudaStream_t s);
int router_bwd(const RouterArgs& a, cudaStream_t s);

}  // namespace lf
