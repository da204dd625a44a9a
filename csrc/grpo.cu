// GRPO token loss, forward and gradient in one pass (fp32 per-token vectors):
//   rho   = exp(logp - logp_old)
//   pg    = -min(rho * A, clip(rho, 1 - eps, 1 + eps) * A)
//   delta = logp_ref - logp ;  kl = exp(delta) - delta - 1        (k3 estimator)
//   loss  = mask * (pg + beta * kl)
//   dloss/dlogp = mask * (-(rho * A if the unclipped branch is active or rho is inside the clip
//                          range else 0) + beta * (1 - exp(delta)))
// Also emits the per-token ratio and kl for logging.
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

__global__ void grpo_loss_kernel(const float* __restrict__ logp, const float* __restrict__ logp_old,
                                 const float* __restrict__ logp_ref, const float* __restrict__ adv,
                                 const float* __restrict__ mask, float* __restrict__ loss, float* __restrict__ dlogp,
                                 float* __restrict__ ratio_out, float* __restrict__ kl_out, long long n, float eps,
                                 float beta) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float mk = mask[i];
  const float lp = logp[i];
  const float a = adv[i];
  const float rho = __expf(lp - logp_old[i]);
  const float clipped = fminf(fmaxf(rho, 1.f - eps), 1.f + eps);
  const float t1 = rho * a, t2 = clipped * a;
  const bool unclipped_active = t1 <= t2;
  const bool in_range = (rho >= 1.f - eps) && (rho <= 1.f + eps);
  const float pg = -fminf(t1, t2);
  const float dpg = -((unclipped_active || in_range) ? rho * a : 0.f);
  float kl = 0.f, dkl = 0.f;
  if (logp_ref != nullptr) {
    const float delta = logp_ref[i] - lp;
    const float ed = __expf(delta);
    kl = ed - delta - 1.f;
    dkl = 1.f - ed;
  }
  loss[i] = mk * (pg + beta * kl);
  dlogp[i] = mk * (dpg + beta * dkl);
  if (ratio_out != nullptr) ratio_out[i] = rho;
  if (kl_out != nullptr) kl_out[i] = kl;
}

}  // namespace icb

ICB_API int icb_grpo_loss(const float* logp, const float* logp_old, const float* logp_ref, const float* adv,
                          const float* mask, float* loss, float* dlogp, float* ratio, float* kl, long long n, float eps,
                          float beta, void* stream) {
  if (n <= 0) return 0;
  const int th = 256;
  const long long bl = (n + th - 1) / th;
  icb::grpo_loss_kernel<<<(unsigned)bl, th, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logp, logp_old, logp_ref, adv, mask, loss, dlogp, ratio, kl, n, eps, beta);
  return icb::check_launch("grpo_loss");
}
