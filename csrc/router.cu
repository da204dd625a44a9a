// Mixture-of-experts router on sm_100a: softmax over the expert logits, top-k selection, the histogram of
// expert loads and the mean routing probabilities in one pass (one warp per token), and its backward.
//
//   forward : probs = softmax(logits[t, :]) ; (w, idx)[t, 0..k) = top-k of probs (optionally renormalised to sum 1);
//             counts[e] += #slots routed to e ; psum[e] += probs[t, e]   (load-balance loss: coeff * E * sum_e f_e P_e
//             with f_e = counts[e] / (T k), P_e = psum[e] / T)
//   backward: dprobs[t, e] = (gradient of the selected weights) + aux_scale * counts[e] ;
//             dlogits = probs * (dprobs - sum_e probs * dprobs)
// The logits come from the tcgen05 GEMM (x @ W_r^T, fp32 output); E <= 256, k <= 8.
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kRouterMaxPerLane = 8;   // E <= 256
constexpr int kRouterMaxK = 8;

__global__ void __launch_bounds__(256)
router_fwd_kernel(const float* __restrict__ logits, int T, int E, int K, int normalize, float* __restrict__ probs,
                  float* __restrict__ w_out, int* __restrict__ idx_out, int* __restrict__ counts,
                  float* __restrict__ psum) {
  __shared__ float sh_p[256];
  __shared__ int sh_c[256];
  for (int i = threadIdx.x; i < E; i += blockDim.x) { sh_p[i] = 0.f; sh_c[i] = 0; }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_lane = (E + 31) >> 5;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    float v[kRouterMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      v[j] = (j < per_lane && e < E) ? logits[(size_t)t * E + e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      v[j] = (v[j] == -INFINITY) ? 0.f : __expf(v[j] - mx);
      s += v[j];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      v[j] *= inv;
      if (j < per_lane && e < E) {
        probs[(size_t)t * E + e] = v[j];
        atomicAdd(&sh_p[e], v[j]);
      }
      // a row of NaN logits (a diverged run) still has to select K valid experts: the probabilities written
      // above carry the NaN to the loss, the selection below sees zeros
      if (!(v[j] >= 0.f)) v[j] = 0.f;
    }
    // top-k by k rounds of warp arg-max (ties: lowest expert index, like torch.topk on distinct values)
    float taken_w[kRouterMaxK];
    int taken_e[kRouterMaxK];
    float wsum = 0.f;
    for (int r = 0; r < K; ++r) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kRouterMaxPerLane; ++j) {
        const int e = j * 32 + lane;
        if (j < per_lane && e < E && (v[j] > best || (v[j] == best && e < best_e))) { best = v[j]; best_e = e; }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      best_e = min(best_e, E - 1);     // (unreachable for K <= E: every round finds an expert)
      taken_w[r] = best;
      taken_e[r] = best_e;
      wsum += best;
      if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;     // remove the winner from the next rounds
    }
    if (lane == 0) {
      const float norm = normalize ? 1.f / fmaxf(wsum, 1e-20f) : 1.f;
      for (int r = 0; r < K; ++r) {
        w_out[(size_t)t * K + r] = taken_w[r] * norm;
        idx_out[(size_t)t * K + r] = taken_e[r];
        atomicAdd(&sh_c[taken_e[r]], 1);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    if (sh_c[i]) atomicAdd(&counts[i], sh_c[i]);
    if (sh_p[i] != 0.f) atomicAdd(&psum[i], sh_p[i]);
  }
}

// dw: [T, K] gradient of the returned weights; aux_scale = d(aux)/d(psum[e]) / counts[e] = coeff * E / (T * T * K)
// times the incoming gradient of the aux loss (a device scalar).
__global__ void __launch_bounds__(256)
router_bwd_kernel(const float* __restrict__ probs, const float* __restrict__ dw, const int* __restrict__ idx,
                  const int* __restrict__ counts, const float* __restrict__ daux, float aux_scale, int T, int E, int K,
                  int normalize, float* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_lane = (E + 31) >> 5;
  const float ga = (daux != nullptr ? *daux : 0.f) * aux_scale;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    float p[kRouterMaxPerLane], dp[kRouterMaxPerLane];
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      const bool ok = j < per_lane && e < E;
      p[j] = ok ? probs[(size_t)t * E + e] : 0.f;
      dp[j] = ok ? ga * static_cast<float>(counts[e]) : 0.f;
    }
    // selected weights: w_r = p[e_r] (or p[e_r] / S with S = sum of the selected): route their gradients to dprobs
    float sel_p[kRouterMaxK], sel_g[kRouterMaxK];
    int sel_e[kRouterMaxK];
    float S = 0.f, dot = 0.f;
    for (int r = 0; r < K; ++r) {
      sel_e[r] = idx[(size_t)t * K + r];
      sel_g[r] = dw[(size_t)t * K + r];
      sel_p[r] = probs[(size_t)t * E + sel_e[r]];
      S += sel_p[r];
      dot += sel_g[r] * sel_p[r];
    }
    S = fmaxf(S, 1e-20f);
    for (int r = 0; r < K; ++r) {
      // d w_r / d p[e_q] = delta_rq / S - p[e_r] / S^2  (normalised) ; delta_rq (plain)
      const float g = normalize ? (sel_g[r] / S - dot / (S * S)) : sel_g[r];
      if ((sel_e[r] & 31) == lane) dp[sel_e[r] >> 5] += g;
    }
    float inner = 0.f;
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) inner += p[j] * dp[j];
    inner = warp_sum(inner);
#pragma unroll
    for (int j = 0; j < kRouterMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      if (j < per_lane && e < E) dlogits[(size_t)t * E + e] = p[j] * (dp[j] - inner);
    }
  }
}

}  // namespace icb

using namespace icb;

// logits, probs: [T, E] fp32; w_out [T, K] fp32; idx_out [T, K] int32; counts [E] int32 and psum [E] fp32 are
// accumulated into (zero them first). E <= 256, K <= 8.
ICB_API int icb_router_fwd(const float* logits, int T, int E, int K, int normalize, float* probs, float* w_out,
                           int* idx_out, int* counts, float* psum, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kRouterMaxPerLane || K < 1 || K > kRouterMaxK || K > E) return -2;
  int blocks = (T + 7) / 8;
  const int cap = num_sms() * 4;
  if (blocks > cap) blocks = cap;
  router_fwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, T, E, K, normalize, probs,
                                                                                 w_out, idx_out, counts, psum);
  return check_launch("router_fwd_kernel");
}

ICB_API int icb_router_bwd(const float* probs, const float* dw, const int* idx, const int* counts, const float* daux,
                           float aux_scale, int T, int E, int K, int normalize, float* dlogits, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kRouterMaxPerLane || K < 1 || K > kRouterMaxK) return -2;
  int blocks = (T + 7) / 8;
  const int cap = num_sms() * 4;
  if (blocks > cap) blocks = cap;
  router_bwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(probs, dw, idx, counts, daux, aux_scale,
                                                                                 T, E, K, normalize, dlogits);
  return check_launch("router_bwd_kernel");
}
