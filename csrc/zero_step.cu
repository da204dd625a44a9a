// ZeRO-1 optimizer step with its collectives inside the kernels, sm_100a.
//
// Data-parallel ranks keep the flat fp32 gradient buffer and the flat 16-bit parameter buffer in
// symmetric memory, so every rank can address every peer's copy over NVLink. Two kernels replace
// reduce-scatter -> norm all-reduce -> Adam -> all-gather:
//
//   zero_reduce_kernel : for the shard [lo, hi) this rank owns, sum the gradient of all ranks
//       (plain P2P loads from every peer, or one multimem.ld_reduce through the NVSwitch multicast
//       address), store the sum in the local buffer, accumulate the weighted sum of squares, and have
//       the last CTA publish this rank's partial norm to every peer.
//   zero_adam_kernel   : wait for all partial norms, derive the clip coefficient, run Adam on the
//       shard (fp32 moments, optional fp32 master weights) and store the updated 16-bit parameters
//       into every rank's parameter buffer (P2P stores, or one multimem.st). The last CTA tells all
//       peers that this rank's parameters are out and waits until every peer said the same, so kernel
//       completion means "all parameters of all shards are in my buffer".
//
// Cross-rank ordering uses three cumulative counters per rank (gradients ready / norms published /
// parameters published), bumped with system-scope release reductions and awaited with bounded acquire
// polls; target = world * epoch with the epoch read from a device word (CUDA-graph safe).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kZeroMaxRegions = 8;
constexpr int kZeroMaxWorld = 16;

struct ZeroRegion {
  long long a, b;     // element range inside the flat buffer, already clipped to [lo, hi); multiples of 8
  float norm_weight;  // weight of this range in the global sum of squares (1/dp^2, / tp for replicated ranges)
  float weight_decay;
  int adam;           // 1: updated by zero_adam_kernel, 0: reduced only (another optimizer owns the update)
};

struct ZeroArgs {
  int rank, world;
  int n_regions;
  ZeroRegion regions[kZeroMaxRegions];
  float* const* peer_grads;     // device array [world]: every rank's flat fp32 gradient buffer
  const float* mc_grads;        // multicast address of the gradient buffer or null
  float* grads;                 // this rank's gradient buffer
  void* const* peer_params;     // device array [world]: every rank's flat 16-bit parameter buffer
  void* mc_params;              // multicast address of the parameter buffer or null
  void* params;                 // this rank's parameter buffer
  float* master;                // fp32 master weights of the shard (index relative to lo) or null
  float* exp_avg;               // fp32 moments of the shard (index relative to lo)
  float* exp_avg_sq;
  long long lo;                 // first element of this rank's shard
  int* const* peer_ctr;         // device array [world]: every rank's int[4] counters
  int* ctr;                     // this rank's counters: [0] grads ready, [1] norms published, [2] params published
  float* const* peer_norm;      // device array [world]: every rank's float[2][kZeroMaxWorld] partial-norm slots
  const float* norm_slots;      // this rank's slots
  const int* epoch_ptr;         // device word: steps completed so far on this workspace
  unsigned int* ticket;         // local: CTA completion ticket (reset by the last CTA)
  float* sumsq_acc;             // local: weighted sum of squares accumulator (reset by the last CTA)
  float* norm_out;              // local: global gradient norm (written by zero_adam_kernel)
  float* coef_out;              // local: clip coefficient
  float lr, beta1, beta2, eps, step_size, grad_scale, clip;
  int p_fmt;                    // 1 bf16, 0 fp16
  int* status;
};

__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ float block_sum_256(float s, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x == 0)
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[w];
  return t;  // valid on thread 0
}

__global__ void __launch_bounds__(256) zero_reduce_kernel(const ZeroArgs args) {
  __shared__ float sh[8];
  __shared__ int ok_sh;
  const int epoch = *args.epoch_ptr + 1;
  // 1. my gradients are complete (stream order): tell every rank, then wait for every rank.
  if (blockIdx.x == 0 && threadIdx.x < args.world) {
    __threadfence_system();
    red_release_sys_add(args.peer_ctr[threadIdx.x] + 0, 1);
  }
  if (threadIdx.x == 0) ok_sh = wait_flag_sys(args.ctr + 0, args.world * epoch, args.status, kTimeoutPeerFlag) ? 1 : 0;
  __syncthreads();
  float acc = 0.f;
  if (ok_sh) {
    const long long stride = (long long)gridDim.x * blockDim.x * 4;
    for (int r = 0; r < args.n_regions; ++r) {
      const ZeroRegion reg = args.regions[r];
      float s = 0.f;
      for (long long i = reg.a + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < reg.b; i += stride) {
        float4 g;
        if (args.mc_grads != nullptr) {
          g = multimem_ld_reduce_f32x4(args.mc_grads + i);
        } else {
          g = make_float4(0.f, 0.f, 0.f, 0.f);
          float4 v[kZeroMaxWorld];
#pragma unroll 8
          for (int p = 0; p < args.world; ++p) v[p] = ld_f4(args.peer_grads[(args.rank + p) % args.world] + i);
#pragma unroll 8
          for (int p = 0; p < args.world; ++p) { g.x += v[p].x; g.y += v[p].y; g.z += v[p].z; g.w += v[p].w; }
        }
        *reinterpret_cast<float4*>(args.grads + i) = g;
        s += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
      }
      acc += s * reg.norm_weight;
    }
  }
  const float total = block_sum_256(acc, sh);
  // 2. last CTA publishes this rank's partial sum of squares to every rank.
  if (threadIdx.x == 0) {
    atomicAdd(args.sumsq_acc, total);
    __threadfence();
    const unsigned int t = atomicAdd(args.ticket, 1u);
    if (t == gridDim.x - 1) {
      __threadfence();
      const float mine = atomicExch(args.sumsq_acc, 0.f);
      *args.ticket = 0u;
      for (int p = 0; p < args.world; ++p) {
        float* slot = args.peer_norm[p] + (epoch & 1) * kZeroMaxWorld + args.rank;
        *reinterpret_cast<volatile float*>(slot) = mine;
      }
      __threadfence_system();
      for (int p = 0; p < args.world; ++p) red_release_sys_add(args.peer_ctr[p] + 1, 1);
    }
  }
}

template <int FMT>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if (FMT == 1) return unpack_bf16x2(w);
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <int FMT>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  return FMT == 1 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

template <int FMT>
__global__ void __launch_bounds__(256) zero_adam_kernel(const ZeroArgs args) {
  __shared__ float coef_sh;
  __shared__ int ok_sh;
  const int epoch = *args.epoch_ptr + 1;
  if (threadIdx.x == 0) {
    const bool ok = wait_flag_sys(args.ctr + 1, args.world * epoch, args.status, kTimeoutPeerFlag);
    float total = 0.f;
    for (int p = 0; p < args.world; ++p)
      total += *reinterpret_cast<const volatile float*>(args.norm_slots + (epoch & 1) * kZeroMaxWorld + p);
    const float nrm = sqrtf(total);
    float c = 1.f;
    if (args.clip > 0.f) c = fminf(1.f, args.clip / (nrm + 1e-6f));
    coef_sh = c;
    ok_sh = ok ? 1 : 0;
    if (blockIdx.x == 0) { *args.norm_out = nrm; *args.coef_out = c; }
  }
  __syncthreads();
  if (ok_sh) {
    const float gs = args.grad_scale * coef_sh;
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (int r = 0; r < args.n_regions; ++r) {
      const ZeroRegion reg = args.regions[r];
      if (!reg.adam) continue;
      const float decay = 1.f - args.lr * reg.weight_decay;
      for (long long i = reg.a + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < reg.b; i += stride) {
        const long long j = i - args.lo;
        float g[8], m[8], v[8], p[8];
        *reinterpret_cast<float4*>(g) = ld_f4(args.grads + i);
        *reinterpret_cast<float4*>(g + 4) = ld_f4(args.grads + i + 4);
        *reinterpret_cast<float4*>(m) = ld_f4(args.exp_avg + j);
        *reinterpret_cast<float4*>(m + 4) = ld_f4(args.exp_avg + j + 4);
        *reinterpret_cast<float4*>(v) = ld_f4(args.exp_avg_sq + j);
        *reinterpret_cast<float4*>(v + 4) = ld_f4(args.exp_avg_sq + j + 4);
        if (args.master != nullptr) {
          *reinterpret_cast<float4*>(p) = ld_f4(args.master + j);
          *reinterpret_cast<float4*>(p + 4) = ld_f4(args.master + j + 4);
        } else {
          const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(args.params) + i);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = unpack2<FMT>(w[t]);
            p[2 * t] = f.x; p[2 * t + 1] = f.y;
          }
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float gg = g[t] * gs;
          m[t] = args.beta1 * m[t] + (1.f - args.beta1) * gg;
          v[t] = args.beta2 * v[t] + (1.f - args.beta2) * gg * gg;
          p[t] = p[t] * decay - args.step_size * m[t] / (sqrtf(v[t]) + args.eps);
        }
        *reinterpret_cast<float4*>(args.exp_avg + j) = *reinterpret_cast<float4*>(m);
        *reinterpret_cast<float4*>(args.exp_avg + j + 4) = *reinterpret_cast<float4*>(m + 4);
        *reinterpret_cast<float4*>(args.exp_avg_sq + j) = *reinterpret_cast<float4*>(v);
        *reinterpret_cast<float4*>(args.exp_avg_sq + j + 4) = *reinterpret_cast<float4*>(v + 4);
        if (args.master != nullptr) {
          *reinterpret_cast<float4*>(args.master + j) = *reinterpret_cast<float4*>(p);
          *reinterpret_cast<float4*>(args.master + j + 4) = *reinterpret_cast<float4*>(p + 4);
        }
        uint4 o;
        o.x = pack2<FMT>(p[0], p[1]); o.y = pack2<FMT>(p[2], p[3]);
        o.z = pack2<FMT>(p[4], p[5]); o.w = pack2<FMT>(p[6], p[7]);
        if (args.mc_params != nullptr) {
          multimem_st_v4(reinterpret_cast<uint16_t*>(args.mc_params) + i, o);
        } else {
          for (int q = 0; q < args.world; ++q) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(args.peer_params[(args.rank + q) % args.world]) + i;
            *reinterpret_cast<uint4*>(dst) = o;
          }
        }
      }
    }
  }
  // All of this rank's parameter stores are out when its last CTA gets here: tell every rank, then wait
  // until every rank has told us, so that whatever follows this kernel reads a complete buffer.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int t = atomicAdd(args.ticket, 1u);
    if (t == gridDim.x - 1) {
      *args.ticket = 0u;
      __threadfence_system();
      for (int p = 0; p < args.world; ++p) red_release_sys_add(args.peer_ctr[p] + 2, 1);
      wait_flag_sys(args.ctr + 2, args.world * epoch, args.status, kTimeoutPeerFlag);
    }
  }
}

}  // namespace icb

using namespace icb;

// One fused ZeRO-1 step over a data-parallel group of `world` ranks (<= 16).
//   regions: host array [n_regions][5] of doubles {a, b, norm_weight, weight_decay, adam} with [a, b) inside this
//            rank's shard [lo, hi), multiples of 8 elements.
//   peer_* : device arrays [world] of symmetric-memory peer pointers; mc_* the multicast addresses or null.
//   ctr / norm_slots: this rank's int[4] counters and float[2][16] slots (zero-initialised symmetric memory);
//   scratch: local device memory, 2 words (ticket, accumulator), zero-initialised once.
//   phase 1 launches the reduction only, phase 2 the Adam + parameter broadcast only, 3 both.
ICB_API int icb_zero_step(int phase, int rank, int world, int n_regions, const double* regions, float* const* peer_grads,
                          const float* mc_grads, float* grads, void* const* peer_params, void* mc_params, void* params,
                          float* master, float* exp_avg, float* exp_avg_sq, long long lo, int* const* peer_ctr, int* ctr,
                          float* const* peer_norm, const float* norm_slots, const int* epoch_ptr, void* scratch,
                          float* norm_out, float* coef_out, float lr, float beta1, float beta2, float eps,
                          float step_size, float grad_scale, float clip, int p_dtype, int* status, void* stream_) {
  if (world < 1 || world > kZeroMaxWorld || n_regions < 0 || n_regions > kZeroMaxRegions) return -2;
  if (p_dtype != kBF16 && p_dtype != 1) return -3;
  ZeroArgs a;
  a.rank = rank; a.world = world; a.n_regions = n_regions;
  long long n_total = 0;
  for (int r = 0; r < n_regions; ++r) {
    a.regions[r].a = (long long)regions[r * 5 + 0];
    a.regions[r].b = (long long)regions[r * 5 + 1];
    a.regions[r].norm_weight = (float)regions[r * 5 + 2];
    a.regions[r].weight_decay = (float)regions[r * 5 + 3];
    a.regions[r].adam = regions[r * 5 + 4] != 0.0 ? 1 : 0;
    if (a.regions[r].a % 8 || a.regions[r].b % 8 || a.regions[r].b < a.regions[r].a) return -4;
    n_total += a.regions[r].b - a.regions[r].a;
  }
  a.peer_grads = peer_grads; a.mc_grads = mc_grads; a.grads = grads;
  a.peer_params = peer_params; a.mc_params = mc_params; a.params = params;
  a.master = master; a.exp_avg = exp_avg; a.exp_avg_sq = exp_avg_sq; a.lo = lo;
  a.peer_ctr = peer_ctr; a.ctr = ctr; a.peer_norm = peer_norm; a.norm_slots = norm_slots;
  a.epoch_ptr = epoch_ptr;
  a.ticket = reinterpret_cast<unsigned int*>(scratch);
  a.sumsq_acc = reinterpret_cast<float*>(scratch) + 1;
  a.norm_out = norm_out; a.coef_out = coef_out;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.step_size = step_size;
  a.grad_scale = grad_scale; a.clip = clip;
  a.p_fmt = (p_dtype == kBF16) ? 1 : 0;
  a.status = status;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  long long blocks = (n_total / 8 + 255) / 256;
  const long long cap = (long long)num_sms() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (phase & 1) {
    zero_reduce_kernel<<<(int)blocks, 256, 0, stream>>>(a);
    int rc = check_launch("zero_reduce_kernel");
    if (rc) return rc;
  }
  if (phase & 2) {
    if (a.p_fmt == 1) zero_adam_kernel<1><<<(int)blocks, 256, 0, stream>>>(a);
    else zero_adam_kernel<0><<<(int)blocks, 256, 0, stream>>>(a);
    return check_launch("zero_adam_kernel");
  }
  return 0;
}
