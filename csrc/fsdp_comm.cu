// FSDP collectives as kernels over symmetric memory, sm_100a (opt-in; the NCCL path is the default).
//
//   fsdp_gather_kernel         : every rank copies its parameter shard into slot `rank` of every rank's full
//                                buffer (16-byte P2P stores, or one multimem.st through the NVSwitch multicast
//                                mapping). Opening barrier: "my full buffer may be overwritten" from all ranks;
//                                closing barrier: "my shard is everywhere" from all ranks, so kernel completion
//                                means the local full buffer is complete.
//   fsdp_reduce_scatter_kernel : after "my flat gradient is complete" from all ranks, the owner of a shard sums
//                                that range over all ranks (P2P loads of 16-bit or fp32 gradients, or one
//                                multimem.ld_reduce) and accumulates it, scaled, into its fp32 gradient shard
//                                (the cast / scale / accumulate of the bucket is fused into the reduction).
//                                Closing barrier: all ranks are done reading, the flat buffers may be reused.
//
// Counters are cumulative (target = world * calls), the call count lives in a device word, waits are bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kFsdpMaxWorld = 16;

struct FsdpArgs {
  int rank, world;
  long long shard_elems;          // elements per shard (multiple of 8)
  // gather
  const void* shard;              // this rank's shard (16-bit)
  void* const* peer_full;         // device array [world]: every rank's full buffer (16-bit, world * shard_elems)
  void* mc_full;                  // multicast address of the full buffer or null
  // reduce-scatter
  const void* const* peer_flat;   // device array [world]: every rank's flat gradient (world * shard_elems)
  const void* mc_flat;            // multicast address of the flat gradient or null
  float* grad_shard;              // this rank's fp32 gradient shard (accumulated into)
  float scale;
  int flat_fmt;                   // 0 fp16, 1 bf16, 2 fp32
  // synchronisation
  int* const* peer_ctr;           // device array [world]: every rank's int[4] counters
  int* ctr;                       // [0] gather open, [1] gather close, [2] reduce open, [3] reduce close
  const int* epoch_ptr;           // device word: calls of this kernel kind completed so far
  unsigned int* ticket;
  int* status;
};

__device__ __forceinline__ bool fsdp_open(const FsdpArgs& a, int idx, int epoch, int* ok_sh) {
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    red_release_sys_add(a.peer_ctr[threadIdx.x] + idx, 1);
  }
  if (threadIdx.x == 0) *ok_sh = wait_flag_sys(a.ctr + idx, a.world * epoch, a.status, kTimeoutPeerFlag) ? 1 : 0;
  __syncthreads();
  return *ok_sh != 0;
}

__device__ __forceinline__ void fsdp_close(const FsdpArgs& a, int idx, int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.ticket, 1u) == gridDim.x - 1) {
      *a.ticket = 0u;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) red_release_sys_add(a.peer_ctr[p] + idx, 1);
      wait_flag_sys(a.ctr + idx, a.world * epoch, a.status, kTimeoutPeerFlag);
    }
  }
}

__global__ void __launch_bounds__(256) fsdp_gather_kernel(const FsdpArgs a) {
  __shared__ int ok_sh;
  const int epoch = *a.epoch_ptr + 1;
  if (fsdp_open(a, 0, epoch, &ok_sh)) {
    const long long n16 = a.shard_elems / 8;                 // 16-byte pieces
    const long long base = (long long)a.rank * n16;
    const uint4* src = reinterpret_cast<const uint4*>(a.shard);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
      const uint4 v = src[i];
      if (a.mc_full != nullptr) {
        multimem_st_v4(reinterpret_cast<uint4*>(a.mc_full) + base + i, v);
      } else {
        for (int q = 0; q < a.world; ++q)
          reinterpret_cast<uint4*>(a.peer_full[(a.rank + q) % a.world])[base + i] = v;
      }
    }
  }
  fsdp_close(a, 1, epoch);
}

__device__ __forceinline__ void acc16(float* s, uint4 u, int fmt) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 f = fmt == 1 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
    s[2 * t] += f.x;
    s[2 * t + 1] += f.y;
  }
}

__global__ void __launch_bounds__(256) fsdp_reduce_scatter_kernel(const FsdpArgs a) {
  __shared__ int ok_sh;
  const int epoch = *a.epoch_ptr + 1;
  if (fsdp_open(a, 2, epoch, &ok_sh)) {
    const long long n8 = a.shard_elems / 8;                  // groups of 8 elements
    const long long base = (long long)a.rank * a.shard_elems;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n8; g += stride) {
      const long long e0 = base + g * 8;
      float s[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = 0.f;
      if (a.flat_fmt == 2) {
        for (int q = 0; q < a.world; ++q) {
          const float* p = reinterpret_cast<const float*>(a.peer_flat[(a.rank + q) % a.world]) + e0;
          const float4 x = *reinterpret_cast<const float4*>(p), y = *reinterpret_cast<const float4*>(p + 4);
          s[0] += x.x; s[1] += x.y; s[2] += x.z; s[3] += x.w;
          s[4] += y.x; s[5] += y.y; s[6] += y.z; s[7] += y.w;
        }
      } else if (a.mc_flat != nullptr) {
        const uint8_t* p = reinterpret_cast<const uint8_t*>(a.mc_flat) + e0 * 2;
        acc16(s, a.flat_fmt == 1 ? multimem_ld_reduce_bf16x8(p) : multimem_ld_reduce_f16x8(p), a.flat_fmt);
      } else {
        for (int q = 0; q < a.world; ++q) {
          const uint4 u = *reinterpret_cast<const uint4*>(
              reinterpret_cast<const uint8_t*>(a.peer_flat[(a.rank + q) % a.world]) + e0 * 2);
          acc16(s, u, a.flat_fmt);
        }
      }
      float* dst = a.grad_shard + g * 8;
      float4 d0 = *reinterpret_cast<float4*>(dst), d1 = *reinterpret_cast<float4*>(dst + 4);
      d0.x += s[0] * a.scale; d0.y += s[1] * a.scale; d0.z += s[2] * a.scale; d0.w += s[3] * a.scale;
      d1.x += s[4] * a.scale; d1.y += s[5] * a.scale; d1.z += s[6] * a.scale; d1.w += s[7] * a.scale;
      *reinterpret_cast<float4*>(dst) = d0;
      *reinterpret_cast<float4*>(dst + 4) = d1;
    }
  }
  fsdp_close(a, 3, epoch);
}

static int fsdp_grid(long long work) {
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)num_sms() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace icb

using namespace icb;

// Parameter all-gather of one FSDP unit: shard [shard_elems] -> slot `rank` of every rank's full buffer.
ICB_API int icb_fsdp_gather(const void* shard, long long shard_elems, void* const* peer_full, void* mc_full, int rank,
                            int world, int* const* peer_ctr, int* ctr, const int* epoch_ptr, void* ticket, int* status,
                            void* stream_) {
  if (world < 1 || world > kFsdpMaxWorld || shard_elems % 8 != 0) return -2;
  FsdpArgs a{};
  a.rank = rank; a.world = world; a.shard_elems = shard_elems;
  a.shard = shard; a.peer_full = peer_full; a.mc_full = mc_full;
  a.peer_ctr = peer_ctr; a.ctr = ctr; a.epoch_ptr = epoch_ptr;
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  a.status = status;
  fsdp_gather_kernel<<<fsdp_grid(shard_elems / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  return check_launch("fsdp_gather_kernel");
}

// Gradient reduce-scatter of one FSDP unit with the accumulate fused:
// grad_shard[i] += scale * sum_r flat_r[rank * shard_elems + i]. flat_dtype: 0 bf16, 1 fp16, 2 fp32 (DType codes).
ICB_API int icb_fsdp_reduce_scatter(const void* const* peer_flat, const void* mc_flat, float* grad_shard,
                                    long long shard_elems, float scale, int flat_dtype, int rank, int world,
                                    int* const* peer_ctr, int* ctr, const int* epoch_ptr, void* ticket, int* status,
                                    void* stream_) {
  if (world < 1 || world > kFsdpMaxWorld || shard_elems % 8 != 0) return -2;
  FsdpArgs a{};
  a.rank = rank; a.world = world; a.shard_elems = shard_elems;
  a.peer_flat = peer_flat; a.mc_flat = (flat_dtype == kF32) ? nullptr : mc_flat;
  a.grad_shard = grad_shard; a.scale = scale;
  a.flat_fmt = flat_dtype == kF32 ? 2 : (flat_dtype == kBF16 ? 1 : 0);
  a.peer_ctr = peer_ctr; a.ctr = ctr; a.epoch_ptr = epoch_ptr;
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  a.status = status;
  fsdp_reduce_scatter_kernel<<<fsdp_grid(shard_elems / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  return check_launch("fsdp_reduce_scatter_kernel");
}
