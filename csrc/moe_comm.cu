// Expert-parallel token exchange of a mixture-of-experts layer inside CUDA kernels, sm_100a.
//
// Every rank of the expert-parallel group owns E / ep experts and a receive buffer in symmetric
// memory laid out exactly as the grouped GEMM wants it: rows sorted by local expert, every expert's
// segment padded to 128 rows. Three kernels replace sort + index_select + all-to-all (x3) + index_copy:
//
//   moe_count_kernel   : histogram of this rank's token slots per expert and the position of every
//                        slot inside its (rank, expert) run; the last CTA stores the histogram row into
//                        every rank's counts matrix and bumps their "counts" counter.
//   moe_push_kernel    : waits for all rows of the counts matrix; every CTA derives (in shared memory)
//                        the segment starts of every owner and this rank's base offset inside each
//                        segment, so the destination row of a slot is base[e] + pos[s] with no further
//                        communication; one warp per slot copies the token's row with 16-byte P2P stores
//                        straight into the owner's receive buffer (dispatch = permute + transfer in one
//                        pass). The owner's CTAs also zero the padding rows of its segments and write the
//                        grouped GEMM's tables (segment offsets, expert of every 128-row tile). The last CTA
//                        bumps every rank's "rows arrived" counter and waits for all ranks, so kernel
//                        completion means the receive buffer is complete.
//                        The same kernel, given destinations, pushes gradient rows in the backward pass.
//   moe_pull_kernel    : signals that this rank's expert outputs are complete, waits for all ranks, then
//                        one warp per token reads its k expert-output rows from the owners with P2P loads,
//                        weights and sums them in fp32 (+ an optional addend) and writes the token's output;
//                        optionally keeps the k gathered rows for the router-weight gradient.
//
// Counters are cumulative (target = ep * calls made, counted in device words per kernel kind) and every wait is
// bounded. Buffers are single: each kernel's closing barrier orders the next writer behind the last reader.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kMoeMaxExperts = 256;
constexpr int kMoeMaxEp = 16;

struct MoeCountArgs {
  const int* expert;        // [S] expert id of every slot
  int S, E, ep, rank;
  int* hist;                // local [E], zero on entry, left zero on exit
  int* pos;                 // [S] out: index of the slot inside this rank's run of its expert
  int* const* peer_counts;  // device array [ep]: every rank's counts matrix [ep][E]
  int* const* peer_ctr;     // device array [ep]: every rank's int[4] counters
  unsigned int* ticket;     // local, zero on entry and exit
};

__global__ void __launch_bounds__(256) moe_count_kernel(const MoeCountArgs a) {
  const int lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long s0 = (long long)blockIdx.x * blockDim.x; s0 < a.S; s0 += stride) {
    const long long s = s0 + threadIdx.x;
    bool valid = s < a.S;
    const int e = valid ? a.expert[s] : -1;
    if (valid && (unsigned)e >= (unsigned)a.E) {   // not an expert id: the slot is dropped (moe_push reports it)
      a.pos[s] = -1;
      valid = false;
    }
    // warp-aggregated atomics: lanes with the same expert take consecutive positions
    const unsigned active = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned peers = __match_any_sync(active, e);
      const int leader = __ffs(peers) - 1;
      const int my = __popc(peers & ((1u << lane) - 1u));
      int base = 0;
      if (lane == leader) base = atomicAdd(a.hist + e, __popc(peers));
      base = __shfl_sync(peers, base, leader);
      a.pos[s] = base + my;
    }
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned int last_sh;
  if (threadIdx.x == 0) {
    __threadfence();
    last_sh = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (last_sh) {
    __threadfence();
    // publish this rank's histogram row to every rank, then reset the local scratch
    for (int i = threadIdx.x; i < a.E; i += blockDim.x) {
      const int c = atomicExch(a.hist + i, 0);
      for (int p = 0; p < a.ep; ++p)
        *reinterpret_cast<volatile int*>(a.peer_counts[p] + a.rank * a.E + i) = c;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < a.ep) {
      __threadfence_system();
      red_release_sys_add(a.peer_ctr[threadIdx.x] + 0, 1);
    }
    if (threadIdx.x == 0) *a.ticket = 0u;
  }
}

struct MoePushArgs {
  const void* rows;          // source rows [n_src_rows, d] 16-bit
  const int* expert;         // [S] global expert id of every slot
  const int* pos;            // [S] from moe_count_kernel (forward) or null when dest_in is given
  const int* dest_in;        // [S] destination rows recorded by the forward pass (backward) or null
  int* dest_out;             // [S] out: destination row inside the owner's buffer (forward) or null
  int S, E, ep, rank, e_local, top_k;
  int rows_per_slot;         // 1: slot s reads row s; 0: slot s reads row s / top_k
  int d;                     // row length in elements (multiple of 8)
  int cap;                   // rows of every receive buffer
  uint8_t* const* peer_recv; // device array [ep]: every rank's receive buffer [cap][d]
  uint8_t* recv;             // this rank's receive buffer
  const int* counts;         // this rank's counts matrix [ep][E] (filled by every rank's moe_count_kernel)
  int* const* peer_ctr;
  int* ctr;
  const int* count_epoch_ptr; // device word: moe_count_kernel calls made so far (counter 0 target = ep * value)
  const int* epoch_ptr;       // device word: moe_push_kernel calls completed so far (counter 1)
  const int* counts_saved;   // [ep][E] copy kept by the forward pass (backward) or null
  int* seg_offsets;          // local out [e_local + 1] (forward) or null
  int* tile_expert;          // local out [cap / 128] (forward) or null
  int* counts_out;           // local out [ep][E]: copy of the counts matrix for the backward pass, or null
  unsigned int* ticket;
  int* status;
};

__global__ void __launch_bounds__(256) moe_push_kernel(const MoePushArgs a) {
  __shared__ int base_sh[kMoeMaxExperts];      // first destination row of this rank's slots of expert e
  __shared__ int seg_start_sh[kMoeMaxExperts]; // first row of expert e's segment on its owner
  __shared__ int total_sh[kMoeMaxExperts];     // rows of expert e over all ranks
  __shared__ int ok_sh;
  const int epoch = *a.epoch_ptr + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* cm = a.counts_saved != nullptr ? a.counts_saved : a.counts;
  if (threadIdx.x == 0) {
    ok_sh = 1;
    if (a.counts_saved == nullptr)
      ok_sh = wait_flag_sys(a.ctr + 0, a.ep * (*a.count_epoch_ptr), a.status, kTimeoutPeerFlag) ? 1 : 0;
  }
  __syncthreads();
  const bool ok = ok_sh != 0;
  if (ok) {
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
      int tot = 0, before = 0;
      for (int r = 0; r < a.ep; ++r) {
        const int c = *reinterpret_cast<const volatile int*>(cm + r * a.E + e);
        if (r < a.rank) before += c;
        tot += c;
      }
      total_sh[e] = tot;
      base_sh[e] = before;
    }
    __syncthreads();
    if (threadIdx.x < a.ep) {   // one thread per owner: exclusive scan of padded totals over its experts
      int off = 0;
      for (int j = 0; j < a.e_local; ++j) {
        const int e = threadIdx.x * a.e_local + j;
        seg_start_sh[e] = off;
        off += (total_sh[e] + 127) & ~127;
      }
      if (off > a.cap && a.status != nullptr) atomicCAS(a.status, 0, kBadArgument);   // receive buffer too small
    }
    __syncthreads();
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) base_sh[e] += seg_start_sh[e];
    __syncthreads();
    // ---- owner-side bookkeeping for the local experts: tables and zero padding rows ----
    const int e0 = a.rank * a.e_local;
    if (blockIdx.x == 0 && a.counts_out != nullptr) {
      // private copy: the shared matrix may be overwritten by a faster rank's next layer as soon as this
      // kernel's closing barrier has been passed
      for (int i = threadIdx.x; i < a.ep * a.E; i += blockDim.x)
        a.counts_out[i] = *reinterpret_cast<const volatile int*>(cm + i);
    }
    if (blockIdx.x == 0 && a.seg_offsets != nullptr) {
      for (int j = threadIdx.x; j <= a.e_local; j += blockDim.x) {
        int v;
        if (j < a.e_local) v = seg_start_sh[e0 + j];
        else v = seg_start_sh[e0 + a.e_local - 1] + ((total_sh[e0 + a.e_local - 1] + 127) & ~127);
        a.seg_offsets[j] = v;
      }
      const int tiles = a.cap >> 7;
      for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
        const int row = t << 7;
        int ex = -1;
        for (int j = 0; j < a.e_local; ++j) {
          const int s0 = seg_start_sh[e0 + j];
          const int s1 = s0 + ((total_sh[e0 + j] + 127) & ~127);
          if (row >= s0 && row < s1) { ex = j; break; }
        }
        a.tile_expert[t] = ex;
      }
    }
    {
      // padding rows [seg_start + total, seg_end) of every local expert: zero them (16 bytes per lane)
      const int row_u4 = a.d >> 3;
      const int gw = blockIdx.x * (blockDim.x >> 5) + warp;
      const int n_gw = gridDim.x * (blockDim.x >> 5);
      for (int j = 0; j < a.e_local; ++j) {
        const int s0 = seg_start_sh[e0 + j] + total_sh[e0 + j];
        const int s1 = seg_start_sh[e0 + j] + ((total_sh[e0 + j] + 127) & ~127);
        // (counts are trusted to be non-negative; a corrupted matrix must still not produce a row below 0)
        for (int row = max(s0, 0) + gw; row < s1 && row < a.cap; row += n_gw) {
          uint4* dst = reinterpret_cast<uint4*>(a.recv + (size_t)row * a.d * 2);
          for (int c = lane; c < row_u4; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    // ---- one warp per slot: copy the row into the owner's buffer ----
    const int row_u4 = a.d >> 3;
    const int gw = blockIdx.x * (blockDim.x >> 5) + warp;
    const int n_gw = gridDim.x * (blockDim.x >> 5);
    for (int s = gw; s < a.S; s += n_gw) {
      const int e = a.expert[s];
      if ((unsigned)e >= (unsigned)a.E) {
        if (lane == 0 && a.dest_out != nullptr) a.dest_out[s] = -1;
        if (lane == 0 && a.status != nullptr) atomicCAS(a.status, 0, kBadArgument);
        continue;
      }
      const int owner = e / a.e_local;
      const int dest = a.dest_in != nullptr ? a.dest_in[s] : base_sh[e] + a.pos[s];
      if (lane == 0 && a.dest_out != nullptr) a.dest_out[s] = dest;
      if (dest < 0 || dest >= a.cap) continue;
      const int src_row = a.rows_per_slot ? s : s / a.top_k;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.rows) + (size_t)src_row * a.d * 2);
      uint4* dst = reinterpret_cast<uint4*>(a.peer_recv[owner] + (size_t)dest * a.d * 2);
      for (int c = lane; c < row_u4; c += 32) dst[c] = src[c];
    }
  }
  if (!ok) {
    // The counts never arrived (the wait ran out or the status block already reports a failure): nothing was
    // pushed. Leave defined tables behind - no slot has a destination, no tile an expert, every count is zero -
    // so that the kernels downstream of this one (grouped GEMMs, combine, the backward pass) do nothing instead
    // of working from uninitialised memory.
    const int gt = blockIdx.x * blockDim.x + threadIdx.x;
    const int nt = gridDim.x * blockDim.x;
    if (a.dest_out != nullptr)
      for (int s = gt; s < a.S; s += nt) a.dest_out[s] = -1;
    if (blockIdx.x == 0) {
      if (a.seg_offsets != nullptr)
        for (int j = threadIdx.x; j <= a.e_local; j += blockDim.x) a.seg_offsets[j] = 0;
      if (a.tile_expert != nullptr)
        for (int t = threadIdx.x; t < (a.cap >> 7); t += blockDim.x) a.tile_expert[t] = -1;
      if (a.counts_out != nullptr)
        for (int i = threadIdx.x; i < a.ep * a.E; i += blockDim.x) a.counts_out[i] = 0;
    }
  }
  // ---- all of this rank's rows are out: tell every rank, wait for every rank ----
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.ticket, 1u) == gridDim.x - 1) {
      *a.ticket = 0u;
      __threadfence_system();
      for (int p = 0; p < a.ep; ++p) red_release_sys_add(a.peer_ctr[p] + 1, 1);
      wait_flag_sys(a.ctr + 1, a.ep * epoch, a.status, kTimeoutPeerFlag);
    }
  }
}

struct MoePullArgs {
  const int* expert;          // [T * k]
  const int* dest;            // [T * k] row inside the owner's buffer
  const float* weight;        // [T * k] fp32 combine weights or null (= 1)
  const void* addend;         // [T, d] 16-bit added to the output or null
  void* out;                  // [T, d] 16-bit
  void* gathered;             // [T * k, d] 16-bit copy of the pulled rows or null
  int T, top_k, e_local, ep, rank, d, cap;
  const uint8_t* const* peer_y; // device array [ep]: every rank's expert-output buffer [cap][d]
  int* const* peer_ctr;
  int* ctr;
  const int* epoch_ptr;
  unsigned int* ticket;
  int fmt;                    // 1 bf16, 0 fp16
  int* status;
};

__global__ void __launch_bounds__(256) moe_pull_kernel(const MoePullArgs a) {
  __shared__ int ok_sh;
  const int epoch = *a.epoch_ptr + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && threadIdx.x < a.ep) {
    __threadfence_system();
    red_release_sys_add(a.peer_ctr[threadIdx.x] + 2, 1);   // my expert outputs are complete (stream order)
  }
  if (threadIdx.x == 0) ok_sh = wait_flag_sys(a.ctr + 2, a.ep * epoch, a.status, kTimeoutPeerFlag) ? 1 : 0;
  __syncthreads();
  if (ok_sh) {
    const int gw = blockIdx.x * (blockDim.x >> 5) + warp;
    const int n_gw = gridDim.x * (blockDim.x >> 5);
    const int row_u4 = a.d >> 3;
    for (int t = gw; t < a.T; t += n_gw) {
      for (int c = lane; c < row_u4; c += 32) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        if (a.addend != nullptr) {
          const uint4 u = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.addend) + (size_t)t * a.d * 2)[c];
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = a.fmt == 1 ? unpack_bf16x2(w[j]) : __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
          }
        }
        for (int k = 0; k < a.top_k; ++k) {
          const int s = t * a.top_k + k;
          const int dest = a.dest[s];
          const int owner = a.expert[s] / a.e_local;
          if (dest < 0 || dest >= a.cap || (unsigned)owner >= (unsigned)a.ep) {
            // a slot without a row (dropped for capacity, or never dispatched): it contributes nothing, and the
            // copy kept for the router-weight gradient is zero rather than uninitialised
            if (a.gathered != nullptr)
              reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.gathered) + (size_t)s * a.d * 2)[c] =
                  make_uint4(0u, 0u, 0u, 0u);
            continue;
          }
          const uint4 u = __ldcv(reinterpret_cast<const uint4*>(a.peer_y[owner] + (size_t)dest * a.d * 2) + c);
          if (a.gathered != nullptr)
            reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.gathered) + (size_t)s * a.d * 2)[c] = u;
          const float wk = a.weight != nullptr ? a.weight[s] : 1.f;
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = a.fmt == 1 ? unpack_bf16x2(w[j]) : __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            acc[2 * j] += wk * f.x; acc[2 * j + 1] += wk * f.y;
          }
        }
        uint4 o;
        if (a.fmt == 1) {
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        } else {
          o.x = pack_f16x2(acc[0], acc[1]); o.y = pack_f16x2(acc[2], acc[3]);
          o.z = pack_f16x2(acc[4], acc[5]); o.w = pack_f16x2(acc[6], acc[7]);
        }
        reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.out) + (size_t)t * a.d * 2)[c] = o;
      }
    }
  }
  // Everybody must be done reading before an owner may overwrite its output buffer: closing barrier.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.ticket, 1u) == gridDim.x - 1) {
      *a.ticket = 0u;
      for (int p = 0; p < a.ep; ++p) red_release_sys_add(a.peer_ctr[p] + 3, 1);
      wait_flag_sys(a.ctr + 3, a.ep * epoch, a.status, kTimeoutPeerFlag);
    }
  }
}

static int moe_grid(long long work_warps) {
  long long blocks = (work_warps + 7) / 8;
  const long long cap = (long long)num_sms() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace icb

using namespace icb;

// Histogram + in-run positions of this rank's slots; publishes the histogram row to every rank and bumps
// counter 0 everywhere. The caller counts these calls in a device word that moe_push reads.
ICB_API int icb_moe_count(const int* expert, int S, int E, int ep, int rank, int* hist, int* pos,
                          int* const* peer_counts, int* const* peer_ctr, void* ticket, void* stream_) {
  if (E < 1 || E > kMoeMaxExperts || ep < 1 || ep > kMoeMaxEp || E % ep != 0) return -2;
  MoeCountArgs a;
  a.expert = expert; a.S = S; a.E = E; a.ep = ep; a.rank = rank; a.hist = hist; a.pos = pos;
  a.peer_counts = peer_counts; a.peer_ctr = peer_ctr;
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  long long blocks = ((long long)S + 255) / 256;
  const long long cap = (long long)num_sms() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  moe_count_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  return check_launch("moe_count_kernel");
}

// Dispatch (forward: pos given, dest_out / seg_offsets / tile_expert written) or gradient push
// (backward: dest_in and counts_saved given). Uses counter 1.
ICB_API int icb_moe_push(const void* rows, const int* expert, const int* pos, const int* dest_in, int* dest_out, int S,
                         int E, int ep, int rank, int top_k, int rows_per_slot, int d, int cap,
                         void* const* peer_recv, void* recv, const int* counts, const int* counts_saved,
                         int* const* peer_ctr, int* ctr, const int* count_epoch_ptr, const int* epoch_ptr,
                         int* seg_offsets, int* tile_expert, int* counts_out, void* ticket, int* status,
                         void* stream_) {
  if (E < 1 || E > kMoeMaxExperts || ep < 1 || ep > kMoeMaxEp || E % ep != 0) return -2;
  if (d % 8 != 0 || cap % 128 != 0) return -7;
  if ((pos == nullptr) == (dest_in == nullptr)) return -3;
  MoePushArgs a;
  a.rows = rows; a.expert = expert; a.pos = pos; a.dest_in = dest_in; a.dest_out = dest_out;
  a.S = S; a.E = E; a.ep = ep; a.rank = rank; a.e_local = E / ep; a.top_k = top_k;
  a.rows_per_slot = rows_per_slot; a.d = d; a.cap = cap;
  a.peer_recv = reinterpret_cast<uint8_t* const*>(peer_recv);
  a.recv = reinterpret_cast<uint8_t*>(recv);
  a.counts = counts; a.counts_saved = counts_saved;
  a.peer_ctr = peer_ctr; a.ctr = ctr; a.count_epoch_ptr = count_epoch_ptr; a.epoch_ptr = epoch_ptr;
  a.seg_offsets = seg_offsets; a.tile_expert = tile_expert; a.counts_out = counts_out;
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  a.status = status;
  moe_push_kernel<<<moe_grid(S), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  return check_launch("moe_push_kernel");
}

// Combine (or gradient gather): out[t] = addend[t] + sum_k weight[t,k] * Y_owner(t,k)[dest[t,k]]. Uses counters 2, 3.
ICB_API int icb_moe_pull(const int* expert, const int* dest, const float* weight, const void* addend, void* out,
                         void* gathered, int T, int top_k, int E, int ep, int rank, int d, int cap,
                         const void* const* peer_y, int* const* peer_ctr, int* ctr, const int* epoch_ptr, void* ticket,
                         int dtype, int* status, void* stream_) {
  if (E < 1 || ep < 1 || ep > kMoeMaxEp || E % ep != 0) return -2;
  if (d % 8 != 0) return -7;
  if (dtype != kBF16 && dtype != 1) return -3;
  MoePullArgs a;
  a.expert = expert; a.dest = dest; a.weight = weight; a.addend = addend; a.out = out; a.gathered = gathered;
  a.T = T; a.top_k = top_k; a.e_local = E / ep; a.ep = ep; a.rank = rank; a.d = d; a.cap = cap;
  a.peer_y = reinterpret_cast<const uint8_t* const*>(peer_y);
  a.peer_ctr = peer_ctr; a.ctr = ctr; a.epoch_ptr = epoch_ptr;
  a.ticket = reinterpret_cast<unsigned int*>(ticket);
  a.fmt = (dtype == kBF16) ? 1 : 0;
  a.status = status;
  moe_pull_kernel<<<moe_grid(T), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a);
  return check_launch("moe_pull_kernel");
}
