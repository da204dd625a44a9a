// Persistent, warp-specialised bf16/fp16 GEMM for sm_100a.
//
//   C[M,N] (+)= A * B  (+ bias[N]) (+ residual[M,N])
//
// * Operands are staged by TMA (128-byte swizzle, no multicast) into a 4-stage
//   shared-memory ring; one elected thread issues tcgen05.mma (128x256x16 per
//   instruction) with fp32 accumulators in tensor memory.
// * TMEM holds two 128x256 accumulators, so the epilogue of tile i (tcgen05.ld
//   -> registers -> swizzled smem -> TMA store) overlaps the main loop of tile i+1.
// * Each operand may be K-major (reduction dim contiguous) or MN-major (output
//   dim contiguous), which covers forward (x@W with W stored [in,out]), dgrad
//   (dy@W^T) and wgrad (x^T@dy) without any transposing copy.
// * Grouped forms for mixture-of-experts: group_mode 1 picks B (and bias) per
//   128-row M tile from a lookup table; group_mode 2 computes one C per group
//   over a K range taken from an offsets table (expert weight gradients).
// * Fused all-gather -> GEMM (template flag AG): A lives in a gathered buffer. Two extra copy
//   warps per CTA push this rank's shard into every peer's buffer over NVLink (plain P2P
//   stores, fire-and-forget, peers visited in ring order) and bump the peer's per-128-row
//   arrival counters with system-scope releases, while the tensor core works on the row
//   blocks that are already there (local shard first, then the shards in the order they
//   arrive). The TMA producer waits (acquire, bounded) on the counters of remote blocks.
// * Split-K (plain problems with few output tiles, e.g. decode steps with a handful of token rows): the
//   work items are (tile, K range) pairs, so a 64 x 2048 x 1536 product runs on 48 CTAs instead of 8 and
//   streams the weights at memory bandwidth; partial tiles are added into a zeroed fp32 C by TMA
//   reduce-add, bias and residual by the first K range only.
// * Every wait is bounded: on timeout a status word is set and the kernel drains.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer, warps 2-5 = epilogue (one TMEM lane quarter each).
#include "host_common.h"
#include "ptx.cuh"

#include "gemm_common.cuh"

namespace icb {

struct GemmArgs {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_groups;
  int group_mode;            // 0 none, 1 B chosen per m-tile, 2 per-group K range
  const int* group_table;    // mode 1: [num_m_tiles] group of each m tile (-1 = skip tile); mode 2: [G+1] k offsets
  const void* bias;          // [N] (mode 1: [G, N]) in input dtype, may be null
  const void* residual;      // [M, ldr] in output dtype, may be null (may alias C)
  long long ldr;
  int in_fmt;                // 0 fp16, 1 bf16
  int out_f32;               // 0: output dtype == input dtype, 1: fp32
  int split_k;               // >1: every output tile is computed by split_k CTAs over disjoint K ranges of
  int k_per_split;           //     k_per_split elements each, accumulated into a zeroed fp32 C with TMA reduce-add
  int* status;
  // ---- fused all-gather (AG kernels only) ----
  int ag_rank, ag_world;            // this rank / group size
  int ag_rows_per_rank;             // token rows per shard (multiple of 128)
  long long ag_row_bytes;           // bytes per token row of the gathered buffer
  uint8_t* ag_local;                // this rank's gathered buffer [world * rows_per_rank, row_bytes]
  uint8_t* const* ag_peers;         // device array [world]: every rank's gathered buffer (peer pointers)
  int* const* ag_peer_signal;       // device array [world]: every rank's shard_ready[world] array
  const int* ag_signal;             // this rank's shard_ready[world] (written by the peers)
  int* ag_ready;                    // this rank's per-128-row-block arrival counters (bumped by the peers)
  int* const* ag_peer_ready;        // device array [world]: every rank's arrival counters
  const int* ag_epoch_ptr;          // device word: calls completed so far on this workspace (this call = +1)
  int ag_chunks_per_block;          // 8 KiB chunks in one 128-row block
  uint8_t* ag_mc;                   // multicast (NVLS) address of the gathered buffer, or null: plain P2P stores
  int ag_batch;                     // chunks a copy warp pushes between two fence + publish steps (1..16)
  int ag_helpers;                   // 1: the four epilogue warps push chunks too before their first tile
  int ag_push;                      // 0: the shards arrive from their producers, this kernel only waits
  unsigned long long* ag_debug;     // optional [grid][4] timestamps (ns): start, push done, first remote block ready, end
};

constexpr int kAgChunkBytes = 8192;  // copy granularity of the all-gather (one warp iteration)

// Position `seq` of the visiting order -> index in rank-major order: shard 0 of the visiting order is
// this rank's own, shard s belongs to rank - s (mod world).
__device__ __forceinline__ int ag_rotate(int seq, int per_shard, int rank, int world) {
  const int s = seq / per_shard;
  const int owner = (rank - s + world) % world;
  return owner * per_shard + (seq - s * per_shard);
}

// Push this rank's shard into every peer's gathered buffer. The shard is streamed as 8 KiB chunks,
// interleaved over `n_cw` warps of the grid (`cw` = this warp's index). Stores need no round trip, so a few
// warps saturate the link. Peers are visited in ring order (rank+1 first): at any moment every rank writes
// to a different peer. Each finished chunk bumps the arrival counter of its 128-row block on the *peer*
// (one system-scope fence per batch, then relaxed reductions); a block is complete at
// epoch * chunks_per_block.
__device__ __noinline__ void ag_push_shard(const GemmArgs& args, int cw, int n_cw, int lane) {
    const long long shard_bytes = (long long)args.ag_rows_per_rank * args.ag_row_bytes;
    const long long block_bytes = 128LL * args.ag_row_bytes;
    const int chunks_per_shard = (int)(shard_bytes / kAgChunkBytes);
    // A system-scope fence waits for the acknowledgement of every remote store, i.e. a full NVLink
    // round trip: issue it once per batch of chunks (up to kAgBatch), then publish the batch.
    constexpr int kAgBatch = 16;
    if (args.ag_mc != nullptr) {
      // NVLS form: one multimem.st per 16 bytes lands in every rank's buffer (the switch replicates),
      // so the shard leaves this GPU once instead of world-1 times. The arrival counters are still
      // bumped per peer, by lanes 0..world-2 in parallel.
      int c = cw;
      while (c < chunks_per_shard) {
        int done_rb[kAgBatch];
        int n_done = 0;
#pragma unroll 1
        for (; c < chunks_per_shard && n_done < args.ag_batch; c += n_cw) {
          const long long off = (long long)args.ag_rank * shard_bytes + (long long)c * kAgChunkBytes;
          const uint4* src = reinterpret_cast<const uint4*>(args.ag_local + off);
          uint4* dst = reinterpret_cast<uint4*>(args.ag_mc + off);
          uint4 v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = src[lane + j * 32];
#pragma unroll
          for (int j = 0; j < 16; ++j) multimem_st_v4(dst + lane + j * 32, v[j]);
          done_rb[n_done] = (int)(off / block_bytes);
          ++n_done;
        }
        __syncwarp();
        for (int p = lane; p < args.ag_world - 1; p += 32) {
          const int q = (args.ag_rank + 1 + p) % args.ag_world;
          __threadfence_system();
          for (int i = 0; i < n_done; ++i) red_relaxed_sys_add(args.ag_peer_ready[q] + done_rb[i], 1);
        }
        __syncwarp();
      }
    } else {
      const int total_chunks = (args.ag_world - 1) * chunks_per_shard;
      int c = cw;
      while (c < total_chunks) {
        int done_q[kAgBatch], done_rb[kAgBatch];
        int n_done = 0;
#pragma unroll 1
        for (; c < total_chunks && n_done < args.ag_batch; c += n_cw) {
          const int step = c / chunks_per_shard + 1;
          const int within = c - (step - 1) * chunks_per_shard;
          const int q = (args.ag_rank + step) % args.ag_world;
          const long long off = (long long)args.ag_rank * shard_bytes + (long long)within * kAgChunkBytes;
          const uint4* src = reinterpret_cast<const uint4*>(args.ag_local + off);
          uint4* dst = reinterpret_cast<uint4*>(args.ag_peers[q] + off);
          uint4 v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = src[lane + j * 32];
#pragma unroll
          for (int j = 0; j < 16; ++j) dst[lane + j * 32] = v[j];
          done_q[n_done] = q;
          done_rb[n_done] = (int)(off / block_bytes);
          ++n_done;
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          for (int i = 0; i < n_done; ++i) red_relaxed_sys_add(args.ag_peer_ready[done_q[i]] + done_rb[i], 1);
        }
        __syncwarp();
      }
    }
}

template <int A_MAJOR, int B_MAJOR, bool AG, int BN>
__global__ void __launch_bounds__(AG ? kGemmThreads + 64 : kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem + GemmSmem::a_off;
  uint8_t* smem_b = smem + GemmSmem::b_off;
  uint8_t* smem_slab = smem + GemmSmem::slab_off;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + GemmSmem::bar_off);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ag_mtiles_per_shard = AG ? max(args.ag_rows_per_rank >> 7, 1) : 1;
  // Flags are cumulative; the sequence number lives on the device so that a captured CUDA graph
  // replays with the right value (the host bumps the word after every call, in stream order).
  const int ag_epoch = AG ? (*args.ag_epoch_ptr + 1) : 0;

  const int tiles_per_group = args.num_m_tiles * args.num_n_tiles;
  const int total_tiles = (args.group_mode == 2 ? args.num_groups : 1) * tiles_per_group;
  const int total_work = total_tiles * (args.split_k > 1 ? args.split_k : 1);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      // Row blocks already seen complete: a system-scope acquire costs about a microsecond, far more
      // than the few hundred nanoseconds of work the 4-stage ring buffers, so each block is polled once.
      unsigned long long ag_seen = 0ull;
      if (AG && args.ag_debug != nullptr) args.ag_debug[blockIdx.x * 4 + 0] = globaltimer_ns();
      bool ag_gave_up = false;   // after one wait ran out the remaining tiles are not waited for
      auto ag_ensure_ready = [&](int rb) {
        if (ag_gave_up || (rb < 64 && ((ag_seen >> rb) & 1ull))) return;
        if (!wait_flag_sys(args.ag_ready + rb, ag_epoch * args.ag_chunks_per_block, args.status, kTimeoutPeerFlag,
                           rb)) {
          ag_gave_up = true;
          return;
        }
        fence_proxy_async_all();
        if (args.ag_debug != nullptr && ag_seen == 0ull) args.ag_debug[blockIdx.x * 4 + 2] = globaltimer_ns();
        if (rb < 64) ag_seen |= (1ull << rb);
      };
      for (int work = blockIdx.x; work < total_work; work += gridDim.x) {
        int grp = 0, k_begin = 0, k_end = args.K;
        int tile = work;
        if (args.split_k > 1) {
          tile = work / args.split_k;
          k_begin = (work - tile * args.split_k) * args.k_per_split;
          k_end = min(args.K, k_begin + args.k_per_split);
        }
        int local = tile;
        if (args.group_mode == 2) {
          grp = tile / tiles_per_group;
          local = tile - grp * tiles_per_group;
          k_begin = args.group_table[grp];
          k_end = args.group_table[grp + 1];
        }
        int mt, nt;
        tile_coords(local, args.num_m_tiles, args.num_n_tiles, mt, nt);
        if (args.group_mode == 1) {
          grp = args.group_table[mt];
          if (grp < 0) continue;
        }
        if (AG && A_MAJOR == 0) {
          // local shard first, then rank-1, rank-2, ... (the order in which the peers' pushes land)
          mt = ag_rotate(mt, ag_mtiles_per_shard, args.ag_rank, args.ag_world);
          if (mt / ag_mtiles_per_shard != args.ag_rank) ag_ensure_ready(mt);
        }
        const int m0 = mt * kBM, n0 = nt * BN;
        const int bz = (args.group_mode == 1) ? grp : 0;
        for (int kseq = k_begin; kseq < k_end; kseq += kBK, ++it) {
          int k0 = kseq;
          if (AG && A_MAJOR == 1) {
            // the reduction runs over token rows: start with the local shard's rows
            k0 = ag_rotate(kseq, args.ag_rows_per_rank, args.ag_rank, args.ag_world);
            if ((k0 & 127) == 0) {
              const int rb = k0 >> 7;
              if (rb / ag_mtiles_per_shard != args.ag_rank) ag_ensure_ready(rb);
            }
          }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
          mbar_expect_tx(&full_bar[s], kAStageBytes + BN * kBK * 2);
          uint8_t* sa = smem_a + s * kAStageBytes;
          uint8_t* sb = smem_b + s * kBStageBytes;
          if (A_MAJOR == 0) {
            tma_load_2d(sa, &tmA, &full_bar[s], k0, m0);
          } else {
            tma_load_2d(sa, &tmA, &full_bar[s], m0, k0);
            tma_load_2d(sa + 8192, &tmA, &full_bar[s], m0 + 64, k0);
          }
          if (B_MAJOR == 0) {
            tma_load_3d(sb, &tmB, &full_bar[s], k0, n0, bz);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * 8192, &tmB, &full_bar[s], n0 + c * 64, k0, bz);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, BN, args.in_fmt, A_MAJOR, B_MAJOR);
      uint32_t it = 0, tcount = 0;
      for (int work = blockIdx.x; work < total_work; work += gridDim.x) {
        int k_begin = 0, k_end = args.K;
        int tile = work;
        if (args.split_k > 1) {
          tile = work / args.split_k;
          k_begin = (work - tile * args.split_k) * args.k_per_split;
          k_end = min(args.K, k_begin + args.k_per_split);
        }
        int local = tile;
        if (args.group_mode == 2) {
          const int grp = tile / tiles_per_group;
          local = tile - grp * tiles_per_group;
          k_begin = args.group_table[grp];
          k_end = args.group_table[grp + 1];
        }
        if (args.group_mode == 1) {
          int mt, nt;
          tile_coords(local, args.num_m_tiles, args.num_n_tiles, mt, nt);
          if (args.group_table[mt] < 0) continue;
        }
        if (k_end <= k_begin) continue;  // the epilogue writes zeros (+residual) without an accumulator
        const uint32_t acc = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, args.status, kTimeoutTmemEmpty);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        uint32_t first = 1;
        for (int k0 = k_begin; k0 < k_end; k0 += kBK, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(&full_bar[s], ph, abort_flag, args.status, kTimeoutSmemFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * kAStageBytes);
          const uint32_t b_addr = smem_u32(smem_b + s * kBStageBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = (A_MAJOR == 0) ? umma_desc_sw128(a_addr + k * 32, 16, 1024)
                                                  : umma_desc_sw128(a_addr + k * 2048, 8192, 1024);
            const uint64_t bdesc = (B_MAJOR == 0) ? umma_desc_sw128(b_addr + k * 32, 16, 1024)
                                                  : umma_desc_sw128(b_addr + k * 2048, 8192, 1024);
            umma_ss(tmem_d, adesc, bdesc, idesc, first ? 0u : 1u);
            first = 0;
          }
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&tfull_bar[acc]);
        ++tcount;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ epilogue ----------------------------------
    if (AG && args.ag_push && args.ag_helpers) ag_push_shard(args, blockIdx.x * 6 + (warp - 2), gridDim.x * 6, lane);
    const int et = threadIdx.x - 64;     // 0..127
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;
    const int esz = args.out_f32 ? 4 : 2;
    const int cols_per_slab = 128 / esz;  // 64 (16-bit) or 32 (fp32)
    uint32_t tcount = 0, slab_count = 0;
    for (int work = blockIdx.x; work < total_work; work += gridDim.x) {
      int grp = 0, k_begin = 0, k_end = args.K;
      int tile = work;
      bool first_split = true;     // bias and residual are added by the first K range only
      if (args.split_k > 1) {
        tile = work / args.split_k;
        const int ks = work - tile * args.split_k;
        k_begin = ks * args.k_per_split;
        k_end = min(args.K, k_begin + args.k_per_split);
        first_split = ks == 0;
      }
      int local = tile;
      if (args.group_mode == 2) {
        grp = tile / tiles_per_group;
        local = tile - grp * tiles_per_group;
        k_begin = args.group_table[grp];
        k_end = args.group_table[grp + 1];
      }
      int mt, nt;
      tile_coords(local, args.num_m_tiles, args.num_n_tiles, mt, nt);
      if (args.group_mode == 1) {
        grp = args.group_table[mt];
        if (grp < 0) continue;
      }
      if (AG && A_MAJOR == 0) mt = ag_rotate(mt, ag_mtiles_per_shard, args.ag_rank, args.ag_world);
      const bool empty_k = (k_end <= k_begin);
      const int m0 = mt * kBM, n0 = nt * BN;
      const uint32_t acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!empty_k) {
        mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, args.status, kTimeoutTmemFull);
        tc_fence_after();
      }
      const long long m_glob = m0 + row;
      const bool row_ok = m_glob < args.M;
      const int cz = (args.group_mode == 2) ? grp : 0;
      const uint8_t* bias_base = nullptr;
      if (args.bias != nullptr)
        bias_base = reinterpret_cast<const uint8_t*>(args.bias) + (args.group_mode == 1 ? (size_t)grp * args.N * 2 : 0);

#pragma unroll 1
      for (int sub = 0; sub < BN / 32; ++sub) {
        const int col0 = sub * 32;
        const int slab_sub = (esz == 2) ? (sub & 1) : 0;
        const bool slab_start = (slab_sub == 0);
        const bool slab_end = (esz == 4) || (sub & 1);
        uint8_t* slab = smem_slab + (slab_count & 1) * kSlabBytes;
        if (slab_start) {
          if (et == 0) tma_store_wait_read<1>();
          named_barrier(1, 128);
        }
        uint32_t r[32];
        if (!empty_k) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + col0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (sub == BN / 32 - 1 && !empty_k) {
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        const int n_glob = n0 + col0;
        if (bias_base != nullptr && first_split) {
          if (n_glob + 32 <= args.N) {
            const uint4* bp = reinterpret_cast<const uint4*>(bias_base + (size_t)n_glob * 2);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 u = __ldg(bp + c);
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                float lo, hi;
                if (args.in_fmt == 1) {
                  const float2 f = unpack_bf16x2(w[t]);
                  lo = f.x; hi = f.y;
                } else {
                  const __half2 h = *reinterpret_cast<const __half2*>(&w[t]);
                  const float2 f = __half22float2(h);
                  lo = f.x; hi = f.y;
                }
                v[c * 8 + t * 2] += lo;
                v[c * 8 + t * 2 + 1] += hi;
              }
            }
          } else {
            for (int j = 0; j < 32; ++j) {
              if (n_glob + j < args.N) {
                const uint16_t raw = reinterpret_cast<const uint16_t*>(bias_base)[n_glob + j];
                float b;
                if (args.in_fmt == 1) b = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw));
                else b = __half2float(*reinterpret_cast<const __half*>(&raw));
                v[j] += b;
              }
            }
          }
        }
        if (args.residual != nullptr && row_ok && first_split) {
          const uint8_t* rp = reinterpret_cast<const uint8_t*>(args.residual) +
                              ((size_t)cz * args.M * args.ldr + (size_t)m_glob * args.ldr + n_glob) * esz;
          const bool vec_ok = (n_glob + 32 <= args.N) && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0);
          if (esz == 4) {
            if (vec_ok) {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const float4 f = *reinterpret_cast<const float4*>(rp + c * 16);
                v[c * 4] += f.x; v[c * 4 + 1] += f.y; v[c * 4 + 2] += f.z; v[c * 4 + 3] += f.w;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (n_glob + j < args.N) v[j] += reinterpret_cast<const float*>(rp)[j];
            }
          } else {
            if (vec_ok) {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const uint4 u = *reinterpret_cast<const uint4*>(rp + c * 16);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  float2 f;
                  if (args.in_fmt == 1) f = unpack_bf16x2(w[t]);
                  else f = __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
                  v[c * 8 + t * 2] += f.x;
                  v[c * 8 + t * 2 + 1] += f.y;
                }
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (n_glob + j < args.N) {
                  const uint16_t raw = reinterpret_cast<const uint16_t*>(rp)[j];
                  float b;
                  if (args.in_fmt == 1) b = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw));
                  else b = __half2float(*reinterpret_cast<const __half*>(&raw));
                  v[j] += b;
                }
              }
            }
          }
        }
        // registers -> swizzled staging slab (row-major 128 B rows, 16 B chunks XOR row%8)
        uint8_t* srow = slab + row * 128;
        if (esz == 4) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int pc = c ^ (row & 7);
            *reinterpret_cast<float4*>(srow + pc * 16) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int pc = (slab_sub * 4 + c) ^ (row & 7);
            uint4 u;
            if (args.in_fmt == 1) {
              u.x = pack_bf16x2(v[c * 8], v[c * 8 + 1]);
              u.y = pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
              u.z = pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
              u.w = pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
            } else {
              u.x = pack_f16x2(v[c * 8], v[c * 8 + 1]);
              u.y = pack_f16x2(v[c * 8 + 2], v[c * 8 + 3]);
              u.z = pack_f16x2(v[c * 8 + 4], v[c * 8 + 5]);
              u.w = pack_f16x2(v[c * 8 + 6], v[c * 8 + 7]);
            }
            *reinterpret_cast<uint4*>(srow + pc * 16) = u;
          }
        }
        if (slab_end) {
          fence_proxy_async_smem();
          named_barrier(1, 128);
          if (et == 0) {
            const int slab_col0 = n0 + col0 - slab_sub * 32;
            if (slab_col0 < args.N) {
              if (args.split_k > 1) tma_reduce_add_3d(&tmC, slab, slab_col0, m0, cz);
              else tma_store_3d(&tmC, slab, slab_col0, m0, cz);
            }
            tma_store_commit();
          }
          ++slab_count;
        }
      }
      if (!empty_k) ++tcount;
    }
    if (et == 0) tma_store_wait<0>();
  }

  if (AG && warp >= 6 && args.ag_push) {
    // ------------------------------ all-gather copy warps ----------------------
    // Two dedicated warps per CTA; with ag_helpers the four epilogue warps have already taken their share
    // of the chunks before their first accumulator was ready (warp slots 0..3), these are slots 4 and 5.
    const int per_cta = args.ag_helpers ? 6 : 2;
    ag_push_shard(args, blockIdx.x * per_cta + (per_cta - 2) + (warp - 6), gridDim.x * per_cta, lane);
  }

  if (AG && args.ag_debug != nullptr) {
    if (warp == 6 && lane == 0) args.ag_debug[blockIdx.x * 4 + 1] = globaltimer_ns();
    if (warp == 2 && lane == 0) args.ag_debug[blockIdx.x * 4 + 3] = globaltimer_ns();
  }
  // Drain: nobody may exit while TMEM is allocated or copies are in flight.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give outstanding TMA loads time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int A_MAJOR, int B_MAJOR, bool AG = false>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const GemmArgs& args,
                       int grid, cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm_kernel<A_MAJOR, B_MAJOR, AG, kBN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) {
      fprintf(stderr, "[ironcore_b200] gemm smem attribute failed: %s\n", cudaGetErrorString(e));
      return -(int)e;
    }
    configured = true;
  }
  kern<<<grid, AG ? kGemmThreads + 64 : kGemmThreads, kGemmSmemBytes, stream>>>(tmA, tmB, tmC, args);
  return check_launch("gemm_kernel");
}

}  // namespace icb

using namespace icb;

// C[M,N] (+)= A*B (+bias) (+residual).
//   a_major 0: A is [M, lda] row-major (K contiguous);  1: A is [K, lda] row-major (M contiguous)
//   b_major 0: B is [N, ldb] row-major (K contiguous);  1: B is [K, ldb] row-major (N contiguous)
//   in_dtype 0 bf16 / 1 fp16; out_f32 selects fp32 output (residual, if any, has the output dtype)
//   group_mode 0: plain. 1: B = B_base + group_table[m_tile]*b_group_stride (elements), bias row per group.
//   group_mode 2: for g in [0,G): C_g[M,N] = A[:, k_g..k_g+1) * B[k range], C_g = C + g*M*ldc
//                 (needs a_major = b_major = 1; K offsets multiples of 64 or zero-padded rows).
// All pitches in elements; pitches * element size and base pointers must be multiples of 16 bytes.
static int gemm_impl(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                     int K, long long lda, long long ldb, long long ldc, long long ldr, int a_major, int b_major,
                     int in_dtype, int out_f32, int group_mode, int num_groups, const int* group_table,
                     long long b_group_stride, int* status, int max_ctas, void* stream_, const GemmArgs* ag,
                     int split_k = 1) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (split_k > 1 && (group_mode != 0 || ag != nullptr || !out_f32)) return -8;
  if (in_dtype != kBF16 && in_dtype != kF16) return -2;
  if (group_mode == 2 && !(a_major == 1 && b_major == 1)) return -3;
  const int es = 2;
  const int oes = out_f32 ? 4 : 2;
  if ((lda * es) % 16 || (ldb * es) % 16 || (ldc * oes) % 16) return -4;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -5;
  if (num_groups < 1) num_groups = 1;

  // 128 x 256 tiles throughout: a 128-column tile costs 0.79 of a 256-column one on B200 (the operand feed,
  // not the tensor pipe, bounds it), so it loses even on shapes with a ragged last wave.
  const int bn = kBN;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  const uint64_t k_rows = (uint64_t)K;
  if (a_major == 0) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * es};
    uint32_t box[2] = {64, (uint32_t)kBM};
    rc = make_tmap(&tmA, in_dtype, 2, A, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)M, k_rows};
    uint64_t str[1] = {(uint64_t)lda * es};
    uint32_t box[2] = {64, (uint32_t)kBK};
    rc = make_tmap(&tmA, in_dtype, 2, A, dims, str, box, true);
  }
  if (rc) return rc;
  const uint64_t bgroups = (group_mode == 1) ? (uint64_t)num_groups : 1;
  if (b_major == 0) {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, bgroups};
    uint64_t str[2] = {(uint64_t)ldb * es, (uint64_t)(group_mode == 1 ? b_group_stride : (long long)N * ldb) * es};
    uint32_t box[3] = {64, (uint32_t)bn, 1};
    rc = make_tmap(&tmB, in_dtype, 3, B, dims, str, box, true);
  } else {
    uint64_t dims[3] = {(uint64_t)N, k_rows, bgroups};
    uint64_t str[2] = {(uint64_t)ldb * es, (uint64_t)(group_mode == 1 ? b_group_stride : (long long)K * ldb) * es};
    uint32_t box[3] = {64, (uint32_t)kBK, 1};
    rc = make_tmap(&tmB, in_dtype, 3, B, dims, str, box, true);
  }
  if (rc) return rc;
  {
    const uint64_t cgroups = (group_mode == 2) ? (uint64_t)num_groups : 1;
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, cgroups};
    uint64_t str[2] = {(uint64_t)ldc * oes, (uint64_t)M * ldc * oes};
    uint32_t box[3] = {(uint32_t)(128 / oes), (uint32_t)kBM, 1};
    rc = make_tmap(&tmC, out_f32 ? kF32 : in_dtype, 3, C, dims, str, box, true);
  }
  if (rc) return rc;

  GemmArgs args;
  if (ag != nullptr) args = *ag;
  else {
    args.ag_rank = 0; args.ag_world = 1; args.ag_rows_per_rank = 0; args.ag_row_bytes = 0;
    args.ag_local = nullptr; args.ag_peers = nullptr; args.ag_peer_signal = nullptr; args.ag_signal = nullptr;
    args.ag_ready = nullptr; args.ag_epoch_ptr = nullptr; args.ag_chunks_per_block = 1; args.ag_peer_ready = nullptr;
    args.ag_mc = nullptr; args.ag_batch = 4; args.ag_debug = nullptr; args.ag_helpers = 0; args.ag_push = 0;
  }
  args.M = M; args.N = N; args.K = K;
  args.num_m_tiles = (M + kBM - 1) / kBM;
  args.num_n_tiles = (N + bn - 1) / bn;
  args.num_groups = num_groups;
  args.group_mode = group_mode;
  args.group_table = group_table;
  args.bias = bias;
  args.residual = residual;
  args.ldr = ldr;
  args.in_fmt = (in_dtype == kBF16) ? 1 : 0;
  args.out_f32 = out_f32;
  args.status = status;
  args.split_k = 1;
  args.k_per_split = K;
  if (split_k > 1) {
    const int kblocks = (K + kBK - 1) / kBK;
    const int per = (kblocks + split_k - 1) / split_k;
    args.k_per_split = per * kBK;
    args.split_k = (kblocks + per - 1) / per;      // no empty K range
  }

  long long total = (long long)args.num_m_tiles * args.num_n_tiles * (group_mode == 2 ? num_groups : 1) *
                    args.split_k;
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (total < grid) grid = (int)total;
  if (grid < 1) grid = 1;

  if (ag != nullptr) {
    if (a_major == 0 && b_major == 0) return launch_gemm<0, 0, true>(tmA, tmB, tmC, args, grid, stream);
    if (a_major == 0 && b_major == 1) return launch_gemm<0, 1, true>(tmA, tmB, tmC, args, grid, stream);
    if (a_major == 1 && b_major == 1) return launch_gemm<1, 1, true>(tmA, tmB, tmC, args, grid, stream);
    return -6;
  }
  if (a_major == 0 && b_major == 0) return launch_gemm<0, 0>(tmA, tmB, tmC, args, grid, stream);
  if (a_major == 0 && b_major == 1) return launch_gemm<0, 1>(tmA, tmB, tmC, args, grid, stream);
  if (a_major == 1 && b_major == 0) return launch_gemm<1, 0>(tmA, tmB, tmC, args, grid, stream);
  return launch_gemm<1, 1>(tmA, tmB, tmC, args, grid, stream);
}

ICB_API int icb_gemm(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                     int K, long long lda, long long ldb, long long ldc, long long ldr, int a_major, int b_major,
                     int in_dtype, int out_f32, int group_mode, int num_groups, const int* group_table,
                     long long b_group_stride, int* status, int max_ctas, void* stream_) {
  return gemm_impl(A, B, C, bias, residual, M, N, K, lda, ldb, ldc, ldr, a_major, b_major, in_dtype, out_f32,
                   group_mode, num_groups, group_table, b_group_stride, status, max_ctas, stream_, nullptr);
}

// icb_gemm with every output tile split over `split_k` CTAs along K. C must be fp32 (out_f32 = 1) and zeroed by the
// caller (stream order): the partial tiles are accumulated into it with TMA reduce-add; bias and residual (fp32,
// must not alias C) enter once. Plain problems only. For a few token rows against a wide weight matrix this turns
// a handful of CTAs into a grid that streams the weights at memory bandwidth.
ICB_API int icb_gemm_splitk(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                            int K, long long lda, long long ldb, long long ldc, long long ldr, int a_major, int b_major,
                            int in_dtype, int split_k, int* status, void* stream_) {
  return gemm_impl(A, B, C, bias, residual, M, N, K, lda, ldb, ldc, ldr, a_major, b_major, in_dtype, 1, 0, 1, nullptr,
                   0, status, 0, stream_, nullptr, split_k);
}

// Optional instrumentation of the fused all-gather kernels: a device buffer of [148][4] 64-bit nanosecond
// timestamps per CTA (producer start, copy warps done, first remote row block ready, epilogue done); null = off.
static unsigned long long* g_ag_debug = nullptr;
ICB_API int icb_set_ag_debug(void* buf) {
  g_ag_debug = reinterpret_cast<unsigned long long*>(buf);
  return 0;
}

// Fused all-gather -> GEMM over a tensor-parallel group (sequence parallelism).
//   gathered : this rank's gathered activation buffer [world * rows_per_rank, width] (16-bit, contiguous);
//              the local shard's rows must already be in place (stream order).
//   peers    : device array [world] of every rank's gathered buffer (symmetric-memory peer pointers).
//   peer_ready : device array [world] of every rank's arrival-counter array; `signal` is unused (reserved).
//   ready    : this rank's int array [world * rows_per_rank / 128] of cumulative arrival counters.
//   epoch_ptr: device int holding the number of calls already made on this workspace (same on every
//              rank); the caller increments it in stream order after this call.
//   a_major 0: C[M = world*rows_per_rank, N] = gathered[M, K = width] * B        (forward / dgrad of a row-parallel layer)
//   a_major 1: C[M = width, N] = gathered^T * B[K = world*rows_per_rank, N]      (wgrad: reduction over gathered rows)
//   flags    : bit 0 = the shards are pushed by their producers (the fused reduce-scatter + norm kernel of
//              every rank writes its normalised rows into all gather buffers and bumps the same counters):
//              this kernel pushes nothing and only waits; bit 1 = the epilogue warps help pushing.
//   gathered_mc: multicast (NVLS) address of `gathered` or null. With it the shard is pushed once with multimem.st
//              and replicated by the NVSwitch; a workspace must use the same form on every call and rank.
// The local shard is pushed to every peer with plain P2P stores by copy warps inside the same kernel;
// the tensor core starts with the local shard and follows the other shards in arrival order.
ICB_API int icb_ag_gemm(void* gathered, const void* const* peers, int* const* peer_ready, const int* signal,
                        int* ready, int rank, int world, int rows_per_rank, int width, const int* epoch_ptr, const void* B,
                        void* C, const void* bias, const void* residual, int N, long long ldb, long long ldc,
                        long long ldr, int a_major, int b_major, int in_dtype, int out_f32, int* status,
                        void* stream_, void* gathered_mc, int flags) {
  if (rows_per_rank % 128 != 0 || width % 32 != 0) return -7;   // 128-row blocks must be whole 8 KiB chunks
  GemmArgs ag;
  ag.ag_rank = rank; ag.ag_world = world; ag.ag_rows_per_rank = rows_per_rank;
  ag.ag_row_bytes = (long long)width * 2;
  ag.ag_local = reinterpret_cast<uint8_t*>(gathered);
  ag.ag_peers = reinterpret_cast<uint8_t* const*>(const_cast<void* const*>(reinterpret_cast<const void* const*>(peers)));
  ag.ag_peer_signal = nullptr;
  ag.ag_peer_ready = peer_ready;
  ag.ag_signal = signal;
  ag.ag_ready = ready;
  ag.ag_epoch_ptr = epoch_ptr;
  ag.ag_mc = reinterpret_cast<uint8_t*>(gathered_mc);
  // Publishing granularity of the push: 4 chunks per fence (fewer make the first remote tiles ready earlier,
  // more amortise the system-scope fence; 4 measured best at 2 ranks).
  ag.ag_batch = 4;
  ag.ag_debug = g_ag_debug;
  ag.ag_push = (flags & 1) ? 0 : 1;
  ag.ag_helpers = (flags & 2) ? 1 : 0;
  ag.ag_chunks_per_block = (int)(128LL * width * 2 / kAgChunkBytes);
  const int rows = world * rows_per_rank;
  const int M = a_major == 0 ? rows : width;
  const int K = a_major == 0 ? width : rows;
  return gemm_impl(gathered, B, C, bias, residual, M, N, K, width, ldb, ldc, ldr, a_major, b_major, in_dtype, out_f32,
                   0, 1, nullptr, 0, status, 0, stream_, &ag);
}
