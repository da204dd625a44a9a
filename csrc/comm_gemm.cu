// Fused GEMM -> reduce-scatter over a tensor-parallel group (sequence parallelism), sm_100a.
//
//   partial[M, N] = A_local[M, K_local] * B_local          (tcgen05, same pipeline as gemm.cu)
//   out_shard[M/t, N] = sum_ranks partial[rows of this rank] (+ bias) (+ residual)
//
// One kernel does both. The epilogue of every 128 x 256 tile converts the accumulator to
// 16-bit and stores it straight into the *owner's* receive buffer (slot of the sending rank)
// with peer-to-peer stores over NVLink, then bumps the owner's per-tile arrival counter with
// a system-scope release. Tiles destined for other ranks are computed first (ring order
// starting at rank+1), the rank's own rows last, so the wire is busy while the tensor core
// still has work. When a CTA runs out of GEMM tiles its warps turn into reducers: they wait
// (bounded, acquire) until all t partials of a 16-row x 256-column unit of this rank's shard
// have arrived, sum them in fp32, add bias / residual and write the output shard.
// Counters are cumulative (target = t * epoch), receive buffers alternate by call parity on
// the host side, so nothing is ever re-zeroed.
//
// Fused follow-up (norm_gamma != null): under sequence parallelism the reduced rows are the residual
// stream, and what comes next is RMSNorm -> all-gather -> column-parallel GEMM. In this mode a reducer
// warp owns whole rows: it sums the partials (+ bias + residual), stores the residual-stream row,
// normalises it (fp32 statistics, gain applied) and stores the normalised row straight into every
// rank's gather buffer of the next GEMM (P2P stores, or one multimem.st through the NVSwitch), then
// bumps the per-128-row arrival counters that the all-gather GEMM kernel polls. The norm kernel, the
// copy into the gather buffer and the push phase of the following all-gather GEMM disappear.
#include "gemm_common.cuh"
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

struct RsArgs {
  int M, N, K;
  int num_m_tiles, num_n_tiles;
  int rank, world;
  int rows_per_rank;               // M / world, multiple of 128
  uint8_t* const* peer_recv;       // device array [world]: every rank's receive buffer [world][rows_per_rank][N] (16-bit)
  int* const* peer_flags;          // device array [world]: every rank's arrival counters [rows_per_rank/128][num_n_tiles]
  const uint8_t* recv;             // this rank's receive buffer
  const int* flags;                // this rank's arrival counters
  void* out;                       // [rows_per_rank, ldo] 16-bit
  long long ldo;
  const void* bias;                // [N] or null
  const void* residual;            // [rows_per_rank, ldr] or null
  long long ldr;
  const int* epoch_ptr;            // device word: calls completed so far on this workspace
  const uint8_t* mc_recv;          // multicast (NVLS) address of the receive buffer, or null (see below)
  int in_fmt;
  int* status;
  // ---- fused RMSNorm + all-gather push of the reduced rows (norm_gamma == null: off) ----
  const void* norm_gamma;          // [N] gain, 16-bit
  float norm_eps, norm_w_offset;   // y = h * rsqrt(mean(h^2) + eps) * (gamma + w_offset)
  float* norm_rstd;                // [rows_per_rank] fp32: written by the forward form, read by the backward form
  int norm_bwd;                    // 0: forward (normalise the reduced rows); 1: backward (see rs_reduce_norm_push)
  const void* norm_x;              // backward: the norm's input rows [rows_per_rank, norm_ldx], 16-bit
  long long norm_ldx;
  void* aux_out;                   // backward: the reduced rows themselves [rows_per_rank, N], 16-bit
  uint8_t* const* ag_peers;        // device array [world]: every rank's gather buffer [world * rows_per_rank][N]
  uint8_t* ag_mc;                  // multicast address of the gather buffer or null (P2P stores)
  int* const* ag_peer_ready;       // device array [world]: every rank's per-128-row arrival counters
  int ag_rows_per_unit;            // consecutive rows a warp finishes before it publishes once
  int ag_add_per_unit;             // counter increment per unit (a 128-row block totals 128 * N * 2 / 8192)
};

template <bool BF16>
__device__ __forceinline__ void rs_acc8(float (&a)[8], const uint4& u) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 f = BF16 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
    a[2 * t] += f.x;
    a[2 * t + 1] += f.y;
  }
}
template <bool BF16>
__device__ __forceinline__ uint4 rs_pack8(const float (&a)[8]) {
  uint4 o;
  if (BF16) {
    o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
  } else {
    o.x = pack_f16x2(a[0], a[1]); o.y = pack_f16x2(a[2], a[3]);
    o.z = pack_f16x2(a[4], a[5]); o.w = pack_f16x2(a[6], a[7]);
  }
  return o;
}

// Row-owning reduce phase with the norm and the all-gather push fused in (see the header comment).
// One warp per unit of `ag_rows_per_unit` consecutive rows; a lane covers 8 columns of every
// 256-column stripe. kCU stripes of kSB source ranks are loaded together, so each lane keeps
// kCU * kSB 16-byte loads in flight (the phase is latency bound: a warp owns only a few rows).
// The counters of a finished unit are published after the loads of the next unit have been issued:
// by then the unit's remote stores have been acknowledged and the system-scope fence is cheap.
//
// BWD = false (forward):  h = sum(partials) + bias + residual  -> out ;  push  h * rstd * (gamma + off)
// BWD = true  (backward of the same boundary): the reduced rows are dn, the gradient of the normalised
//   activations. dn -> aux_out (kept for the gain's gradient); with xh = x * rstd and g = dn * (gamma + off):
//   dx = rstd * (g - xh * mean(g * xh)) + residual  -> out and pushed (the input gradient of the
//   row-parallel layer that produced x, gathered for that layer's dgrad and wgrad).
template <bool BF16, int kCU, int kSB, bool BWD>
__device__ __noinline__ void rs_reduce_norm_push(const RsArgs& args, int warp, int lane) {
  const int nwarps = kGemmThreads / 32;
  const int gw = blockIdx.x * nwarps + warp;
  const int n_gw = gridDim.x * nwarps;
  const int N = args.N;
  const int units = args.rows_per_rank / args.ag_rows_per_unit;
  const int target = args.world * (*args.epoch_ptr + 1);
  const size_t slot_stride = (size_t)args.rows_per_rank * N * 2;   // bytes between two source ranks' slots
  const uint8_t* gamma = reinterpret_cast<const uint8_t*>(args.norm_gamma);
  int checked_lm = -1, checked_ok = 0;
  int pending_rb = -1;                                             // unit whose counters are not yet published
  auto publish = [&](int rb) {
    __syncwarp();
    for (int p = lane; p < args.world - 1; p += 32) {
      const int q = (args.rank + 1 + p) % args.world;
      __threadfence_system();
      red_relaxed_sys_add(args.ag_peer_ready[q] + rb, args.ag_add_per_unit);
    }
    __syncwarp();
  };
  for (int u = gw; u < units; u += n_gw) {
    const int row0 = u * args.ag_rows_per_unit;
    const int lm = row0 >> 7;
    if (lm != checked_lm) {
      // all column tiles of this 128-row block must have arrived from every rank
      int ok = 1;
      for (int nt = lane; nt < args.num_n_tiles; nt += 32)
        ok &= wait_flag_sys(args.flags + lm * args.num_n_tiles + nt, target, args.status, kTimeoutPeerFlag,
                            lm * args.num_n_tiles + nt) ? 1 : 0;
      checked_ok = __all_sync(0xffffffffu, ok);
      checked_lm = lm;
    }
    if (!checked_ok) continue;
    for (int r = 0; r < args.ag_rows_per_unit; ++r) {
      const int lrow = row0 + r;
      uint8_t* out_row = reinterpret_cast<uint8_t*>(args.out) + (size_t)lrow * args.ldo * 2;
      // forward: the reduced row itself is the first output; backward: it goes to the auxiliary output
      uint8_t* red_row = BWD ? reinterpret_cast<uint8_t*>(args.aux_out) + (size_t)lrow * N * 2 : out_row;
      const uint8_t* res_row = args.residual != nullptr
                                   ? reinterpret_cast<const uint8_t*>(args.residual) + (size_t)lrow * args.ldr * 2
                                   : nullptr;
      const uint8_t* x_row = BWD ? reinterpret_cast<const uint8_t*>(args.norm_x) + (size_t)lrow * args.norm_ldx * 2
                                 : nullptr;
      const float rstd_in = BWD ? args.norm_rstd[lrow] : 0.f;
      // ---- pass 1: sum of the partials -> reduced row; row statistic (sum of squares / <g, xh>)
      float ss = 0.f;
      for (int c0 = lane * 8; c0 < N; c0 += 256 * kCU) {
        float acc[kCU][8];
#pragma unroll
        for (int i = 0; i < kCU; ++i) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        }
        uint4 rv[kCU];     // forward: residual; backward: x (the norm's input)
        const uint8_t* side_row = BWD ? x_row : res_row;
        if (side_row != nullptr) {
#pragma unroll
          for (int i = 0; i < kCU; ++i) {
            const int col = c0 + i * 256;
            if (col < N) rv[i] = *reinterpret_cast<const uint4*>(side_row + (size_t)col * 2);
          }
        }
        if (args.mc_recv != nullptr) {
          uint4 v[kCU];
#pragma unroll
          for (int i = 0; i < kCU; ++i) {
            const int col = c0 + i * 256;
            if (col < N) {
              const uint8_t* p = args.mc_recv + (((size_t)args.rank * args.rows_per_rank + lrow) * N + col) * 2;
              v[i] = BF16 ? multimem_ld_reduce_bf16x8(p) : multimem_ld_reduce_f16x8(p);
            }
          }
#pragma unroll
          for (int i = 0; i < kCU; ++i)
            if (c0 + i * 256 < N) rs_acc8<BF16>(acc[i], v[i]);
        } else {
          const uint8_t* base = args.recv + ((size_t)lrow * N) * 2;
          for (int s0 = 0; s0 < args.world; s0 += kSB) {
            uint4 v[kSB][kCU];
#pragma unroll
            for (int sb = 0; sb < kSB; ++sb) {
              if (s0 + sb < args.world) {
#pragma unroll
                for (int i = 0; i < kCU; ++i) {
                  const int col = c0 + i * 256;
                  if (col < N)
                    v[sb][i] = __ldcv(reinterpret_cast<const uint4*>(base + (s0 + sb) * slot_stride + (size_t)col * 2));
                }
              }
            }
#pragma unroll
            for (int sb = 0; sb < kSB; ++sb) {
              if (s0 + sb < args.world) {
#pragma unroll
                for (int i = 0; i < kCU; ++i)
                  if (c0 + i * 256 < N) rs_acc8<BF16>(acc[i], v[sb][i]);
              }
            }
          }
        }
        if (pending_rb >= 0) {      // the previous unit's stores have had a whole load round trip to land
          publish(pending_rb);
          pending_rb = -1;
        }
#pragma unroll
        for (int i = 0; i < kCU; ++i) {
          const int col = c0 + i * 256;
          if (col < N) {
            if (args.bias != nullptr)
              rs_acc8<BF16>(acc[i], *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(args.bias) +
                                                                     (size_t)col * 2));
            if (!BWD && res_row != nullptr) rs_acc8<BF16>(acc[i], rv[i]);
            const uint4 o = rs_pack8<BF16>(acc[i]);
            *reinterpret_cast<uint4*>(red_row + (size_t)col * 2) = o;
            // statistics of the rounded values: what a separate norm kernel would read back
            float hr[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) hr[j] = 0.f;
            rs_acc8<BF16>(hr, o);
            if (!BWD) {
#pragma unroll
              for (int j = 0; j < 8; ++j) ss += hr[j] * hr[j];
            } else {
              float xv[8], g[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) { xv[j] = 0.f; g[j] = args.norm_w_offset; }
              rs_acc8<BF16>(xv, rv[i]);
              rs_acc8<BF16>(g, *reinterpret_cast<const uint4*>(gamma + (size_t)col * 2));
#pragma unroll
              for (int j = 0; j < 8; ++j) ss += hr[j] * g[j] * (xv[j] * rstd_in);
            }
          }
        }
      }
      ss = warp_sum(ss);
      const float rstd = BWD ? rstd_in : rsqrtf(ss / N + args.norm_eps);
      const float c1 = ss / N;                                   // backward: mean(g * xh)
      if (!BWD && lane == 0 && args.norm_rstd != nullptr) args.norm_rstd[lrow] = rstd;
      // ---- pass 2: normalise / norm backward (this lane re-reads its own stores) and push into every gather buffer
      const size_t g_row = ((size_t)args.rank * args.rows_per_rank + lrow) * N * 2;
      for (int c0 = lane * 8; c0 < N; c0 += 256 * kCU) {
        uint4 y[kCU];
#pragma unroll
        for (int i = 0; i < kCU; ++i) {
          const int col = c0 + i * 256;
          if (col < N) {
            float h[8], g[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { h[j] = 0.f; g[j] = args.norm_w_offset; }
            rs_acc8<BF16>(h, *reinterpret_cast<const uint4*>(red_row + (size_t)col * 2));
            rs_acc8<BF16>(g, *reinterpret_cast<const uint4*>(gamma + (size_t)col * 2));
            if (!BWD) {
#pragma unroll
              for (int j = 0; j < 8; ++j) h[j] = h[j] * rstd * g[j];
            } else {
              float xv[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) xv[j] = 0.f;
              rs_acc8<BF16>(xv, *reinterpret_cast<const uint4*>(x_row + (size_t)col * 2));
#pragma unroll
              for (int j = 0; j < 8; ++j) h[j] = rstd * (h[j] * g[j] - xv[j] * rstd * c1);
              if (res_row != nullptr) rs_acc8<BF16>(h, *reinterpret_cast<const uint4*>(res_row + (size_t)col * 2));
            }
            y[i] = rs_pack8<BF16>(h);
            if (BWD) *reinterpret_cast<uint4*>(out_row + (size_t)col * 2) = y[i];
          }
        }
        if (args.ag_mc != nullptr) {
#pragma unroll
          for (int i = 0; i < kCU; ++i) {
            const int col = c0 + i * 256;
            if (col < N) multimem_st_v4(args.ag_mc + g_row + (size_t)col * 2, y[i]);
          }
        } else {
          for (int q = 0; q < args.world; ++q) {
            uint8_t* dst = args.ag_peers[(args.rank + q) % args.world] + g_row;
#pragma unroll
            for (int i = 0; i < kCU; ++i) {
              const int col = c0 + i * 256;
              if (col < N) *reinterpret_cast<uint4*>(dst + (size_t)col * 2) = y[i];
            }
          }
        }
      }
    }
    pending_rb = (args.rank * args.rows_per_rank + row0) >> 7;
  }
  if (pending_rb >= 0) publish(pending_rb);
}

template <bool BF16, bool BWD>
__device__ __forceinline__ void rs_reduce_norm_dispatch(const RsArgs& args, int warp, int lane) {
  // 16 loads per lane in flight whatever the group size: two source ranks x 8 stripes, or four x 4
  if (args.world <= 2) rs_reduce_norm_push<BF16, 8, 2, BWD>(args, warp, lane);
  else rs_reduce_norm_push<BF16, 4, 4, BWD>(args, warp, lane);
}

template <int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ RsArgs args) {
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
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = args.num_m_tiles * args.num_n_tiles;
  const int mtiles_per_shard = args.rows_per_rank >> 7;
  // tile -> (m tile, n tile): remote owners first in ring order, own shard last
  auto coords = [&](int tile, int& mt, int& nt) {
    tile_coords(tile, args.num_m_tiles, args.num_n_tiles, mt, nt);
    mt = (mt + (args.rank + 1) * mtiles_per_shard) % args.num_m_tiles;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int mt, nt;
        coords(tile, mt, nt);
        const int m0 = mt * kBM, n0 = nt * kBN;
        for (int k0 = 0; k0 < args.K; k0 += kBK, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
          mbar_expect_tx(&full_bar[s], kAStageBytes + kBStageBytes);
          uint8_t* sa = smem_a + s * kAStageBytes;
          uint8_t* sb = smem_b + s * kBStageBytes;
          tma_load_2d(sa, &tmA, &full_bar[s], k0, m0);
          if (B_MAJOR == 0) {
            tma_load_2d(sb, &tmB, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < kBN / 64; ++c) tma_load_2d(sb + c * 8192, &tmB, &full_bar[s], n0 + c * 64, k0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, kBN, args.in_fmt, 0, B_MAJOR);
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const uint32_t acc = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, args.status, kTimeoutTmemEmpty);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        uint32_t first = 1;
        for (int k0 = 0; k0 < args.K; k0 += kBK, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(&full_bar[s], ph, abort_flag, args.status, kTimeoutSmemFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * kAStageBytes);
          const uint32_t b_addr = smem_u32(smem_b + s * kBStageBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = umma_desc_sw128(a_addr + k * 32, 16, 1024);
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
  } else {
    // ---------------- epilogue: accumulator -> owner's receive slot (P2P stores) ----------------
    const int et = threadIdx.x - 64;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int mt, nt;
      coords(tile, mt, nt);
      const int owner = mt / mtiles_per_shard;
      const int lm = mt - owner * mtiles_per_shard;
      const int n0 = nt * kBN;
      const uint32_t acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, args.status, kTimeoutTmemFull);
      tc_fence_after();
      // Rows of this tile inside the owner's receive slot of the sending rank.
      // NVLS form: the partial tile stays in this rank's own buffer, laid out [M][N]; the owner sums all
      // ranks' copies with one multimem.ld_reduce per 16 bytes, so only the arrival counter crosses NVLink
      // from here and the owner's ingress is 1x instead of world x.
      const size_t slot_row0 = args.mc_recv != nullptr
                                   ? (size_t)owner * args.rows_per_rank + (size_t)lm * 128
                                   : (size_t)args.rank * args.rows_per_rank + (size_t)lm * 128;
      uint8_t* dst_tile = args.peer_recv[args.mc_recv != nullptr ? args.rank : owner] + slot_row0 * args.N * 2;
      // The accumulator leaves in two halves of 128 columns. Each half is staged in shared memory
      // (two 128-byte-swizzled slabs) and then written out cooperatively so that every warp store
      // covers two rows x 256 contiguous bytes: NVLink sees full-line writes instead of 16-byte pieces.
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
#pragma unroll 1
        for (int sub = 0; sub < 4; ++sub) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kBN + half * 128 + sub * 32, r);
          tmem_ld_wait();
          if (half == 1 && sub == 3) {
            tc_fence_before();
            mbar_arrive(&tempty_bar[acc]);
          }
          uint8_t* srow = smem_slab + (sub >> 1) * kSlabBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 u;
            if (args.in_fmt == 1) {
              u.x = pack_bf16x2(__uint_as_float(r[c * 8]), __uint_as_float(r[c * 8 + 1]));
              u.y = pack_bf16x2(__uint_as_float(r[c * 8 + 2]), __uint_as_float(r[c * 8 + 3]));
              u.z = pack_bf16x2(__uint_as_float(r[c * 8 + 4]), __uint_as_float(r[c * 8 + 5]));
              u.w = pack_bf16x2(__uint_as_float(r[c * 8 + 6]), __uint_as_float(r[c * 8 + 7]));
            } else {
              u.x = pack_f16x2(__uint_as_float(r[c * 8]), __uint_as_float(r[c * 8 + 1]));
              u.y = pack_f16x2(__uint_as_float(r[c * 8 + 2]), __uint_as_float(r[c * 8 + 3]));
              u.z = pack_f16x2(__uint_as_float(r[c * 8 + 4]), __uint_as_float(r[c * 8 + 5]));
              u.w = pack_f16x2(__uint_as_float(r[c * 8 + 6]), __uint_as_float(r[c * 8 + 7]));
            }
            const int piece = (sub & 1) * 4 + c;
            *reinterpret_cast<uint4*>(srow + ((piece ^ (row & 7)) << 4)) = u;
          }
        }
        named_barrier(1, 128);
        const int col_base = n0 + half * 128;
#pragma unroll 4
        for (int k = 0; k < 16; ++k) {
          const int idx = k * 128 + et;
          const int rr = idx >> 4;            // row of the tile
          const int p16 = idx & 15;           // 16-byte piece inside the 256-byte half row
          const int col = col_base + p16 * 8;
          if (col < args.N) {
            const uint4 u = *reinterpret_cast<const uint4*>(smem_slab + (p16 >> 3) * kSlabBytes + rr * 128 +
                                                            (((p16 & 7) ^ (rr & 7)) << 4));
            *reinterpret_cast<uint4*>(dst_tile + ((size_t)rr * args.N + col) * 2) = u;
          }
        }
        named_barrier(1, 128);
      }
      // publish the tile: all 128 rows are written -> one arrival on the owner's counter. The barrier
      // orders every thread's stores before thread 0, whose system-scope fence + release are cumulative.
      named_barrier(1, 128);
      if (et == 0) {
        __threadfence_system();
        red_release_sys_add(args.peer_flags[owner] + lm * args.num_n_tiles + nt, 1);
      }
      ++tcount;
    }
  }

  // ---------------- reduce phase: every warp of the CTA sums arrived partials ----------------
  if (args.norm_gamma != nullptr) {
    if (args.in_fmt == 1) {
      if (args.norm_bwd) rs_reduce_norm_dispatch<true, true>(args, warp, lane);
      else rs_reduce_norm_dispatch<true, false>(args, warp, lane);
    } else {
      if (args.norm_bwd) rs_reduce_norm_dispatch<false, true>(args, warp, lane);
      else rs_reduce_norm_dispatch<false, false>(args, warp, lane);
    }
  } else {
    const int nwarps = kGemmThreads / 32;
    const int gw = blockIdx.x * nwarps + warp;
    const int n_gw = gridDim.x * nwarps;
    const int units = mtiles_per_shard * args.num_n_tiles * 8;   // 16 rows x 256 columns each
    const int target = args.world * (*args.epoch_ptr + 1);
    for (int u = gw; u < units; u += n_gw) {
      const int rg = u & 7;
      const int tn = u >> 3;
      const int nt = tn % args.num_n_tiles;
      const int lm = tn / args.num_n_tiles;
      int ok = 1;
      if (lane == 0)
        ok = wait_flag_sys(args.flags + lm * args.num_n_tiles + nt, target, args.status, kTimeoutPeerFlag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) continue;
      const int col = nt * kBN + lane * 8;
      if (col >= args.N) continue;
      float bias_v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) bias_v[j] = 0.f;
      if (args.bias != nullptr) {
        const uint4 ub = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(args.bias) + (size_t)col * 2);
        const uint32_t w[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float2 f = args.in_fmt == 1 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
          bias_v[2 * t] = f.x; bias_v[2 * t + 1] = f.y;
        }
      }
      // four rows per pass: all partial loads of the pass are issued before any is consumed
#pragma unroll 1
      for (int i0 = 0; i0 < 16; i0 += 4) {
        float acc[4][8];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[r][j] = bias_v[j];
        uint4 resv[4];
        if (args.residual != nullptr) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int lrow = lm * 128 + rg * 16 + i0 + r;
            resv[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(args.residual) +
                                                      ((size_t)lrow * args.ldr + col) * 2);
          }
        }
        if (args.mc_recv != nullptr) {
          uint4 v[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int lrow = lm * 128 + rg * 16 + i0 + r;
            const uint8_t* p = args.mc_recv + (((size_t)args.rank * args.rows_per_rank + lrow) * args.N + col) * 2;
            v[r] = args.in_fmt == 1 ? multimem_ld_reduce_bf16x8(p) : multimem_ld_reduce_f16x8(p);
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              float2 f = args.in_fmt == 1 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
              acc[r][2 * t] += f.x; acc[r][2 * t + 1] += f.y;
            }
          }
        } else
        for (int src = 0; src < args.world; ++src) {
          uint4 v[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int lrow = lm * 128 + rg * 16 + i0 + r;
            v[r] = __ldcv(reinterpret_cast<const uint4*>(
                args.recv + (((size_t)src * args.rows_per_rank + lrow) * args.N + col) * 2));
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              float2 f = args.in_fmt == 1 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
              acc[r][2 * t] += f.x; acc[r][2 * t + 1] += f.y;
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int lrow = lm * 128 + rg * 16 + i0 + r;
          if (args.residual != nullptr) {
            const uint32_t w[4] = {resv[r].x, resv[r].y, resv[r].z, resv[r].w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              float2 f = args.in_fmt == 1 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
              acc[r][2 * t] += f.x; acc[r][2 * t + 1] += f.y;
            }
          }
          uint4 o;
          if (args.in_fmt == 1) {
            o.x = pack_bf16x2(acc[r][0], acc[r][1]); o.y = pack_bf16x2(acc[r][2], acc[r][3]);
            o.z = pack_bf16x2(acc[r][4], acc[r][5]); o.w = pack_bf16x2(acc[r][6], acc[r][7]);
          } else {
            o.x = pack_f16x2(acc[r][0], acc[r][1]); o.y = pack_f16x2(acc[r][2], acc[r][3]);
            o.z = pack_f16x2(acc[r][4], acc[r][5]); o.w = pack_f16x2(acc[r][6], acc[r][7]);
          }
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(args.out) + ((size_t)lrow * args.ldo + col) * 2) = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int B_MAJOR>
static int launch_gemm_rs(const CUtensorMap& tmA, const CUtensorMap& tmB, const RsArgs& args, int grid,
                          cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm_rs_kernel<B_MAJOR>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(tmA, tmB, args);
  return check_launch("gemm_rs_kernel");
}

}  // namespace icb

using namespace icb;

// out_shard[rows_per_rank, N] = reduce_scatter_rows(A[M, K] * B) (+bias) (+residual), M = world * rows_per_rank.
//   A: [M, lda] row-major (K contiguous). b_major 0: B [N, ldb] (K contiguous); 1: B [K, ldb] (N contiguous).
//   peer_recv / peer_flags: device arrays [world] of peer pointers to every rank's receive buffer
//   ([world][rows_per_rank][N] 16-bit) and arrival counters ([rows_per_rank/128][ceil(N/256)] int).
//   mc_recv: multicast (NVLS) address of the receive buffer or null. With it partial tiles stay local ([M][N]) and the
//   owner reduces them through the switch (multimem.ld_reduce); same form on every call and rank of a workspace.
//   N must be a multiple of 8; rows_per_rank a multiple of 128; epoch_ptr = device int with the number of calls already
//   made on this pair of buffers (same on every rank; the caller increments it after the call).
static int gemm_rs_impl(const void* A, const void* B, void* out, const void* bias, const void* residual, int M, int N,
                        int K, long long lda, long long ldb, long long ldo, long long ldr, int b_major, int in_dtype,
                        const void* const* peer_recv, int* const* peer_flags, const void* recv, const int* flags,
                        int rank, int world, const int* epoch_ptr, int* status, void* stream_, const void* mc_recv,
                        const RsArgs* fused) {
  if (world < 1 || M % world != 0) return -2;
  const int rows_per_rank = M / world;
  if (rows_per_rank % 128 != 0 || N % 8 != 0) return -7;
  if ((lda * 2) % 16 || (ldb * 2) % 16 || (ldo * 2) % 16) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, (uint32_t)kBM};
    rc = make_tmap(&tmA, in_dtype, 2, A, dims, str, box, true);
    if (rc) return rc;
  }
  if (b_major == 0) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, (uint32_t)kBN};
    rc = make_tmap(&tmB, in_dtype, 2, B, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, (uint32_t)kBK};
    rc = make_tmap(&tmB, in_dtype, 2, B, dims, str, box, true);
  }
  if (rc) return rc;
  RsArgs a{};
  if (fused != nullptr) a = *fused;
  a.M = M; a.N = N; a.K = K;
  a.num_m_tiles = M / kBM;
  a.num_n_tiles = (N + kBN - 1) / kBN;
  a.rank = rank; a.world = world; a.rows_per_rank = rows_per_rank;
  a.peer_recv = reinterpret_cast<uint8_t* const*>(const_cast<void* const*>(reinterpret_cast<const void* const*>(peer_recv)));
  a.peer_flags = peer_flags;
  a.recv = reinterpret_cast<const uint8_t*>(recv);
  a.flags = flags;
  a.out = out; a.ldo = ldo;
  a.bias = bias; a.residual = residual; a.ldr = ldr;
  a.epoch_ptr = epoch_ptr;
  a.mc_recv = reinterpret_cast<const uint8_t*>(mc_recv);
  a.in_fmt = (in_dtype == kBF16) ? 1 : 0;
  a.status = status;
  int grid = num_sms();
  const int total = a.num_m_tiles * a.num_n_tiles;
  if (total < grid) grid = total;
  if (b_major == 0) return launch_gemm_rs<0>(tmA, tmB, a, grid, stream);
  return launch_gemm_rs<1>(tmA, tmB, a, grid, stream);
}

ICB_API int icb_gemm_rs(const void* A, const void* B, void* out, const void* bias, const void* residual, int M, int N,
                        int K, long long lda, long long ldb, long long ldo, long long ldr, int b_major, int in_dtype,
                        const void* const* peer_recv, int* const* peer_flags, const void* recv, const int* flags,
                        int rank, int world, const int* epoch_ptr, int* status, void* stream_, const void* mc_recv) {
  return gemm_rs_impl(A, B, out, bias, residual, M, N, K, lda, ldb, ldo, ldr, b_major, in_dtype, peer_recv, peer_flags,
                      recv, flags, rank, world, epoch_ptr, status, stream_, mc_recv, nullptr);
}

// icb_gemm_rs followed, inside the same kernel, by RMSNorm of the reduced rows and their all-gather:
//   out[rows_per_rank, N]     = reduce_scatter_rows(A * B) (+ bias) (+ residual)        (the residual stream)
//   gather_r[rank rows, N]    = out * rsqrt(mean(out^2) + eps) * (gamma + w_offset)      on every rank r
//   rstd[rows_per_rank]       = the reciprocal root mean squares (fp32), for the backward pass
// ag_peers / ag_peer_ready are the gather buffers ([world * rows_per_rank, N], 16-bit) and per-128-row arrival
// counters of the all-gather GEMM that consumes the rows (icb_ag_gemm with flags bit 0); ag_mc is the multicast
// address of that gather buffer or null. N * 2 bytes must divide 8192 or be a multiple of it (the counters
// count 8 KiB chunks, as the push of icb_ag_gemm does).
ICB_API int icb_gemm_rs_norm_ag(const void* A, const void* B, void* out, const void* bias, const void* residual, int M,
                                int N, int K, long long lda, long long ldb, long long ldo, long long ldr, int b_major,
                                int in_dtype, const void* const* peer_recv, int* const* peer_flags, const void* recv,
                                const int* flags, int rank, int world, const int* epoch_ptr, int* status, void* stream_,
                                const void* mc_recv, const void* gamma, float eps, float w_offset, float* rstd,
                                void* const* ag_peers, void* ag_mc, int* const* ag_peer_ready) {
  if (gamma == nullptr || ag_peers == nullptr || ag_peer_ready == nullptr) return -2;
  const long long row_bytes = (long long)N * 2;
  RsArgs f{};
  if (row_bytes >= 8192) {
    if (row_bytes % 8192) return -8;
    f.ag_rows_per_unit = 1;
    f.ag_add_per_unit = (int)(row_bytes / 8192);
  } else {
    if (8192 % row_bytes) return -8;
    f.ag_rows_per_unit = (int)(8192 / row_bytes);
    f.ag_add_per_unit = 1;
  }
  f.norm_gamma = gamma; f.norm_eps = eps; f.norm_w_offset = w_offset; f.norm_rstd = rstd;
  f.ag_peers = reinterpret_cast<uint8_t* const*>(ag_peers);
  f.ag_mc = reinterpret_cast<uint8_t*>(ag_mc);
  f.ag_peer_ready = ag_peer_ready;
  return gemm_rs_impl(A, B, out, bias, residual, M, N, K, lda, ldb, ldo, ldr, b_major, in_dtype, peer_recv, peer_flags,
                      recv, flags, rank, world, epoch_ptr, status, stream_, mc_recv, &f);
}

// Backward of the same boundary: the column-parallel layer's input gradient is reduced, taken through the RMSNorm
// backward and gathered for the row-parallel layer's backward, in the kernel that computes the partial products.
//   dn[rows_per_rank, N]   = reduce_scatter_rows(A * B)                       (gradient of the normalised rows)
//   out[rows_per_rank, N]  = rstd * (dn * g - xh * mean(dn * g * xh)) (+ residual),  xh = x * rstd, g = gamma + w_offset
//   every rank's gather buffer receives `out` at this rank's rows (P2P stores / multimem.st) and the arrival
//   counters are bumped, as in icb_gemm_rs_norm_ag. x / rstd: the norm's input rows and the statistics its forward
//   wrote; residual: the gradient arriving over the residual path. dn is kept for the gain's gradient.
ICB_API int icb_gemm_rs_norm_bwd_ag(const void* A, const void* B, void* out, const void* residual, int M, int N, int K,
                                    long long lda, long long ldb, long long ldo, long long ldr, int b_major,
                                    int in_dtype, const void* const* peer_recv, int* const* peer_flags,
                                    const void* recv, const int* flags, int rank, int world, const int* epoch_ptr,
                                    int* status, void* stream_, const void* mc_recv, const void* gamma, float w_offset,
                                    const float* rstd, const void* x, long long ldx, void* dn, void* const* ag_peers,
                                    void* ag_mc, int* const* ag_peer_ready) {
  if (gamma == nullptr || ag_peers == nullptr || ag_peer_ready == nullptr || rstd == nullptr || x == nullptr ||
      dn == nullptr)
    return -2;
  const long long row_bytes = (long long)N * 2;
  RsArgs f{};
  if (row_bytes >= 8192) {
    if (row_bytes % 8192) return -8;
    f.ag_rows_per_unit = 1;
    f.ag_add_per_unit = (int)(row_bytes / 8192);
  } else {
    if (8192 % row_bytes) return -8;
    f.ag_rows_per_unit = (int)(8192 / row_bytes);
    f.ag_add_per_unit = 1;
  }
  f.norm_gamma = gamma; f.norm_eps = 0.f; f.norm_w_offset = w_offset;
  f.norm_rstd = const_cast<float*>(rstd);
  f.norm_bwd = 1; f.norm_x = x; f.norm_ldx = ldx; f.aux_out = dn;
  f.ag_peers = reinterpret_cast<uint8_t* const*>(ag_peers);
  f.ag_mc = reinterpret_cast<uint8_t*>(ag_mc);
  f.ag_peer_ready = ag_peer_ready;
  return gemm_rs_impl(A, B, out, nullptr, residual, M, N, K, lda, ldb, ldo, ldr, b_major, in_dtype, peer_recv,
                      peer_flags, recv, flags, rank, world, epoch_ptr, status, stream_, mc_recv, &f);
}
