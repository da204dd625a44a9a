// Two-SM tcgen05 GEMM for sm_100a: the default kernel for large plain problems (see ops/kernels.py).
//
// A thread-block cluster of two CTAs on neighbouring SMs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own 128 columns of B
// (32 KiB per k-block instead of the 48 KiB a single-CTA 128 x 256 tile needs), the leader CTA's MMA
// thread issues one instruction that reads both CTAs' shared memory, and each CTA's TMEM receives the
// 128 accumulator rows it owns. Less operand traffic per flop and a 6-stage ring (instead of 4) give the
// TMA pipeline 1.5 x more latency tolerance, which is what bounds the single-CTA kernel.
//
// Synchronisation inside the pair (all mbarriers live at the same offsets in both CTAs):
//   full[s]   (leader's is used): 2 arrivals. Each CTA's producer adds its transaction bytes with
//             arrive.expect_tx (the peer does so remotely) and its TMA loads complete on the leader's barrier.
//   empty[s]  (own): the leader's tcgen05.commit arrives on both CTAs' barriers.
//   tfull[a]  (own): commit to both CTAs when a tile's accumulator is complete.
//   tempty[a] (leader's): all 256 epilogue threads of the pair arrive (the peer's remotely).
// No TMA load is multicast; every wait is bounded (status word, drain, TMEM freed).

#include "gemm_common.cuh"
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int k2Stages = 6;
constexpr int k2AStage = 128 * kBK * 2;   // 16 KiB: this CTA's 128 rows of A
constexpr int k2BStage = 128 * kBK * 2;   // 16 KiB: this CTA's 128 columns of B
struct Gemm2Smem {
  static constexpr int a_off = 0;
  static constexpr int b_off = k2Stages * k2AStage;
  static constexpr int bar_off = b_off + k2Stages * k2BStage;
  static constexpr int total = bar_off + 256;
};
constexpr int kGemm2SmemBytes = Gemm2Smem::total + 1024;

struct Gemm2Args {
  int M, N, K;
  int num_m_tiles, num_n_tiles;   // 256 x 256 tiles
  void* C;
  long long ldc;
  const void* bias;               // [N] 16-bit or null
  const void* residual;           // same dtype and pitch rules as C, or null
  long long ldr;
  int in_fmt;                     // 1 bf16, 0 fp16
  int out_f32;
  int* status;
};

// ---- cluster / pair primitives ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier of the CTA pair
// (`bar_cluster_addr` may belong to the peer).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

template <int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Gemm2Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem + Gemm2Smem::a_off;
  uint8_t* smem_b = smem + Gemm2Smem::b_off;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Gemm2Smem::bar_off);
  uint64_t* empty_bar = full_bar + k2Stages;
  uint64_t* tfull_bar = empty_bar + k2Stages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();     // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(&full_bar[s], 2);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 256);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anybody signals the peer
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = args.num_m_tiles * args.num_n_tiles;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < total_tiles; tile += num_pairs) {
        int mt, nt;
        tile_coords(tile, args.num_m_tiles, args.num_n_tiles, mt, nt);
        const int m0 = mt * 256 + (int)cta * 128;       // this CTA's rows of A
        const int n0 = nt * 256 + (int)cta * 128;       // this CTA's columns of B
        for (int k0 = 0; k0 < args.K; k0 += kBK, ++it) {
          const int s = it % k2Stages;
          const uint32_t ph = (it / k2Stages) & 1;
          mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
          mbar_expect_tx_cluster(full_leader, k2AStage + k2BStage);
          uint8_t* sa = smem_a + s * k2AStage;
          uint8_t* sb = smem_b + s * k2BStage;
          if (A_MAJOR == 0) {
            tma_load_2d_pair(sa, &tmA, full_leader, k0, m0);
          } else {
            tma_load_2d_pair(sa, &tmA, full_leader, m0, k0);
            tma_load_2d_pair(sa + 8192, &tmA, full_leader, m0 + 64, k0);
          }
          if (B_MAJOR == 0) {
            tma_load_2d_pair(sb, &tmB, full_leader, k0, n0);
          } else {
            tma_load_2d_pair(sb, &tmB, full_leader, n0, k0);
            tma_load_2d_pair(sb + 8192, &tmB, full_leader, n0 + 64, k0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = umma_idesc(256, 256, args.in_fmt, A_MAJOR, B_MAJOR);
      uint32_t it = 0, tcount = 0;
      for (int tile = pair; tile < total_tiles; tile += num_pairs) {
        const uint32_t acc = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, args.status, kTimeoutTmemEmpty);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * 256;
        uint32_t first = 1;
        for (int k0 = 0; k0 < args.K; k0 += kBK, ++it) {
          const int s = it % k2Stages;
          const uint32_t ph = (it / k2Stages) & 1;
          mbar_wait(&full_bar[s], ph, abort_flag, args.status, kTimeoutSmemFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + s * k2AStage);
          const uint32_t b_addr = smem_u32(smem_b + s * k2BStage);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc = (A_MAJOR == 0) ? umma_desc_sw128(a_addr + k * 32, 16, 1024)
                                                  : umma_desc_sw128(a_addr + k * 2048, 8192, 1024);
            const uint64_t bdesc = (B_MAJOR == 0) ? umma_desc_sw128(b_addr + k * 32, 16, 1024)
                                                  : umma_desc_sw128(b_addr + k * 2048, 8192, 1024);
            umma_ss_pair(tmem_d, adesc, bdesc, idesc, first ? 0u : 1u);
            first = 0;
          }
          umma_commit_pair(&empty_bar[s]);
        }
        umma_commit_pair(&tfull_bar[acc]);
        ++tcount;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int esz = args.out_f32 ? 4 : 2;
    uint32_t tcount = 0;
    for (int tile = pair; tile < total_tiles; tile += num_pairs) {
      int mt, nt;
      tile_coords(tile, args.num_m_tiles, args.num_n_tiles, mt, nt);
      const int m0 = mt * 256 + (int)cta * 128;
      const int n0 = nt * 256;
      const uint32_t acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, args.status, kTimeoutTmemFull);
      tc_fence_after();
      const long long m_glob = m0 + row;
      const bool row_ok = m_glob < args.M;
#pragma unroll 1
      for (int sub = 0; sub < 8; ++sub) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256 + sub * 32, r);
        tmem_ld_wait();
        if (sub == 7) {
          tc_fence_before();
          const uint32_t te = map_to_cta(smem_u32(&tempty_bar[acc]), 0);
          mbar_arrive_cluster(te);
        }
        const int n_glob = n0 + sub * 32;
        if (!row_ok || n_glob >= args.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        const bool full32 = n_glob + 32 <= args.N;
        if (args.bias != nullptr) {
          for (int j = 0; j < 32; ++j) {
            if (n_glob + j < args.N) {
              const uint16_t raw = reinterpret_cast<const uint16_t*>(args.bias)[n_glob + j];
              v[j] += args.in_fmt == 1 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                                       : __half2float(*reinterpret_cast<const __half*>(&raw));
            }
          }
        }
        if (args.residual != nullptr) {
          const uint8_t* rp = reinterpret_cast<const uint8_t*>(args.residual) + ((size_t)m_glob * args.ldr + n_glob) * esz;
          if (esz == 4) {
            if (full32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
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
            for (int j = 0; j < 32; ++j) {
              if (n_glob + j < args.N) {
                const uint16_t raw = reinterpret_cast<const uint16_t*>(rp)[j];
                v[j] += args.in_fmt == 1 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                                         : __half2float(*reinterpret_cast<const __half*>(&raw));
              }
            }
          }
        }
        uint8_t* cp = reinterpret_cast<uint8_t*>(args.C) + ((size_t)m_glob * args.ldc + n_glob) * esz;
        const bool vec = full32 && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
        if (esz == 4) {
          if (vec) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<float4*>(cp + c * 16) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (n_glob + j < args.N) reinterpret_cast<float*>(cp)[j] = v[j];
          }
        } else {
          if (vec) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 u;
              if (args.in_fmt == 1) {
                u.x = pack_bf16x2(v[c * 8], v[c * 8 + 1]); u.y = pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
                u.z = pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]); u.w = pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
              } else {
                u.x = pack_f16x2(v[c * 8], v[c * 8 + 1]); u.y = pack_f16x2(v[c * 8 + 2], v[c * 8 + 3]);
                u.z = pack_f16x2(v[c * 8 + 4], v[c * 8 + 5]); u.w = pack_f16x2(v[c * 8 + 6], v[c * 8 + 7]);
              }
              *reinterpret_cast<uint4*>(cp + c * 16) = u;
            }
          } else {
            for (int j = 0; j < 32; ++j) {
              if (n_glob + j < args.N) {
                if (args.in_fmt == 1) reinterpret_cast<__nv_bfloat16*>(cp)[j] = __float2bfloat16(v[j]);
                else reinterpret_cast<__half*>(cp)[j] = __float2half(v[j]);
              }
            }
          }
        }
      }
      ++tcount;
    }
  }

  // Drain: nobody leaves while the pair's TMEM is allocated, copies are in flight or the peer may still
  // signal a barrier in this CTA's shared memory.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int A_MAJOR, int B_MAJOR>
static int launch_gemm2sm(const CUtensorMap& tmA, const CUtensorMap& tmB, const Gemm2Args& args, int grid,
                          cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm2sm_kernel<A_MAJOR, B_MAJOR>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemm2SmemBytes);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  kern<<<grid, kGemmThreads, kGemm2SmemBytes, stream>>>(tmA, tmB, args);
  return check_launch("gemm2sm_kernel");
}

}  // namespace icb

using namespace icb;

// C[M, N] = A * B (+ bias) (+ residual) with 256 x 256 tiles on CTA pairs. Same operand conventions as icb_gemm
// (a_major / b_major 0 = K contiguous, 1 = M / N contiguous; pitches in elements, 16-byte aligned rows);
// plain problems only (no grouping), M and N of any size (edge tiles are clipped by TMA / bounds checks).
ICB_API int icb_gemm_2sm(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                         int K, long long lda, long long ldb, long long ldc, long long ldr, int a_major, int b_major,
                         int in_dtype, int out_f32, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (in_dtype != kBF16 && in_dtype != kF16) return -2;
  const int oes = out_f32 ? 4 : 2;
  if ((lda * 2) % 16 || (ldb * 2) % 16 || (ldc * oes) % 16) return -4;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -5;
  CUtensorMap tmA, tmB;
  int rc;
  if (a_major == 0) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, 128};
    rc = make_tmap(&tmA, in_dtype, 2, A, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, (uint32_t)kBK};
    rc = make_tmap(&tmA, in_dtype, 2, A, dims, str, box, true);
  }
  if (rc) return rc;
  if (b_major == 0) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, 128};
    rc = make_tmap(&tmB, in_dtype, 2, B, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, (uint32_t)kBK};
    rc = make_tmap(&tmB, in_dtype, 2, B, dims, str, box, true);
  }
  if (rc) return rc;
  Gemm2Args a;
  a.M = M; a.N = N; a.K = K;
  a.num_m_tiles = (M + 255) / 256;
  a.num_n_tiles = (N + 255) / 256;
  a.C = C; a.ldc = ldc; a.bias = bias; a.residual = residual; a.ldr = ldr;
  a.in_fmt = (in_dtype == kBF16) ? 1 : 0;
  a.out_f32 = out_f32;
  a.status = status;
  int grid = num_sms() & ~1;
  const int total = a.num_m_tiles * a.num_n_tiles;
  if (total * 2 < grid) grid = total * 2;
  if (a_major == 0 && b_major == 0) return launch_gemm2sm<0, 0>(tmA, tmB, a, grid, stream);
  if (a_major == 0 && b_major == 1) return launch_gemm2sm<0, 1>(tmA, tmB, a, grid, stream);
  if (a_major == 1 && b_major == 0) return launch_gemm2sm<1, 0>(tmA, tmB, a, grid, stream);
  return launch_gemm2sm<1, 1>(tmA, tmB, a, grid, stream);
}
