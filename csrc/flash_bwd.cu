// Flash attention backward for sm_100a (causal / full, GQA, cu_seqlens, head_dim 64/128).
//
// One CTA owns a 128-row K/V tile of one KV head and walks every query head of the group
// and every query tile that can see it. Per step five tcgen05 GEMMs run on tiles that are
// loaded once: S = Q K^T and dP = dO V^T (K-major reads), then dV += P^T dO, dK += dS^T Q
// and dQ = dS K, which read the *same* shared-memory bytes through MN-major descriptors,
// so nothing is transposed or copied. TMEM holds S, dP, dV and dK (4 x 128 columns for
// head_dim 128); dQ reuses the dP columns once the softmax warps have consumed dP. Q is double buffered:
// the next step's Q tile is loaded while this step runs and its S = Q K^T is issued right behind this step's
// dQ, so that it executes while dQ is drained.
// Warps 2-9 are two groups of four; a thread owns one query row (TMEM lane) and its group one half of
// the columns. Per step they first turn S into P = exp2(S*scale - lse) (kept in registers, written as bf16 into a
// 128-byte-swizzled tile) and publish it, so that dV = P^T dO runs while they wait for dP and form
// dS' = P (dP - delta); then they copy dQ from TMEM into an fp32 staging tile (the P tile and the step's Q buffer,
// both free by then) that one thread adds to a zeroed fp32 scratch with TMA bulk reduce-adds (converted to 16-bit
// and scaled by a follow-up kernel) and, at the end, dK (first group) / dV (second group; TMEM lane == kv row).
// dK/dV need no atomics: the group's heads are accumulated in place.
// Barriers of one step: s_full (S done) -> p_full (P written) -> dV; dp_full (dP done) -> pds_full (dS written)
// -> dK, dQ -> dq_full -> drain -> dq_empty (dP columns free). Every wait is bounded (status word + drain on
// timeout).
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

// Cycle counters for `python -m benchmarks.flash_bwd_trace` (a separate build with -DICB_FB_TRACE; the product
// library compiles these macros away): where each role of the kernel spends a step, summed over all CTAs.
#ifdef ICB_FB_TRACE
__device__ unsigned long long g_fb_trace[16];
#define FB_T0(v) long long v = clock64()
#define FB_TSET(v) v = clock64()
#define FB_TADD(i, v) atomicAdd(&g_fb_trace[i], (unsigned long long)(clock64() - (v)))
#define FB_TCOUNT(i) atomicAdd(&g_fb_trace[i], 1ull)
#else
#define FB_T0(v)
#define FB_TSET(v)
#define FB_TADD(i, v)
#define FB_TCOUNT(i)
#endif

constexpr int kFbThreads = 320;           // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr int kFbSoftmaxThreads = 256;
constexpr int kFbTmemCols = 512;

int make_head_tmap(CUtensorMap* tm, const void* base, int hd, int heads, long long tokens, long long row_stride,
                   int dtype);

struct FlashBwdArgs {
  int batch, seq_len, hq, hkv;
  const int* cu_seqlens;
  const float* lse;      // [hq, T]
  const float* delta;    // [hq, T]  rowsum(dO * O)
  float* dq_acc;         // [T, hq, HD] fp32, zero-initialised
  void* dk;              // first element of dK inside rows of dkv_stride elements
  void* dv;
  long long dkv_stride;
  long long total_tokens;
  float scale, scale_log2;
  int causal;
  int in_fmt;
  int* status;
  const unsigned long long* drop_seed;  // the device word the forward pass was given
  int drop_thr;
  float drop_scale;
};

template <int HD>
struct FbSmem {
  static constexpr int kChunks = HD / 64;
  static constexpr int tile_bytes = 128 * HD * 2;
  static constexpr int p_bytes = 128 * 128 * 2;
  static constexpr int k_off = 0;
  static constexpr int v_off = k_off + tile_bytes;
  static constexpr int q_off = v_off + tile_bytes;          // two Q buffers
  static constexpr int do_off = q_off + 2 * tile_bytes;
  static constexpr int p_off = do_off + tile_bytes;
  static constexpr int ds_off = p_off + p_bytes;
  static constexpr int bar_off = ds_off + p_bytes;
  static constexpr int total = bar_off + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2_b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint4 fb_pack8(const float (&f)[8], int in_fmt) {
  uint4 u;
  if (in_fmt == 1) {
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  } else {
    u.x = pack_f16x2(f[0], f[1]); u.y = pack_f16x2(f[2], f[3]);
    u.z = pack_f16x2(f[4], f[5]); u.w = pack_f16x2(f[6], f[7]);
  }
  return u;
}
// byte offset of the 16-byte piece that holds columns col0 .. col0 + 7 of a row in a 128-byte-swizzled tile of
// 64-column (16 KiB) chunks; row7 = row & 7
__device__ __forceinline__ int fb_piece_off(int col0, int row7) {
  return (col0 >> 6) * 16384 + ((((col0 & 63) >> 3) ^ row7) << 4);
}

// The softmax / dS phase of one query row, in two parts per 32-column chunk so that P can be published (and
// dV = P^T dO started) before dP has even arrived:
//   part 1: P = exp2(S*scale - lse) (masked), kept in registers and written for the dV product;
//   part 2: dS' = P (dP - delta), written for dK and dQ (the softmax scale that dS carries is applied where dK
//           and dQ leave the chip).
// MASK: the tile crosses the diagonal, the end of the sequence or holds rows past it. DROP: attention dropout
// (dV takes the masked, rescaled P; dP arrives as d(masked P) and is masked the same way; delta = rowsum(dO O)
// already includes the mask).
template <bool MASK, bool DROP>
__device__ __forceinline__ void fb_p_chunk(const uint32_t (&sr)[32], float (&pv)[32], int col_base, uint8_t* prow,
                                           int row7, float scale_log2, float lse2, bool q_valid, int kv0, int q_idx,
                                           int seq_len, int causal, int in_fmt, unsigned long long drop_key,
                                           unsigned long long drop_row, int drop_thr, float drop_scale) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float p[8];
    unsigned long long h = 0ull;
    if (DROP) h = dropout_hash(drop_key, drop_row + (unsigned)((kv0 + col_base + g * 8) >> 3));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = fast_exp2_b(__uint_as_float(sr[g * 8 + i]) * scale_log2 - lse2);
      if (MASK) {
        const int kv_idx = kv0 + col_base + g * 8 + i;
        const bool keep = q_valid && kv_idx < seq_len && !(causal && kv_idx > q_idx);
        v = keep ? v : 0.f;
      }
      pv[g * 8 + i] = v;
      p[i] = DROP ? ((int)((h >> (8 * i)) & 0xffull) >= drop_thr ? v * drop_scale : 0.f) : v;
    }
    *reinterpret_cast<uint4*>(prow + fb_piece_off(col_base + g * 8, row7)) = fb_pack8(p, in_fmt);
  }
}
template <bool DROP>
__device__ __forceinline__ void fb_ds_chunk(const uint32_t (&dr)[32], const float (&pv)[32], int col_base,
                                            uint8_t* dsrow, int row7, float dlt, int kv0, int in_fmt,
                                            unsigned long long drop_key, unsigned long long drop_row, int drop_thr,
                                            float drop_scale) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float ds[8];
    unsigned long long h = 0ull;
    if (DROP) h = dropout_hash(drop_key, drop_row + (unsigned)((kv0 + col_base + g * 8) >> 3));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float dp = __uint_as_float(dr[g * 8 + i]);
      if (DROP) dp = (int)((h >> (8 * i)) & 0xffull) >= drop_thr ? dp * drop_scale : 0.f;
      ds[i] = pv[g * 8 + i] * (dp - dlt);
    }
    *reinterpret_cast<uint4*>(dsrow + fb_piece_off(col_base + g * 8, row7)) = fb_pack8(ds, in_fmt);
  }
}

template <int HD>
__global__ void __launch_bounds__(kFbThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, const FlashBwdArgs args) {
  using L = FbSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::k_off;
  uint8_t* sV = smem + L::v_off;
  uint8_t* sQ = smem + L::q_off;
  uint8_t* sDO = smem + L::do_off;
  uint8_t* sP = smem + L::p_off;
  uint8_t* sDS = smem + L::ds_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;        // 2
  uint64_t* q_empty = bars + 3;       // 2
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;
  uint64_t* dp_full = bars + 7;
  uint64_t* pds_full = bars + 8;
  uint64_t* dq_full = bars + 9;
  uint64_t* dq_empty = bars + 10;
  uint64_t* stage_free = bars + 11;   // 2: the dQ staging that borrowed Q buffer i has been read by its reduce
  uint64_t* s_full = bars + 13;
  uint64_t* p_full = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  FB_T0(t_cta);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int b = blockIdx.z;
  const int group = args.hq / args.hkv;

  int seq_start, seq_len;
  if (args.cu_seqlens != nullptr) {
    seq_start = args.cu_seqlens[b];
    seq_len = args.cu_seqlens[b + 1] - seq_start;
  } else {
    seq_start = b * args.seq_len;
    seq_len = args.seq_len;
  }
  const int n_tiles = (seq_len + 127) >> 7;
  const int jt = blockIdx.x;  // kv tile; low tiles (most work under a causal mask) are scheduled first
  if (jt >= n_tiles) return;
  const int kv0 = jt * 128;
  const int i_begin = args.causal ? jt : 0;
  const int iters_per_head = n_tiles - i_begin;
  const int n_iters = iters_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(dp_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, kFbSoftmaxThreads);
    mbar_init(pds_full, kFbSoftmaxThreads);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, kFbSoftmaxThreads);
    mbar_init(&stage_free[0], 1);
    mbar_init(&stage_free[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kFbTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base;
  const uint32_t tm_dp = tmem_base + 128;   // also dQ, once the softmax warps have consumed dP
  const uint32_t tm_dv = tmem_base + 256;
  const uint32_t tm_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::tile_bytes);
#pragma unroll
      for (int c = 0; c < L::kChunks; ++c) {
        tma_load_3d(sK + c * 16384, &tmK, kv_full, c * 64, kv_head, seq_start + kv0);
        tma_load_3d(sV + c * 16384, &tmV, kv_full, c * 64, kv_head, seq_start + kv0);
      }
      for (int it = 0; it < n_iters; ++it) {
        const uint32_t ph = it & 1;
        const int head = kv_head * group + it / iters_per_head;
        const int t0 = seq_start + (i_begin + it % iters_per_head) * 128;
        const int qb = it & 1;
        FB_T0(tt);
        mbar_wait(&q_empty[qb], ((it >> 1) & 1) ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
        FB_TADD(0, tt);
        FB_TSET(tt);
        mbar_wait(&stage_free[qb], ((it >> 1) & 1) ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
        FB_TADD(12, tt);
        mbar_expect_tx(&q_full[qb], L::tile_bytes);
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_3d(sQ + qb * L::tile_bytes + c * 16384, &tmQ, &q_full[qb], c * 64, head, t0);
        FB_TSET(tt);
        mbar_wait(do_empty, ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
        FB_TADD(1, tt);
        mbar_expect_tx(do_full, L::tile_bytes);
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c) tma_load_3d(sDO + c * 16384, &tmDO, do_full, c * 64, head, t0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_kk = umma_idesc(128, 128, args.in_fmt, 0, 0);   // S, dP
      const uint32_t idesc_mm = umma_idesc(128, HD, args.in_fmt, 1, 1);    // dV, dK
      const uint32_t idesc_km = umma_idesc(128, HD, args.in_fmt, 0, 1);    // dQ
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      const uint32_t aP = smem_u32(sP), aDS = smem_u32(sDS);
      mbar_wait(kv_full, 0, abort_flag, args.status, kTimeoutSmemFull);
      // S of step it + 1 is issued right behind dQ of step it (Q is double buffered and the S columns were
      // consumed before P / dS were published), so the tensor core works on it while dQ is drained; dP has to
      // wait for that drain because dQ uses its columns.
      auto issue_s = [&](int it) {
        const uint32_t q_addr = aQ + (it & 1) * L::tile_bytes;
        FB_T0(tq);
        mbar_wait(&q_full[it & 1], (it >> 1) & 1, abort_flag, args.status, kTimeoutSmemFull);
        FB_TADD(2, tq);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_ss(tm_s, umma_desc_sw128(q_addr + off, 16, 1024), umma_desc_sw128(aK + off, 16, 1024), idesc_kk,
                  k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      };
      if (n_iters > 0) issue_s(0);
      for (int it = 0; it < n_iters; ++it) {
        const uint32_t ph = it & 1;
        const uint32_t q_addr = aQ + (it & 1) * L::tile_bytes;
        FB_T0(tm);
        mbar_wait(do_full, ph, abort_flag, args.status, kTimeoutSmemFull);
        FB_TADD(3, tm);
        FB_TSET(tm);
        mbar_wait(dq_empty, ph ^ 1, abort_flag, args.status, kTimeoutTmemEmpty);
        FB_TADD(4, tm);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_ss(tm_dp, umma_desc_sw128(aDO + off, 16, 1024), umma_desc_sw128(aV + off, 16, 1024), idesc_kk,
                  k > 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        FB_TSET(tm);
        mbar_wait(p_full, ph, abort_flag, args.status, kTimeoutLocalFlag);
        FB_TADD(5, tm);
        tc_fence_after();
        const uint32_t acc = it > 0 ? 1u : 0u;
        // dV += P^T dO   (A = P read MN-major: M = kv, K = q rows; B = dO read MN-major)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tm_dv, umma_desc_sw128(aP + k * 2048, 16384, 1024), umma_desc_sw128(aDO + k * 2048, 16384, 1024),
                  idesc_mm, (acc | (k > 0 ? 1u : 0u)));
        umma_commit(do_empty);
        mbar_wait(pds_full, ph, abort_flag, args.status, kTimeoutLocalFlag);
        tc_fence_after();
        // dK += dS^T Q
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tm_dk, umma_desc_sw128(aDS + k * 2048, 16384, 1024), umma_desc_sw128(q_addr + k * 2048, 16384, 1024),
                  idesc_mm, (acc | (k > 0 ? 1u : 0u)));
        umma_commit(&q_empty[it & 1]);
        // dQ = dS K   (A = dS read K-major: M = q rows, K = kv; B = K tile read MN-major)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tm_dp, umma_desc_sw128(aDS + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                  umma_desc_sw128(aK + k * 2048, 16384, 1024), idesc_km, k > 0 ? 1u : 0u);
        umma_commit(dq_full);
        if (it + 1 < n_iters) issue_s(it + 1);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;       // column half of this warp's group
    const int row = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const float log2e = 1.4426950408889634f;
    const bool dropout = args.drop_thr > 0;
    const unsigned long long drop_key = dropout ? *args.drop_seed : 0ull;
    for (int it = 0; it < n_iters; ++it) {
      const uint32_t ph = it & 1;
      const int head = kv_head * group + it / iters_per_head;
      const int it_q = i_begin + it % iters_per_head;
      const int q_idx = it_q * 128 + row;
      const bool q_valid = q_idx < seq_len;
      const long long tok = (long long)seq_start + q_idx;
      float lse2 = 0.f, dlt = 0.f;
      if (q_valid) {
        lse2 = args.lse[(size_t)head * args.total_tokens + tok] * log2e;
        dlt = args.delta[(size_t)head * args.total_tokens + tok];
      }
      const bool need_mask = (args.causal && it_q == jt) || (kv0 + 128 > seq_len) || (it_q * 128 + 128 > seq_len);
      const unsigned long long drop_row = dropout_row_counter(b, args.hq, head, args.seq_len, q_idx);
      FB_T0(ts);
      mbar_wait(s_full, ph, abort_flag, args.status, kTimeoutTmemFull);
      if (threadIdx.x == 64) {
        FB_TADD(6, ts);
        FB_TCOUNT(15);
      }
      FB_TSET(ts);
      tc_fence_after();
      if (it > 0) {
        // the P tile staged the first half of the previous step's dQ: that bulk reduce (the older of the two
        // groups) must have read it
        if (threadIdx.x == 64) tma_store_wait_read<1>();
        named_barrier(1, kFbSoftmaxThreads);
      }
      if (threadIdx.x == 64) FB_TADD(11, ts);
      uint8_t* prow = sP + row * 128;
      uint8_t* dsrow = sDS + row * 128;
      const int row7 = row & 7;
      float pv[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col_base = half * 64 + cc * 32;
        uint32_t sr[32];
        tmem_ld_32x32(tm_s + lane_off + col_base, sr);
        tmem_ld_wait();
#define ICB_FB_P(M, D)                                                                                               \
  fb_p_chunk<M, D>(sr, pv[cc], col_base, prow, row7, args.scale_log2, lse2, q_valid, kv0, q_idx, seq_len,            \
                   args.causal, args.in_fmt, drop_key, drop_row, args.drop_thr, args.drop_scale)
        if (dropout) {
          if (need_mask) ICB_FB_P(true, true);
          else ICB_FB_P(false, true);
        } else {
          if (need_mask) ICB_FB_P(true, false);
          else ICB_FB_P(false, false);
        }
#undef ICB_FB_P
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(p_full);                // dV = P^T dO may start
      FB_T0(t2);
      mbar_wait(dp_full, ph, abort_flag, args.status, kTimeoutTmemFull);
      if (threadIdx.x == 64) FB_TADD(13, t2);
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col_base = half * 64 + cc * 32;
        uint32_t dr[32];
        tmem_ld_32x32(tm_dp + lane_off + col_base, dr);
        tmem_ld_wait();
        if (dropout)
          fb_ds_chunk<true>(dr, pv[cc], col_base, dsrow, row7, dlt, kv0, args.in_fmt, drop_key, drop_row,
                            args.drop_thr, args.drop_scale);
        else
          fb_ds_chunk<false>(dr, pv[cc], col_base, dsrow, row7, dlt, kv0, args.in_fmt, drop_key, drop_row,
                             args.drop_thr, args.drop_scale);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(pds_full);
      if (threadIdx.x == 64) FB_TADD(7, ts);
      FB_TSET(ts);
      // drain dQ: TMEM -> fp32 staging in the 128-byte swizzle of the tensor map, then one thread adds the tile to
      // the fp32 accumulator in global memory with bulk reduce-adds: whole 128-byte lines instead of one 16-byte
      // atomic per thread and row. The first 64 columns are staged in the P tile and the rest in this step's Q
      // buffer (both free once dq_full fired): the next softmax only has to wait for the reduce of the first half,
      // the second half may take until the Q buffer is loaded again a step later.
      if (it > 0 && threadIdx.x == 64) {
        tma_store_wait_read<0>();                      // both groups of the previous step: long done by now
        mbar_arrive(&stage_free[(it - 1) & 1]);
      }
      mbar_wait(dq_full, ph, abort_flag, args.status, kTimeoutTmemFull);
      if (threadIdx.x == 64) FB_TADD(8, ts);
      FB_TSET(ts);
      tc_fence_after();
      uint8_t* stage_hi = sQ + (it & 1) * L::tile_bytes;
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tm_dp + lane_off + c * 32, o);
        tmem_ld_wait();
        uint8_t* brow = (c < 2 ? sP + c * 16384 : stage_hi + (c - 2) * 16384) + row * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(brow + ((g ^ (row & 7)) << 4)) = make_uint4(o[g * 4], o[g * 4 + 1], o[g * 4 + 2], o[g * 4 + 3]);
      }
      tc_fence_before();
      mbar_arrive(dq_empty);              // the dP columns are free: the next step's dP = dO V^T may be issued
      fence_proxy_async_smem();
      named_barrier(1, kFbSoftmaxThreads);
      if (threadIdx.x == 64) {
        const int t0 = seq_start + it_q * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) tma_reduce_add_3d(&tmDQ, sP + c * 16384, c * 32, head, t0);
        tma_store_commit();
#pragma unroll
        for (int c = 2; c < HD / 32; ++c) tma_reduce_add_3d(&tmDQ, stage_hi + (c - 2) * 16384, c * 32, head, t0);
        tma_store_commit();                              // (an empty group for head_dim 64)
      }
      if (threadIdx.x == 64) FB_TADD(9, ts);
    }
    if (threadIdx.x == 64) tma_store_wait<0>();
    // ---- epilogue: dK, dV (lane == kv row). The last dq_full wait implies every MMA finished.
    {
      const int kv_idx = kv0 + row;
      const bool valid = kv_idx < seq_len;
      const long long tok = (long long)seq_start + kv_idx;
      uint8_t* dkrow = reinterpret_cast<uint8_t*>(args.dk) + ((size_t)tok * args.dkv_stride + (size_t)kv_head * HD) * 2;
      uint8_t* dvrow = reinterpret_cast<uint8_t*>(args.dv) + ((size_t)tok * args.dkv_stride + (size_t)kv_head * HD) * 2;
      tc_fence_after();
      {
        const int which = half;
        const float out_scale = which == 0 ? args.scale : 1.0f;   // dK = scale * dS'^T Q
        const uint32_t tm = which == 0 ? tm_dk : tm_dv;
        uint8_t* orow = which == 0 ? dkrow : dvrow;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tm + lane_off + c * 32, o);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[g * 8 + i]) * out_scale;
              uint4 u;
              if (args.in_fmt == 1) {
                u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
                u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
              } else {
                u.x = pack_f16x2(f[0], f[1]); u.y = pack_f16x2(f[2], f[3]);
                u.z = pack_f16x2(f[4], f[5]); u.w = pack_f16x2(f[6], f[7]);
              }
              *reinterpret_cast<uint4*>(orow + (c * 32 + g * 8) * 2) = u;
            }
          }
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
    tmem_dealloc(tmem_base, kFbTmemCols);
  }
  if (threadIdx.x == 0) {
    FB_TADD(10, t_cta);
    FB_TCOUNT(14);
  }
}

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (token, head).
template <bool BF16>
__global__ void flash_delta_kernel(const uint16_t* __restrict__ dO, const uint16_t* __restrict__ O,
                                   float* __restrict__ delta, long long T, int hq, int hd) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * hq) return;
  const long long t = w / hq;
  const int h = (int)(w - t * hq);
  const size_t base = ((size_t)t * hq + h) * hd;
  float s = 0.f;
  for (int i = lane * 2; i < hd; i += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(dO + base + i);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(O + base + i);
    float2 fa, fb;
    if (BF16) { fa = unpack_bf16x2(a); fb = unpack_bf16x2(b); }
    else {
      fa = __half22float2(*reinterpret_cast<const __half2*>(&a));
      fb = __half22float2(*reinterpret_cast<const __half2*>(&b));
    }
    s += fa.x * fb.x + fa.y * fb.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(size_t)h * T + t] = s;
}

// fp32 [T, width] * scale -> 16-bit rows of pitch out_stride
template <bool BF16>
__global__ void flash_dq_convert_kernel(const float* __restrict__ acc, uint16_t* __restrict__ out, long long T,
                                        int width, long long out_stride, float scale) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = width >> 3;
  if (idx >= T * vecs) return;
  const long long t = idx / vecs;
  const int v = (int)(idx - t * vecs);
  float4 a = *reinterpret_cast<const float4*>(acc + (size_t)t * width + v * 8);
  float4 b = *reinterpret_cast<const float4*>(acc + (size_t)t * width + v * 8 + 4);
  a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;     // dQ = scale * dS' K
  b.x *= scale; b.y *= scale; b.z *= scale; b.w *= scale;
  uint4 u;
  if (BF16) {
    u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w); u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
  } else {
    u.x = pack_f16x2(a.x, a.y); u.y = pack_f16x2(a.z, a.w); u.z = pack_f16x2(b.x, b.y); u.w = pack_f16x2(b.z, b.w);
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + v * 8) = u;
}

template <int HD>
static int launch_flash_bwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                            const CUtensorMap& tmDO, const CUtensorMap& tmDQ, const FlashBwdArgs& args, dim3 grid,
                            cudaStream_t stream) {
  static bool configured = false;
  auto kern = flash_bwd_kernel<HD>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSmem<HD>::total);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  kern<<<grid, kFbThreads, FbSmem<HD>::total, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, args);
  return check_launch("flash_bwd_kernel");
}

}  // namespace icb

using namespace icb;

#ifdef ICB_FB_TRACE
// Copies the 16 counters out (and clears them): [0] tma: q_empty, [1] tma: do_empty, [2] mma: q_full, [3] mma: do_full,
// [4] mma: dq_empty, [5] mma: p_full, [6] softmax: s_full, [7] softmax: s_full .. dS published, [8] softmax: dq_full,
// [9] softmax: dQ drain, [10] whole CTA, [11] of [7]: wait for the staging tile, [12] tma: stage_free,
// [13] of [7]: dp_full, [14] CTAs, [15] steps.
ICB_API int icb_flash_bwd_trace_read(unsigned long long* out, int reset) {
  if (cudaMemcpyFromSymbol(out, icb::g_fb_trace, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  if (reset) {
    unsigned long long z[16] = {0};
    if (cudaMemcpyToSymbol(icb::g_fb_trace, z, sizeof(z)) != cudaSuccess) return -1;
  }
  return 0;
}
#endif

// Scratch: delta fp32 [hq * T] and dq_acc fp32 [T * hq * hd] (zeroed here). dq/dk/dv point at the
// first element of each gradient inside rows of dqkv_stride elements (packed layout or separate).
// dropout_p / dropout_seed: the values the forward pass was given (the mask is recomputed, never stored).
ICB_API int icb_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out,
                          const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_acc, int batch,
                          int seq_len, long long total_tokens, int hq, int hkv, int hd, long long q_stride,
                          long long kv_stride, long long dq_stride, long long dkv_stride, const int* cu_seqlens,
                          int causal, float scale, int dtype, int* status, void* stream_, float dropout_p,
                          const unsigned long long* dropout_seed) {
  if (hd != 64 && hd != 128) return -2;
  if (hq % hkv != 0) return -3;
  if (batch <= 0 || seq_len <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool bf16 = dtype == kBF16;
  {
    const long long warps = total_tokens * hq;
    const int th = 256;
    const long long blocks = (warps * 32 + th - 1) / th;
    if (bf16)
      flash_delta_kernel<true><<<(unsigned)blocks, th, 0, stream>>>(reinterpret_cast<const uint16_t*>(dout),
                                                                   reinterpret_cast<const uint16_t*>(out), delta,
                                                                   total_tokens, hq, hd);
    else
      flash_delta_kernel<false><<<(unsigned)blocks, th, 0, stream>>>(reinterpret_cast<const uint16_t*>(dout),
                                                                    reinterpret_cast<const uint16_t*>(out), delta,
                                                                    total_tokens, hq, hd);
    int rc = check_launch("flash_delta");
    if (rc) return rc;
  }
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)total_tokens * hq * hd * sizeof(float), stream);
  if (e != cudaSuccess) return -(int)e;

  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ;
  int rc = make_head_tmap(&tmQ, q, hd, hq, total_tokens, q_stride, dtype);
  if (rc) return rc;
  rc = make_head_tmap(&tmK, k, hd, hkv, total_tokens, kv_stride, dtype);
  if (rc) return rc;
  rc = make_head_tmap(&tmV, v, hd, hkv, total_tokens, kv_stride, dtype);
  if (rc) return rc;
  rc = make_head_tmap(&tmDO, dout, hd, hq, total_tokens, (long long)hq * hd, dtype);
  if (rc) return rc;
  {
    // fp32 accumulator [T, hq, hd] seen as (hd, hq, T); boxes of 32 floats (one 128-byte swizzle row) x 128 tokens
    uint64_t dims[3] = {(uint64_t)hd, (uint64_t)hq, (uint64_t)total_tokens};
    uint64_t str[2] = {(uint64_t)hd * 4, (uint64_t)hq * hd * 4};
    uint32_t box[3] = {32, 1, 128};
    rc = make_tmap(&tmDQ, kF32, 3, dq_acc, dims, str, box, true);
    if (rc) return rc;
  }
  FlashBwdArgs a;
  a.batch = batch; a.seq_len = seq_len; a.hq = hq; a.hkv = hkv;
  a.cu_seqlens = cu_seqlens;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dk = dk; a.dv = dv; a.dkv_stride = dkv_stride;
  a.total_tokens = total_tokens;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.in_fmt = bf16 ? 1 : 0;
  a.status = status;
  a.drop_thr = icb_dropout_threshold(dropout_p);
  if (a.drop_thr > 0 && dropout_seed == nullptr) return -4;
  a.drop_seed = dropout_seed;
  a.drop_scale = 256.0f / (256 - a.drop_thr);
  dim3 grid((seq_len + 127) / 128, hkv, batch);
  rc = (hd == 64) ? launch_flash_bwd<64>(tmQ, tmK, tmV, tmDO, tmDQ, a, grid, stream)
                  : launch_flash_bwd<128>(tmQ, tmK, tmV, tmDO, tmDQ, a, grid, stream);
  if (rc) return rc;
  {
    const int width = hq * hd;
    const long long n = total_tokens * (width / 8);
    const int th = 256;
    const long long blocks = (n + th - 1) / th;
    if (bf16)
      flash_dq_convert_kernel<true><<<(unsigned)blocks, th, 0, stream>>>(dq_acc, reinterpret_cast<uint16_t*>(dq),
                                                                        total_tokens, width, dq_stride, scale);
    else
      flash_dq_convert_kernel<false><<<(unsigned)blocks, th, 0, stream>>>(dq_acc, reinterpret_cast<uint16_t*>(dq),
                                                                         total_tokens, width, dq_stride, scale);
  }
  return check_launch("flash_dq_convert");
}
