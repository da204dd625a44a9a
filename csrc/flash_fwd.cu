// Flash attention forward for sm_100a: causal / full, GQA, optional document
// boundaries (cu_seqlens), head_dim 64 or 128, bf16 or fp16.
//
// One CTA owns 128 query rows of one head. Warp 0 streams K and V tiles (128 rows)
// with TMA into 2-stage rings, warp 1 issues tcgen05.mma for S = Q K^T (TMEM,
// double buffered) and O += P V (TMEM accumulator), warps 2-5 hold one query row per
// thread (TMEM lane == row, so row max / row sum need no shuffles): they read S with
// tcgen05.ld, apply the mask and the online softmax in the exp2 domain, and write P
// (bf16) into a 128-byte-swizzled shared-memory tile that feeds the second MMA.
// S_{j+1} is issued before P_j V_j, so the tensor core computes the next score tile
// while the softmax of the current one runs. The accumulator is only rescaled when
// the running max grows by more than 2^8 (exact: the final normalisation uses the
// same reference max), which keeps TMEM read-modify-write off the steady state.
// Two tilings: BN = 128 key rows per step with one CTA per SM (double-buffered P), and BN = 64 with two
// CTAs per SM (half the shared memory and TMEM each, single P buffer): two independent pipelines per SM
// give every warp scheduler two softmax warps, which hides the latency of the row-wise exp / max / sum
// chain that one warp per scheduler cannot.
// Every wait is bounded; on timeout the status word is set and the CTA drains.
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kFaThreads = 192;

struct FlashFwdArgs {
  int batch, seq_len, hq, hkv;        // seq_len: tokens per sequence (max when cu_seqlens is used)
  const int* cu_seqlens;              // [batch + 1] or null (then sequence b spans [b*seq_len, (b+1)*seq_len))
  void* out;                          // [T, hq, HD]
  float* lse;                         // [hq, T] natural-log sum-exp
  long long total_tokens;
  float scale_log2;                   // softmax scale * log2(e)
  int causal;
  int in_fmt;                         // 1 bf16, 0 fp16
  int* status;
  const unsigned long long* drop_seed;  // device word; read when drop_thr > 0
  int drop_thr;                       // keep a probability when its hash byte >= drop_thr (0: no dropout)
  float drop_scale;                   // 256 / (256 - drop_thr)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD, int BN>
struct FaSmem {
  static constexpr int kChunks = HD / 64;            // 64-element (128 B) column chunks per row
  static constexpr int kPStages = BN == 128 ? 2 : 1;
  static constexpr int q_bytes = 128 * HD * 2;
  static constexpr int kv_bytes = BN * HD * 2;
  static constexpr int kv_chunk = BN * 128;          // bytes of one 64-column chunk of a K / V tile
  static constexpr int p_bytes = 128 * BN * 2;
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + q_bytes;
  static constexpr int v_off = k_off + 2 * kv_bytes;
  static constexpr int p_off = v_off + 2 * kv_bytes;
  static constexpr int bar_off = p_off + kPStages * p_bytes;
  // BN = 128: manual 1 KiB alignment slack. BN = 64: the declaration is 1 KiB aligned (checked in the
  // kernel), so that two CTAs fit into one SM's shared memory.
  static constexpr int total = bar_off + 256 + (BN == 128 ? 1024 : 0);
  static constexpr int tmem_cols = BN == 128 ? 512 : 256;
  static constexpr int tmem_o = 2 * BN;
};

template <int HD, int BN>
__global__ void __launch_bounds__(kFaThreads, BN == 128 ? 1 : 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashFwdArgs args) {
  using L = FaSmem<HD, BN>;
  constexpr int PS = L::kPStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (BN != 128 && smem != smem_raw) {
    // the two-CTA layout has no room for alignment slack
    if (threadIdx.x == 0 && args.status != nullptr) atomicCAS(args.status, 0, kBadArgument);
    return;
  }
  uint8_t* sQ = smem + L::q_off;
  uint8_t* sK = smem + L::k_off;
  uint8_t* sV = smem + L::v_off;
  uint8_t* sP = smem + L::p_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2
  uint64_t* p_full = bars + 13;       // 2
  uint64_t* p_empty = bars + 15;      // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int kv_head = head / (args.hq / args.hkv);

  int seq_start, seq_len;
  if (args.cu_seqlens != nullptr) {
    seq_start = args.cu_seqlens[b];
    seq_len = args.cu_seqlens[b + 1] - seq_start;
  } else {
    seq_start = b * args.seq_len;
    seq_len = args.seq_len;
  }
  const int num_q_tiles = (seq_len + 127) >> 7;
  // heaviest (latest) query tiles first
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
  if (qt >= num_q_tiles) return;
  const int q0 = qt * 128;
  const int n_kv_total = (seq_len + BN - 1) / BN;
  const int n_kv = args.causal ? min((q0 + 128 + BN - 1) / BN, n_kv_total) : n_kv_total;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&p_empty[i], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + L::tmem_o;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, L::q_bytes);
#pragma unroll
      for (int c = 0; c < L::kChunks; ++c) tma_load_3d(sQ + c * 16384, &tmQ, q_full, c * 64, head, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int t0 = seq_start + j * BN;
        mbar_wait(&k_empty[s], ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
        mbar_expect_tx(&k_full[s], L::kv_bytes);
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_3d(sK + s * L::kv_bytes + c * L::kv_chunk, &tmK, &k_full[s], c * 64, kv_head, t0);
        mbar_wait(&v_empty[s], ph ^ 1, abort_flag, args.status, kTimeoutSmemEmpty);
        mbar_expect_tx(&v_full[s], L::kv_bytes);
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_3d(sV + s * L::kv_bytes + c * L::kv_chunk, &tmV, &v_full[s], c * 64, kv_head, t0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(128, BN, args.in_fmt, 0, 0);
      const uint32_t idesc_pv = umma_idesc(128, HD, args.in_fmt, 0, 1);
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t k_addr = smem_u32(sK + s * L::kv_bytes);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t q_off = (k >> 2) * 16384 + (k & 3) * 32;
          const uint32_t k_off = (k >> 2) * L::kv_chunk + (k & 3) * 32;
          umma_ss(tmem_base + s * BN, umma_desc_sw128(q_addr + q_off, 16, 1024),
                  umma_desc_sw128(k_addr + k_off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
      };
      mbar_wait(q_full, 0, abort_flag, args.status, kTimeoutSmemFull);
      mbar_wait(&k_full[0], 0, abort_flag, args.status, kTimeoutSmemFull);
      tc_fence_after();
      issue_s(0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) & 1;
          const uint32_t ph1 = ((j + 1) >> 1) & 1;
          mbar_wait(&k_full[s1], ph1, abort_flag, args.status, kTimeoutSmemFull);
          if (j + 1 >= 2) mbar_wait(&s_empty[s1], ph1 ^ 1, abort_flag, args.status, kTimeoutTmemEmpty);
          tc_fence_after();
          issue_s(j + 1);
        }
        const int sp = j % PS;
        const uint32_t php = (j / PS) & 1;
        mbar_wait(&v_full[s], ph, abort_flag, args.status, kTimeoutSmemFull);
        mbar_wait(&p_full[sp], php, abort_flag, args.status, kTimeoutLocalFlag);
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP + sp * L::p_bytes);
        const uint32_t v_addr = smem_u32(sV + s * L::kv_bytes);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t adesc = umma_desc_sw128(p_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = umma_desc_sw128(v_addr + k * 2048, L::kv_chunk, 1024);
          umma_ss(tmem_o, adesc, bdesc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&p_empty[sp]);
        umma_commit(&v_empty[s]);
      }
    }
    __syncwarp();
  } else {
    // ----------------------------- softmax / correction / epilogue -----------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int q_idx = q0 + row;  // position inside the sequence
    float m_ref = -INFINITY;     // reference max (log2 domain, scaled)
    float l_sum = 0.f;
    const bool dropout = args.drop_thr > 0;
    const unsigned long long drop_key = dropout ? *args.drop_seed : 0ull;
    const unsigned long long drop_row = dropout_row_counter(b, args.hq, head, args.seq_len, q_idx);
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      mbar_wait(&s_full[s], ph, abort_flag, args.status, kTimeoutTmemFull);
      tc_fence_after();
      constexpr int NC = BN / 32;
      uint32_t r[NC][32];
#pragma unroll
      for (int c = 0; c < NC; ++c) tmem_ld_32x32(tmem_base + lane_off + s * BN + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[s]);
      const int kv0 = j * BN;
      const bool need_mask = (args.causal && kv0 + BN > q0) || (kv0 + BN > seq_len);
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(r[c][i]) * args.scale_log2;
          if (need_mask) {
            const int kv_idx = kv0 + c * 32 + i;
            if (kv_idx >= seq_len || (args.causal && kv_idx > q_idx)) x = -INFINITY;
          }
          r[c][i] = __float_as_uint(x);
          m_tile = fmaxf(m_tile, x);
        }
      }
      float m_new = fmaxf(m_ref, m_tile);
      if (m_new == -INFINITY) m_new = 0.f;
      const bool grow = m_new > m_ref + 8.0f;
      const unsigned any_grow = __ballot_sync(0xffffffffu, grow);
      if (any_grow) {
        const float factor = grow ? fast_exp2(m_ref - m_new) : 1.0f;
        if (grow) {
          l_sum *= factor;
          m_ref = m_new;
        }
        if (j > 0) {
          // the accumulator must be complete up to P_{j-1} V_{j-1} before it is rescaled
          const int spp = (j - 1) % PS;
          mbar_wait(&p_empty[spp], ((j - 1) / PS) & 1, abort_flag, args.status, kTimeoutTmemFull);
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32(tmem_o + lane_off + c * 32, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
      }
      // P buffer sp was last read by P_{j-PS} V_{j-PS}
      const int sp = j % PS;
      const uint32_t php = (j / PS) & 1;
      if (j >= PS) mbar_wait(&p_empty[sp], php ^ 1, abort_flag, args.status, kTimeoutLocalFlag);
      uint8_t* prow = sP + sp * L::p_bytes + row * 128;
      float lsum_tile = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            p[i] = fast_exp2(__uint_as_float(r[c][g * 8 + i]) - m_ref);
            lsum_tile += p[i];
          }
          if (dropout) {
            // the row sum keeps every probability (softmax first, dropout second); only P V sees the mask
            const unsigned long long h = dropout_hash(drop_key, drop_row + (unsigned)((kv0 + c * 32 + g * 8) >> 3));
#pragma unroll
            for (int i = 0; i < 8; ++i)
              p[i] = (int)((h >> (8 * i)) & 0xffull) >= args.drop_thr ? p[i] * args.drop_scale : 0.f;
          }
          uint4 u;
          if (args.in_fmt == 1) {
            u.x = pack_bf16x2(p[0], p[1]); u.y = pack_bf16x2(p[2], p[3]);
            u.z = pack_bf16x2(p[4], p[5]); u.w = pack_bf16x2(p[6], p[7]);
          } else {
            u.x = pack_f16x2(p[0], p[1]); u.y = pack_f16x2(p[2], p[3]);
            u.z = pack_f16x2(p[4], p[5]); u.w = pack_f16x2(p[6], p[7]);
          }
          const int col = c * 32 + g * 8;          // first kv column of this 16-byte piece
          const int chunk = col >> 6;              // 64-column chunk (16 KiB each)
          const int piece = (col & 63) >> 3;       // 16-byte piece inside the 128-byte row
          *reinterpret_cast<uint4*>(prow + chunk * 16384 + ((piece ^ (row & 7)) << 4)) = u;
        }
      }
      l_sum += lsum_tile;
      fence_proxy_async_smem();
      mbar_arrive(&p_full[sp]);
    }
    // ---- epilogue: O / l, log-sum-exp ----
    {
      const int last = n_kv - 1;
      mbar_wait(&p_empty[last % PS], (last / PS) & 1, abort_flag, args.status, kTimeoutTmemFull);
      tc_fence_after();
      const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      const bool valid = q_idx < seq_len;
      const long long tok = (long long)seq_start + q_idx;
      uint8_t* orow = reinterpret_cast<uint8_t*>(args.out) + ((size_t)tok * args.hq + head) * HD * 2;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_off + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[g * 8 + i]) * inv_l;
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
      if (valid) args.lse[(size_t)head * args.total_tokens + tok] = (m_ref + log2f(l_sum)) * 0.6931471805599453f;
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
    tmem_dealloc(tmem_base, L::tmem_cols);
  }
}

template <int HD, int BN>
static int launch_flash_fwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                            const FlashFwdArgs& args, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  auto kern = flash_fwd_kernel<HD, BN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSmem<HD, BN>::total);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  kern<<<grid, kFaThreads, FaSmem<HD, BN>::total, stream>>>(tmQ, tmK, tmV, args);
  return check_launch("flash_fwd_kernel");
}

// 3-D view (head_dim, heads, tokens) of a [T, row_stride] matrix whose heads start at `base`.
int make_head_tmap_rows(CUtensorMap* tm, const void* base, int hd, int heads, long long tokens, long long row_stride,
                        int dtype, int box_rows) {
  uint64_t dims[3] = {(uint64_t)hd, (uint64_t)heads, (uint64_t)tokens};
  uint64_t str[2] = {(uint64_t)hd * 2, (uint64_t)row_stride * 2};
  uint32_t box[3] = {64, 1, (uint32_t)box_rows};
  return make_tmap(tm, dtype, 3, base, dims, str, box, true);
}
int make_head_tmap(CUtensorMap* tm, const void* base, int hd, int heads, long long tokens, long long row_stride,
                   int dtype) {
  return make_head_tmap_rows(tm, base, hd, heads, tokens, row_stride, dtype, 128);
}

// Key rows per step: 64 (two CTAs per SM; measured 0.270 ms against 0.452 ms for 128 rows with one CTA per SM
// at s = 4096, 32 heads x 128). `wide` selects the 128-row tiling.
static int flash_fwd_bn(int wide) { return wide ? 128 : 64; }

}  // namespace icb

using namespace icb;

// q/k/v: first element of each operand inside rows of `row_stride` elements (packed qkv or separate
// tensors). out: [T, hq, hd] contiguous. lse: [hq, T] fp32. cu_seqlens (optional, device int32
// [batch + 1]) gives document boundaries in the flat token stream; seq_len is then the maximum length.
// dropout_p > 0 drops attention probabilities with probability round(256 p) / 256 under the mask that the
// device word *dropout_seed selects (the backward pass must be given the same word).
ICB_API int icb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int seq_len,
                          long long total_tokens, int hq, int hkv, int hd, long long q_stride, long long kv_stride,
                          const int* cu_seqlens, int causal, float scale, int dtype, int* status, void* stream_,
                          float dropout_p, const unsigned long long* dropout_seed, int wide) {
  if (hd != 64 && hd != 128) return -2;
  if (hq % hkv != 0) return -3;
  if (batch <= 0 || seq_len <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_head_tmap(&tmQ, q, hd, hq, total_tokens, q_stride, dtype);
  if (rc) return rc;
  const int bn = flash_fwd_bn(wide);
  rc = make_head_tmap_rows(&tmK, k, hd, hkv, total_tokens, kv_stride, dtype, bn);
  if (rc) return rc;
  rc = make_head_tmap_rows(&tmV, v, hd, hkv, total_tokens, kv_stride, dtype, bn);
  if (rc) return rc;
  FlashFwdArgs a;
  a.batch = batch; a.seq_len = seq_len; a.hq = hq; a.hkv = hkv;
  a.cu_seqlens = cu_seqlens;
  a.out = out; a.lse = lse; a.total_tokens = total_tokens;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.in_fmt = (dtype == kBF16) ? 1 : 0;
  a.status = status;
  a.drop_thr = icb_dropout_threshold(dropout_p);
  if (a.drop_thr > 0 && dropout_seed == nullptr) return -4;
  a.drop_seed = dropout_seed;
  a.drop_scale = 256.0f / (256 - a.drop_thr);
  dim3 grid((seq_len + 127) / 128, hq, batch);
  if (bn == 64) {
    if (hd == 64) return launch_flash_fwd<64, 64>(tmQ, tmK, tmV, a, grid, stream);
    return launch_flash_fwd<128, 64>(tmQ, tmK, tmV, a, grid, stream);
  }
  if (hd == 64) return launch_flash_fwd<64, 128>(tmQ, tmK, tmV, a, grid, stream);
  return launch_flash_fwd<128, 128>(tmQ, tmK, tmV, a, grid, stream);
}
