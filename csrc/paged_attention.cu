// Block (paged) KV cache kernels for rollout / decode on sm_100a.
//
// Cache layout per layer: k_cache, v_cache [num_blocks, block_size, hkv, hd] (16-bit);
// block_table [num_seqs, max_blocks] int32 maps a sequence's logical page to a physical block.
//
//  * kv_append      : scatter the new tokens' K / V rows (already rotated) into their slots.
//  * paged_decode   : one query token per sequence. A CTA owns (sequence, kv head) and serves the
//                     whole GQA group from one pass over that head's pages, so K and V are read once
//                     per group (decode is bound by KV bytes, not FLOPs). Each warp walks pages with
//                     an online softmax (two lanes per token for the q.k dot products, four output
//                     dims per lane for p.V), and the eight warps are merged through shared memory.
//                     All loads of a 16-token step (the K half rows, then the 16 V rows) are issued
//                     before they are consumed: a warp owns only a few steps, so the kernel is bound
//                     by load latency unless a step keeps many loads in flight.
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

template <bool BF16>
__device__ __forceinline__ float cvt16(uint16_t v) {
  if (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v));
  return __half2float(*reinterpret_cast<const __half*>(&v));
}

// k, v: [T, hkv*hd] rows with pitch `stride`; slot[t] = block * block_size + offset (or < 0 to skip)
__global__ void kv_append_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                                 uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                                 const long long* __restrict__ slots, int T, int row_elems, long long k_stride,
                                 long long v_stride) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const long long slot = slots[t];
  if (slot < 0) return;
  const int nvec = row_elems >> 3;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 a = *reinterpret_cast<const uint4*>(k + (size_t)t * k_stride + i * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(v + (size_t)t * v_stride + i * 8);
    *reinterpret_cast<uint4*>(k_cache + (size_t)slot * row_elems + i * 8) = a;
    *reinterpret_cast<uint4*>(v_cache + (size_t)slot * row_elems + i * 8) = b;
  }
}

constexpr int kPdWarps = 8;
constexpr int kPdMaxGroup = 8;

template <int HD, bool BF16>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_kernel(const uint16_t* __restrict__ q, long long q_stride, const uint16_t* __restrict__ k_cache,
                    const uint16_t* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, uint16_t* __restrict__ out, float* __restrict__ lse_out,
                    int hq, int hkv, int block_size, int max_blocks, float scale) {
  constexpr int HALF = HD / 2;       // elements of a K row handled by one of the two lanes of a token
  constexpr int OD = HD / 32;        // output dims owned by one lane
  const int seq = blockIdx.x;
  const int kvh = blockIdx.y;
  const int G = hq / hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = seq_lens[seq];
  __shared__ float sq[kPdMaxGroup][HD];
  __shared__ float sm_m[kPdWarps][kPdMaxGroup], sm_l[kPdWarps][kPdMaxGroup];
  __shared__ float sm_o[kPdWarps][kPdMaxGroup][HD];
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    const int g = i / HD, d = i - g * HD;
    sq[g][d] = cvt16<BF16>(q[(size_t)seq * q_stride + (size_t)(kvh * G + g) * HD + d]) * scale;
  }
  __syncthreads();
  float m[kPdMaxGroup], l[kPdMaxGroup], o[kPdMaxGroup][OD];
#pragma unroll
  for (int g = 0; g < kPdMaxGroup; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < OD; ++d) o[g][d] = 0.f;
  }
  const int row_elems = hkv * HD;
  const int tok_in_pair = lane >> 1;        // token handled by this lane pair (16 per step)
  const int half = lane & 1;
  const int n_pages = (ctx + block_size - 1) / block_size;
  // a "step" covers 16 consecutive tokens; block_size is a multiple of 16
  const int steps_per_page = block_size / 16;
  for (int step = warp; step < n_pages * steps_per_page; step += kPdWarps) {
    const int page = step / steps_per_page;
    const int blk = block_table[(size_t)seq * max_blocks + page];
    const int tok0 = page * block_size + (step - page * steps_per_page) * 16;
    const int in_blk0 = tok0 - page * block_size;
    // ---- the step's 16 V rows (4 output dims per lane) are requested before anything is computed ----
    const int n_tok = min(16, ctx - tok0);
    const uint16_t* vbase = v_cache + ((size_t)blk * block_size + in_blk0) * row_elems + kvh * HD + lane * OD;
    uint2 vu[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      vu[t] = make_uint2(0u, 0u);
      if (t < n_tok) {
        if (OD == 4) vu[t] = *reinterpret_cast<const uint2*>(vbase + (size_t)t * row_elems);
        else vu[t].x = *reinterpret_cast<const uint32_t*>(vbase + (size_t)t * row_elems);
      }
    }
    // ---- scores for 16 tokens x G heads ----
    const int my_tok = tok0 + tok_in_pair;
    const bool tok_ok = my_tok < ctx;
    float s[kPdMaxGroup];
#pragma unroll
    for (int g = 0; g < kPdMaxGroup; ++g) s[g] = 0.f;
    if (tok_ok) {
      const uint16_t* kr = k_cache + ((size_t)blk * block_size + in_blk0 + tok_in_pair) * row_elems + kvh * HD + half * HALF;
      uint4 ku[HALF / 8];
#pragma unroll
      for (int c = 0; c < HALF / 8; ++c) ku[c] = *reinterpret_cast<const uint4*>(kr + c * 8);
#pragma unroll
      for (int c = 0; c < HALF / 8; ++c) {
        const uint32_t w[4] = {ku[c].x, ku[c].y, ku[c].z, ku[c].w};
        float kf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = BF16 ? unpack_bf16x2(w[i]) : __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          kf[2 * i] = f.x; kf[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < kPdMaxGroup; ++g) {
          if (g < G) {
            const float* qg = &sq[g][half * HALF + c * 8];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[g] += kf[i] * qg[i];
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kPdMaxGroup; ++g) {
      if (g < G) {
        s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
        if (!tok_ok) s[g] = -INFINITY;
      }
    }
    // ---- online softmax per head over these 16 tokens ----
    float p[kPdMaxGroup];
#pragma unroll
    for (int g = 0; g < kPdMaxGroup; ++g) {
      if (g < G) {
        float mx = s[g];
#pragma unroll
        for (int off = 16; off >= 2; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_new = fmaxf(m[g], mx);
        const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
        p[g] = (s[g] == -INFINITY) ? 0.f : __expf(s[g] - m_new);
        float ps = (half == 0) ? p[g] : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        l[g] = l[g] * corr + ps;
        m[g] = m_new;
#pragma unroll
        for (int d = 0; d < OD; ++d) o[g][d] *= corr;
      }
    }
    // ---- O += P V : lane owns OD output dims of the 16 rows fetched above ----
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      float vf[OD];
      if (OD == 4) {
        float2 a = BF16 ? unpack_bf16x2(vu[t].x) : __half22float2(*reinterpret_cast<const __half2*>(&vu[t].x));
        float2 b = BF16 ? unpack_bf16x2(vu[t].y) : __half22float2(*reinterpret_cast<const __half2*>(&vu[t].y));
        vf[0] = a.x; vf[1] = a.y; vf[2 % OD] = b.x; vf[3 % OD] = b.y;
      } else {
        float2 a = BF16 ? unpack_bf16x2(vu[t].x) : __half22float2(*reinterpret_cast<const __half2*>(&vu[t].x));
        vf[0] = a.x; vf[1 % OD] = a.y;
      }
#pragma unroll
      for (int g = 0; g < kPdMaxGroup; ++g) {
        if (g < G) {
          const float pt = __shfl_sync(0xffffffffu, p[g], 2 * t);   // 0 for tokens past the context
#pragma unroll
          for (int d = 0; d < OD; ++d) o[g][d] += pt * vf[d];
        }
      }
    }
  }
  // ---- merge the warps ----
#pragma unroll
  for (int g = 0; g < kPdMaxGroup; ++g) {
    if (g < G) {
      if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
      for (int d = 0; d < OD; ++d) sm_o[warp][g][lane * OD + d] = o[g][d];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    const int g = i / HD, d = i - g * HD;
    float mm = -INFINITY;
    for (int w = 0; w < kPdWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, acc = 0.f;
    for (int w = 0; w < kPdWarps; ++w) {
      const float c = (sm_m[w][g] == -INFINITY) ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      acc += sm_o[w][g][d] * c;
    }
    const float val = ll > 0.f ? acc / ll : 0.f;
    const size_t oi = ((size_t)seq * hq + kvh * G + g) * HD + d;
    if (BF16) reinterpret_cast<__nv_bfloat16*>(out)[oi] = __float2bfloat16(val);
    else reinterpret_cast<__half*>(out)[oi] = __float2half(val);
    if (d == 0 && lse_out != nullptr) lse_out[(size_t)seq * hq + kvh * G + g] = mm + logf(fmaxf(ll, 1e-30f));
  }
}


// ---------------------------------------------------------------------------------------------------------
// Tensor-core form of paged_decode (head_dim 128). The scalar kernel above issues about 2800 instructions per
// warp for every 16 tokens and is bound by instruction issue (ncu: 22 % issue slots busy with 2 warps per
// scheduler, 0.6 TB/s of KV traffic). Here the GQA group (at most 8 query heads) is the M dimension of
// mma.sync.m16n8k16 (rows 8..15 are padding): S = Q K^T and O += P V for 16 tokens take 32 MMAs, and every
// operand is fetched with 16-byte loads straight into its fragment:
//   * Q K^T: the contraction index is the head dimension, whose order inside a 32-element group is free as long
//     as Q and K use the same one; thread (r, c) of a warp takes elements [32 g + 8 c, 32 g + 8 c + 8) of K row
//     r (token) and of Q row r (head), which fills b0, b1 / a0, a2 of two consecutive k-steps.
//   * P V: thread (r, c) needs V[token][col] for tokens {2c, 2c+1, 2c+8, 2c+9} of the step and one column per
//     8-column output tile; the output columns are assigned as col = 16 r + tile, so those are 32 contiguous
//     bytes per token, and the pairs of tokens are interleaved into b0 / b1 with one byte permute per tile.
// Grid (sequence, kv head, split): a split owns a contiguous range of 16-token steps; with more than one split
// the partial (max, sum, unnormalised output) records go to scratch and paged_decode_merge_kernel combines them.
// ---------------------------------------------------------------------------------------------------------
constexpr int kPmWarps = 4;

template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if (BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  return BF16 ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
}

template <bool BF16>
__global__ void __launch_bounds__(kPmWarps * 32)
paged_decode_mma_kernel(const uint16_t* __restrict__ q, long long q_stride, const uint16_t* __restrict__ k_cache,
                        const uint16_t* __restrict__ v_cache, const int* __restrict__ block_table,
                        const int* __restrict__ seq_lens, uint16_t* __restrict__ out, float* __restrict__ lse_out,
                        float* __restrict__ part, int hq, int hkv, int block_size, int max_blocks, float scale,
                        int nsplit) {
  constexpr int HD = 128;
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = hq / hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int ctx = seq_lens[seq];
  const int row_elems = hkv * HD;
  const int total_steps = (ctx + 15) >> 4;
  const int steps_per_split = (total_steps + nsplit - 1) / nsplit;
  const int step_begin = split * steps_per_split;
  const int step_end = min(total_steps, step_begin + steps_per_split);

  // Q fragments of head r (zero for the padding rows)
  uint32_t qa[4][4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (r < G) u = *reinterpret_cast<const uint4*>(q + (size_t)seq * q_stride + (size_t)(kvh * G + r) * HD + g * 32 + c * 8);
    qa[g][0] = u.x; qa[g][1] = u.y; qa[g][2] = u.z; qa[g][3] = u.w;
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m = -INFINITY, l = 0.f;       // running max of row r (uniform over the 4 lanes of the row), partial sum

  for (int step = step_begin + warp; step < step_end; step += kPmWarps) {
    const int tok0 = step << 4;
    const int page = tok0 / block_size;
    const int blk = block_table[(size_t)seq * max_blocks + page];
    const size_t row0 = (size_t)blk * block_size + (tok0 - page * block_size);   // cache row of the step's first token
    // ---- K: rows (tokens) r and r + 8 of the step, this lane's 8-element slices; V: four token rows, 16 columns
    uint4 ku[2][4], vu[4][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint16_t* kr = k_cache + (row0 + j * 8 + r) * row_elems + kvh * HD + c * 8;
#pragma unroll
      for (int g = 0; g < 4; ++g) ku[j][g] = *reinterpret_cast<const uint4*>(kr + g * 32);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int tk = 2 * c + (t & 1) + (t >> 1) * 8;          // tokens 2c, 2c+1, 2c+8, 2c+9 of the step
      const uint16_t* vr = v_cache + (row0 + tk) * row_elems + kvh * HD + r * 16;
      if (tok0 + tk < ctx) {
        vu[t][0] = *reinterpret_cast<const uint4*>(vr);
        vu[t][1] = *reinterpret_cast<const uint4*>(vr + 8);
      } else {
        vu[t][0] = vu[t][1] = make_uint4(0u, 0u, 0u, 0u);      // never multiply a stale row, even by zero
      }
    }
    // ---- S = Q K^T for two 8-token tiles
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        mma_16816<BF16>(sc[j], qa[g][0], 0u, qa[g][1], 0u, ku[j][g].x, ku[j][g].y);
        mma_16816<BF16>(sc[j], qa[g][2], 0u, qa[g][3], 0u, ku[j][g].z, ku[j][g].w);
      }
    }
    // ---- online softmax of row r: this lane holds tokens j * 8 + 2c, + 1
    float p[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tk = tok0 + j * 8 + 2 * c + e;
        p[j][e] = tk < ctx ? sc[j][e] * scale : -INFINITY;
        mx = fmaxf(mx, p[j][e]);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
    float ps = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[j][e] = (p[j][e] == -INFINITY) ? 0.f : __expf(p[j][e] - m_new);
        ps += p[j][e];
      }
    }
    l = l * corr + ps;
    m = m_new;
    const uint32_t pa0 = pack16x2<BF16>(p[0][0], p[0][1]);     // k slots 2c, 2c+1   (tokens 2c, 2c+1)
    const uint32_t pa2 = pack16x2<BF16>(p[1][0], p[1][1]);     // k slots 2c+8, 2c+9 (tokens 2c+8, 2c+9)
    // ---- O = O * corr + P V over 16 output tiles (column 16 r' + i of tile i belongs to B lane group r')
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int w = i >> 1;
      const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
      const uint32_t* v0 = reinterpret_cast<const uint32_t*>(&vu[0][0]);
      const uint32_t* v1 = reinterpret_cast<const uint32_t*>(&vu[1][0]);
      const uint32_t* v2 = reinterpret_cast<const uint32_t*>(&vu[2][0]);
      const uint32_t* v3 = reinterpret_cast<const uint32_t*>(&vu[3][0]);
      const uint32_t b0 = __byte_perm(v0[w], v1[w], sel);
      const uint32_t b1 = __byte_perm(v2[w], v3[w], sel);
      o[i][0] *= corr; o[i][1] *= corr;
      mma_16816<BF16>(o[i], pa0, 0u, pa2, 0u, b0, b1);
    }
  }
  // ---- merge the warps of the CTA: row r's (m, l) and its 128 output values
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  __shared__ float sm_m[kPmWarps][8], sm_l[kPmWarps][8];
  __shared__ float sm_o[kPmWarps][8][HD];
  if (c == 0) { sm_m[warp][r] = m; sm_l[warp][r] = l; }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    sm_o[warp][r][(2 * c) * 16 + i] = o[i][0];
    sm_o[warp][r][(2 * c + 1) * 16 + i] = o[i][1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, d = idx - g * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPmWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kPmWarps; ++w) {
      const float f = (sm_m[w][g] == -INFINITY) ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * f;
      acc += sm_o[w][g][d] * f;
    }
    const int head = kvh * G + g;
    if (nsplit == 1) {
      const float val = ll > 0.f ? acc / ll : 0.f;
      const size_t oi = ((size_t)seq * hq + head) * HD + d;
      if (BF16) reinterpret_cast<__nv_bfloat16*>(out)[oi] = __float2bfloat16(val);
      else reinterpret_cast<__half*>(out)[oi] = __float2half(val);
      if (d == 0 && lse_out != nullptr) lse_out[(size_t)seq * hq + head] = mm + logf(fmaxf(ll, 1e-30f));
    } else {
      // partial record of (seq, head, split): [HD] unnormalised output, then max and sum
      float* rec = part + (((size_t)seq * hq + head) * nsplit + split) * (HD + 2);
      rec[d] = acc;
      if (d == 0) { rec[HD] = mm; rec[HD + 1] = ll; }
    }
  }
}

template <bool BF16>
__global__ void paged_decode_merge_kernel(const float* __restrict__ part, uint16_t* __restrict__ out,
                                          float* __restrict__ lse_out, int nsplit) {
  constexpr int HD = 128;
  const size_t row = blockIdx.x;                 // seq * hq + head
  const int d = threadIdx.x;                     // 128 threads
  const float* rec = part + row * nsplit * (HD + 2);
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, rec[s * (HD + 2) + HD]);
  float ll = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = rec[s * (HD + 2) + HD];
    const float f = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += rec[s * (HD + 2) + HD + 1] * f;
    acc += rec[s * (HD + 2) + d] * f;
  }
  const float val = ll > 0.f ? acc / ll : 0.f;
  if (BF16) reinterpret_cast<__nv_bfloat16*>(out)[row * HD + d] = __float2bfloat16(val);
  else reinterpret_cast<__half*>(out)[row * HD + d] = __float2half(val);
  if (d == 0 && lse_out != nullptr) lse_out[row] = mm + logf(fmaxf(ll, 1e-30f));
}

}  // namespace icb

using namespace icb;

ICB_API int icb_kv_append(const void* k, const void* v, void* k_cache, void* v_cache, const long long* slots, int T,
                          int row_elems, long long k_stride, long long v_stride, void* stream) {
  if (T <= 0) return 0;
  if (row_elems % 8) return -2;
  kv_append_kernel<<<T, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint16_t*>(k), reinterpret_cast<const uint16_t*>(v), reinterpret_cast<uint16_t*>(k_cache),
      reinterpret_cast<uint16_t*>(v_cache), slots, T, row_elems, k_stride, v_stride);
  return check_launch("kv_append");
}

// q: [S, hq*hd] rows of pitch q_stride; out: [S, hq*hd]; lse (optional): [S, hq]. hq/hkv <= 8,
// block_size a multiple of 16, hd 64 or 128. scratch != null selects the tensor-core kernel (hd 128 only; q rows,
// cache rows 16-byte aligned): the context is cut into `nsplit` ranges handled by different CTAs, and scratch
// must hold num_seqs * hq * nsplit * (hd + 2) floats.
ICB_API int icb_paged_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                             const int* block_table, const int* seq_lens, void* out, float* lse, int num_seqs, int hq,
                             int hkv, int hd, int block_size, int max_blocks, float scale, int dtype, void* stream,
                             void* scratch, int nsplit) {
  if (num_seqs <= 0) return 0;
  if (hq % hkv || hq / hkv > kPdMaxGroup || block_size % 16) return -2;
  dim3 grid(num_seqs, hkv);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto Q = reinterpret_cast<const uint16_t*>(q);
  auto K = reinterpret_cast<const uint16_t*>(k_cache);
  auto V = reinterpret_cast<const uint16_t*>(v_cache);
  auto O = reinterpret_cast<uint16_t*>(out);
#define ICB_PD(HD_, BF_) \
  paged_decode_kernel<HD_, BF_><<<grid, kPdWarps * 32, 0, st>>>(Q, q_stride, K, V, block_table, seq_lens, O, lse, hq, \
                                                                 hkv, block_size, max_blocks, scale)
  if (hd == 128 && scratch != nullptr && nsplit >= 1) {
    // tensor-core kernel; `scratch` holds num_seqs * hq * nsplit records of hd + 2 floats (unused when nsplit == 1)
    dim3 g3(num_seqs, hkv, nsplit);
    if (dtype == kBF16) {
      paged_decode_mma_kernel<true><<<g3, kPmWarps * 32, 0, st>>>(Q, q_stride, K, V, block_table, seq_lens, O, lse,
                                                                 reinterpret_cast<float*>(scratch), hq, hkv, block_size,
                                                                 max_blocks, scale, nsplit);
      if (nsplit > 1)
        paged_decode_merge_kernel<true><<<num_seqs * hq, 128, 0, st>>>(reinterpret_cast<const float*>(scratch), O, lse,
                                                                       nsplit);
    } else {
      paged_decode_mma_kernel<false><<<g3, kPmWarps * 32, 0, st>>>(Q, q_stride, K, V, block_table, seq_lens, O, lse,
                                                                  reinterpret_cast<float*>(scratch), hq, hkv, block_size,
                                                                  max_blocks, scale, nsplit);
      if (nsplit > 1)
        paged_decode_merge_kernel<false><<<num_seqs * hq, 128, 0, st>>>(reinterpret_cast<const float*>(scratch), O, lse,
                                                                        nsplit);
    }
    return check_launch("paged_decode_mma");
  }
  if (hd == 128 && dtype == kBF16) ICB_PD(128, true);
  else if (hd == 128) ICB_PD(128, false);
  else if (hd == 64 && dtype == kBF16) ICB_PD(64, true);
  else if (hd == 64) ICB_PD(64, false);
  else return -3;
#undef ICB_PD
  return check_launch("paged_decode");
}
