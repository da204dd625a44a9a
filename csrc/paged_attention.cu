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
// block_size a multiple of 16, hd 64 or 128.
ICB_API int icb_paged_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                             const int* block_table, const int* seq_lens, void* out, float* lse, int num_seqs, int hq,
                             int hkv, int hd, int block_size, int max_blocks, float scale, int dtype, void* stream) {
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
  if (hd == 128 && dtype == kBF16) ICB_PD(128, true);
  else if (hd == 128) ICB_PD(128, false);
  else if (hd == 64 && dtype == kBF16) ICB_PD(64, true);
  else if (hd == 64) ICB_PD(64, false);
  else return -3;
#undef ICB_PD
  return check_launch("paged_decode");
}
