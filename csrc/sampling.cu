// Token sampling for rollout on sm_100a: one pass over a row of (vocabulary-sharded) logits yields the
// Gumbel-max sample and the softmax statistics of the row.
//
//   sample_gumbel_kernel : for every row r of logits[S, V] (16-bit or fp32, any row pitch), with x = logit / T:
//        best  = argmax_c ( x[c] - log(-log(u[r, c])) )      u uniform in (0, 1) from a counter-based hash
//        stats = { best perturbed value, x[best], max_c x[c], sum_c exp(x[c] - max) }
//     arg max of Gumbel-perturbed logits is an exact sample of softmax(x); under tensor parallelism every
//     rank runs the kernel on its shard (the hash is keyed by the global column) and the ranks combine
//     five scalars per row instead of gathering the vocabulary. Columns >= valid are ignored (padding).
//     The row is read once (16-byte loads); no [S, V] intermediate is written.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kSampleThreads = 256;

// splitmix64 finaliser: a bijective mix of the 64-bit counter; the top 24 bits give u in (0, 1)
__device__ __forceinline__ float uniform_from_counter(unsigned long long key) {
  key += 0x9E3779B97F4A7C15ull;
  key = (key ^ (key >> 30)) * 0xBF58476D1CE4E5B9ull;
  key = (key ^ (key >> 27)) * 0x94D049BB133111EBull;
  key ^= key >> 31;
  return (static_cast<float>(static_cast<uint32_t>(key >> 40)) + 0.5f) * (1.0f / 16777216.0f);
}

struct SampleAcc {
  float best, best_x, mx, sum;
  int idx;
};

__device__ __forceinline__ void sample_visit(SampleAcc& a, float x, int col, unsigned long long row_key,
                                             long long col0) {
  const float u = uniform_from_counter(row_key + static_cast<unsigned long long>(col0 + col));
  const float pert = x - __logf(-__logf(u));
  if (pert > a.best) { a.best = pert; a.best_x = x; a.idx = col; }
  if (x > a.mx) { a.sum = a.sum * __expf(a.mx - x) + 1.f; a.mx = x; }
  else a.sum += __expf(x - a.mx);
}

__device__ __forceinline__ void sample_merge(SampleAcc& a, const SampleAcc& b) {
  if (b.best > a.best || (b.best == a.best && b.idx < a.idx && b.idx >= 0)) {
    a.best = b.best; a.best_x = b.best_x; a.idx = b.idx;
  }
  const float m = fmaxf(a.mx, b.mx);
  const float sa = (a.mx == -INFINITY) ? 0.f : a.sum * __expf(a.mx - m);
  const float sb = (b.mx == -INFINITY) ? 0.f : b.sum * __expf(b.mx - m);
  a.sum = sa + sb;
  a.mx = m;
}

// FMT: 0 bf16, 1 fp16, 2 fp32. Grid (S, parts): CTA (r, p) scans columns [p * span, (p + 1) * span) of row r
// (span a multiple of 8) and writes one partial record; with parts == 1 the record is the result.
template <int FMT>
__global__ void __launch_bounds__(kSampleThreads)
sample_gumbel_kernel(const void* __restrict__ logits, long long row_stride, int V, int valid, float inv_temp,
                     unsigned long long seed, unsigned long long draw, long long col0, int span,
                     float* __restrict__ stats, int* __restrict__ index) {
  const int row = blockIdx.x;
  // one 2^24-wide counter range per (draw, row): columns never collide across rows or draws
  const unsigned long long row_key = seed * 0xD1342543DE82EF95ull + ((draw * gridDim.x + row) << 24);
  SampleAcc acc{-INFINITY, 0.f, -INFINITY, 0.f, -1};
  const int n = min(V, valid);
  const int c_begin = blockIdx.y * span;
  const int c_end = min(n, c_begin + span);
  if (FMT == 2) {
    const float* p = reinterpret_cast<const float*>(logits) + (size_t)row * row_stride;
    for (int c = c_begin + threadIdx.x; c < c_end; c += kSampleThreads)
      sample_visit(acc, p[c] * inv_temp, c, row_key, col0);
  } else {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(logits) + (size_t)row * row_stride;
    const bool vec = ((reinterpret_cast<uintptr_t>(p) & 15) == 0);
    const int v_begin = c_begin >> 3;
    const int v_end = vec ? max(v_begin, c_end >> 3) : v_begin;
    for (int i = v_begin + threadIdx.x; i < v_end; i += kSampleThreads) {
      const uint4 u = *reinterpret_cast<const uint4*>(p + i * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = FMT == 0 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
        sample_visit(acc, f.x * inv_temp, i * 8 + 2 * t, row_key, col0);
        sample_visit(acc, f.y * inv_temp, i * 8 + 2 * t + 1, row_key, col0);
      }
    }
    for (int c = v_end * 8 + threadIdx.x; c < c_end; c += kSampleThreads) {
      const uint16_t raw = p[c];
      const float x = FMT == 0 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                               : __half2float(*reinterpret_cast<const __half*>(&raw));
      sample_visit(acc, x * inv_temp, c, row_key, col0);
    }
  }
  // warp, then block reduction
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    SampleAcc o;
    o.best = __shfl_xor_sync(0xffffffffu, acc.best, off);
    o.best_x = __shfl_xor_sync(0xffffffffu, acc.best_x, off);
    o.mx = __shfl_xor_sync(0xffffffffu, acc.mx, off);
    o.sum = __shfl_xor_sync(0xffffffffu, acc.sum, off);
    o.idx = __shfl_xor_sync(0xffffffffu, acc.idx, off);
    sample_merge(acc, o);
  }
  __shared__ SampleAcc sh[kSampleThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    SampleAcc r = sh[0];
    for (int w = 1; w < kSampleThreads / 32; ++w) sample_merge(r, sh[w]);
    const size_t o = (size_t)row * gridDim.y + blockIdx.y;
    stats[o * 4 + 0] = r.best;
    stats[o * 4 + 1] = r.best_x;
    stats[o * 4 + 2] = r.mx;
    stats[o * 4 + 3] = r.sum;
    index[o] = r.idx;
  }
}

// merge the `parts` partial records of every row: one thread per row
__global__ void sample_merge_kernel(const float* __restrict__ part_stats, const int* __restrict__ part_index, int S,
                                    int parts, float* __restrict__ stats, int* __restrict__ index) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= S) return;
  SampleAcc r{-INFINITY, 0.f, -INFINITY, 0.f, -1};
  for (int p = 0; p < parts; ++p) {
    const size_t o = (size_t)row * parts + p;
    const SampleAcc b{part_stats[o * 4], part_stats[o * 4 + 1], part_stats[o * 4 + 2], part_stats[o * 4 + 3],
                      part_index[o]};
    sample_merge(r, b);
  }
  stats[row * 4 + 0] = r.best;
  stats[row * 4 + 1] = r.best_x;
  stats[row * 4 + 2] = r.mx;
  stats[row * 4 + 3] = r.sum;
  index[row] = r.idx;
}

}  // namespace icb

using namespace icb;

// How many column ranges a row is split into (the scratch of icb_sample_gumbel holds S * parts records of 5 words).
ICB_API int icb_sample_parts(int S, int V) {
  if (S <= 0 || V <= 0) return 1;
  int parts = (4 * num_sms() + S - 1) / S;                 // about four CTAs per SM in total
  const int max_parts = (V + 8 * kSampleThreads - 1) / (8 * kSampleThreads);   // at least one vector per thread
  if (parts > max_parts) parts = max_parts;
  return parts < 1 ? 1 : parts;
}

// logits: [S, V] rows of pitch row_stride (elements), dtype 0 bf16 / 1 fp16 / 2 fp32. Columns >= valid are padding.
// stats: [S, 4] fp32 = {best perturbed value, scaled logit at the sample, row max, sum exp(x - max)};
// index: [S] int32 local column of the sample (-1 when the shard has no valid column).
// scratch: S * icb_sample_parts(S, V) * 5 words (partial records), unused when parts == 1.
// (seed, draw) select the noise: the same pair reproduces the same samples; col0 is the global index of column 0.
ICB_API int icb_sample_gumbel(const void* logits, long long row_stride, int S, int V, int valid, float temperature,
                              unsigned long long seed, unsigned long long draw, long long col0, int dtype, float* stats,
                              int* index, void* scratch, void* stream_) {
  if (S <= 0) return 0;
  if (temperature <= 0.f || V <= 0) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const float inv_t = 1.0f / temperature;
  const int parts = icb_sample_parts(S, V);
  if (parts > 1 && scratch == nullptr) return -3;
  int span = ((V + parts - 1) / parts + 7) & ~7;
  float* pstats = parts > 1 ? reinterpret_cast<float*>(scratch) : stats;
  int* pindex = parts > 1 ? reinterpret_cast<int*>(reinterpret_cast<float*>(scratch) + (size_t)S * parts * 4) : index;
  const dim3 grid(S, parts);
  if (dtype == kBF16)
    sample_gumbel_kernel<0><<<grid, kSampleThreads, 0, st>>>(logits, row_stride, V, valid, inv_t, seed, draw, col0, span,
                                                             pstats, pindex);
  else if (dtype == kF16)
    sample_gumbel_kernel<1><<<grid, kSampleThreads, 0, st>>>(logits, row_stride, V, valid, inv_t, seed, draw, col0, span,
                                                             pstats, pindex);
  else
    sample_gumbel_kernel<2><<<grid, kSampleThreads, 0, st>>>(logits, row_stride, V, valid, inv_t, seed, draw, col0, span,
                                                             pstats, pindex);
  int rc = check_launch("sample_gumbel_kernel");
  if (rc || parts == 1) return rc;
  sample_merge_kernel<<<(S + 127) / 128, 128, 0, st>>>(pstats, pindex, S, parts, stats, index);
  return check_launch("sample_merge_kernel");
}
