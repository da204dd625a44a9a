// RMSNorm / LayerNorm forward and backward for 16-bit activations (bf16/fp16),
// fp32 statistics. One 128-thread CTA walks rows that one of its threads streams into a shared-memory ring with
// bulk asynchronous copies, several rows ahead of the reduction; every tensor is read from memory once and
// written once.
//
// forward : (optionally h = x + residual, stored) ; y = norm(h) * (w + w_offset) (+ b)
// backward: dx = d norm / dh (+ dres_in), per-CTA partial dw/db in fp32 scratch,
//           then a second kernel reduces the partials (deterministic, no atomics).
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

constexpr int kNormThreads = 128;

template <bool BF16>
__device__ __forceinline__ void load8(const void* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t;
    if (BF16) t = unpack_bf16x2(w[i]);
    else t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <bool BF16>
__device__ __forceinline__ void store8(void* p, const float (&f)[8]) {
  uint4 u;
  if (BF16) {
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  } else {
    u.x = pack_f16x2(f[0], f[1]); u.y = pack_f16x2(f[2], f[3]);
    u.z = pack_f16x2(f[4], f[5]); u.w = pack_f16x2(f[6], f[7]);
  }
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float block_sum_128(float v, float* sh) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  return sh[0] + sh[1] + sh[2] + sh[3];
}

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t;
    if (BF16) t = unpack_bf16x2(w[i]);
    else t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 ldg16(const uint16_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// VPT = 16-byte vectors per thread; D == VPT*128*8 is not required: tail vectors are masked.
// Forward. Rows (x and, when given, the residual) reach the CTA through a ring of shared-memory stages that one
// thread fills with bulk asynchronous copies, two to four rows ahead of the one being reduced; both passes over
// the row (statistics, then y) read shared memory, so the registers hold only the packed weights.
template <bool BF16, int VPT, bool RMS>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ res, const uint16_t* __restrict__ w,
                const uint16_t* __restrict__ b, uint16_t* __restrict__ y, uint16_t* __restrict__ h_out,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int D, float eps, float w_offset,
                int stages, int* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float sh[4];
  const int nvec = D >> 3;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const bool has_res = res != nullptr;
  const uint32_t stage_bytes = row_bytes * (has_res ? 2u : 1u);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)stages * stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(full + stages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  auto fill = [&](int row, int s) {   // thread 0
    uint8_t* st = ring + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], stage_bytes);
    bulk_load_g2s(st, x + (size_t)row * D, row_bytes, &full[s]);
    if (has_res) bulk_load_g2s(st + row_bytes, res + (size_t)row * D, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      const long long row = (long long)blockIdx.x + (long long)i * gridDim.x;
      if (row < M) fill((int)row, i);
    }
  }
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  uint4 wraw[VPT], braw[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * kNormThreads;
    wraw[i] = vi < nvec ? ldg16(w + vi * 8) : zero4;
    braw[i] = (vi < nvec && b != nullptr) ? ldg16(b + vi * 8) : zero4;
  }
  const bool round_h = has_res && h_out != nullptr;
  int it = 0;
  for (int row = blockIdx.x; row < M; row += gridDim.x, ++it) {
    const int s = it % stages;
    const size_t base = (size_t)row * D;
    mbar_wait(&full[s], (uint32_t)((it / stages) & 1), abort_flag, status, kTimeoutSmemFull);
    const uint4* sx = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
    const uint4* sres = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes + row_bytes);
    // h = x (+ residual), rounded to the 16-bit value that is stored for the backward pass when it is stored
    auto load_h = [&](int vi, float (&h)[8]) -> uint4 {
      unpack8<BF16>(sx[vi], h);
      uint4 packed = sx[vi];
      if (has_res) {
        float rv[8];
        unpack8<BF16>(sres[vi], rv);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] += rv[j];
        if (round_h) {
          if (BF16) {
            packed.x = pack_bf16x2(h[0], h[1]); packed.y = pack_bf16x2(h[2], h[3]);
            packed.z = pack_bf16x2(h[4], h[5]); packed.w = pack_bf16x2(h[6], h[7]);
          } else {
            packed.x = pack_f16x2(h[0], h[1]); packed.y = pack_f16x2(h[2], h[3]);
            packed.z = pack_f16x2(h[4], h[5]); packed.w = pack_f16x2(h[6], h[7]);
          }
          unpack8<BF16>(packed, h);
        }
      }
      return packed;
    };
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        float h[8];
        const uint4 packed = load_h(vi, h);
        if (round_h) *reinterpret_cast<uint4*>(h_out + base + vi * 8) = packed;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += RMS ? h[j] * h[j] : h[j];
      }
    }
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(block_sum_128(sum, sh) / D + eps);
    } else {
      mean = block_sum_128(sum, sh) / D;
      float s2 = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * kNormThreads;
        if (vi < nvec) {
          float h[8];
          load_h(vi, h);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float d = h[j] - mean; s2 += d * d; }
        }
      }
      rstd = rsqrtf(block_sum_128(s2, sh) / D + eps);
    }
    if (threadIdx.x == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        float h[8], o[8], wv[8], bv[8];
        load_h(vi, h);
        unpack8<BF16>(wraw[i], wv);
        unpack8<BF16>(braw[i], bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (h[j] - mean) * rstd * (wv[j] + w_offset) + bv[j];
        store8<BF16>(y + base + vi * 8, o);
      }
    }
    __syncthreads();                       // every thread is done with stage s
    if (threadIdx.x == 0) {
      const long long next = (long long)row + (long long)stages * gridDim.x;
      if (next < M) fill((int)next, s);
    }
  }
}

// Backward. Rows reach the CTA through a ring of shared-memory stages that one thread fills with bulk
// asynchronous copies (dy, x and, when given, the incoming residual gradient of a row: up to 3 x 2 D bytes per
// stage), two to four rows ahead of the one being reduced, so that every CTA keeps tens of KiB in flight
// across its two block-wide reductions; both passes over the row (statistics, then dx) read shared memory.
// DB: the bias gradient is wanted (LayerNorm with bias).
template <bool BF16, int VPT, bool RMS, bool DB>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                const uint16_t* __restrict__ dres_in, uint16_t* __restrict__ dx, float* __restrict__ dw_part,
                float* __restrict__ db_part, int M, int D, float w_offset, int stages, int* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float sh[4];
  const int nvec = D >> 3;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const bool has_res = dres_in != nullptr;
  const uint32_t stage_bytes = row_bytes * (has_res ? 3u : 2u);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)stages * stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(full + stages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  auto fill = [&](int row, int s) {   // thread 0
    uint8_t* st = ring + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], stage_bytes);
    bulk_load_g2s(st, dy + (size_t)row * D, row_bytes, &full[s]);
    bulk_load_g2s(st + row_bytes, x + (size_t)row * D, row_bytes, &full[s]);
    if (has_res) bulk_load_g2s(st + 2 * row_bytes, dres_in + (size_t)row * D, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      const long long row = (long long)blockIdx.x + (long long)i * gridDim.x;
      if (row < M) fill((int)row, i);
    }
  }
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  uint4 wraw[VPT];
  float dwv[VPT][8], dbv[DB ? VPT : 1][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dwv[i][j] = 0.f;
      if (DB) dbv[i][j] = 0.f;
    }
    wraw[i] = vi < nvec ? ldg16(w + vi * 8) : zero4;
  }
  int it = 0;
  for (int row = blockIdx.x; row < M; row += gridDim.x, ++it) {
    const int s = it % stages;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    mbar_wait(&full[s], (uint32_t)((it / stages) & 1), abort_flag, status, kTimeoutSmemFull);
    const uint4* sdy = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
    const uint4* sx = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes + row_bytes);
    const uint4* sres = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes + 2 * row_bytes);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        float dyv[8], xh[8], wv[8];
        unpack8<BF16>(sdy[vi], dyv);
        unpack8<BF16>(sx[vi], xh);
        unpack8<BF16>(wraw[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xn = (xh[j] - mean) * rstd;
          const float g = dyv[j] * (wv[j] + w_offset);
          s1 += g * xn;
          if (!RMS) s2 += g;
          dwv[i][j] += dyv[j] * xn;
          if (DB) dbv[i][j] += dyv[j];
        }
      }
    }
    const float c1 = block_sum_128(s1, sh) / D;
    const float c2 = RMS ? 0.f : block_sum_128(s2, sh) / D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        float dyv[8], xh[8], wv[8], a[8], o[8];
        unpack8<BF16>(sdy[vi], dyv);
        unpack8<BF16>(sx[vi], xh);
        unpack8<BF16>(wraw[i], wv);
        unpack8<BF16>(has_res ? sres[vi] : zero4, a);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o[j] = rstd * (dyv[j] * (wv[j] + w_offset) - c2 - (xh[j] - mean) * rstd * c1) + a[j];
        store8<BF16>(dx + (size_t)row * D + vi * 8, o);
      }
    }
    __syncthreads();                       // every thread is done with stage s
    if (threadIdx.x == 0) {
      const long long next = (long long)row + (long long)stages * gridDim.x;
      if (next < M) fill((int)next, s);
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * kNormThreads;
    if (vi < nvec) {
      float* p = dw_part + (size_t)blockIdx.x * D + vi * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dwv[i][0], dwv[i][1], dwv[i][2], dwv[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dwv[i][4], dwv[i][5], dwv[i][6], dwv[i][7]);
      if (DB) {
        float* q = db_part + (size_t)blockIdx.x * D + vi * 8;
        *reinterpret_cast<float4*>(q) = make_float4(dbv[i][0], dbv[i][1], dbv[i][2], dbv[i][3]);
        *reinterpret_cast<float4*>(q + 4) = make_float4(dbv[i][4], dbv[i][5], dbv[i][6], dbv[i][7]);
      }
    }
  }
}

// out[d] (+)= sum_p part[p, d]; writes 16-bit or fp32 output. blockDim = (32, 8): 32 columns per CTA,
// the partial rows are split over 8 thread rows (4 loads in flight each) and folded through smem.
template <bool BF16>
__global__ void reduce_partials_kernel(const float* __restrict__ part, int P, int D, void* __restrict__ out,
                                       int out_f32, int accumulate) {
  __shared__ float sh[8][33];
  const int d = blockIdx.x * 32 + threadIdx.x;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (d < D) {
    int p = threadIdx.y;
    for (; p + 24 < P; p += 32) {
      s0 += part[(size_t)p * D + d];
      s1 += part[(size_t)(p + 8) * D + d];
      s2 += part[(size_t)(p + 16) * D + d];
      s3 += part[(size_t)(p + 24) * D + d];
    }
    for (; p < P; p += 8) s0 += part[(size_t)p * D + d];
  }
  sh[threadIdx.y][threadIdx.x] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (threadIdx.y != 0 || d >= D) return;
  float s = 0.f;
#pragma unroll
  for (int y = 0; y < 8; ++y) s += sh[y][threadIdx.x];
  if (out_f32) {
    float* o = reinterpret_cast<float*>(out);
    o[d] = accumulate ? o[d] + s : s;
  } else if (BF16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
    o[d] = __float2bfloat16(accumulate ? __bfloat162float(o[d]) + s : s);
  } else {
    __half* o = reinterpret_cast<__half*>(out);
    o[d] = __float2half(accumulate ? __half2float(o[d]) + s : s);
  }
}

// Ring depth for a stage of `stage_bytes`: as many stages as fit into about 52 KiB (four CTAs per SM), 2 to 4.
static int norm_ring_stages(int stage_bytes) {
  int st = (52 * 1024) / stage_bytes;
  return st < 2 ? 2 : (st > 4 ? 4 : st);
}

template <bool BF16, int VPT, bool RMS>
static int norm_fwd_launch(int grid, cudaStream_t st, const uint16_t* x, const uint16_t* res, const uint16_t* w,
                           const uint16_t* b, uint16_t* y, uint16_t* h, float* mean, float* rstd, int M, int D,
                           float eps, float woff, int* status) {
  const int stage_bytes = D * 2 * (res != nullptr ? 2 : 1);
  const int stages = norm_ring_stages(stage_bytes);
  const size_t smem = (size_t)stages * stage_bytes + (size_t)stages * 8 + 16;
  auto kern = norm_fwd_kernel<BF16, VPT, RMS>;
  static size_t configured = 0;      // per instantiation: largest dynamic shared memory size enabled so far
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -(int)e;
    configured = smem;
  }
  kern<<<grid, kNormThreads, smem, st>>>(x, res, w, b, y, h, mean, rstd, M, D, eps, woff, stages, status);
  return 0;
}

template <bool BF16, bool RMS>
static int norm_fwd_dispatch(int vpt, int grid, cudaStream_t st, const uint16_t* x, const uint16_t* res,
                             const uint16_t* w, const uint16_t* b, uint16_t* y, uint16_t* h, float* mean, float* rstd,
                             int M, int D, float eps, float woff, int* status) {
  int rc = 0;
#define ICB_NF(V) rc = norm_fwd_launch<BF16, V, RMS>(grid, st, x, res, w, b, y, h, mean, rstd, M, D, eps, woff, status)
  switch (vpt) {
    case 1: ICB_NF(1); break;
    case 2: ICB_NF(2); break;
    case 3: case 4: ICB_NF(4); break;
    case 5: case 6: ICB_NF(6); break;
    case 7: case 8: ICB_NF(8); break;
    default: return -2;
  }
#undef ICB_NF
  if (rc) return rc;
  return check_launch("norm_fwd");
}

template <bool BF16, int VPT, bool RMS, bool DB>
static int norm_bwd_launch(int grid, cudaStream_t st, const uint16_t* dy, const uint16_t* x, const uint16_t* w,
                           const float* mean, const float* rstd, const uint16_t* dres, uint16_t* dx, float* dwp,
                           float* dbp, int M, int D, float woff, int* status) {
  const int stages = norm_ring_stages(D * 2 * (dres != nullptr ? 3 : 2));
  const size_t smem = (size_t)stages * D * 2 * (dres != nullptr ? 3 : 2) + (size_t)stages * 8 + 16;
  auto kern = norm_bwd_kernel<BF16, VPT, RMS, DB>;
  static size_t configured = 0;      // per instantiation: largest dynamic shared memory size enabled so far
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return -(int)e;
    configured = smem;
  }
  kern<<<grid, kNormThreads, smem, st>>>(dy, x, w, mean, rstd, dres, dx, dwp, dbp, M, D, woff, stages, status);
  return 0;
}

template <bool BF16, bool RMS>
static int norm_bwd_dispatch(int vpt, int grid, cudaStream_t st, const uint16_t* dy, const uint16_t* x,
                             const uint16_t* w, const float* mean, const float* rstd, const uint16_t* dres,
                             uint16_t* dx, float* dwp, float* dbp, int M, int D, float woff, int* status) {
  int rc = 0;
#define ICB_NB(V)                                                                                                  \
  rc = dbp != nullptr ? norm_bwd_launch<BF16, V, RMS, true>(grid, st, dy, x, w, mean, rstd, dres, dx, dwp, dbp, M, \
                                                            D, woff, status)                                       \
                      : norm_bwd_launch<BF16, V, RMS, false>(grid, st, dy, x, w, mean, rstd, dres, dx, dwp, dbp,   \
                                                             M, D, woff, status)
  switch (vpt) {
    case 1: ICB_NB(1); break;
    case 2: ICB_NB(2); break;
    case 3: case 4: ICB_NB(4); break;
    case 5: case 6: ICB_NB(6); break;
    case 7: case 8: ICB_NB(8); break;
    default: return -2;
  }
#undef ICB_NB
  if (rc) return rc;
  return check_launch("norm_bwd");
}

}  // namespace icb

using namespace icb;

// Number of CTAs (= rows of the partial-sum scratch) the backward kernel uses for M rows.
ICB_API int icb_norm_bwd_parts(int M) {
  int g = num_sms() * 4;
  return M < g ? M : g;
}

// dtype: 0 bf16, 1 fp16. rms: 1 RMSNorm, 0 LayerNorm. D must be a multiple of 8 and <= 8192.
// res/h_out/b/mean may be null. If res is given, h = x + res is normalised and (if h_out) stored.
ICB_API int icb_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out,
                         float* mean, float* rstd, int M, int D, float eps, float w_offset, int rms, int dtype,
                         void* stream, int* status) {
  if (M <= 0) return 0;
  if (D % 8 != 0 || D > 8192) return -2;
  const int vpt = (D / 8 + kNormThreads - 1) / kNormThreads;
  int grid = num_sms() * 8;
  if (M < grid) grid = M;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const uint16_t*>(x);
  auto R = reinterpret_cast<const uint16_t*>(res);
  auto W = reinterpret_cast<const uint16_t*>(w);
  auto B = reinterpret_cast<const uint16_t*>(b);
  auto Y = reinterpret_cast<uint16_t*>(y);
  auto H = reinterpret_cast<uint16_t*>(h_out);
  if (dtype == kBF16)
    return rms ? norm_fwd_dispatch<true, true>(vpt, grid, st, X, R, W, B, Y, H, mean, rstd, M, D, eps, w_offset, status)
               : norm_fwd_dispatch<true, false>(vpt, grid, st, X, R, W, B, Y, H, mean, rstd, M, D, eps, w_offset, status);
  return rms ? norm_fwd_dispatch<false, true>(vpt, grid, st, X, R, W, B, Y, H, mean, rstd, M, D, eps, w_offset, status)
             : norm_fwd_dispatch<false, false>(vpt, grid, st, X, R, W, B, Y, H, mean, rstd, M, D, eps, w_offset, status);
}

// scratch: fp32 [(db ? 2 : 1) * icb_norm_bwd_parts(M) * D]. dw/db are written (or accumulated into)
// in the 16-bit dtype (grad_f32 = 0) or fp32 (grad_f32 = 1). dres_in (optional) is added to dx.
ICB_API int icb_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                         const void* dres_in, void* dx, void* dw, void* db, float* scratch, int M, int D,
                         float w_offset, int rms, int dtype, int grad_f32, int accumulate, void* stream, int* status) {
  if (M <= 0) return 0;
  if (D % 8 != 0 || D > 8192) return -2;
  const int vpt = (D / 8 + kNormThreads - 1) / kNormThreads;
  const int grid = icb_norm_bwd_parts(M);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* dwp = scratch;
  float* dbp = (db != nullptr) ? scratch + (size_t)grid * D : nullptr;
  auto DY = reinterpret_cast<const uint16_t*>(dy);
  auto X = reinterpret_cast<const uint16_t*>(x);
  auto W = reinterpret_cast<const uint16_t*>(w);
  auto DR = reinterpret_cast<const uint16_t*>(dres_in);
  auto DX = reinterpret_cast<uint16_t*>(dx);
  int rc;
  if (dtype == kBF16)
    rc = rms ? norm_bwd_dispatch<true, true>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status)
             : norm_bwd_dispatch<true, false>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status);
  else
    rc = rms ? norm_bwd_dispatch<false, true>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status)
             : norm_bwd_dispatch<false, false>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status);
  if (rc) return rc;
  const dim3 th(32, 8); const int bl = (D + 31) / 32;
  if (dtype == kBF16) {
    reduce_partials_kernel<true><<<bl, th, 0, st>>>(dwp, grid, D, dw, grad_f32, accumulate);
    if (db != nullptr) reduce_partials_kernel<true><<<bl, th, 0, st>>>(dbp, grid, D, db, grad_f32, accumulate);
  } else {
    reduce_partials_kernel<false><<<bl, th, 0, st>>>(dwp, grid, D, dw, grad_f32, accumulate);
    if (db != nullptr) reduce_partials_kernel<false><<<bl, th, 0, st>>>(dbp, grid, D, db, grad_f32, accumulate);
  }
  return check_launch("norm_bwd_reduce");
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared and documented in no_alloc.h).
// ---------------------------------------------------------------------------------------
#include "no_alloc.h"

namespace icb {
// Partial sums of dw (first half) and db (second half); lives in the library's device image.
static __device__ __align__(256) float g_norm_bwd_scratch[2 * ICB_NOALLOC_PARTS * ICB_NOALLOC_MAX_D];

// The array's name is only a host-side stand-in for the symbol: the device address has to be
// asked for, once per device, with that device current.
static float* noalloc_scratch_for_current_device(int* rc) {
  static float* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = ICB_NOALLOC_SETUP_FAILED;
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[ironcore_b200] icb_norm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      *rc = ICB_NOALLOC_SETUP_FAILED;
      return nullptr;
    }
    cache[dev] = p;
  }
  *rc = 0;
  return cache[dev];
}
}  // namespace icb

ICB_API int icb_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                 const void* dres_in, void* dx, void* dw, void* db, int M, int D, float w_offset,
                                 int rms, int dtype, int grad_f32, int accumulate, void* stream) {
  if (M <= 0) return 0;
  if (D % 8 != 0) return -2;
  if (D > ICB_NOALLOC_MAX_D) {
    fprintf(stderr,
            "[ironcore_b200] icb_norm_bwd_noalloc: row length %d exceeds the built-in scratch limit of %d; "
            "use icb_norm_bwd with a caller-provided scratch buffer\n", D, ICB_NOALLOC_MAX_D);
    return ICB_NOALLOC_TOO_LARGE;
  }
  int rc = 0;
  int* status = nullptr;     // no status block: the ring's waits then use the default limit and only drain
  float* scratch = noalloc_scratch_for_current_device(&rc);
  if (scratch == nullptr) return rc;
  const int vpt = (D / 8 + kNormThreads - 1) / kNormThreads;
  const int grid = M < ICB_NOALLOC_PARTS ? M : ICB_NOALLOC_PARTS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* dwp = scratch;
  float* dbp = (db != nullptr) ? scratch + (size_t)ICB_NOALLOC_PARTS * ICB_NOALLOC_MAX_D : nullptr;
  auto DY = reinterpret_cast<const uint16_t*>(dy);
  auto X = reinterpret_cast<const uint16_t*>(x);
  auto W = reinterpret_cast<const uint16_t*>(w);
  auto DR = reinterpret_cast<const uint16_t*>(dres_in);
  auto DX = reinterpret_cast<uint16_t*>(dx);
  if (dtype == kBF16)
    rc = rms ? norm_bwd_dispatch<true, true>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status)
             : norm_bwd_dispatch<true, false>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status);
  else
    rc = rms ? norm_bwd_dispatch<false, true>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status)
             : norm_bwd_dispatch<false, false>(vpt, grid, st, DY, X, W, mean, rstd, DR, DX, dwp, dbp, M, D, w_offset, status);
  if (rc) return rc;
  const dim3 th(32, 8); const int bl = (D + 31) / 32;
  if (dtype == kBF16) {
    reduce_partials_kernel<true><<<bl, th, 0, st>>>(dwp, grid, D, dw, grad_f32, accumulate);
    if (db != nullptr) reduce_partials_kernel<true><<<bl, th, 0, st>>>(dbp, grid, D, db, grad_f32, accumulate);
  } else {
    reduce_partials_kernel<false><<<bl, th, 0, st>>>(dwp, grid, D, dw, grad_f32, accumulate);
    if (db != nullptr) reduce_partials_kernel<false><<<bl, th, 0, st>>>(dbp, grid, D, db, grad_f32, accumulate);
  }
  return check_launch("norm_bwd_noalloc_reduce");
}
