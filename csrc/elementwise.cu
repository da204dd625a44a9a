// Memory-bound building blocks: rotary embedding, gated / plain activations,
// embedding gather and scatter-add, vocab-(parallel) cross entropy statistics and
// in-place gradient, multi-tensor Adam on flat buffers, squared-norm reduction and
// the clip coefficient. 16-bit activations (bf16/fp16), fp32 math, 16-byte accesses.
#include "host_common.h"
#include "ptx.cuh"

namespace icb {

template <bool BF16>
__device__ __forceinline__ float ld16(const uint16_t* p) {
  if (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  return __half2float(*reinterpret_cast<const __half*>(p));
}
template <bool BF16>
__device__ __forceinline__ void st16(uint16_t* p, float v) {
  if (BF16) *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16(v);
  else *reinterpret_cast<__half*>(p) = __float2half(v);
}
template <bool BF16>
__device__ __forceinline__ void ld8(const uint16_t* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t;
    if (BF16) t = unpack_bf16x2(w[i]);
    else t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
template <bool BF16>
__device__ __forceinline__ void st8(uint16_t* p, const float (&f)[8]) {
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

// ---------------------------------------------------------------------------
// Rotary position embedding. x: [T, nheads, hd] with row pitch `row_stride`
// elements (so q and k can be rotated inside a packed qkv row). One thread owns
// one (token, frequency) pair and walks the heads, so sin/cos are evaluated once.
// interleaved = 1: pairs (2i, 2i+1); 0: pairs (i, i + hd/2) ("rotate half").
// inverse = 1 applies the transpose rotation (the backward pass).
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void rope_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, const int* __restrict__ pos_ids,
                            int T, int nheads, int hd, long long row_stride, long long out_stride, int seq_len,
                            float base, float scale, int offset, int interleaved, int inverse, int rot_dim) {
  // partial rotary: only the first rot_dim elements of every head rotate (frequencies over rot_dim); the rest
  // of the head is left as it is, so rot_dim < hd is an in-place operation (out == x)
  const int half = rot_dim >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * half) return;
  const int t = (int)(idx / half);
  const int i = (int)(idx - (long long)t * half);
  const int pos = (pos_ids != nullptr) ? pos_ids[t] : (t % seq_len);
  const float inv_freq = powf(base, -2.0f * (float)i / (float)rot_dim);
  float s, c;
  sincosf((float)(pos + offset) * scale * inv_freq, &s, &c);
  if (inverse) s = -s;
  const uint16_t* xr = x + (size_t)t * row_stride;
  uint16_t* orow = out + (size_t)t * out_stride;
  const int i0 = interleaved ? 2 * i : i;
  const int i1 = interleaved ? 2 * i + 1 : i + half;
  for (int h = 0; h < nheads; ++h) {
    const float a = ld16<BF16>(xr + h * hd + i0);
    const float b = ld16<BF16>(xr + h * hd + i1);
    st16<BF16>(orow + h * hd + i0, a * c - b * s);
    st16<BF16>(orow + h * hd + i1, b * c + a * s);
  }
}

// ---------------------------------------------------------------------------
// Activations. kind: 0 relu, 1 gelu (erf), 2 gelu (tanh), 3 silu, 4 sigmoid(identity-gate, for GLU)
// Gated: x = [f | g] halves of the last dim, y = act(f) * g   (swiglu: act = silu;
// geglu: act = gelu; reglu: relu; "glu": y = f * sigmoid(g)).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_f(int kind, float x) {
  switch (kind) {
    case 0: return x > 0.f ? x : 0.f;
    case 1: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 3: return __fdividef(x, 1.f + __expf(-x));
    default: return __fdividef(1.f, 1.f + __expf(-x));
  }
}
__device__ __forceinline__ float act_df(int kind, float x) {
  switch (kind) {
    case 0: return x > 0.f ? 1.f : 0.f;
    case 1: {
      const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
      return cdf + x * pdf;
    }
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
    }
    case 3: {
      const float sg = __fdividef(1.f, 1.f + __expf(-x));
      return sg * (1.f + x * (1.f - sg));
    }
    default: {
      const float sg = __fdividef(1.f, 1.f + __expf(-x));
      return sg * (1.f - sg);
    }
  }
}

// KIND >= 0 fixes the activation at compile time (3 = silu: the SwiGLU of every Llama-style model); KIND = -1
// reads it from the argument. Every thread owns two 8-element vectors half the problem apart and issues the
// loads of both before it computes, which doubles the bytes each SM keeps in flight.
template <bool BF16, int KIND, bool LIMIT>
__global__ void __launch_bounds__(256) glu_fwd_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                                      long long M, int F, int kind_arg, int gate_is_act,
                                                      const int* __restrict__ row_limit) {
  const int kind = KIND >= 0 ? KIND : kind_arg;
  const int vecs = F >> 3;
  const long long total = M * vecs;
  const long long half = (total + 1) >> 1;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i0 >= half) return;
  // rows from *row_limit on hold nothing (unused capacity of a padded expert layout): zeros are written for them
  const long long live = LIMIT ? (long long)*row_limit : M;
  const long long i1 = i0 + half;
  const bool two = i1 < total;
  const long long m0 = i0 / vecs, m1 = two ? i1 / vecs : m0;
  const int v0 = (int)(i0 - m0 * vecs), v1 = two ? (int)(i1 - m1 * vecs) : v0;
  // dead rows are not read: their loads go to row 0 instead (always inside the buffer), unconditionally, so that
  // the four loads are issued back to back; the select below discards what they return
  const bool live0 = !LIMIT || m0 < live, live1 = two && (!LIMIT || m1 < live);
  const uint16_t* r0 = x + (size_t)(live0 ? m0 : 0) * 2 * F + v0 * 8;
  const uint16_t* r1 = x + (size_t)(live1 ? m1 : 0) * 2 * F + v1 * 8;
  float f0[8], g0[8], f1[8], g1[8], o[8];
  ld8<BF16>(r0, f0);
  ld8<BF16>(r0 + F, g0);
  ld8<BF16>(r1, f1);
  ld8<BF16>(r1 + F, g1);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    o[j] = !live0 ? 0.f : (gate_is_act ? f0[j] * act_f(kind, g0[j]) : act_f(kind, f0[j]) * g0[j]);
  st8<BF16>(y + (size_t)m0 * F + v0 * 8, o);
  if (two) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      o[j] = !live1 ? 0.f : (gate_is_act ? f1[j] * act_f(kind, g1[j]) : act_f(kind, f1[j]) * g1[j]);
    st8<BF16>(y + (size_t)m1 * F + v1 * 8, o);
  }
}
template <bool BF16, int KIND, bool LIMIT>
__global__ void __launch_bounds__(256) glu_bwd_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x,
                                                      uint16_t* __restrict__ dx, long long M, int F, int kind_arg,
                                                      int gate_is_act, const int* __restrict__ row_limit) {
  const int kind = KIND >= 0 ? KIND : kind_arg;
  const long long live = LIMIT ? (long long)*row_limit : M;
  const int vecs = F >> 3;
  const long long total = M * vecs;
  const long long half = (total + 1) >> 1;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i0 >= half) return;
  const long long i1 = i0 + half;
  const int n = i1 < total ? 2 : 1;
  long long mm[2];
  int vv[2];
  float f[2][8], g[2][8], d[2][8];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const long long idx = (u == 0 || n == 2) ? (u == 0 ? i0 : i1) : i0;
    mm[u] = idx / vecs;
    vv[u] = (int)(idx - mm[u] * vecs);
    const long long src = (!LIMIT || mm[u] < live) ? mm[u] : 0;   // dead rows: loads from row 0, discarded
    ld8<BF16>(x + (size_t)src * 2 * F + vv[u] * 8, f[u]);
    ld8<BF16>(x + (size_t)src * 2 * F + F + vv[u] * 8, g[u]);
    ld8<BF16>(dy + (size_t)src * F + vv[u] * 8, d[u]);
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (u < n) {
      float df[8], dg[8];
      const bool dead = LIMIT && mm[u] >= live;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (dead) {
          df[j] = 0.f;
          dg[j] = 0.f;
        } else if (gate_is_act) {
          df[j] = d[u][j] * act_f(kind, g[u][j]);
          dg[j] = d[u][j] * f[u][j] * act_df(kind, g[u][j]);
        } else {
          df[j] = d[u][j] * g[u][j] * act_df(kind, f[u][j]);
          dg[j] = d[u][j] * act_f(kind, f[u][j]);
        }
      }
      st8<BF16>(dx + (size_t)mm[u] * 2 * F + vv[u] * 8, df);
      st8<BF16>(dx + (size_t)mm[u] * 2 * F + F + vv[u] * 8, dg);
    }
  }
}
template <bool BF16>
__global__ void act_fwd_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, long long nvec, int kind) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nvec) return;
  float f[8], o[8];
  ld8<BF16>(x + idx * 8, f);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = act_f(kind, f[j]);
  st8<BF16>(y + idx * 8, o);
}
template <bool BF16>
__global__ void act_bwd_kernel(const uint16_t* __restrict__ dy, const uint16_t* __restrict__ x,
                               uint16_t* __restrict__ dx, long long nvec, int kind) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nvec) return;
  float f[8], d[8], o[8];
  ld8<BF16>(x + idx * 8, f);
  ld8<BF16>(dy + idx * 8, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = d[j] * act_df(kind, f[j]);
  st8<BF16>(dx + idx * 8, o);
}

// ---------------------------------------------------------------------------
// Embedding: out[t] = W[ids[t] - vocab_start] (zero row when the id lives on
// another vocab shard) + pos_table[pos[t]] (optional). One warp per token.
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const uint16_t* __restrict__ W,
                                     const uint16_t* __restrict__ pos_table, const int* __restrict__ pos_ids,
                                     uint16_t* __restrict__ out, int T, int D, int vocab_start, int vocab_rows,
                                     int seq_len) {
  const int warps_per_block = blockDim.x >> 5;
  const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  const long long id = ids[t] - vocab_start;
  const bool mine = id >= 0 && id < vocab_rows;
  const int pos = (pos_ids != nullptr) ? pos_ids[t] : (t % seq_len);
  for (int v = lane; v < (D >> 3); v += 32) {
    float a[8];
    if (mine) ld8<BF16>(W + (size_t)id * D + v * 8, a);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
    }
    if (pos_table != nullptr) {
      float p[8];
      ld8<BF16>(pos_table + (size_t)pos * D + v * 8, p);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += p[j];
    }
    st8<BF16>(out + (size_t)t * D + v * 8, a);
  }
}
// dW[row[t]] += dy[t] with fp32 atomics (dW fp32) — rows out of range are skipped.
template <bool BF16>
__global__ void embedding_bwd_kernel(const long long* __restrict__ rows, const uint16_t* __restrict__ dy,
                                     float* __restrict__ dW, int T, int D, int row_start, int nrows) {
  const int warps_per_block = blockDim.x >> 5;
  const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  const long long id = rows[t] - row_start;
  if (id < 0 || id >= nrows) return;
  for (int v = lane; v < (D >> 3); v += 32) {
    float a[8];
    ld8<BF16>(dy + (size_t)t * D + v * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dW + (size_t)id * D + v * 8 + j, a[j]);
  }
}

// ---------------------------------------------------------------------------
// Cross entropy over a vocab shard. One 256-thread CTA per token row.
// stats: row max, sum exp(logit - max), logit of the target if it lives here.
// grad : logits <- (exp(logit - lse) - onehot) * gscale[row]   (in place)
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(256)
ce_stats_kernel(const uint16_t* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ rmax,
                float* __restrict__ rsum, float* __restrict__ rtgt, int T, int V, long long ld, int vocab_start,
                int vocab_valid) {
  __shared__ float shm[8], shs[8];
  const int row = blockIdx.x;
  const uint16_t* lr = logits + (size_t)row * ld;
  float mx = -INFINITY, sm = 0.f;
  const int nvec = vocab_valid >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    ld8<BF16>(lr + v * 8, f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > mx) { sm *= __expf(mx - lm); mx = lm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm += __expf(f[j] - mx);
  }
  for (int j = nvec * 8 + threadIdx.x; j < vocab_valid; j += blockDim.x) {
    const float f = ld16<BF16>(lr + j);
    if (f > mx) { sm *= __expf(mx - f); mx = f; }
    sm += __expf(f - mx);
  }
  // combine (max, sum) pairs across the CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o);
    const float os = __shfl_xor_sync(0xffffffffu, sm, o);
    const float nm = fmaxf(mx, om);
    sm = (mx == -INFINITY ? 0.f : sm * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    mx = nm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { shm[warp] = mx; shs[warp] = sm; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = shm[0], s = shs[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) {
      const float nm = fmaxf(m, shm[w]);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (shm[w] == -INFINITY ? 0.f : shs[w] * __expf(shm[w] - nm));
      m = nm;
    }
    rmax[row] = m;
    rsum[row] = s;
    const long long tg = targets[row] - vocab_start;
    rtgt[row] = (tg >= 0 && tg < vocab_valid) ? ld16<BF16>(lr + tg) : 0.f;
  }
}
template <bool BF16>
__global__ void __launch_bounds__(256)
ce_grad_kernel(uint16_t* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ lse,
               const float* __restrict__ gscale, int T, int V, long long ld, int vocab_start, int vocab_valid) {
  const int row = blockIdx.x;
  uint16_t* lr = logits + (size_t)row * ld;
  const float l = lse[row];
  const float gs = gscale[row];
  const long long tg = targets[row] - vocab_start;
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    ld8<BF16>(lr + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = v * 8 + j;
      float p = (col < vocab_valid) ? __expf(f[j] - l) : 0.f;
      if (col == tg && col < vocab_valid) p -= 1.f;   // a target that names a padding column is not on this shard
      f[j] = p * gs;
    }
    st8<BF16>(lr + v * 8, f);
  }
  for (int col = nvec * 8 + threadIdx.x; col < V; col += blockDim.x) {
    float p = (col < vocab_valid) ? __expf(ld16<BF16>(lr + col) - l) : 0.f;
    if (col == tg && col < vocab_valid) p -= 1.f;
    st16<BF16>(lr + col, p * gs);
  }
}

// ---------------------------------------------------------------------------
// Adam on a flat range (decoupled weight decay, bias correction folded into
// step_size = lr*sqrt(1-b2^t)/(1-b1^t), denom = sqrt(v)+eps, fp32 moments,
// parameter updated in its own dtype — no fp32 master copy):
//   g' = g * gscale * (*gscale_dev) ; m = b1 m + (1-b1) g' ; v = b2 v + (1-b2) g'^2
//   p  = p (1 - lr wd) - step_size * m / (sqrt(v) + eps)
// ---------------------------------------------------------------------------
template <int PT, int GT>  // 0 bf16, 1 fp16, 2 fp32
__global__ void adam_kernel(void* __restrict__ p_, const void* __restrict__ g_, float* __restrict__ m,
                            float* __restrict__ v, long long n, float lr, float b1, float b2, float eps, float wd,
                            float step_size, float gscale, const float* __restrict__ gscale_dev) {
  const float gs = gscale * (gscale_dev != nullptr ? *gscale_dev : 1.f);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g;
    if (GT == 2) g = reinterpret_cast<const float*>(g_)[i];
    else if (GT == 0) g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g_)[i]);
    else g = __half2float(reinterpret_cast<const __half*>(g_)[i]);
    g *= gs;
    float p;
    if (PT == 2) p = reinterpret_cast<float*>(p_)[i];
    else if (PT == 0) p = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(p_)[i]);
    else p = __half2float(reinterpret_cast<__half*>(p_)[i]);
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p = p * (1.f - lr * wd) - step_size * mi / (sqrtf(vi) + eps);
    if (PT == 2) reinterpret_cast<float*>(p_)[i] = p;
    else if (PT == 0) reinterpret_cast<__nv_bfloat16*>(p_)[i] = __float2bfloat16(p);
    else reinterpret_cast<__half*>(p_)[i] = __float2half(p);
  }
}

// Four elements per thread and step (16-byte loads of the fp32 streams, two steps in flight): the form that runs
// whenever the four pointers are aligned for it; the element-wise kernel above takes the ragged tail.
template <int T>
__device__ __forceinline__ void adam_load4(const void* base, long long i4, float (&f)[4]) {
  if (T == 2) {
    const float4 t = reinterpret_cast<const float4*>(base)[i4];
    f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
  } else {
    const uint2 u = reinterpret_cast<const uint2*>(base)[i4];
    if (T == 0) {
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    } else {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    }
  }
}
template <int T>
__device__ __forceinline__ void adam_store4(void* base, long long i4, const float (&f)[4]) {
  if (T == 2) {
    reinterpret_cast<float4*>(base)[i4] = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    uint2 u;
    if (T == 0) { u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); }
    else { u.x = pack_f16x2(f[0], f[1]); u.y = pack_f16x2(f[2], f[3]); }
    reinterpret_cast<uint2*>(base)[i4] = u;
  }
}
template <int PT, int GT>
__global__ void __launch_bounds__(256)
adam_vec4_kernel(void* __restrict__ p_, const void* __restrict__ g_, float* __restrict__ m, float* __restrict__ v,
                 long long n4, float lr, float b1, float b2, float eps, float wd, float step_size, float gscale,
                 const float* __restrict__ gscale_dev) {
  const float gs = gscale * (gscale_dev != nullptr ? *gscale_dev : 1.f);
  const float decay = 1.f - lr * wd;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
    const long long idx[2] = {i, i + stride};
    const int cnt = idx[1] < n4 ? 2 : 1;
    float g[2][4], p[2][4], mm[2][4], vv[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u < cnt) {
        adam_load4<GT>(g_, idx[u], g[u]);
        adam_load4<PT>(p_, idx[u], p[u]);
        adam_load4<2>(m, idx[u], mm[u]);
        adam_load4<2>(v, idx[u], vv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u < cnt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float gj = g[u][j] * gs;
          mm[u][j] = b1 * mm[u][j] + (1.f - b1) * gj;
          vv[u][j] = b2 * vv[u][j] + (1.f - b2) * gj * gj;
          p[u][j] = p[u][j] * decay - step_size * mm[u][j] / (sqrtf(vv[u][j]) + eps);
        }
        adam_store4<2>(m, idx[u], mm[u]);
        adam_store4<2>(v, idx[u], vv[u]);
        adam_store4<PT>(p_, idx[u], p[u]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Sum of squares of a flat range: per-CTA partials in scratch, then one CTA
// folds them (optionally adding to what `out` already holds).
// ---------------------------------------------------------------------------
template <int GT>
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const void* __restrict__ g_, long long n, float* __restrict__ part) {
  __shared__ float sh[8];
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g;
    if (GT == 2) g = reinterpret_cast<const float*>(g_)[i];
    else if (GT == 0) g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g_)[i]);
    else g = __half2float(reinterpret_cast<const __half*>(g_)[i]);
    s += g * g;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sh[w];
    part[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(256) sumsq_final_kernel(const float* __restrict__ part, int P,
                                                          float* __restrict__ out, int accumulate) {
  __shared__ float sh[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += part[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sh[w];
    *out = accumulate ? *out + t : t;
  }
}
// norm = sqrt(total_sq); coef = min(1, clip / (norm + 1e-6)) (coef = 1 when clip <= 0)
__global__ void clip_coef_kernel(const float* __restrict__ total_sq, float clip, float* __restrict__ norm_out,
                                 float* __restrict__ coef_out) {
  const float nrm = sqrtf(*total_sq);
  *norm_out = nrm;
  float c = 1.f;
  if (clip > 0.f) c = fminf(1.f, clip / (nrm + 1e-6f));
  *coef_out = c;
}

template <bool BF16>
__global__ void cast_add_kernel(const float* __restrict__ acc, const uint16_t* __restrict__ residual,
                                uint16_t* __restrict__ out, long long M, int N, long long ldr, long long ldo) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vec_per_row = N >> 3;
  if (i >= M * vec_per_row) return;
  const long long row = i / vec_per_row;
  const int col = (int)(i - row * vec_per_row) * 8;
  const float4 a = *reinterpret_cast<const float4*>(acc + row * N + col);
  const float4 b = *reinterpret_cast<const float4*>(acc + row * N + col + 4);
  float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  if (residual != nullptr) {
    const uint4 u = *reinterpret_cast<const uint4*>(residual + row * ldr + col);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = BF16 ? unpack_bf16x2(w[t]) : __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
      v[2 * t] += f.x;
      v[2 * t + 1] += f.y;
    }
  }
  uint4 o;
  if (BF16) {
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  } else {
    o.x = pack_f16x2(v[0], v[1]); o.y = pack_f16x2(v[2], v[3]);
    o.z = pack_f16x2(v[4], v[5]); o.w = pack_f16x2(v[6], v[7]);
  }
  *reinterpret_cast<uint4*>(out + row * ldo + col) = o;
}

}  // namespace icb

using namespace icb;

#define ICB_ST(s) reinterpret_cast<cudaStream_t>(s)
#define ICB_U16(p) reinterpret_cast<const uint16_t*>(p)
#define ICB_U16M(p) reinterpret_cast<uint16_t*>(p)

ICB_API int icb_rope(const void* x, void* out, const int* pos_ids, int T, int nheads, int hd, long long row_stride,
                     long long out_stride, int seq_len, float base, float scale, int offset, int interleaved,
                     int inverse, int dtype, void* stream, int rot_dim) {
  if (T <= 0 || nheads <= 0) return 0;
  if (rot_dim <= 0) rot_dim = hd;
  if (hd % 2 || rot_dim % 2 || rot_dim > hd) return -2;
  if (rot_dim < hd && x != out) return -3;       // partial rotary leaves the tail of each head in place
  const long long n = (long long)T * (rot_dim / 2);
  const int th = 256;
  const int bl = (int)((n + th - 1) / th);
  if (dtype == kBF16)
    rope_kernel<true><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(x), ICB_U16M(out), pos_ids, T, nheads, hd, row_stride,
                                                     out_stride, seq_len, base, scale, offset, interleaved, inverse,
                                                     rot_dim);
  else
    rope_kernel<false><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(x), ICB_U16M(out), pos_ids, T, nheads, hd, row_stride,
                                                      out_stride, seq_len, base, scale, offset, interleaved, inverse,
                                                      rot_dim);
  return check_launch("rope");
}

// row_limit (optional, device int32): rows from *row_limit on are not read and get zeros.
ICB_API int icb_glu_fwd(const void* x, void* y, long long M, int F, int kind, int gate_is_act, int dtype,
                        void* stream, const int* row_limit) {
  if (M <= 0) return 0;
  if (F % 8) return -2;
  const long long n = (M * (F / 8) + 1) / 2;
  const int th = 256;
  const int bl = (int)((n + th - 1) / th);
  const bool silu = kind == 3 && !gate_is_act;
#define ICB_GLU_FWD(B16, K, L) \
  glu_fwd_kernel<B16, K, L><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(x), ICB_U16M(y), M, F, kind, gate_is_act, row_limit)
#define ICB_GLU_FWD_L(B16, K)            \
  do {                                   \
    if (row_limit != nullptr) ICB_GLU_FWD(B16, K, true); \
    else ICB_GLU_FWD(B16, K, false);     \
  } while (0)
  if (dtype == kBF16) {
    if (silu) ICB_GLU_FWD_L(true, 3);
    else ICB_GLU_FWD_L(true, -1);
  } else {
    if (silu) ICB_GLU_FWD_L(false, 3);
    else ICB_GLU_FWD_L(false, -1);
  }
#undef ICB_GLU_FWD_L
#undef ICB_GLU_FWD
  return check_launch("glu_fwd");
}
ICB_API int icb_glu_bwd(const void* dy, const void* x, void* dx, long long M, int F, int kind, int gate_is_act,
                        int dtype, void* stream, const int* row_limit) {
  if (M <= 0) return 0;
  if (F % 8) return -2;
  const long long n = (M * (F / 8) + 1) / 2;
  const int th = 256;
  const int bl = (int)((n + th - 1) / th);
  const bool silu = kind == 3 && !gate_is_act;
#define ICB_GLU_BWD(B16, K, L)                                                                                     \
  glu_bwd_kernel<B16, K, L><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(dy), ICB_U16(x), ICB_U16M(dx), M, F, kind,      \
                                                           gate_is_act, row_limit)
#define ICB_GLU_BWD_L(B16, K)            \
  do {                                   \
    if (row_limit != nullptr) ICB_GLU_BWD(B16, K, true); \
    else ICB_GLU_BWD(B16, K, false);     \
  } while (0)
  if (dtype == kBF16) {
    if (silu) ICB_GLU_BWD_L(true, 3);
    else ICB_GLU_BWD_L(true, -1);
  } else {
    if (silu) ICB_GLU_BWD_L(false, 3);
    else ICB_GLU_BWD_L(false, -1);
  }
#undef ICB_GLU_BWD_L
#undef ICB_GLU_BWD
  return check_launch("glu_bwd");
}
// out[M, N] (16-bit, pitch ldo) = acc[M, N] (fp32, contiguous) (+ residual[M, N], 16-bit, pitch ldr): the closing
// step of a split-K product, whose partial tiles were summed in fp32. N a multiple of 8; 16-byte aligned rows.
ICB_API int icb_cast_add(const float* acc, const void* residual, void* out, long long M, int N, long long ldr,
                         long long ldo, int dtype, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 8 || (dtype != kBF16 && dtype != kF16)) return -2;
  const long long nvec = M * (N / 8);
  const int threads = 256;
  const int blocks = (int)((nvec + threads - 1) / threads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    cast_add_kernel<true><<<blocks, threads, 0, st>>>(acc, reinterpret_cast<const uint16_t*>(residual),
                                                      reinterpret_cast<uint16_t*>(out), M, N, ldr, ldo);
  else
    cast_add_kernel<false><<<blocks, threads, 0, st>>>(acc, reinterpret_cast<const uint16_t*>(residual),
                                                       reinterpret_cast<uint16_t*>(out), M, N, ldr, ldo);
  return check_launch("cast_add_kernel");
}

ICB_API int icb_act_fwd(const void* x, void* y, long long n, int kind, int dtype, void* stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  const long long nv = n / 8;
  const int th = 256;
  const int bl = (int)((nv + th - 1) / th);
  if (dtype == kBF16) act_fwd_kernel<true><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(x), ICB_U16M(y), nv, kind);
  else act_fwd_kernel<false><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(x), ICB_U16M(y), nv, kind);
  return check_launch("act_fwd");
}
ICB_API int icb_act_bwd(const void* dy, const void* x, void* dx, long long n, int kind, int dtype, void* stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  const long long nv = n / 8;
  const int th = 256;
  const int bl = (int)((nv + th - 1) / th);
  if (dtype == kBF16) act_bwd_kernel<true><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(dy), ICB_U16(x), ICB_U16M(dx), nv, kind);
  else act_bwd_kernel<false><<<bl, th, 0, ICB_ST(stream)>>>(ICB_U16(dy), ICB_U16(x), ICB_U16M(dx), nv, kind);
  return check_launch("act_bwd");
}

ICB_API int icb_embedding_fwd(const long long* ids, const void* W, const void* pos_table, const int* pos_ids,
                              void* out, int T, int D, int vocab_start, int vocab_rows, int seq_len, int dtype,
                              void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -2;
  const int th = 128, wpb = th / 32;
  const int bl = (T + wpb - 1) / wpb;
  if (dtype == kBF16)
    embedding_fwd_kernel<true><<<bl, th, 0, ICB_ST(stream)>>>(ids, ICB_U16(W), ICB_U16(pos_table), pos_ids,
                                                              ICB_U16M(out), T, D, vocab_start, vocab_rows, seq_len);
  else
    embedding_fwd_kernel<false><<<bl, th, 0, ICB_ST(stream)>>>(ids, ICB_U16(W), ICB_U16(pos_table), pos_ids,
                                                               ICB_U16M(out), T, D, vocab_start, vocab_rows, seq_len);
  return check_launch("embedding_fwd");
}
ICB_API int icb_embedding_bwd(const long long* rows, const void* dy, float* dW, int T, int D, int row_start,
                              int nrows, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -2;
  const int th = 128, wpb = th / 32;
  const int bl = (T + wpb - 1) / wpb;
  if (dtype == kBF16)
    embedding_bwd_kernel<true><<<bl, th, 0, ICB_ST(stream)>>>(rows, ICB_U16(dy), dW, T, D, row_start, nrows);
  else
    embedding_bwd_kernel<false><<<bl, th, 0, ICB_ST(stream)>>>(rows, ICB_U16(dy), dW, T, D, row_start, nrows);
  return check_launch("embedding_bwd");
}

// logits: [T, ld] 16-bit; columns [vocab_valid, V) are padding (ignored by stats, zero gradient).
ICB_API int icb_ce_stats(const void* logits, const long long* targets, float* rmax, float* rsum, float* rtgt, int T,
                         int V, long long ld, int vocab_start, int vocab_valid, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -2;
  if (dtype == kBF16)
    ce_stats_kernel<true><<<T, 256, 0, ICB_ST(stream)>>>(ICB_U16(logits), targets, rmax, rsum, rtgt, T, V, ld,
                                                         vocab_start, vocab_valid);
  else
    ce_stats_kernel<false><<<T, 256, 0, ICB_ST(stream)>>>(ICB_U16(logits), targets, rmax, rsum, rtgt, T, V, ld,
                                                          vocab_start, vocab_valid);
  return check_launch("ce_stats");
}
ICB_API int icb_ce_grad(void* logits, const long long* targets, const float* lse, const float* gscale, int T, int V,
                        long long ld, int vocab_start, int vocab_valid, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -2;
  if (dtype == kBF16)
    ce_grad_kernel<true><<<T, 256, 0, ICB_ST(stream)>>>(ICB_U16M(logits), targets, lse, gscale, T, V, ld, vocab_start,
                                                        vocab_valid);
  else
    ce_grad_kernel<false><<<T, 256, 0, ICB_ST(stream)>>>(ICB_U16M(logits), targets, lse, gscale, T, V, ld,
                                                         vocab_start, vocab_valid);
  return check_launch("ce_grad");
}

ICB_API int icb_adam(void* p, const void* g, float* m, float* v, long long n, float lr, float b1, float b2, float eps,
                     float wd, float step_size, float gscale, const float* gscale_dev, int p_dtype, int g_dtype,
                     void* stream) {
  if (n <= 0) return 0;
  const int th = 256;
  const long long cap = (long long)num_sms() * 16;
  const size_t psz = p_dtype == 2 ? 4 : 2, gsz = g_dtype == 2 ? 4 : 2;
  const bool aligned = reinterpret_cast<uintptr_t>(p) % (4 * psz) == 0 && reinterpret_cast<uintptr_t>(g) % (4 * gsz) == 0 &&
                       reinterpret_cast<uintptr_t>(m) % 16 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0;
  const long long n4 = aligned ? n / 4 : 0;        // vectors of four elements for the wide kernel
  const long long done = n4 * 4;
  const long long tail = n - done;
  const long long vblocks = (n4 + 2 * th - 1) / (2 * th);
  const int vbl = (int)(vblocks < cap ? vblocks : cap);
  const long long tblocks = (tail + th - 1) / th;
  const int bl = (int)(tblocks < cap ? tblocks : cap);
  void* pt = reinterpret_cast<char*>(p) + done * psz;
  const void* gt = reinterpret_cast<const char*>(g) + done * gsz;
#define ICB_ADAM(PT, GT)                                                                                            \
  do {                                                                                                              \
    if (n4 > 0)                                                                                                     \
      adam_vec4_kernel<PT, GT><<<vbl, th, 0, ICB_ST(stream)>>>(p, g, m, v, n4, lr, b1, b2, eps, wd, step_size,      \
                                                               gscale, gscale_dev);                                 \
    if (tail > 0)                                                                                                   \
      adam_kernel<PT, GT><<<bl, th, 0, ICB_ST(stream)>>>(pt, gt, m + done, v + done, tail, lr, b1, b2, eps, wd,     \
                                                         step_size, gscale, gscale_dev);                            \
  } while (0)
  if (p_dtype == 0 && g_dtype == 0) ICB_ADAM(0, 0);
  else if (p_dtype == 0 && g_dtype == 2) ICB_ADAM(0, 2);
  else if (p_dtype == 1 && g_dtype == 1) ICB_ADAM(1, 1);
  else if (p_dtype == 1 && g_dtype == 2) ICB_ADAM(1, 2);
  else if (p_dtype == 2 && g_dtype == 2) ICB_ADAM(2, 2);
  else if (p_dtype == 2 && g_dtype == 0) ICB_ADAM(2, 0);
  else return -2;
#undef ICB_ADAM
  return check_launch("adam");
}

ICB_API int icb_sumsq_parts(long long n) {
  long long blocks = (n + 256 * 8 - 1) / (256 * 8);
  const long long cap = (long long)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
// scratch: fp32 [icb_sumsq_parts(n)]. out: one float on the device.
ICB_API int icb_sumsq(const void* g, long long n, float* scratch, float* out, int accumulate, int dtype,
                      void* stream) {
  const int bl = icb_sumsq_parts(n);
  if (dtype == 0) sumsq_partial_kernel<0><<<bl, 256, 0, ICB_ST(stream)>>>(g, n, scratch);
  else if (dtype == 1) sumsq_partial_kernel<1><<<bl, 256, 0, ICB_ST(stream)>>>(g, n, scratch);
  else sumsq_partial_kernel<2><<<bl, 256, 0, ICB_ST(stream)>>>(g, n, scratch);
  sumsq_final_kernel<<<1, 256, 0, ICB_ST(stream)>>>(scratch, bl, out, accumulate);
  return check_launch("sumsq");
}
ICB_API int icb_clip_coef(const float* total_sq, float clip, float* norm_out, float* coef_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, ICB_ST(stream)>>>(total_sq, clip, norm_out, coef_out);
  return check_launch("clip_coef");
}
