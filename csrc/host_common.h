// Host-side helpers shared by every translation unit: TMA descriptor encoding
// through the driver entry point (no link-time dependency on libcuda), launch
// error handling and the C ABI conventions of the library.
//
// ABI: every exported function is `extern "C" int icb_*(...)`, takes raw device
// pointers plus sizes plus a cudaStream_t (as void*), allocates nothing unless
// its comment says otherwise, and returns 0 or a negative error / cudaError code.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define ICB_API extern "C" __attribute__((visibility("default")))

namespace icb {

enum DType : int { kBF16 = 0, kF16 = 1, kF32 = 2 };

inline int dtype_bytes(int dt) { return dt == kF32 ? 4 : 2; }
// 8-bit threshold of the attention dropout mask: a probability is dropped when its hash byte is below it.
inline int icb_dropout_threshold(float p) {
  if (!(p > 0.f)) return 0;
  int t = (int)(p * 256.0f + 0.5f);
  return t < 1 ? 1 : (t > 255 ? 255 : t);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[ironcore_b200] cuTensorMapEncodeTiled entry point unavailable (%d)\n", (int)e);
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

inline CUtensorMapDataType tmap_dtype(int dt) {
  switch (dt) {
    case kBF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case kF16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

// Row-major tensor of up to 4 dims; dims[0] is the contiguous one. strides_bytes
// has rank-1 entries (stride of dims[1..]). Box inner extent * element size must
// be 128 bytes when swizzle128 is set.
inline int make_tmap(CUtensorMap* out, int dt, int rank, const void* base, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -100;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, tmap_dtype(dt), (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[ironcore_b200] cuTensorMapEncodeTiled failed (%d): rank=%d base=%p dims=[%llu,%llu,%llu] "
            "stride0=%llu box=[%u,%u,%u]\n",
            (int)r, rank, base, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
            (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 1 ? strides_bytes[0] : 0),
            box[0], rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0);
    return -101;
  }
  return 0;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[ironcore_b200] launch of %s failed: %s\n", what, cudaGetErrorString(e));
    return -(int)e;
  }
  return 0;
}

inline int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace icb
