// Tile geometry shared by the GEMM kernels: 128 x 256 x 64 CTA tiles, a 4-stage TMA ring,
// two 128 x 256 fp32 accumulators in TMEM and two 16 KiB epilogue staging slabs.
#pragma once

#include "ptx.cuh"

namespace icb {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kAStageBytes = kBM * kBK * 2;   // 16 KiB
constexpr int kBStageBytes = kBN * kBK * 2;   // 32 KiB
constexpr int kSlabBytes = kBM * 128;         // 128 rows x 128 B
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;

struct GemmSmem {
  // offsets from the 1024-aligned base
  static constexpr int a_off = 0;
  static constexpr int b_off = kStages * kAStageBytes;
  static constexpr int slab_off = b_off + kStages * kBStageBytes;
  static constexpr int bar_off = slab_off + 2 * kSlabBytes;
  static constexpr int total = bar_off + 256;
};
constexpr int kGemmSmemBytes = GemmSmem::total + 1024;  // slack for manual alignment

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mt, int& nt) {
  const int per_group = kGroupM * num_n;
  const int g = tile / per_group;
  const int first_m = g * kGroupM;
  const int gsz = min(num_m - first_m, kGroupM);
  const int r = tile - g * per_group;
  mt = first_m + r % gsz;
  nt = r / gsz;
}


}  // namespace icb
