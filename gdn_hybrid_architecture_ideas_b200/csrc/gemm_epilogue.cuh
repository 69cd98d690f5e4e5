// bf16 epilogue of the tcgen05 GEMM kernels: accumulator rows leave tensor memory 64 columns at a time, are rounded to
// bf16 into a 128-byte-swizzled shared-memory slab (128 rows x 128 bytes) and a TMA tile store writes the slab, so the
// output leaves in full 128-byte lines issued by one thread instead of 16-byte pieces of 32 different rows per warp
// instruction, and the tile's edges are clipped by the tensor map. Two slabs alternate: the store of one overlaps
// the conversion of the next, and the tensor-memory loads of the next 64 columns are in flight while this slab is
// converted. Called by the four epilogue warps of a CTA (128 threads, named barrier 1).
#pragma once
#include "sm100.cuh"

namespace ghb {

constexpr uint32_t EPI_SLAB_BYTES = 128 * 128;          // 128 rows x 64 bf16
constexpr uint32_t EPI_SMEM_BYTES = 2 * EPI_SLAB_BYTES;

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// taddr: tensor-memory address of this warp's lane quadrant at the accumulator's first column. slabs: 1024-byte aligned.
// (m0, n0): the tile's first row / column; N: columns of the output. slab_count: running slab number of this CTA
// (selects the buffer). acc_free: the accumulator's "drained" barrier, arrived on (one lane per warp) as soon as the last
// column has left tensor memory.
template <int BN>
__device__ __forceinline__ void epilogue_store_bf16(uint32_t taddr, uint8_t* slabs, const CUtensorMap* tma_c, int m0, int n0, int N, int quad,
                                                    int lane, uint32_t& slab_count, uint64_t* acc_free) {
  using namespace sm100;
  constexpr int SLABS = BN / 64;
  const int row = quad * 32 + lane;
  const bool issuer = quad == 0 && lane == 0;
  uint32_t r[2][64];
  tmem_ld_x32(taddr, r[0]);
  tmem_ld_x32(taddr + 32, r[0] + 32);
#pragma unroll
  for (int j = 0; j < SLABS; ++j) {
    tmem_ld_wait();
    if (j + 1 < SLABS) {
      tmem_ld_x32(taddr + (j + 1) * 64, r[(j + 1) & 1]);
      tmem_ld_x32(taddr + (j + 1) * 64 + 32, r[(j + 1) & 1] + 32);
    } else {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_free);
    }
    if (n0 + j * 64 >= N) continue;          // the same for every thread of the CTA
    uint8_t* slab = slabs + (slab_count & 1) * EPI_SLAB_BYTES;
    ++slab_count;
    const uint32_t* v = r[j & 1];
    const uint32_t base = smem_u32(slab) + row * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[c * 8 + 2 * e]), __uint_as_float(v[c * 8 + 2 * e + 1]));
        p[e] = *reinterpret_cast<uint32_t*>(&h);
      }
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + ((c ^ (row & 7)) << 4)), "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3]) : "memory");
    }
    fence_proxy_async();
    if (issuer) tma_store_wait_read<0>();    // the store issued one slab ago has read the other buffer: it is free for the next slab
    epi_bar_sync();
    if (issuer) {
      tma_store_2d(tma_c, slab, n0 + j * 64, m0);
      tma_store_commit();
    }
  }
}

// Before the CTA leaves: every store issued by the issuing thread has completed.
__device__ __forceinline__ void epilogue_store_drain(int quad, int lane) {
  if (quad == 0 && lane == 0) sm100::tma_store_wait<0>();
}

}  // namespace ghb
