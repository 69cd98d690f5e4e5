// bf16 GEMM on tcgen05 tensor cores: D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
//
// One persistent CTA per SM walks output tiles of 128 x BN. Warp roles: warp 0 issues TMA tile loads into a ring of
// shared-memory stages, warp 1 (one thread) issues tcgen05.mma and commits stage releases, warps 2-5 drain the
// accumulator from tensor memory (tcgen05.ld) and store the tile (bf16 tiles through swizzled shared-memory slabs and TMA
// tile stores, csrc/gemm_epilogue.cuh; fp32 tiles straight from registers). Two accumulators alternate so the epilogue
// of tile i overlaps the main loop of tile i+1. Each operand may be K-major (reduction dimension contiguous: forward
// y = x W^T) or MN-major (dgrad dx = dy W, wgrad dW = dy^T x), selected in the UMMA instruction descriptor; the
// shared-memory tiles are 128-byte swizzled in both cases. Output: bf16, fp32, fp32 accumulated in place
// (main-gradient accumulation), or fp32 reduced into the output by several slices of the reduction dimension (split-K
// for weight gradients, whose few output tiles would otherwise leave most SMs idle). No cluster multicast is used.
//
// Replaces the cuBLAS calls behind every nn.Linear of the reference (ced/model/gdn.py:599-849,
// ced/model/attention.py:836-900, ced/model/mlp.py:20-36) and its fp32 wgrad accumulation
// (ced/train/wgrad_accum.py:100-145).
#include "kernels.h"
#include "sm100.cuh"
#include "gemm_epilogue.cuh"
#include <cstdlib>

namespace ghb {
using namespace sm100;

constexpr int BM = 128, BK = 64, UK = 16;
constexpr int GEMM_THREADS = 192;

template <int BN> struct GemmCfg {
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr uint32_t SMEM = STAGES * (A_BYTES + B_BYTES) + EPI_SMEM_BYTES + 256 + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // groups of 8 row-tiles; inside a group the column index runs fastest, so co-resident CTAs share A and B tiles in L2
  constexpr int G = 8;
  int per_group = G * tiles_n;
  int g = tile / per_group, r = tile % per_group;
  int rows = min(G, tiles_m - g * G);
  tm = g * G + r % rows;
  tn = r / rows;
}

template <int BN, bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const __grid_constant__ CUtensorMap tma_c,
            void* __restrict__ Cout, long ldc, int M, int N, int K, int splits, int* __restrict__ err) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
  uint8_t* slabs = smem + STAGES * (Cfg::A_BYTES + Cfg::B_BYTES);      // bf16 output staging (1024-byte aligned)
  uint64_t* full = reinterpret_cast<uint64_t*>(slabs + EPI_SMEM_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int kbs = (num_kb + splits - 1) / splits;      // k-blocks per split; the host guarantees every split is non-empty
  const int units = tiles * splits;                    // work unit = (output tile, slice of the reduction)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (OUT == 0) tma_prefetch_desc(&tma_c);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        int tm, tn; tile_coords(unit % tiles, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = (unit / tiles) * kbs, kb1 = min(num_kb, kb0 + kbs);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 101); ok = false; break; }
          mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          uint8_t* a = sA + s * Cfg::A_BYTES; uint8_t* b = sB + s * Cfg::B_BYTES;
          if (!A_MN) tma_load_2d(a, &tma_a, &full[s], kb * BK, m0);
          else for (int j = 0; j < BM / 64; ++j) tma_load_2d(a + j * (BK * 128), &tma_a, &full[s], m0 + j * 64, kb * BK);
          if (!B_MN) tma_load_2d(b, &tma_b, &full[s], kb * BK, n0);
          else for (int j = 0; j < BN / 64; ++j) tma_load_2d(b + j * (BK * 128), &tma_b, &full[s], n0 + j * 64, kb * BK);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) __nanosleep(100000);   // let copies already issued land before the CTA leaves
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0; uint32_t ph = 0; int it = 0; bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++it) {
        const int acc = it & 1; const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1)) { atomicExch(err, 102); ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        const int kb0 = (unit / tiles) * kbs, kb1 = min(num_kb, kb0 + kbs);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph)) { atomicExch(err, 103); ok = false; break; }
          tc_fence_after();
          const uint32_t a = smem_u32(sA + s * Cfg::A_BYTES), b = smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(a + k * UK * 128, BK * 128, 1024) : umma_desc_sw128(a + k * UK * 2, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(b + k * UK * 128, BK * 128, 1024) : umma_desc_sw128(b + k * UK * 2, 16, 1024);
            umma_bf16(d, da, db, idesc, kb != kb0 || k != 0);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int quad = warp & 3;   // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    int it = 0; bool ok = true;
    uint32_t slab_count = 0;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++it) {
      const int acc = it & 1; const uint32_t aph = (it >> 1) & 1;
      int tm, tn; tile_coords(unit % tiles, tiles_m, tiles_n, tm, tn);
      if (!mbar_wait(&tfull[acc], aph)) { if (lane == 0) atomicExch(err, 104); ok = false; break; }
      tc_fence_after();
      const long row = static_cast<long>(tm) * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (OUT == 0) {      // bf16: through the swizzled staging slabs and TMA tile stores
        epilogue_store_bf16<BN>(taddr, slabs, &tma_c, tm * BM, n0, N, quad, lane, slab_count, &tempty[acc]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          {
            float* out = reinterpret_cast<float*>(Cout) + row * ldc + col;
            if (OUT == 3) {          // slices of one tile's reduction meet in the output through fp32 reductions in L2
              if (col + 32 <= N) {
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + e), "f"(__uint_as_float(r[e])), "f"(__uint_as_float(r[e + 1])),
                               "f"(__uint_as_float(r[e + 2])), "f"(__uint_as_float(r[e + 3])) : "memory");
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) if (col + e < N) atomicAdd(out + e, __uint_as_float(r[e]));
              }
            } else if (col + 32 <= N) {
              float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 x = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                       __uint_as_float(r[4 * v + 3]));
                if (OUT == 2) { float4 y = o4[v]; x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
                o4[v] = x;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) if (col + e < N) out[e] = (OUT == 2 ? out[e] : 0.f) + __uint_as_float(r[e]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (OUT == 0) epilogue_store_drain(quad, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------ host side

static bool encode_operand(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, bool mn_major, int block_mn) {
  // K-major operand: matrix [rows = MN][cols = K], row stride ld; box = 64 (K) x block_mn rows.
  // MN-major operand: stored [K][MN] with row stride ld; box = 64 (MN) x BK rows.
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (!mn_major) { dims[0] = cols; dims[1] = rows; box[0] = BK; box[1] = block_mn; }
  else { dims[0] = rows; dims[1] = cols; box[0] = 64; box[1] = BK; }
  strides[0] = static_cast<uint64_t>(ld) * 2;
  return encode_tensor_map_2d(map, ptr, /*bf16*/ 2, dims, strides, box, /*swizzle128*/ true);
}

template <int BN, bool A_MN, bool B_MN, int OUT>
static int launch_cfg(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc, int splits, int* err,
                      int sms, cudaStream_t stream) {
  CUtensorMap ta, tb, tc;
  if (!encode_operand(&ta, A, M, K, lda, A_MN, BM)) return 21;
  if (!encode_operand(&tb, B, N, K, ldb, B_MN, BN)) return 22;
  if (OUT == 0) {      // bf16 output tiles leave through TMA stores of 64-column slabs
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)}, strides[1] = {static_cast<uint64_t>(ldc) * 2};
    const uint32_t box[2] = {64, BM};
    if (!encode_tensor_map_2d(&tc, C, 2, dims, strides, box, true)) return 23;
  } else {
    tc = ta;
  }
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, OUT>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return 3;
    attr_done = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  kern<<<min(tiles * splits, sms), GEMM_THREADS, Cfg::SMEM, stream>>>(ta, tb, tc, C, ldc, M, N, K, splits, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <int BN, int OUT>
static int launch_major(bool a_mn, bool b_mn, const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                        long ldc, int splits, int* err, int sms, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_cfg<BN, false, false, OUT>(A, B, C, M, N, K, lda, ldb, ldc, splits, err, sms, st);
  if (!a_mn && b_mn) return launch_cfg<BN, false, true, OUT>(A, B, C, M, N, K, lda, ldb, ldc, splits, err, sms, st);
  if (a_mn && !b_mn) return launch_cfg<BN, true, false, OUT>(A, B, C, M, N, K, lda, ldb, ldc, splits, err, sms, st);
  return launch_cfg<BN, true, true, OUT>(A, B, C, M, N, K, lda, ldb, ldc, splits, err, sms, st);
}

// D = A B^T. a_mn / b_mn: the operand is stored with its M (N) dimension contiguous, i.e. as [K][M] ([K][N]) with row
// stride lda (ldb); otherwise as [M][K] ([N][K]). out: 0 bf16, 1 fp32, 2 fp32 accumulate. Returns 0 on a clean launch.
int gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc, bool a_mn, bool b_mn,
              int out, int* err, int sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (lda % 8) return 11;                       // TMA: row strides are multiples of 16 bytes
  if (ldb % 8) return 12;
  if (ldc % (out == 0 ? 8 : 4)) return 13;      // vectorised epilogue stores
  if (reinterpret_cast<uintptr_t>(A) & 15) return 14;
  if (reinterpret_cast<uintptr_t>(B) & 15) return 15;
  if (reinterpret_cast<uintptr_t>(C) & 15) return 16;
  int bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
  if (bn == 256 && out == 0) {     // few 128 x 256 tiles and no split-K (bf16 output): narrower tiles fill more SMs
    const long t256 = static_cast<long>((M + BM - 1) / BM) * ((N + 255) / 256), t128 = static_cast<long>((M + BM - 1) / BM) * ((N + 127) / 128);
    auto waves = [&](long t) { return (t + sms - 1) / sms; };
    // time ~ waves x tile width, and a 128-wide tile runs at about 0.8 of the 256-wide tile's rate (measured: 970 against
    // 1220 TFLOP/s at 65536 x 2816 x 1024): take the narrow tiles only when they save more than that in waves
    if (waves(t128) * 128 * 10 < waves(t256) * 256 * 7) bn = 128;
  }
  static const int forced_bn = [] { const char* e = getenv("GHB_GEMM_BN"); return e ? atoi(e) : 0; }();     // measurement knob
  if (N > 128 && (forced_bn == 128 || forced_bn == 256)) bn = forced_bn;
  // A long reduction into few output tiles (weight gradients: K = tokens) leaves most SMs idle; slice the reduction so
  // that the units fill the machine. Only the fp32 outputs can be reduced into: out 1 is zeroed first, out 2 already
  // holds the running sum. Slices meet through floating-point reductions, so the summation order is not fixed.
  int splits = 1;
  if (out != 0) {
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn), num_kb = (K + BK - 1) / BK;
    splits = max(1, min(min(sms / tiles, num_kb / 16), 16));
    while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;     // no empty slice
    if (splits > 1) {
      if (out == 1 && cudaMemset2DAsync(C, ldc * 4, 0, static_cast<size_t>(N) * 4, M, stream) != cudaSuccess) return 5;
      out = 3;
    }
  }
#define GHB_DISPATCH(BN)                                                                                              \
  switch (out) {                                                                                                      \
    case 0: return launch_major<BN, 0>(a_mn, b_mn, A, B, C, M, N, K, lda, ldb, ldc, 1, err, sms, stream);              \
    case 1: return launch_major<BN, 1>(a_mn, b_mn, A, B, C, M, N, K, lda, ldb, ldc, 1, err, sms, stream);              \
    case 2: return launch_major<BN, 2>(a_mn, b_mn, A, B, C, M, N, K, lda, ldb, ldc, 1, err, sms, stream);              \
    default: return launch_major<BN, 3>(a_mn, b_mn, A, B, C, M, N, K, lda, ldb, ldc, splits, err, sms, stream);        \
  }
  if (bn == 256) { GHB_DISPATCH(256) }
  if (bn == 128) { GHB_DISPATCH(128) }
  GHB_DISPATCH(64)
#undef GHB_DISPATCH
}

}  // namespace ghb
