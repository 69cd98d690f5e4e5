// MXFP8 on the tensor cores: the quantiser that produces E4M3 values with one E8M0 scale per 32 elements, and the
// block-scaled GEMM D[M,N] = A[M,K] * B[N,K]^T that multiplies them with `tcgen05.mma.kind::mxf8f6f4.block_scale`
// (scale factors in tensor memory, fp32 accumulation in tensor memory).
//
// Quantiser (one read of the input, both block orientations): for x [R, C] it writes
//   * q_row [R, C] E4M3 with blocks along C (the operand of a GEMM that reduces over C), and / or
//   * q_col [C, R] E4M3, the TRANSPOSE, with blocks along R (the operand of a GEMM that reduces over R),
// each with its scales in the layout the tensor core reads: for every (128 rows) x (4 blocks = 128 elements) tile a
// 512-byte cell, byte (row % 32) * 16 + (row % 128 / 32) * 4 + (block % 4); cells ordered [row tile][reduction tile].
// Values and exponents are byte-identical to the reference's emulation (ced/model/mxfp8.py:86-188): exponent of
// amax / 448 rounded up to a power of two, elements scaled, clamped to +-448, rounded to nearest even; a block holding a
// non-finite element becomes all NaN with exponent 255.
//
// GEMM: the same persistent warp-specialised structure as the bf16 kernel (csrc/gemm.cu): warp 0 feeds a ring of
// shared-memory stages (two TMA tile loads, 128-byte swizzle, and two 512-byte bulk copies of scale cells per stage),
// one thread of warp 1 copies the stage's scale cells into tensor memory (`tcgen05.cp`, each stage its own columns)
// and issues four K = 32 MMAs whose instruction descriptors select the block's scale byte, warps 2-5 drain one of two
// accumulators while the other is being filled (bf16 tiles leave through swizzled slabs and TMA tile stores). All three GEMMs of a linear (ced/model/fp8.py:223-291) take this form:
// forward x_q W_q^T, input gradient dy_q (W^T)_q^T, weight gradient (dy^T)_q (x^T)_q^T.
#include "kernels.h"
#include "sm100.cuh"
#include "gemm_epilogue.cuh"
#include <cuda_fp8.h>

namespace ghb {
using namespace sm100;

// ================================================================================================ quantiser
namespace {

__device__ __forceinline__ int mxq_exponent(float amax) {
  const int bits = __float_as_int(amax * (1.0f / 448.0f));
  const int e = (bits >> 23) & 0xFF, m = bits & 0x7FFFFF;
  if (e == 255) return m == 0 ? 254 : 255;
  const bool bump = m > 0 && e != 254 && (e != 0 || m > 0x400000);
  return e + (bump ? 1 : 0);
}
// Two values at once through the paired conversion instruction; low byte = a, high byte = b.
__device__ __forceinline__ uint32_t mxq_pair(float a, float b, float inv) {
  const float ya = fminf(fmaxf(a * inv, -448.f), 448.f), yb = fminf(fmaxf(b * inv, -448.f), 448.f);
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(ya, yb), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float mxq_inverse_scale(int b) { return __int_as_float(b == 254 ? 0x00400000 : (254 - b) << 23); }
__device__ __forceinline__ long mxq_scale_offset(long row, long block, long k_tiles) {
  return ((row >> 7) * k_tiles + (block >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (block & 3);
}

constexpr int QT = 128;            // tile edge
constexpr int QS = QT + 4;         // shared-memory row stride in floats (16-byte aligned rows)

// grid-stride over 128 x 128 tiles; 256 threads. R, C multiples of 32.
template <typename T>
__global__ void __launch_bounds__(256)
mx_quant_kernel(const T* __restrict__ x, long R, long C, long ld, uint8_t* __restrict__ q_row, uint8_t* __restrict__ sf_row,
                uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ float tile[];      // [QT][QS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long tiles_c = (C + QT - 1) / QT, tiles_r = (R + QT - 1) / QT;
  const long kt_row = tiles_c, kt_col = tiles_r;
  for (long t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
    const long r0 = (t / tiles_c) * QT, c0 = (t % tiles_c) * QT;
    // ---- load 16 rows per warp, 4 consecutive columns per lane; blocks along C are 8 lanes wide
    const long c = c0 + lane * 4;
#pragma unroll 4
    for (int i = 0; i < QT / 8; ++i) {
      const int rr = warp + i * 8;
      const long r = r0 + rr;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < R && c < C) {
        if constexpr (sizeof(T) == 4) {
          const float4 f = *reinterpret_cast<const float4*>(x + r * ld + c);
          v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(x + r * ld + c);
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
          v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
        }
      }
      if (q_col) *reinterpret_cast<float4*>(tile + rr * QS + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
      if (q_row) {
        float amax = 0.f; bool bad = false;
#pragma unroll
        for (int e = 0; e < 4; ++e) { bad |= !isfinite(v[e]); amax = fmaxf(amax, isnan(v[e]) ? 0.f : fabsf(v[e])); }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          bad |= __shfl_xor_sync(0xffffffffu, static_cast<int>(bad), o) != 0;
        }
        const int b = bad ? 255 : mxq_exponent(amax);
        if (r < R && c < C) {
          const float inv = mxq_inverse_scale(b);
          const uint32_t packed = bad ? 0x7F7F7F7Fu : (mxq_pair(v[0], v[1], inv) | (mxq_pair(v[2], v[3], inv) << 16));
          *reinterpret_cast<uint32_t*>(q_row + r * C + c) = packed;
          if ((lane & 7) == 0) sf_row[mxq_scale_offset(r, c >> 5, kt_row)] = static_cast<uint8_t>(b);
        }
      }
    }
    if (q_col) {
      __syncthreads();
      // ---- blocks along R: a thread owns (column, block of 32 rows); neighbouring threads own neighbouring columns
#pragma unroll 1
      for (int u = threadIdx.x; u < QT * (QT / 32); u += 256) {
        const int cc = u % QT, rb = u / QT;
        const long col = c0 + cc, row_b = r0 + rb * 32;
        if (col >= C || row_b >= R) continue;
        float f[32];      // the block's 32 values, read from shared memory once
        float amax = 0.f; bool bad = false;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          f[i] = tile[(rb * 32 + i) * QS + cc];
          bad |= !isfinite(f[i]);
          amax = fmaxf(amax, isnan(f[i]) ? 0.f : fabsf(f[i]));
        }
        const int b = bad ? 255 : mxq_exponent(amax);
        const float inv = mxq_inverse_scale(b);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          w[i] = bad ? 0x7F7F7F7Fu : (mxq_pair(f[4 * i], f[4 * i + 1], inv) | (mxq_pair(f[4 * i + 2], f[4 * i + 3], inv) << 16));
        uint4* dst = reinterpret_cast<uint4*>(q_col + col * R + row_b);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        sf_col[mxq_scale_offset(col, row_b >> 5, kt_col)] = static_cast<uint8_t>(b);
      }
      __syncthreads();
    }
  }
}

}  // namespace

long mx_scale_bytes(long rows, long k) { return ((rows + 127) / 128) * ((k + 127) / 128) * 512; }

// x [R, C] (row stride ld elements) -> q_row [R, C] + sf_row (blocks along C) and / or q_col [C, R] + sf_col (blocks
// along R); a null pair is skipped. R and C must be multiples of 32 (whole blocks; 16-byte rows of both outputs).
int mx_quantize(const void* x, bool x_bf16, long R, long C, long ld, void* q_row, void* sf_row, void* q_col, void* sf_col, int sms,
                cudaStream_t st) {
  if (R <= 0 || C <= 0) return 0;
  if (R % 32 || C % 32 || ld % 4 || (!q_row && !q_col) || (q_row && !sf_row) || (q_col && !sf_col)) return 1;
  const long tiles = ((R + QT - 1) / QT) * ((C + QT - 1) / QT);
  const int grid = static_cast<int>(tiles < static_cast<long>(sms) * 3 ? tiles : static_cast<long>(sms) * 3);
  const size_t smem = q_col ? sizeof(float) * QT * QS : 0;
  auto* qr = static_cast<uint8_t*>(q_row); auto* sr = static_cast<uint8_t*>(sf_row);
  auto* qc = static_cast<uint8_t*>(q_col); auto* sc = static_cast<uint8_t*>(sf_col);
  if (x_bf16) {
    auto kern = mx_quant_kernel<__nv_bfloat16>;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(float) * QT * QS) != cudaSuccess) return 3; done = true; }
    kern<<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), R, C, ld, qr, sr, qc, sc);
  } else {
    auto kern = mx_quant_kernel<float>;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(float) * QT * QS) != cudaSuccess) return 3; done = true; }
    kern<<<grid, 256, smem, st>>>(static_cast<const float*>(x), R, C, ld, qr, sr, qc, sc);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ block-scaled GEMM
namespace {

constexpr int MBM = 128, MBN = 128, MBK = 128, MUK = 32;      // K in elements = bytes
constexpr int MX_THREADS = 192;
constexpr int MX_STAGES = 5;
constexpr uint32_t MX_A_BYTES = MBM * MBK, MX_B_BYTES = MBN * MBK, MX_SF_BYTES = 512;
constexpr uint32_t MX_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 2 * MX_SF_BYTES;
constexpr uint32_t MX_SMEM = MX_STAGES * MX_STAGE_BYTES + EPI_SMEM_BYTES + 256 + 1024;
constexpr uint32_t MX_TMEM_COLS = 512;        // two 128-column accumulators, then 8 scale columns per stage from column 256
constexpr uint32_t MX_SF_COL0 = 2 * MBN;

// Instruction descriptor, kind::mxf8f6f4 with block scales: E4M3 x E4M3 (format code 0), both K-major, E8M0 scales;
// bits [4,6) and [29,31) select which byte of the 32-bit scale column this K = 32 step reads (B and A).
__host__ __device__ constexpr uint32_t mx_idesc(int M, int N) {
  return (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(M >> 4) << 24);
}
// Unswizzled K-major descriptor of a 32-row x 16-byte scale cell quarter: 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // stride between 8-row groups
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t tmem_col, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                          bool accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mx_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 8;
  const int per_group = G * tiles_n;
  const int g = tile / per_group, r = tile % per_group;
  const int rows = min(G, tiles_m - g * G);
  tm = g * G + r % rows;
  tn = r / rows;
}

// OUT: 0 bf16, 1 fp32, 2 fp32 accumulated in place, 3 fp32 reduced into the output by `splits` slices of K.
template <int OUT>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const __grid_constant__ CUtensorMap tma_c,
               const uint8_t* __restrict__ sfa,
               const uint8_t* __restrict__ sfb, void* __restrict__ Cout, long ldc, int M, int N, int K, int splits, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + MX_STAGES * MX_A_BYTES;
  uint8_t* slabs = sB + MX_STAGES * MX_B_BYTES;          // bf16 output staging (1024-byte aligned)
  uint8_t* sSA = slabs + EPI_SMEM_BYTES;
  uint8_t* sSB = sSA + MX_STAGES * MX_SF_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sSB + MX_STAGES * MX_SF_BYTES);
  uint64_t* empty = full + MX_STAGES;
  uint64_t* tfull = empty + MX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + MBM - 1) / MBM, tiles_n = (N + MBN - 1) / MBN, tiles = tiles_m * tiles_n;
  const int num_kb = K / MBK;                          // the host guarantees K % 128 == 0
  const int kbs = (num_kb + splits - 1) / splits;
  const int units = tiles * splits;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    for (int s = 0; s < MX_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, MX_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        int tm, tn; mx_tile_coords(unit % tiles, tiles_m, tiles_n, tm, tn);
        const int kb0 = (unit / tiles) * kbs, kb1 = min(num_kb, kb0 + kbs);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 111); ok = false; break; }
          mbar_expect_tx(&full[s], MX_STAGE_BYTES);
          tma_load_2d(sA + s * MX_A_BYTES, &tma_a, &full[s], kb * MBK, tm * MBM);
          tma_load_2d(sB + s * MX_B_BYTES, &tma_b, &full[s], kb * MBK, tn * MBN);
          bulk_load(sSA + s * MX_SF_BYTES, sfa + (static_cast<long>(tm) * num_kb + kb) * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
          bulk_load(sSB + s * MX_SF_BYTES, sfb + (static_cast<long>(tn) * num_kb + kb) * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) __nanosleep(100000);   // let copies already issued land before the CTA leaves
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = mx_idesc(MBM, MBN);
      int s = 0; uint32_t ph = 0; int it = 0; bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++it) {
        const int acc = it & 1; const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1)) { atomicExch(err, 112); ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * MBN;
        const int kb0 = (unit / tiles) * kbs, kb1 = min(num_kb, kb0 + kbs);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph)) { atomicExch(err, 113); ok = false; break; }
          tc_fence_after();
          const uint32_t a = smem_u32(sA + s * MX_A_BYTES), b = smem_u32(sB + s * MX_B_BYTES);
          const uint32_t col_a = tmem_base + MX_SF_COL0 + s * 8, col_b = col_a + 4;
          tmem_cp_32x128b_warpx4(col_a, sf_desc(smem_u32(sSA + s * MX_SF_BYTES)));
          tmem_cp_32x128b_warpx4(col_b, sf_desc(smem_u32(sSB + s * MX_SF_BYTES)));
#pragma unroll
          for (int k = 0; k < MBK / MUK; ++k) {
            const uint64_t da = umma_desc_sw128(a + k * MUK, 16, 1024), db = umma_desc_sw128(b + k * MUK, 16, 1024);
            umma_mxf8(d, da, db, idesc | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4), col_a, col_b, kb != kb0 || k != 0);
          }
          umma_commit(&empty[s]);
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
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
      int tm, tn; mx_tile_coords(unit % tiles, tiles_m, tiles_n, tm, tn);
      if (!mbar_wait(&tfull[acc], aph)) { if (lane == 0) atomicExch(err, 114); ok = false; break; }
      tc_fence_after();
      const long row = static_cast<long>(tm) * MBM + quad * 32 + lane;
      const int n0 = tn * MBN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * MBN;
      if (OUT == 0) {      // bf16: through the swizzled staging slabs and TMA tile stores
        epilogue_store_bf16<MBN>(taddr, slabs, &tma_c, tm * MBM, n0, N, quad, lane, slab_count, &tempty[acc]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < MBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          {
            float* out = reinterpret_cast<float*>(Cout) + row * ldc + col;
            if (OUT == 3) {
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
  if (warp == 1) tmem_dealloc(tmem_base, MX_TMEM_COLS);
}

template <int OUT>
int launch_mx(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const void* sfa, const void* sfb, void* C, long ldc, int M, int N, int K, int splits,
              int* err, int sms, cudaStream_t st) {
  auto kern = gemm_mx_kernel<OUT>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM) != cudaSuccess) return 3;
    attr_done = true;
  }
  const int tiles = ((M + MBM - 1) / MBM) * ((N + MBN - 1) / MBN);
  kern<<<min(tiles * splits, sms), MX_THREADS, MX_SMEM, st>>>(ta, tb, tc, static_cast<const uint8_t*>(sfa), static_cast<const uint8_t*>(sfb), C, ldc, M, N, K,
                                                              splits, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace

// D = A B^T with A [M, K], B [N, K] E4M3 (row stride K bytes) and their scale cells from `mx_quantize`.
// out: 0 bf16, 1 fp32, 2 fp32 accumulate. K must be a multiple of 128. Returns 0 on a clean launch.
int gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long ldc, int out, int* err,
               int sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % MBK) return 11;
  if (ldc % (out == 0 ? 8 : 4)) return 13;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(sfa) |
       reinterpret_cast<uintptr_t>(sfb)) & 15) return 14;
  CUtensorMap ta, tb;
  const uint64_t da[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)}, db[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
  const uint64_t strides[1] = {static_cast<uint64_t>(K)};
  const uint32_t box_a[2] = {MBK, MBM}, box_b[2] = {MBK, MBN};
  if (!encode_tensor_map_2d(&ta, A, 1, da, strides, box_a, true)) return 21;
  if (!encode_tensor_map_2d(&tb, B, 1, db, strides, box_b, true)) return 22;
  CUtensorMap tc = ta;
  if (out == 0) {      // bf16 output tiles leave through TMA stores of 64-column slabs
    const uint64_t dc[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)}, sc[1] = {static_cast<uint64_t>(ldc) * 2};
    const uint32_t box_c[2] = {64, MBM};
    if (!encode_tensor_map_2d(&tc, C, 2, dc, sc, box_c, true)) return 23;
  }
  int splits = 1;
  if (out != 0) {       // a long reduction into few tiles (weight gradients): slice it over the idle SMs, as the bf16 kernel does
    const int tiles = ((M + MBM - 1) / MBM) * ((N + MBN - 1) / MBN), num_kb = K / MBK;
    splits = max(1, min(min(sms / tiles, num_kb / 8), 16));
    while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
    if (splits > 1) {
      if (out == 1 && cudaMemset2DAsync(C, ldc * 4, 0, static_cast<size_t>(N) * 4, M, stream) != cudaSuccess) return 5;
      out = 3;
    }
  }
  switch (out) {
    case 0: return launch_mx<0>(ta, tb, tc, sfa, sfb, C, ldc, M, N, K, 1, err, sms, stream);
    case 1: return launch_mx<1>(ta, tb, tc, sfa, sfb, C, ldc, M, N, K, 1, err, sms, stream);
    case 2: return launch_mx<2>(ta, tb, tc, sfa, sfb, C, ldc, M, N, K, 1, err, sms, stream);
    default: return launch_mx<3>(ta, tb, tc, sfa, sfb, C, ldc, M, N, K, splits, err, sms, stream);
  }
}

}  // namespace ghb
