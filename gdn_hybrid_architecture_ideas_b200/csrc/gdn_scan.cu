// Sequential state pass of the chunked gated delta rule on tcgen05 tensor cores, forward and backward.
//
// Per (batch row, value head, 128-wide slice of the value dimension) one CTA walks the chunks of 64 tokens in order,
// holding the transposed state h^T [128 value channels x 128 key channels] in registers (fp32, one value channel per
// thread) with a bf16 copy in shared memory as the tensor-core operand. Per chunk, with the chunk-local operands
// U, W, q_in, k_out, Aqk prepared by the chunk-local stage (already decayed and document-masked):
//
//   v_new = U - W h            o = q_in h + Aqk v_new            h <- carry h + k_out^T v_new
//
// computed in transposed form so every MMA has M = 128 (value channels on TMEM lanes):
//   T1^T = h^T W^T, O^T = h^T q_in^T (+)= v_new^T Aqk^T, D^T = v_new^T k_out.
// The backward kernel walks the chunks in reverse with dS^T in registers and produces dU, dW, dq_in, dk_out, dcarry and
// dS0; it reads the per-chunk entry states h^T and v_new saved by the forward.
// Reference: the chunk loop of ced/model/gdn_chunked.py:142-160 (PyTorch, one launch group per chunk) and the Triton
// state kernels ced/kernels/gdn_triton.py:378-444, 540-639 (which refuse value dimension 256).
#include "kernels.h"
#include "sm100.cuh"

namespace ghb {
using namespace sm100;

constexpr int GC = 64;            // chunk length
constexpr int GK = 128;           // key head dimension
constexpr int GV = 128;           // value slice per CTA
constexpr uint32_t B8K = 8192;    // a [64 rows][64 bf16] swizzled box
constexpr uint32_t B16K = 16384;  // a [128 rows][64 bf16] swizzled box

// 8 consecutive bf16 of operand row `row`, columns col0..col0+7, into a tile of 64-column blocks of `block_bytes`.
__device__ __forceinline__ void st_sw128(uint8_t* base, uint32_t block_bytes, int row, int col0, const float* v8) {
  const int kb = col0 >> 6, c = (col0 & 63) >> 3;
  __nv_bfloat162 a = __floats2bfloat162_rn(v8[0], v8[1]), b = __floats2bfloat162_rn(v8[2], v8[3]);
  __nv_bfloat162 cc = __floats2bfloat162_rn(v8[4], v8[5]), d = __floats2bfloat162_rn(v8[6], v8[7]);
  uint4 pk;
  pk.x = *reinterpret_cast<uint32_t*>(&a); pk.y = *reinterpret_cast<uint32_t*>(&b);
  pk.z = *reinterpret_cast<uint32_t*>(&cc); pk.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(base + kb * block_bytes + row * 128 + ((c ^ (row & 7)) << 4)) = pk;
}
__device__ __forceinline__ void ld_sw128(const uint8_t* base, uint32_t block_bytes, int row, int col0, float* v8) {
  const int kb = col0 >> 6, c = (col0 & 63) >> 3;
  const uint4 pk = *reinterpret_cast<const uint4*>(base + kb * block_bytes + row * 128 + ((c ^ (row & 7)) << 4));
  const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
    v8[2 * e] = f.x; v8[2 * e + 1] = f.y;
  }
}

struct ScanMaps {
  CUtensorMap w, q, k, a, u, h, vn, dO;   // forward uses w, q, k, a, u; backward also h (saved h^T), vn (saved v_new), dO
};

// ================================================================================================ forward
constexpr uint32_t FS_STAGE = 3 * 2 * B8K + B8K + GC * GV * 2;          // W, Qin, Kout (16 KB each), Aqk 8 KB, U 16 KB = 72 KB
constexpr uint32_t FS_SMEM = 2 * FS_STAGE + 2 * B16K + B16K + 256 + 1024;

__global__ void __launch_bounds__(160, 1)
gdn_scan_fwd_kernel(const __grid_constant__ ScanMaps maps, const float* __restrict__ carry, const float* __restrict__ S0,
                    __nv_bfloat16* __restrict__ O, float* __restrict__ Sfinal, __nv_bfloat16* __restrict__ Hsave,
                    __nv_bfloat16* __restrict__ Vnew, int L, int H, int dv, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage0 = smem;
  uint8_t* sHT = smem + 2 * FS_STAGE;         // 32 KB: h^T as [128 v rows][2 blocks of 64 key channels]
  uint8_t* sVn = sHT + 2 * B16K;              // 16 KB: v_new^T as [128 v rows][64 tokens]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sVn + B16K);
  uint64_t* kv_full = bars; uint64_t* kv_empty = bars + 2;
  uint64_t* bar_a = bars + 4; uint64_t* bar_b = bars + 5; uint64_t* bar_c = bars + 6; uint64_t* bar_d = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vs = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const long bh = static_cast<long>(b) * H + h;
  const int NT = L / GC;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(bar_a, 1); mbar_init(bar_b, 128); mbar_init(bar_c, 1); mbar_init(bar_d, 128);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tT1 = tmem, tO = tmem + 64, tD = tmem + 128;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t id_n64 = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t id_n128_bmn = umma_idesc_bf16(128, 128, false, true);
      bool ok = true;
      auto load_chunk = [&](int c, int s) {
        uint8_t* st = stage0 + s * FS_STAGE;
        const int row = static_cast<int>(bh * L + static_cast<long>(c) * GC);
        mbar_expect_tx(&kv_full[s], FS_STAGE);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_2d(st + kb * B8K, &maps.w, &kv_full[s], kb * 64, row);
          tma_load_2d(st + 2 * B8K + kb * B8K, &maps.q, &kv_full[s], kb * 64, row);
          tma_load_2d(st + 4 * B8K + kb * B8K, &maps.k, &kv_full[s], kb * 64, row);
        }
        tma_load_2d(st + 6 * B8K, &maps.a, &kv_full[s], 0, row);
        tma_load_2d(st + 7 * B8K, &maps.u, &kv_full[s], vs * GV, row);
      };
      load_chunk(0, 0);
      uint32_t ph_full[2] = {0, 0}, ph_empty[2] = {0, 0}, ph_b = 0, ph_d = 0;
      for (int c = 0; c < NT && ok; ++c) {
        const int s = c & 1;
        if (c + 1 < NT) {
          if (c >= 1) { if (!mbar_wait(&kv_empty[s ^ 1], ph_empty[s ^ 1])) { atomicExch(err, 301); ok = false; break; } ph_empty[s ^ 1] ^= 1; }
          load_chunk(c + 1, s ^ 1);
        }
        if (!mbar_wait(&kv_full[s], ph_full[s])) { atomicExch(err, 302); ok = false; break; }
        ph_full[s] ^= 1;
        if (!mbar_wait(bar_d, ph_d)) { atomicExch(err, 303); ok = false; break; }     // h^T operand of this chunk is in place
        ph_d ^= 1;
        tc_fence_after();
        const uint32_t st = smem_u32(stage0 + s * FS_STAGE);
        const uint32_t aH = smem_u32(sHT), aV = smem_u32(sVn);
        const uint32_t bW = st, bQ = st + 2 * B8K, bK = st + 4 * B8K, bA = st + 6 * B8K;
#pragma unroll
        for (int k = 0; k < GK / 16; ++k) {
          const uint64_t da = umma_desc_sw128(aH + (k >> 2) * B16K + (k & 3) * 32, 16, 1024);
          umma_bf16(tT1, da, umma_desc_sw128(bW + (k >> 2) * B8K + (k & 3) * 32, 16, 1024), id_n64, k != 0);
          umma_bf16(tO, da, umma_desc_sw128(bQ + (k >> 2) * B8K + (k & 3) * 32, 16, 1024), id_n64, k != 0);
        }
        umma_commit(bar_a);
        if (!mbar_wait(bar_b, ph_b)) { atomicExch(err, 304); ok = false; break; }
        ph_b ^= 1;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < GC / 16; ++k) {
          const uint64_t da = umma_desc_sw128(aV + k * 32, 16, 1024);
          umma_bf16(tO, da, umma_desc_sw128(bA + k * 32, 16, 1024), id_n64, true);
          umma_bf16(tD, da, umma_desc_sw128(bK + k * 2048, B8K, 1024), id_n128_bmn, k != 0);
        }
        umma_commit(bar_c);
        umma_commit(&kv_empty[s]);
      }
      if (!ok) __nanosleep(100000);
    }
  } else {
    const int t = threadIdx.x;                 // value channel vs*128 + t = TMEM lane t
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const long vcol = static_cast<long>(vs) * GV + t;
    float hT[GK];
    if (S0) {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) hT[kk] = S0[(bh * GK + kk) * dv + vcol];
    } else {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) hT[kk] = 0.f;
    }
    uint32_t ph_full[2] = {0, 0}, ph_a = 0, ph_c = 0;
    bool ok = true;
    for (int c = 0; c < NT && ok; ++c) {
      const int s = c & 1;
      // publish the state entering this chunk: shared-memory operand (bf16) and, when asked, the saved copy
#pragma unroll
      for (int g = 0; g < GK / 8; ++g) st_sw128(sHT, B16K, t, g * 8, hT + g * 8);
      if (Hsave) {
        __nv_bfloat16* hs = Hsave + ((bh * NT + c) * dv + vcol) * GK;
#pragma unroll
        for (int g = 0; g < GK / 8; ++g) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) { __nv_bfloat162 x = __floats2bfloat162_rn(hT[g * 8 + 2 * e], hT[g * 8 + 2 * e + 1]); pk[e] = *reinterpret_cast<uint32_t*>(&x); }
          reinterpret_cast<uint4*>(hs)[g] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_d);
      if (!mbar_wait(&kv_full[s], ph_full[s])) { if (lane == 0) atomicExch(err, 305); ok = false; break; }   // U tile of this chunk
      ph_full[s] ^= 1;
      if (!mbar_wait(bar_a, ph_a)) { if (lane == 0) atomicExch(err, 306); ok = false; break; }
      ph_a ^= 1;
      tc_fence_after();
      const __nv_bfloat16* sU = reinterpret_cast<const __nv_bfloat16*>(stage0 + s * FS_STAGE + 7 * B8K);   // [64 tokens][128] plain
      const long tok0 = bh * L + static_cast<long>(c) * GC;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t tv[32];
        tmem_ld_x32(tT1 + lane_off + half * 32, tv);
        tmem_ld_wait();
        float vn[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) vn[e] = __bfloat162float(sU[(half * 32 + e) * GV + t]) - __uint_as_float(tv[e]);
#pragma unroll
        for (int g = 0; g < 4; ++g) st_sw128(sVn, B16K, t, half * 32 + g * 8, vn + g * 8);
        if (Vnew) {
#pragma unroll
          for (int e = 0; e < 32; ++e) Vnew[(tok0 + half * 32 + e) * dv + vcol] = __float2bfloat16(vn[e]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_b);
      if (!mbar_wait(bar_c, ph_c)) { if (lane == 0) atomicExch(err, 307); ok = false; break; }
      ph_c ^= 1;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t ov[32];
        tmem_ld_x32(tO + lane_off + half * 32, ov);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e)      // token-major output [B, L, H, dv]: what the gated norm and the out-projection read
          O[((static_cast<long>(b) * L + c * GC + half * 32 + e) * H + h) * dv + vcol] = __float2bfloat16(__uint_as_float(ov[e]));
      }
      const float cy = carry[bh * NT + c];
#pragma unroll
      for (int q = 0; q < GK / 32; ++q) {
        uint32_t dvv[32];
        tmem_ld_x32(tD + lane_off + q * 32, dvv);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) hT[q * 32 + e] = hT[q * 32 + e] * cy + __uint_as_float(dvv[e]);
      }
      tc_fence_before();
    }
    if (ok && Sfinal) {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) Sfinal[(bh * GK + kk) * dv + vcol] = hT[kk];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// ================================================================================================ backward
// stage layout: dO 16 KB | Aqk 8 KB | Kout 16 KB | Qin 16 KB | W 16 KB | h^T 32 KB | v_new 16 KB = 120 KB
constexpr uint32_t BS_DO = 0, BS_A = 2 * B8K, BS_K = 3 * B8K, BS_Q = 5 * B8K, BS_W = 7 * B8K, BS_H = 9 * B8K, BS_VN = 13 * B8K;
constexpr uint32_t BS_STAGE = 15 * B8K;
constexpr uint32_t BS_SMEM = BS_STAGE + 2 * B16K + B16K + 256 + 1024;

__global__ void __launch_bounds__(160, 1)
gdn_scan_bwd_kernel(const __grid_constant__ ScanMaps maps, const float* __restrict__ carry, const float* __restrict__ dSfinal,
                    __nv_bfloat16* __restrict__ dU, float* __restrict__ dWp, float* __restrict__ dQp, float* __restrict__ dKp,
                    float* __restrict__ dcarry, float* __restrict__ dS0, int L, int H, int dv, long part_stride, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* st = smem;
  uint8_t* sDS = smem + BS_STAGE;             // 32 KB: dS^T as [128 v rows][2 blocks of 64 key channels]
  uint8_t* sVn = sDS + 2 * B16K;              // 16 KB: -dv_new^T as [128 v rows][64 tokens]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sVn + B16K);
  uint64_t* bar_full = bars; uint64_t* bar_free = bars + 1;
  uint64_t* bar_a = bars + 2; uint64_t* bar_b = bars + 3; uint64_t* bar_c = bars + 4; uint64_t* bar_d = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vs = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const long bh = static_cast<long>(b) * H + h;
  const int NT = L / GC;

  if (threadIdx.x == 0) {
    mbar_init(bar_full, 1); mbar_init(bar_free, 1); mbar_init(bar_a, 1); mbar_init(bar_b, 128); mbar_init(bar_c, 1); mbar_init(bar_d, 128);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tVn = tmem, tP = tmem + 64, tW = tmem + 192, tQ = tmem + 256, tK = tmem + 320;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t id64_mm = umma_idesc_bf16(128, 64, true, true);
      constexpr uint32_t id64_kk = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t id64_mk = umma_idesc_bf16(128, 64, true, false);
      constexpr uint32_t id128_mm = umma_idesc_bf16(128, 128, true, true);
      constexpr uint32_t id128_km = umma_idesc_bf16(128, 128, false, true);
      bool ok = true;
      uint32_t ph_full = 0, ph_free = 0, ph_b = 0, ph_d = 0;
      for (int c = NT - 1; c >= 0 && ok; --c) {
        // the operand buffers are free once last chunk's MMAs are done (bar_free) and its readers are done (bar_d)
        if (c != NT - 1) { if (!mbar_wait(bar_free, ph_free)) { atomicExch(err, 311); ok = false; break; } ph_free ^= 1; }
        if (!mbar_wait(bar_d, ph_d)) { atomicExch(err, 312); ok = false; break; }
        ph_d ^= 1;
        const int row = static_cast<int>(bh * L + static_cast<long>(c) * GC);
        mbar_expect_tx(bar_full, BS_STAGE);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_2d(st + BS_DO + kb * B8K, &maps.dO, bar_full, h * dv + vs * GV + kb * 64, static_cast<int>(static_cast<long>(b) * L + c * GC));
          tma_load_2d(st + BS_K + kb * B8K, &maps.k, bar_full, kb * 64, row);
          tma_load_2d(st + BS_Q + kb * B8K, &maps.q, bar_full, kb * 64, row);
          tma_load_2d(st + BS_W + kb * B8K, &maps.w, bar_full, kb * 64, row);
          tma_load_2d(st + BS_H + kb * B16K, &maps.h, bar_full, kb * 64, static_cast<int>((bh * NT + c) * dv + static_cast<long>(vs) * GV));
          tma_load_2d(st + BS_VN + kb * B8K, &maps.vn, bar_full, vs * GV + kb * 64, row);
        }
        tma_load_2d(st + BS_A, &maps.a, bar_full, 0, row);
        if (!mbar_wait(bar_full, ph_full)) { atomicExch(err, 313); ok = false; break; }
        ph_full ^= 1;
        tc_fence_after();
        const uint32_t s0 = smem_u32(st), aS = smem_u32(sDS), aV = smem_u32(sVn);
        // dv_new^T = dO^T Aqk + dS^T k_out^T
#pragma unroll
        for (int k = 0; k < GC / 16; ++k)
          umma_bf16(tVn, umma_desc_sw128(s0 + BS_DO + k * 2048, B8K, 1024), umma_desc_sw128(s0 + BS_A + k * 2048, B8K, 1024), id64_mm, k != 0);
#pragma unroll
        for (int k = 0; k < GK / 16; ++k)
          umma_bf16(tVn, umma_desc_sw128(aS + (k >> 2) * B16K + (k & 3) * 32, 16, 1024),
                    umma_desc_sw128(s0 + BS_K + (k >> 2) * B8K + (k & 3) * 32, 16, 1024), id64_kk, true);
        umma_commit(bar_a);
        if (!mbar_wait(bar_b, ph_b)) { atomicExch(err, 314); ok = false; break; }
        ph_b ^= 1;
        tc_fence_after();
        // P = dO^T q_in - dv_new^T W   (the shared tile holds -dv_new^T)
#pragma unroll
        for (int k = 0; k < GC / 16; ++k) {
          umma_bf16(tP, umma_desc_sw128(s0 + BS_DO + k * 2048, B8K, 1024), umma_desc_sw128(s0 + BS_Q + k * 2048, B8K, 1024), id128_mm, k != 0);
        }
#pragma unroll
        for (int k = 0; k < GC / 16; ++k)
          umma_bf16(tP, umma_desc_sw128(aV + k * 32, 16, 1024), umma_desc_sw128(s0 + BS_W + k * 2048, B8K, 1024), id128_km, true);
        // dW^T = h (-dv_new^T as B), dq_in^T = h dO^T, dk_out^T = dS v_new^T   (A operands read MN-major: [value rows][key channels])
#pragma unroll
        for (int k = 0; k < GV / 16; ++k) {
          const uint64_t dh = umma_desc_sw128(s0 + BS_H + k * 2048, B16K, 1024);
          const uint32_t koff = (k >> 2) * B8K + (k & 3) * 32;
          umma_bf16(tW, dh, umma_desc_sw128(aV + k * 2048, B16K, 1024), id64_mm, k != 0);
          umma_bf16(tQ, dh, umma_desc_sw128(s0 + BS_DO + koff, 16, 1024), id64_mk, k != 0);
          umma_bf16(tK, umma_desc_sw128(aS + k * 2048, B16K, 1024), umma_desc_sw128(s0 + BS_VN + koff, 16, 1024), id64_mk, k != 0);
        }
        umma_commit(bar_c);
        umma_commit(bar_free);
      }
      if (!ok) __nanosleep(100000);
    }
  } else {
    const int t = threadIdx.x;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const long vcol = static_cast<long>(vs) * GV + t;
    float dS[GK];
    if (dSfinal) {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) dS[kk] = dSfinal[(bh * GK + kk) * dv + vcol];
    } else {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) dS[kk] = 0.f;
    }
    uint32_t ph_a = 0, ph_c = 0;
    bool ok = true;
    for (int c = NT - 1; c >= 0 && ok; --c) {
#pragma unroll
      for (int g = 0; g < GK / 8; ++g) st_sw128(sDS, B16K, t, g * 8, dS + g * 8);
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_d);
      if (!mbar_wait(bar_a, ph_a)) { if (lane == 0) atomicExch(err, 315); ok = false; break; }
      ph_a ^= 1;
      tc_fence_after();
      const long tok0 = bh * L + static_cast<long>(c) * GC;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t tv[32];
        tmem_ld_x32(tVn + lane_off + half * 32, tv);
        tmem_ld_wait();
        float neg[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float g = __uint_as_float(tv[e]);
          dU[(tok0 + half * 32 + e) * dv + vcol] = __float2bfloat16(g);
          neg[e] = -g;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) st_sw128(sVn, B16K, t, half * 32 + g * 8, neg + g * 8);
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(bar_b);
      if (!mbar_wait(bar_c, ph_c)) { if (lane == 0) atomicExch(err, 316); ok = false; break; }
      ph_c ^= 1;
      tc_fence_after();
      // dcarry = <dS, h> with h^T read back from the operand tile (rows = value channels)
      float dot = 0.f;
#pragma unroll
      for (int g = 0; g < GK / 8; ++g) {
        float hv[8];
        ld_sw128(st + BS_H, B16K, t, g * 8, hv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot += dS[g * 8 + e] * hv[e];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) atomicAdd(dcarry + bh * NT + c, dot);
      const float cy = carry[bh * NT + c];
#pragma unroll
      for (int q = 0; q < GK / 32; ++q) {
        uint32_t pv[32];
        tmem_ld_x32(tP + lane_off + q * 32, pv);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) dS[q * 32 + e] = dS[q * 32 + e] * cy + __uint_as_float(pv[e]);
      }
      // partial gradients of this value slice: lane = key channel t, columns = tokens
      float* outs[3] = {dWp, dQp, dKp};
      const uint32_t tms[3] = {tW, tQ, tK};
#pragma unroll
      for (int w = 0; w < 3; ++w) {
        float* dst = outs[w] + static_cast<long>(vs) * part_stride;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t gv[32];
          tmem_ld_x32(tms[w] + lane_off + half * 32, gv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) dst[(tok0 + half * 32 + e) * GK + t] = __uint_as_float(gv[e]);
        }
      }
      tc_fence_before();
    }
    if (ok && dS0) {
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) dS0[(bh * GK + kk) * dv + vcol] = dS[kk];
    }
    // a final arrival so the issuer's count of bar_d phases stays aligned is not needed: the issuer leaves after chunk 0
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------ host side
static bool map2d(CUtensorMap* m, const void* p, long rows, int cols, int box_cols, int box_rows, bool swizzle) {
  const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  const uint64_t strides[1] = {static_cast<uint64_t>(cols) * 2};
  const uint32_t box[2] = {static_cast<uint32_t>(box_cols), static_cast<uint32_t>(box_rows)};
  return encode_tensor_map_2d(m, p, 2, dims, strides, box, swizzle);
}

// W, Qin, Kout: [B*H*L, 128]; Aqk: [B*H*L, 64]; U: [B*H*L, dv] (bf16, chunks of 64 rows); carry: [B*H*NT] fp32;
// S0 / Sfinal: [B, H, 128, dv] fp32 or null; O: [B, L, H, dv] bf16 (token-major); Hsave: [B*H*NT*dv, 128] bf16 or null; Vnew like U or null.
int gdn_scan_fwd(const void* W, const void* Qin, const void* Kout, const void* Aqk, const void* U, const float* carry, const float* S0,
                 void* O, float* Sfinal, void* Hsave, void* Vnew, int B, int H, int L, int dv, int* err, cudaStream_t st) {
  if (L % GC || dv % GV) return 1;
  ScanMaps m;
  const long rows = static_cast<long>(B) * H * L;
  if (!map2d(&m.w, W, rows, GK, 64, 64, true) || !map2d(&m.q, Qin, rows, GK, 64, 64, true) || !map2d(&m.k, Kout, rows, GK, 64, 64, true) ||
      !map2d(&m.a, Aqk, rows, GC, 64, 64, true) || !map2d(&m.u, U, rows, dv, GV, 64, false)) return 2;
  m.h = m.w; m.vn = m.u; m.dO = m.u;
  static bool attr = false;
  if (!attr) { if (cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FS_SMEM) != cudaSuccess) return 3; attr = true; }
  dim3 grid(dv / GV, H, B);
  gdn_scan_fwd_kernel<<<grid, 160, FS_SMEM, st>>>(m, carry, S0, static_cast<__nv_bfloat16*>(O), Sfinal, static_cast<__nv_bfloat16*>(Hsave),
                                                  static_cast<__nv_bfloat16*>(Vnew), L, H, dv, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// dWp, dQp, dKp: [dv/128, B*H*L, 128] fp32 partials per value slice (summed by the caller); dcarry: [B*H*NT] fp32 zeroed by the caller.
int gdn_scan_bwd(const void* W, const void* Qin, const void* Kout, const void* Aqk, const void* Hsave, const void* Vnew, const void* dO,
                 const float* carry, const float* dSfinal, void* dU, float* dWp, float* dQp, float* dKp, float* dcarry, float* dS0, int B, int H,
                 int L, int dv, int* err, cudaStream_t st) {
  if (L % GC || dv % GV) return 1;
  ScanMaps m;
  const long rows = static_cast<long>(B) * H * L;
  const long hrows = static_cast<long>(B) * H * (L / GC) * dv;
  if (!map2d(&m.w, W, rows, GK, 64, 64, true) || !map2d(&m.q, Qin, rows, GK, 64, 64, true) || !map2d(&m.k, Kout, rows, GK, 64, 64, true) ||
      !map2d(&m.a, Aqk, rows, GC, 64, 64, true) || !map2d(&m.h, Hsave, hrows, GK, 64, 128, true) || !map2d(&m.vn, Vnew, rows, dv, 64, 64, true) ||
      !map2d(&m.dO, dO, static_cast<long>(B) * L, H * dv, 64, 64, true)) return 2;     // dO is token-major [B, L, H, dv]
  m.u = m.vn;
  static bool attr = false;
  if (!attr) { if (cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BS_SMEM) != cudaSuccess) return 3; attr = true; }
  dim3 grid(dv / GV, H, B);
  gdn_scan_bwd_kernel<<<grid, 160, BS_SMEM, st>>>(m, carry, dSfinal, static_cast<__nv_bfloat16*>(dU), dWp, dQp, dKp, dcarry, dS0, L, H, dv,
                                                  rows * GK, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
