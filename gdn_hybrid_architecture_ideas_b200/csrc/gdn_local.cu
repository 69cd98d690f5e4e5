// Chunk-local stage of the gated delta rule: everything that does not depend on the state carried between chunks.
// One CTA per (batch row, value head, chunk of 64 tokens); two CTAs share an SM (107 KB of shared memory, <= 128 registers).
//
//   c_i = cumulative log decay inside the chunk, seg_i = number of document starts at or before i (0 = the document
//   that continues from the previous chunk), E_ij = exp(c_i - c_j) for j <= i in the same segment;
//   G = (K K^T) E (strictly lower), A = diag(beta) G, T = (I + A)^-1 by a blocked inverse: the four 16 x 16 diagonal
//   blocks by substitution (one column per thread), then two merge levels [[P, 0], [C, Q]]^-1 = [[P^-1, 0],
//   [-Q^-1 C P^-1, Q^-1]] as small tf32 products (the form ced/kernels/gdn_triton.py:133-325 uses).
// Forward: U = (T diag(beta)) V, W = (T diag(beta gamma first)) K, Aqk = (Q K^T) E (lower), q_in = q gamma first,
//   k_out = k exp(c_last - c) last, carry = gamma_last if the chunk has no document start else 0: the operands of the
//   sequential state pass (gdn_scan.cu). Same function as the PyTorch statement `reference.chunk_local`; the reference
//   computes it with batched matmuls and solve_triangular (ced/model/gdn_chunked.py:100-140) or its Triton kernels.
// Backward: gradients of the above given the state pass's dU, partial sums of dW / dq_in / dk_out, dO and v_new (it
//   forms dAqk = dO v_new^T itself):  dR = T^T dX per block of 128 columns of X = [U | W];  dA = -dR X^T;  dbeta, dc,
//   dKK = dG E from A_ij = beta_i G_ij;  dQK, dc from Aqk;  dk = (dKK + dKK^T) K + dQK^T Q + diagonal terms,
//   dq = dQK K + diagonal term, dv = beta dR_u, dg = reverse cumulative sum of dc.
// Tiles that are bf16 in memory (K, Q, V, U, W, dU, dO, v_new) are copied to shared memory as they are and fed to
// mma.sync m16n8k16 through ldmatrix, plain or transposed, so no tile is stored twice; fp32 matrices that become MMA
// operands (T, its scaled forms) enter as a bf16 pair (value + residual).
#include "kernels.h"
#include <cuda_bf16.h>
#include <cstdlib>

namespace ghb {

constexpr int LC = 64;          // chunk length
constexpr int LK = 128;         // key head dimension
constexpr int BS = 68;          // row stride (elements) of the fp32 64 x 64 matrices
constexpr int TS = 136;         // row stride (elements) of the 64 x 128 bf16 tiles: 272 bytes, conflict-free for ldmatrix
constexpr int MS = 72;          // row stride (elements) of the 64 x 64 bf16 matrices


struct LocalIn {
  const __nv_bfloat16* q; const __nv_bfloat16* k; const __nv_bfloat16* v;   // token-major with per-token strides
  long q_tok, k_tok, v_tok;                                                 // elements between consecutive tokens
  const float* g; const float* beta;                                        // [B, L, Hv]
  const unsigned char* start;                                               // [B, L] document-start flags
  int L, Hv, rep;                                                           // rep = Hv / Hk
};

struct alignas(16) ChunkScalars {     // 16-byte multiple: the buffers laid out after it are read as 16-byte vectors
  float c[LC], beta[LC], gamma[LC], to_end[LC];
  int seg[LC];
  float carry;
  int last_seg;
};

__device__ __forceinline__ void load_scalars(const LocalIn& in, int b, int hv, int chunk, ChunkScalars* s) {
  const int t = threadIdx.x;
  if (t < LC) {
    const long tok = static_cast<long>(b) * in.L + chunk * LC + t;
    s->c[t] = in.g[tok * in.Hv + hv];
    s->beta[t] = in.beta[tok * in.Hv + hv];
    s->seg[t] = in.start[tok] ? 1 : 0;
  }
  __syncthreads();
  if (t == 0) {
    float acc = 0.f; int sg = 0;
    for (int i = 0; i < LC; ++i) { acc += s->c[i]; sg += s->seg[i]; s->c[i] = acc; s->seg[i] = sg; }
    s->last_seg = sg;
    s->carry = sg == 0 ? __expf(acc) : 0.f;
  }
  __syncthreads();
  if (t < LC) {
    s->gamma[t] = __expf(s->c[t]);
    s->to_end[t] = __expf(s->c[LC - 1] - s->c[t]);
  }
  __syncthreads();
}

struct LocalGrads {
  const __nv_bfloat16* U; const __nv_bfloat16* W;       // the forward's outputs (X = [U | W])
  const __nv_bfloat16* dU;                               // [B, H, L, DV]
  const float* dWp; const float* dQp; const float* dKp;  // per value-slice partial sums [n_part, B, H, L, 128] of dW, dq_in, dk_out
  long part_stride; int n_part;
  const __nv_bfloat16* dO; const __nv_bfloat16* Vnew;     // dO token-major [B, L, H, DV]; v_new [B, H, L, DV]: dAqk = dO v_new^T is formed here
  const float* dcarry;
  float* dq; float* dk;            // [B, L, Hv, 128] fp32 (per value head; heads sharing a key head are summed by the caller), or null:
  __nv_bfloat16* dq16; __nv_bfloat16* dk16; long qk_tok;   // bf16 rows [token][head][128] with token stride qk_tok (one value head per key head only)
  __nv_bfloat16* dv; long dv_tok;  // [token][Hv][DV] with token stride dv_tok
  float* dg; float* dbeta;         // [B, L, Hv]
};

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Accumulator fragments (both MMA shapes used here): g = lane / 4, t = lane % 4; c0 (g, 2t) c1 (g, 2t+1) c2 (g+8, 2t)
// c3 (g+8, 2t+1). tf32 m16n8k8 operands: a0 (g, t) a1 (g+8, t) a2 (g, t+4) a3 (g+8, t+4); b0 (t, g) b1 (t+4, g).
template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
}

template <int NP>
__device__ __forceinline__ void sum8(const float* p, long stride, float (&f)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = 0.f;
#pragma unroll
  for (int s = 0; s < NP; ++s) {
    const float4 a = *reinterpret_cast<const float4*>(p + s * stride), c = *reinterpret_cast<const float4*>(p + s * stride + 4);
    f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w; f[4] += c.x; f[5] += c.y; f[6] += c.z; f[7] += c.w;
  }
}
template <int NP>
__device__ __forceinline__ float2 sum2(const float* p, long stride) {
  float2 r = make_float2(0.f, 0.f);
#pragma unroll
  for (int s = 0; s < NP; ++s) { const float2 a = *reinterpret_cast<const float2*>(p + s * stride); r.x += a.x; r.y += a.y; }
  return r;
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// One warp: acc (16 x 8 NT) += A (16 x K) B (K x 8 NT) on bf16 tiles in shared memory. A points at the tile's first row
// (A_T false: stored [m][k]) or first column (A_T true: stored [k][m]); B at its first column (B_KN true: stored
// [k][n]) or first row (B_KN false: stored [n][k]). K a multiple of 16, NT even.
template <int NT, bool A_T, bool B_KN>
__device__ __forceinline__ void wgemm(const __nv_bfloat16* A, int lda, const __nv_bfloat16* B, int ldb, int K, float (&acc)[NT][4], int lane) {
  const int j = lane >> 3, r = lane & 7;
  const __nv_bfloat16* pa = A_T ? A + (r + (j >> 1) * 8) * lda + (j & 1) * 8 : A + (r + (j & 1) * 8) * lda + (j >> 1) * 8;
  const __nv_bfloat16* pb = B_KN ? B + (r + (j & 1) * 8) * ldb + (j >> 1) * 8 : B + (r + (j >> 1) * 8) * ldb + (j & 1) * 8;
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 16) {
    uint32_t a[4];
    if (A_T) ldsm_x4_t(a, pa + k0 * lda); else ldsm_x4(a, pa + k0);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b[4];
      if (B_KN) ldsm_x4_t(b, pb + k0 * ldb + n2 * 16); else ldsm_x4(b, pb + n2 * 16 * ldb + k0);
      mma_bf16(acc[2 * n2], a, b[0], b[1]);
      mma_bf16(acc[2 * n2 + 1], a, b[2], b[3]);
    }
  }
}
// 64 rows x 128 bf16 of a global row-major block -> a shared tile (16-byte copies, no conversion)
__device__ __forceinline__ void copy_tile(const __nv_bfloat16* base, long row_stride, __nv_bfloat16* tile) {
  for (int idx = threadIdx.x; idx < LC * 16; idx += blockDim.x) {
    const int row = idx >> 4, c8 = (idx & 15) * 8;
    *reinterpret_cast<uint4*>(tile + row * TS + c8) = *reinterpret_cast<const uint4*>(base + row * row_stride + c8);
  }
}
// out (16 x 16, C fragments of two n-tiles) = P (16 x K) Q (K x 16) on fp32 shared memory with tf32 tensor cores; P rows may
// carry a per-row factor (beta). P at its first row / column, Q at its first row / column, both row-major with stride BS.
__device__ __forceinline__ void small_tf32(const float* P, const float* rowf, const float* Q, int K, float (&acc)[2][4], int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float f0 = rowf ? rowf[g] : 1.f, f1 = rowf ? rowf[g + 8] : 1.f;
  for (int k0 = 0; k0 < K; k0 += 8) {
    uint32_t a[4];
    a[0] = to_tf32(P[g * BS + k0 + t] * f0); a[1] = to_tf32(P[(g + 8) * BS + k0 + t] * f1);
    a[2] = to_tf32(P[g * BS + k0 + t + 4] * f0); a[3] = to_tf32(P[(g + 8) * BS + k0 + t + 4] * f1);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      mma_tf32(acc[nt], a, to_tf32(Q[(k0 + t) * BS + nt * 8 + g]), to_tf32(Q[(k0 + t + 4) * BS + nt * 8 + g]));
  }
}

// T = (I + diag(beta) G)^-1 into sT (fp32, stride BS) from the strictly lower G in sG. Every thread of the CTA calls it.
__device__ __forceinline__ void blocked_inverse(const float* sG, float* sT, const ChunkScalars* sc) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, tq = lane & 3;
  for (int idx = t; idx < LC * BS; idx += blockDim.x) sT[idx] = 0.f;
  __syncthreads();
  if (t < LC) {                         // the four 16 x 16 diagonal blocks, one column per thread
    const int base = (t >> 4) * 16, c = t & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = (i == c) ? 1.f : 0.f;
#pragma unroll
    for (int i = 1; i < 16; ++i) {
      float s = 0.f;
#pragma unroll
      for (int m = 0; m < i; ++m) s += sG[(base + i) * BS + base + m] * x[m];
      x[i] -= sc->beta[base + i] * s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) sT[(base + i) * BS + base + c] = x[i];
  }
  __syncthreads();
  if (warp < 2) {                       // 32 x 32 diagonal blocks: T_10 = -D1^-1 (A_10 D0^-1), one warp per pair
    const int lo = warp * 32, hi = lo + 16;
    float x[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, y[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    small_tf32(sG + hi * BS + lo, sc->beta + hi, sT + lo * BS + lo, 16, x, lane);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sT[(hi + g) * BS + lo + nt * 8 + 2 * tq] = x[nt][0]; sT[(hi + g) * BS + lo + nt * 8 + 2 * tq + 1] = x[nt][1];
      sT[(hi + g + 8) * BS + lo + nt * 8 + 2 * tq] = x[nt][2]; sT[(hi + g + 8) * BS + lo + nt * 8 + 2 * tq + 1] = x[nt][3];
    }
    __syncwarp();
    small_tf32(sT + hi * BS + hi, nullptr, sT + hi * BS + lo, 16, y, lane);
    __syncwarp();
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sT[(hi + g) * BS + lo + nt * 8 + 2 * tq] = -y[nt][0]; sT[(hi + g) * BS + lo + nt * 8 + 2 * tq + 1] = -y[nt][1];
      sT[(hi + g + 8) * BS + lo + nt * 8 + 2 * tq] = -y[nt][2]; sT[(hi + g + 8) * BS + lo + nt * 8 + 2 * tq + 1] = -y[nt][3];
    }
  }
  __syncthreads();
  // the 64 x 64 matrix: T_low = -Q^-1 (C P^-1) with P^-1 = T[0:32, 0:32], Q^-1 = T[32:64, 32:64], C = beta G[32:64, 0:32]
  const int mi = (warp & 1) * 16, nj = (warp >> 1) * 16;       // warps 0-3: one 16 x 16 block each
  float y[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, z[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  if (warp < 4) {
    small_tf32(sG + (32 + mi) * BS, sc->beta + 32 + mi, sT + nj, 32, y, lane);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sT[(32 + mi + g) * BS + nj + nt * 8 + 2 * tq] = y[nt][0]; sT[(32 + mi + g) * BS + nj + nt * 8 + 2 * tq + 1] = y[nt][1];
      sT[(32 + mi + g + 8) * BS + nj + nt * 8 + 2 * tq] = y[nt][2]; sT[(32 + mi + g + 8) * BS + nj + nt * 8 + 2 * tq + 1] = y[nt][3];
    }
  }
  __syncthreads();
  if (warp < 4) small_tf32(sT + (32 + mi) * BS + 32, nullptr, sT + 32 * BS + nj, 32, z, lane);
  __syncthreads();
  if (warp < 4) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sT[(32 + mi + g) * BS + nj + nt * 8 + 2 * tq] = -z[nt][0]; sT[(32 + mi + g) * BS + nj + nt * 8 + 2 * tq + 1] = -z[nt][1];
      sT[(32 + mi + g + 8) * BS + nj + nt * 8 + 2 * tq] = -z[nt][2]; sT[(32 + mi + g + 8) * BS + nj + nt * 8 + 2 * tq + 1] = -z[nt][3];
    }
  }
  __syncthreads();
}

struct BwdSmem {
  static constexpr size_t TILE = LC * TS * 2;             // 17408
  static constexpr size_t MAT32 = LC * BS * 4;            // 17408
  static constexpr size_t MAT16 = LC * MS * 2;            // 9216
  static constexpr size_t OFF_R1 = 0;                     // sK | sQ, later sX | sDX
  static constexpr size_t OFF_DR = 2 * TILE;
  static constexpr size_t OFF_G = OFF_DR + TILE;
  static constexpr size_t OFF_T = OFF_G + MAT32;          // T fp32, later dKK bf16
  static constexpr size_t OFF_TH = OFF_T + MAT32;         // T high part bf16, later dQK bf16
  static constexpr size_t OFF_TL = OFF_TH + MAT16;
  static constexpr size_t OFF_SC = OFF_TL + MAT16;
  static constexpr size_t TOTAL = OFF_SC + sizeof(ChunkScalars) + 2 * LC * sizeof(float);
};

template <int DV>
__global__ void __launch_bounds__(256, 2)
gdn_local_bwd_kernel(LocalIn in, LocalGrads gr) {
  extern __shared__ __align__(16) unsigned char smb[];
  using S = BwdSmem;
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_R1);
  __nv_bfloat16* sQ = sK + LC * TS;
  __nv_bfloat16* sX = sK;                 // the K / Q region holds the X and dX blocks between the score products
  __nv_bfloat16* sDX = sQ;
  __nv_bfloat16* sDR = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_DR);
  float* sG = reinterpret_cast<float*>(smb + S::OFF_G);
  float* sT = reinterpret_cast<float*>(smb + S::OFF_T);
  __nv_bfloat16* sKK = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_T);
  __nv_bfloat16* sTh = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_TH);
  __nv_bfloat16* sQK = sTh;
  __nv_bfloat16* sTl = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_TL);
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(smb + S::OFF_SC);
  float* sdc = reinterpret_cast<float*>(sc + 1);
  float* sdb = sdc + LC;

  const int chunk = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / in.rep;
  const int NT_ = in.L / LC;
  const long tok0 = static_cast<long>(b) * in.L + chunk * LC;
  const long row0 = (static_cast<long>(b) * in.Hv + hv) * in.L + chunk * LC;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = (warp & 3) * 16;
  constexpr int NP = DV / 128;

  load_scalars(in, b, hv, chunk, sc);
  copy_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  if (t < LC) { sdc[t] = 0.f; sdb[t] = 0.f; }
  __syncthreads();
  {   // G = (K K^T) E, strictly lower, fp32
    const int n0 = (warp >> 2) * 32;
    float kk[4][4];
    zero_acc(kk);
    wgemm<4, false, false>(sK + m0 * TS, TS, sK + n0 * TS, TS, LK, kk, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + nt * 8 + 2 * tq + (e & 1);
        sG[i * BS + j] = (j < i && sc->seg[i] == sc->seg[j]) ? kk[nt][e] * __expf(sc->c[i] - sc->c[j]) : 0.f;
      }
  }
  __syncthreads();
  blocked_inverse(sG, sT, sc);
  for (int idx = t; idx < LC * LC; idx += 256) {       // T as a bf16 pair
    const int i = idx >> 6, j = idx & 63;
    const float v = sT[i * BS + j];
    const __nv_bfloat16 h = __float2bfloat16(v);
    sTh[i * MS + j] = h;
    sTl[i * MS + j] = __float2bfloat16(v - __bfloat162float(h));
  }
  // ---- dAqk = dO v_new^T over the value dimension, 128 columns at a time (warp tile 16 x 32), kept in registers
  float dAq[4][4];
  zero_acc(dAq);
#pragma unroll 1
  for (int vb = 0; vb < DV / 128; ++vb) {
    __syncthreads();
    copy_tile(gr.dO + (tok0 * in.Hv + hv) * DV + vb * 128, static_cast<long>(in.Hv) * DV, sDX);
    copy_tile(gr.Vnew + row0 * DV + vb * 128, DV, sX);
    __syncthreads();
    wgemm<4, false, false>(sDX + m0 * TS, TS, sX + (warp >> 2) * 32 * TS, TS, 128, dAq, lane);
  }
  // ---- per block of 128 columns of [U | W]: dR = T^T dX (warp tile 16 x 64), dA += dR X^T (warp tile 16 x 32)
  float dA[4][4];
  zero_acc(dA);
  constexpr int COLS = DV + LK;
#pragma unroll 1
  for (int blk = 0; blk < COLS / 128; ++blk) {
    const bool is_u = blk * 128 < DV;
    const int c0 = is_u ? blk * 128 : 0;
    __syncthreads();
    if (is_u) {
      copy_tile(gr.U + row0 * DV + c0, DV, sX);
      copy_tile(gr.dU + row0 * DV + c0, DV, sDX);
    } else {
      copy_tile(gr.W + row0 * LK, LK, sX);
      for (int idx = t; idx < LC * 16; idx += 256) {
        const int row = idx >> 4, c8 = (idx & 15) * 8;
        float fa[8];
        sum8<NP>(gr.dWp + (row0 + row) * LK + c8, gr.part_stride, fa);
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) { __nv_bfloat162 h = __floats2bfloat162_rn(fa[2 * e], fa[2 * e + 1]); pk[e] = *reinterpret_cast<uint32_t*>(&h); }
        *reinterpret_cast<uint4*>(sDX + row * TS + c8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
    __syncthreads();
    {
      const int n0 = (warp >> 2) * 64;
      float dr[8][4];
      zero_acc(dr);
      wgemm<8, true, true>(sTh + m0, MS, sDX + n0, TS, LC, dr, lane);      // A(i, j) = T[j][i], B(j, col) = dX[j][col]
      wgemm<8, true, true>(sTl + m0, MS, sDX + n0, TS, LC, dr, lane);
      float pb0 = 0.f, pb1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = m0 + g + h * 8, col = n0 + nt * 8 + 2 * tq;
          const float v0 = dr[nt][2 * h], v1 = dr[nt][2 * h + 1];
          *reinterpret_cast<__nv_bfloat162*>(sDR + i * TS + col) = __floats2bfloat162_rn(v0, v1);
          if (is_u) {
            const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(in.v + (tok0 + i) * in.v_tok + static_cast<long>(hv) * DV + c0 + col));
            const float pv = v0 * vv.x + v1 * vv.y;
            if (h) pb1 += pv; else pb0 += pv;
            const float bi = sc->beta[i];
            *reinterpret_cast<__nv_bfloat162*>(gr.dv + (tok0 + i) * gr.dv_tok + static_cast<long>(hv) * DV + c0 + col) = __floats2bfloat162_rn(bi * v0, bi * v1);
          }
        }
      if (is_u) {
        pb0 += __shfl_xor_sync(0xffffffffu, pb0, 1); pb0 += __shfl_xor_sync(0xffffffffu, pb0, 2);
        pb1 += __shfl_xor_sync(0xffffffffu, pb1, 1); pb1 += __shfl_xor_sync(0xffffffffu, pb1, 2);
        if (tq == 0) { atomicAdd(&sdb[m0 + g], pb0); atomicAdd(&sdb[m0 + g + 8], pb1); }
      }
    }
    __syncthreads();
    wgemm<4, false, false>(sDR + m0 * TS, TS, sX + (warp >> 2) * 32 * TS, TS, 128, dA, lane);   // dR X^T
  }
  __syncthreads();
  // sDR now holds dR of the W columns. Reload K and Q over the X / dX blocks.
  copy_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  copy_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  __syncthreads();
  // ---- score matrices: beta / decay gradients; dKK and dQK as bf16 operands of the output products
  {
    const int n0 = (warp >> 2) * 32;
    float qk[4][4];
    zero_acc(qk);
    wgemm<4, false, false>(sQ + m0 * TS, TS, sK + n0 * TS, TS, LK, qk, lane);
    float rb[2] = {0.f, 0.f}, rc[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float kkv[2], qkv[2];
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int e = 2 * h + e2;
          const int i = m0 + g + h * 8, j = n0 + nt * 8 + 2 * tq + e2;
          const bool same = sc->seg[i] == sc->seg[j];
          const float ex = (j <= i && same) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
          const float G = sG[i * BS + j];
          const float da = (j < i && same) ? -dA[nt][e] : 0.f;
          const float dG = da * sc->beta[i];
          const float t1 = dG * G;
          const float dq_ij = (j <= i && same) ? dAq[nt][e] : 0.f;
          const float t2 = dq_ij * qk[nt][e] * ex;
          rb[h] += da * G;
          rc[h] += t1 + t2;
          atomicAdd(&sdc[j], -(t1 + t2));
          kkv[e2] = dG * ex;
          qkv[e2] = dq_ij * ex;
        }
        const int i = m0 + g + h * 8, j = n0 + nt * 8 + 2 * tq;
        *reinterpret_cast<__nv_bfloat162*>(sKK + i * MS + j) = __floats2bfloat162_rn(kkv[0], kkv[1]);
        *reinterpret_cast<__nv_bfloat162*>(sQK + i * MS + j) = __floats2bfloat162_rn(qkv[0], qkv[1]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rb[h] += __shfl_xor_sync(0xffffffffu, rb[h], 1); rb[h] += __shfl_xor_sync(0xffffffffu, rb[h], 2);
      rc[h] += __shfl_xor_sync(0xffffffffu, rc[h], 1); rc[h] += __shfl_xor_sync(0xffffffffu, rc[h], 2);
      if (tq == 0) { atomicAdd(&sdb[m0 + g + 8 * h], rb[h]); atomicAdd(&sdc[m0 + g + 8 * h], rc[h]); }
    }
  }
  __syncthreads();
  // ---- outputs: dk = (dKK + dKK^T) K + dQK^T Q + diagonal terms ; dq = dQK K + diagonal term (warp tile 16 x 64)
  {
    const int n0 = (warp >> 2) * 64;
    float dk[8][4], dq[8][4];
    zero_acc(dk); zero_acc(dq);
    wgemm<8, false, true>(sKK + m0 * MS, MS, sK + n0, TS, LC, dk, lane);        // dKK K
    wgemm<8, true, true>(sKK + m0, MS, sK + n0, TS, LC, dk, lane);              // dKK^T K
    wgemm<8, true, true>(sQK + m0, MS, sQ + n0, TS, LC, dk, lane);              // dQK^T Q
    wgemm<8, false, true>(sQK + m0 * MS, MS, sK + n0, TS, LC, dq, lane);        // dQK K
    float dots[2][3] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = m0 + g + 8 * h;
      const float fq = sc->seg[r] == 0 ? sc->gamma[r] : 0.f;
      const float fk = sc->seg[r] == sc->last_seg ? sc->to_end[r] : 0.f;
      const float br = sc->beta[r];
      float* dqo = gr.dq16 ? nullptr : gr.dq + ((tok0 + r) * in.Hv + hv) * LK;
      float* dko = gr.dq16 ? nullptr : gr.dk + ((tok0 + r) * in.Hv + hv) * LK;
      __nv_bfloat16* dqh = gr.dq16 ? gr.dq16 + (tok0 + r) * gr.qk_tok + static_cast<long>(hv) * LK : nullptr;
      __nv_bfloat16* dkh = gr.dq16 ? gr.dk16 + (tok0 + r) * gr.qk_tok + static_cast<long>(hv) * LK : nullptr;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int kk = n0 + nt * 8 + 2 * tq;
        const float2 drw = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sDR + r * TS + kk));
        const float2 kre = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sK + r * TS + kk));
        const float2 qre = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sQ + r * TS + kk));
        const float2 dqi = sum2<NP>(gr.dQp + (row0 + r) * LK + kk, gr.part_stride);
        const float2 dkv = sum2<NP>(gr.dKp + (row0 + r) * LK + kk, gr.part_stride);
        float2 ok, oq;
        ok.x = dk[nt][2 * h] + br * fq * drw.x + fk * dkv.x; ok.y = dk[nt][2 * h + 1] + br * fq * drw.y + fk * dkv.y;
        oq.x = dq[nt][2 * h] + fq * dqi.x; oq.y = dq[nt][2 * h + 1] + fq * dqi.y;
        if (dqh) {
          *reinterpret_cast<__nv_bfloat162*>(dkh + kk) = __floats2bfloat162_rn(ok.x, ok.y);
          *reinterpret_cast<__nv_bfloat162*>(dqh + kk) = __floats2bfloat162_rn(oq.x, oq.y);
        } else {
          *reinterpret_cast<float2*>(dko + kk) = ok;
          *reinterpret_cast<float2*>(dqo + kk) = oq;
        }
        dots[h][0] += drw.x * kre.x + drw.y * kre.y;
        dots[h][1] += dqi.x * qre.x + dqi.y * qre.y;
        dots[h][2] += dkv.x * kre.x + dkv.y * kre.y;
      }
#pragma unroll
      for (int w = 0; w < 3; ++w) { dots[h][w] += __shfl_xor_sync(0xffffffffu, dots[h][w], 1); dots[h][w] += __shfl_xor_sync(0xffffffffu, dots[h][w], 2); }
      if (tq == 0) {
        atomicAdd(&sdb[r], fq * dots[h][0]);
        atomicAdd(&sdc[r], br * fq * dots[h][0] + fq * dots[h][1] - fk * dots[h][2]);
        atomicAdd(&sdc[LC - 1], fk * dots[h][2]);
      }
    }
  }
  __syncthreads();
  if (t == 0) {
    sdc[LC - 1] += sc->carry * gr.dcarry[(static_cast<long>(b) * in.Hv + hv) * NT_ + chunk];
    float acc = 0.f;
    for (int i = LC - 1; i >= 0; --i) { acc += sdc[i]; sdc[i] = acc; }      // dg_m = sum_{i >= m} dc_i
  }
  __syncthreads();
  if (t < LC) {
    gr.dg[(tok0 + t) * in.Hv + hv] = sdc[t];
    gr.dbeta[(tok0 + t) * in.Hv + hv] = sdb[t];
  }
}

// ================================================================================================ forward
// U = (T diag(beta)) V and W = (T diag(beta gamma first)) K: the scaled inverses enter as bf16 pairs, so V and K are
// multiplied exactly as stored (no rounding of beta v).
struct FwdSmem {
  static constexpr size_t TILE = LC * TS * 2, MAT32 = LC * BS * 4, MAT16 = LC * MS * 2;
  static constexpr size_t OFF_K = 0, OFF_Q = TILE, OFF_G = 2 * TILE, OFF_T = OFF_G + MAT32, OFF_M = OFF_T + MAT32;    // Q tile later holds V blocks
  static constexpr size_t OFF_SC = OFF_M + 4 * MAT16;
  static constexpr size_t TOTAL = OFF_SC + sizeof(ChunkScalars);
};

template <int DV>
__global__ void __launch_bounds__(256, 2)
gdn_local_fwd_kernel(LocalIn in, __nv_bfloat16* __restrict__ U, __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ Aqk,
                      __nv_bfloat16* __restrict__ Qin, __nv_bfloat16* __restrict__ Kout, float* __restrict__ carry) {
  extern __shared__ __align__(16) unsigned char smb[];
  using S = FwdSmem;
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_K);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_Q);
  __nv_bfloat16* sV = sQ;
  float* sG = reinterpret_cast<float*>(smb + S::OFF_G);
  float* sT = reinterpret_cast<float*>(smb + S::OFF_T);
  __nv_bfloat16* sUh = reinterpret_cast<__nv_bfloat16*>(smb + S::OFF_M);      // T diag(beta): value and residual
  __nv_bfloat16* sUl = sUh + LC * MS;
  __nv_bfloat16* sWh = sUl + LC * MS;                                          // T diag(beta gamma first)
  __nv_bfloat16* sWl = sWh + LC * MS;
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(smb + S::OFF_SC);

  const int chunk = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / in.rep;
  const int NT_ = in.L / LC;
  const long tok0 = static_cast<long>(b) * in.L + chunk * LC;
  const long row0 = (static_cast<long>(b) * in.Hv + hv) * in.L + chunk * LC;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = (warp & 3) * 16;

  load_scalars(in, b, hv, chunk, sc);
  copy_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  copy_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  __syncthreads();
  if (t == 0) carry[(static_cast<long>(b) * in.Hv + hv) * NT_ + chunk] = sc->carry;
  {
    const int n0 = (warp >> 2) * 32;
    float kk[4][4], qk[4][4];
    zero_acc(kk); zero_acc(qk);
    wgemm<4, false, false>(sK + m0 * TS, TS, sK + n0 * TS, TS, LK, kk, lane);
    wgemm<4, false, false>(sQ + m0 * TS, TS, sK + n0 * TS, TS, LK, qk, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = m0 + g + h * 8, j = n0 + nt * 8 + 2 * tq;
        float a[2];
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int jj = j + e2;
          const float ex = (jj <= i && sc->seg[i] == sc->seg[jj]) ? __expf(sc->c[i] - sc->c[jj]) : 0.f;
          sG[i * BS + jj] = (jj < i) ? kk[nt][2 * h + e2] * ex : 0.f;
          a[e2] = qk[nt][2 * h + e2] * ex;
        }
        *reinterpret_cast<__nv_bfloat162*>(Aqk + (row0 + i) * LC + j) = __floats2bfloat162_rn(a[0], a[1]);
      }
  }
  // q_in = q gamma (rows of the continuing document), k_out = k exp(c_last - c) (rows of the last document)
  for (int idx = t; idx < LC * LK / 2; idx += 256) {
    const int row = idx / (LK / 2), c2 = (idx % (LK / 2)) * 2;
    const float fq = sc->seg[row] == 0 ? sc->gamma[row] : 0.f;
    const float fk = sc->seg[row] == sc->last_seg ? sc->to_end[row] : 0.f;
    const float2 qv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sQ + row * TS + c2));
    const float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sK + row * TS + c2));
    reinterpret_cast<__nv_bfloat162*>(Qin + (row0 + row) * LK)[c2 / 2] = __floats2bfloat162_rn(qv.x * fq, qv.y * fq);
    reinterpret_cast<__nv_bfloat162*>(Kout + (row0 + row) * LK)[c2 / 2] = __floats2bfloat162_rn(kv.x * fk, kv.y * fk);
  }
  __syncthreads();
  blocked_inverse(sG, sT, sc);
  for (int idx = t; idx < LC * LC; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    const float bj = sc->beta[j];
    const float u = sT[i * BS + j] * bj;
    const float w = sc->seg[j] == 0 ? u * sc->gamma[j] : 0.f;
    const __nv_bfloat16 uh = __float2bfloat16(u), wh = __float2bfloat16(w);
    sUh[i * MS + j] = uh; sUl[i * MS + j] = __float2bfloat16(u - __bfloat162float(uh));
    sWh[i * MS + j] = wh; sWl[i * MS + j] = __float2bfloat16(w - __bfloat162float(wh));
  }
  __syncthreads();
  const int n0 = (warp >> 2) * 64;
  {   // W = (T diag(beta gamma first)) K
    float acc[8][4];
    zero_acc(acc);
    wgemm<8, false, true>(sWh + m0 * MS, MS, sK + n0, TS, LC, acc, lane);
    wgemm<8, false, true>(sWl + m0 * MS, MS, sK + n0, TS, LC, acc, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<__nv_bfloat162*>(W + (row0 + m0 + g + h * 8) * LK + n0 + nt * 8 + 2 * tq) = __floats2bfloat162_rn(acc[nt][2 * h], acc[nt][2 * h + 1]);
  }
#pragma unroll 1
  for (int vb = 0; vb < DV / 128; ++vb) {   // U = (T diag(beta)) V, 128 value columns at a time (the Q tile's buffer holds them)
    __syncthreads();
    copy_tile(in.v + tok0 * in.v_tok + static_cast<long>(hv) * DV + vb * 128, in.v_tok, sV);
    __syncthreads();
    float acc[8][4];
    zero_acc(acc);
    wgemm<8, false, true>(sUh + m0 * MS, MS, sV + n0, TS, LC, acc, lane);
    wgemm<8, false, true>(sUl + m0 * MS, MS, sV + n0, TS, LC, acc, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<__nv_bfloat162*>(U + (row0 + m0 + g + h * 8) * DV + vb * 128 + n0 + nt * 8 + 2 * tq) = __floats2bfloat162_rn(acc[nt][2 * h], acc[nt][2 * h + 1]);
  }
}

int gdn_local_bwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, const void* U, const void* W, const void* dU,
                  const float* dWp, const float* dQp, const float* dKp, int n_part, const void* dO, const void* Vnew, const float* dcarry,
                  float* dq, float* dk, void* dq16, void* dk16, long qk_tok, void* dvv, long dv_tok, float* dg, float* dbeta, cudaStream_t st) {
  if (L % LC || (dv != 128 && dv != 256) || Hv % Hk || n_part != dv / 128) return 1;
  if (dq16 ? (Hv != Hk || !dk16 || qk_tok % 2) : (!dq || !dk)) return 1;
  if (dv_tok % 2) return 1;
  LocalIn in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), q_tok, k_tok, v_tok,
             g, beta, start, L, Hv, Hv / Hk};
  LocalGrads gr{static_cast<const __nv_bfloat16*>(U), static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(dU), dWp, dQp, dKp,
                static_cast<long>(B) * Hv * L * LK, n_part, static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(Vnew), dcarry,
                dq, dk, static_cast<__nv_bfloat16*>(dq16), static_cast<__nv_bfloat16*>(dk16), qk_tok, static_cast<__nv_bfloat16*>(dvv), dv_tok, dg, dbeta};
  dim3 grid(L / LC, Hv, B);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_local_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(BwdSmem::TOTAL));
    cudaFuncSetAttribute(gdn_local_bwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(BwdSmem::TOTAL));
    cudaFuncSetAttribute(gdn_local_bwd_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(gdn_local_bwd_kernel<256>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attr = true;
  }
  if (dv == 128) gdn_local_bwd_kernel<128><<<grid, 256, BwdSmem::TOTAL, st>>>(in, gr);
  else gdn_local_bwd_kernel<256><<<grid, 256, BwdSmem::TOTAL, st>>>(in, gr);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int gdn_local_fwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, void* U, void* W, void* Aqk, void* Qin, void* Kout,
                  float* carry, cudaStream_t st) {
  if (L % LC || (dv != 128 && dv != 256) || Hv % Hk) return 1;
  LocalIn in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), q_tok, k_tok, v_tok,
             g, beta, start, L, Hv, Hv / Hk};
  dim3 grid(L / LC, Hv, B);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_local_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FwdSmem::TOTAL));
    cudaFuncSetAttribute(gdn_local_fwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(FwdSmem::TOTAL));
    cudaFuncSetAttribute(gdn_local_fwd_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(gdn_local_fwd_kernel<256>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attr = true;
  }
  auto* u = static_cast<__nv_bfloat16*>(U); auto* w = static_cast<__nv_bfloat16*>(W); auto* a = static_cast<__nv_bfloat16*>(Aqk);
  auto* qi = static_cast<__nv_bfloat16*>(Qin); auto* ko = static_cast<__nv_bfloat16*>(Kout);
  if (dv == 128) gdn_local_fwd_kernel<128><<<grid, 256, FwdSmem::TOTAL, st>>>(in, u, w, a, qi, ko, carry);
  else gdn_local_fwd_kernel<256><<<grid, 256, FwdSmem::TOTAL, st>>>(in, u, w, a, qi, ko, carry);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
