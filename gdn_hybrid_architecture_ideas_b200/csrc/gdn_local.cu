// Chunk-local stage of the gated delta rule: everything that does not depend on the state carried between chunks.
//
// Forward, one CTA per (batch row, value head, chunk of 64 tokens), fp32 maths:
//   c_i = cumulative log decay inside the chunk, seg_i = number of document starts at or before i (0 = the document
//   that continues from the previous chunk), E_ij = exp(c_i - c_j) for j <= i in the same segment;
//   A_ij = beta_i (k_i . k_j) E_ij (j < i);  X = (I + A)^-1 [beta v | beta gamma first k] by forward substitution, one
//   column per thread held in registers (columns are independent, so the solve needs no synchronisation);
//   outputs U, W (the two column blocks of X), Aqk_ij = (q_i . k_j) E_ij (j <= i), q_in = q gamma first,
//   k_out = k exp(c_last - c) last, carry = gamma_last if the chunk has no document start else 0.
// These are the operands of the sequential state pass (gdn_scan.cu). Same function as the PyTorch statement
// `reference.chunk_local`; the reference computes it with batched matmuls and solve_triangular
// (ced/model/gdn_chunked.py:100-140) or its Triton kernels for value dimension 128 (ced/kernels/gdn_triton.py:96-374).
#include "kernels.h"
#include <cuda_bf16.h>
#include <cstdlib>

namespace ghb {

constexpr int LC = 64;          // chunk length
constexpr int LK = 128;         // key head dimension
constexpr int KS = 132;         // padded row stride of the fp32 q / k tiles in shared memory
constexpr int AS = 65;          // padded row stride of the 64 x 64 matrices

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

// fp32 tile [64][KS] of one head's rows of q or k for this chunk
__device__ __forceinline__ void load_tile(const __nv_bfloat16* base, long tok_stride, float* tile) {
  for (int idx = threadIdx.x; idx < LC * (LK / 8); idx += blockDim.x) {
    const int row = idx / (LK / 8), c8 = (idx % (LK / 8)) * 8;
    const uint4 pk = *reinterpret_cast<const uint4*>(base + row * tok_stride + c8);
    const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
      tile[row * KS + c8 + 2 * e] = f.x; tile[row * KS + c8 + 2 * e + 1] = f.y;
    }
  }
}

// acc[ii][jj] = sum_kk X[i][kk] * Y[j][kk] for i = ty + 16 ii, j = tx + 16 jj (interleaved rows: conflict-free float4 loads)
__device__ __forceinline__ void tile_dot(const float* X, const float* Y, int ty, int tx, float (&acc)[4][4]) {
#pragma unroll
  for (int ii = 0; ii < 4; ++ii)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.f;
#pragma unroll 4
  for (int kk = 0; kk < LK; kk += 4) {
    float4 a[4], bq[4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) a[ii] = *reinterpret_cast<const float4*>(X + (ty + 16 * ii) * KS + kk);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) bq[jj] = *reinterpret_cast<const float4*>(Y + (tx + 16 * jj) * KS + kk);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        acc[ii][jj] += a[ii].x * bq[jj].x + a[ii].y * bq[jj].y + a[ii].z * bq[jj].z + a[ii].w * bq[jj].w;
  }
}

template <int DV>
__global__ void __launch_bounds__(256)
gdn_local_fwd_kernel(LocalIn in, __nv_bfloat16* __restrict__ U, __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ Aqk,
                     __nv_bfloat16* __restrict__ Qin, __nv_bfloat16* __restrict__ Kout, float* __restrict__ carry) {
  extern __shared__ __align__(16) float sm[];
  float* sK = sm;                       // [64][KS]
  float* sQ = sK + LC * KS;             // [64][KS]
  float* sA = sQ + LC * KS;             // [64][AS]
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(sA + LC * AS);
  __nv_bfloat16* sAq = reinterpret_cast<__nv_bfloat16*>(sc + 1);   // [64][64] staging of Aqk

  const int chunk = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / in.rep;
  const int NT = in.L / LC;
  const long tok0 = static_cast<long>(b) * in.L + chunk * LC;
  const long out_row0 = (static_cast<long>(b) * in.Hv + hv) * in.L + chunk * LC;

  load_scalars(in, b, hv, chunk, sc);
  load_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  load_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  __syncthreads();
  if (threadIdx.x == 0) carry[(static_cast<long>(b) * in.Hv + hv) * NT + chunk] = sc->carry;

  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  {
    float kk[4][4], qk[4][4];
    tile_dot(sK, sK, ty, tx, kk);
    tile_dot(sQ, sK, ty, tx, qk);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int i = ty + 16 * ii, j = tx + 16 * jj;
        const bool same = sc->seg[i] == sc->seg[j];
        const float e = (j <= i && same) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
        sA[i * AS + j] = (j < i) ? sc->beta[i] * kk[ii][jj] * e : 0.f;
        sAq[i * LC + j] = __float2bfloat16(qk[ii][jj] * e);
      }
  }
  __syncthreads();
  // Aqk, q_in, k_out (coalesced bf16 rows)
  for (int idx = threadIdx.x; idx < LC * LC / 8; idx += blockDim.x)
    reinterpret_cast<uint4*>(Aqk + out_row0 * LC)[idx] = reinterpret_cast<const uint4*>(sAq)[idx];
  for (int idx = threadIdx.x; idx < LC * LK / 2; idx += blockDim.x) {
    const int row = idx / (LK / 2), c2 = (idx % (LK / 2)) * 2;
    const float fq = sc->seg[row] == 0 ? sc->gamma[row] : 0.f;
    const float fk = sc->seg[row] == sc->last_seg ? sc->to_end[row] : 0.f;
    reinterpret_cast<__nv_bfloat162*>(Qin + (out_row0 + row) * LK)[c2 / 2] = __floats2bfloat162_rn(sQ[row * KS + c2] * fq, sQ[row * KS + c2 + 1] * fq);
    reinterpret_cast<__nv_bfloat162*>(Kout + (out_row0 + row) * LK)[c2 / 2] = __floats2bfloat162_rn(sK[row * KS + c2] * fk, sK[row * KS + c2 + 1] * fk);
  }
  // forward substitution, one column of [U | W] per thread (a second column for the first DV + 128 - 256 threads)
  constexpr int COLS = DV + LK;
#pragma unroll 1
  for (int rep = 0; rep < (COLS + 255) / 256; ++rep) {
    const int col = rep * 256 + threadIdx.x;
    if (col >= COLS) break;
    float x[LC];
    if (col < DV) {
      const __nv_bfloat16* vp = in.v + tok0 * in.v_tok + static_cast<long>(hv) * DV + col;
#pragma unroll
      for (int i = 0; i < LC; ++i) x[i] = sc->beta[i] * __bfloat162float(vp[i * in.v_tok]);
    } else {
#pragma unroll
      for (int i = 0; i < LC; ++i) x[i] = sc->seg[i] == 0 ? sc->beta[i] * sc->gamma[i] * sK[i * KS + (col - DV)] : 0.f;
    }
#pragma unroll
    for (int i = 1; i < LC; ++i) {
      float acc = x[i];
#pragma unroll
      for (int j = 0; j < i; ++j) acc -= sA[i * AS + j] * x[j];
      x[i] = acc;
    }
    if (col < DV) {
#pragma unroll
      for (int i = 0; i < LC; ++i) U[(out_row0 + i) * DV + col] = __float2bfloat16(x[i]);
    } else {
#pragma unroll
      for (int i = 0; i < LC; ++i) W[(out_row0 + i) * LK + (col - DV)] = __float2bfloat16(x[i]);
    }
  }
}

static_assert(sizeof(ChunkScalars) % 16 == 0 && (LC * KS * 4) % 16 == 0 && (LC * AS * 4) % 16 == 0, "16-byte aligned shared-memory carve-up");
constexpr size_t LOCAL_FWD_SMEM = (2 * LC * KS + LC * AS) * sizeof(float) + sizeof(ChunkScalars) + LC * LC * 2 + 64;

int gdn_local_fwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, void* U, void* W, void* Aqk, void* Qin, void* Kout,
                  float* carry, cudaStream_t st) {
  if (L % LC || (dv != 128 && dv != 256) || Hv % Hk) return 1;
  LocalIn in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), q_tok, k_tok, v_tok,
             g, beta, start, L, Hv, Hv / Hk};
  dim3 grid(L / LC, Hv, B);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_local_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_FWD_SMEM));
    cudaFuncSetAttribute(gdn_local_fwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_FWD_SMEM));
    attr = true;
  }
  auto* u = static_cast<__nv_bfloat16*>(U); auto* w = static_cast<__nv_bfloat16*>(W); auto* a = static_cast<__nv_bfloat16*>(Aqk);
  auto* qi = static_cast<__nv_bfloat16*>(Qin); auto* ko = static_cast<__nv_bfloat16*>(Kout);
  if (dv == 128) gdn_local_fwd_kernel<128><<<grid, 256, LOCAL_FWD_SMEM, st>>>(in, u, w, a, qi, ko, carry);
  else gdn_local_fwd_kernel<256><<<grid, 256, LOCAL_FWD_SMEM, st>>>(in, u, w, a, qi, ko, carry);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb

// ================================================================================================ backward
// Gradients of the chunk-local stage, one CTA per (batch row, value head, chunk). Inputs: the forward inputs, the
// forward's outputs X = [U | W], and the gradients of U, W, q_in, k_out, Aqk, carry handed back by the state pass.
//   T = (I + A)^-1 explicitly (one column per thread), then every product is a warp-level tensor-core GEMM
//   (mma.sync m16n8k8, tf32 operands, fp32 accumulation) on fp32 tiles in shared memory:
//   dR = T^T dX per block of 128 columns;  dA = -dR X^T;  A_ij = beta_i G_ij, G = (K K^T) E  ->  dbeta, dc, dKK = dG E;
//   Aqk = (Q K^T) E -> dQK, dc;  dk = (dKK + dKK^T) K + dQK^T Q + diagonal terms, dq = dQK K + diagonal term,
//   dv = beta dR_u, dg = reverse cumulative sum of dc.
namespace ghb {

constexpr int BS = 68;          // padded row stride of the 64 x 64 matrices of the backward kernel

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
// One warp accumulates a 16 x (8 NT) tile: acc[nt] += A(16 x K) B(K x 8 nt). A points at the tile's first row, B at its first
// column. A_T: A(m, k) is stored at A[k * lda + m] (else A[m * lda + k]). B_K: B(k, n) is stored at B[k * ldb + n] (else B[n * ldb + k]).
// Fragment layout of mma.m16n8k8: g = lane / 4, t = lane % 4; a0 (g, t) a1 (g+8, t) a2 (g, t+4) a3 (g+8, t+4); b0 (t, g) b1 (t+4, g);
// c0 (g, 2t) c1 (g, 2t+1) c2 (g+8, 2t) c3 (g+8, 2t+1).
template <int NT, bool A_T, bool B_K>
__device__ __forceinline__ void warp_gemm(const float* A, int lda, const float* B, int ldb, int K, float (&acc)[NT][4], int lane) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll 2
  for (int k0 = 0; k0 < K; k0 += 8) {
    uint32_t a[4];
    if (A_T) {
      a[0] = to_tf32(A[(k0 + t) * lda + g]); a[1] = to_tf32(A[(k0 + t) * lda + g + 8]);
      a[2] = to_tf32(A[(k0 + t + 4) * lda + g]); a[3] = to_tf32(A[(k0 + t + 4) * lda + g + 8]);
    } else {
      a[0] = to_tf32(A[g * lda + k0 + t]); a[1] = to_tf32(A[(g + 8) * lda + k0 + t]);
      a[2] = to_tf32(A[g * lda + k0 + t + 4]); a[3] = to_tf32(A[(g + 8) * lda + k0 + t + 4]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      uint32_t b0, b1;
      if (B_K) { b0 = to_tf32(B[(k0 + t) * ldb + nt * 8 + g]); b1 = to_tf32(B[(k0 + t + 4) * ldb + nt * 8 + g]); }
      else { b0 = to_tf32(B[(nt * 8 + g) * ldb + k0 + t]); b1 = to_tf32(B[(nt * 8 + g) * ldb + k0 + t + 4]); }
      mma_tf32(acc[nt], a, b0, b1);
    }
  }
}
template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])); f[2 * e] = v.x; f[2 * e + 1] = v.y; }
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

template <int DV>
__global__ void __launch_bounds__(256, 1)
gdn_local_bwd_kernel(LocalIn in, LocalGrads gr) {
  extern __shared__ __align__(16) float sm[];
  float* sK = sm;                       // [64][KS]
  float* sQ = sK + LC * KS;             // [64][KS] (also the staging of dX blocks)
  float* sDR = sQ + LC * KS;            // dR block [64][KS]
  float* sX = sDR + LC * KS;            // X block  [64][KS]
  float* sG = sX + LC * KS;             // G, later S = dKK + dKK^T   [64][BS]
  float* sAq = sG + LC * BS;            // Aqk, later dQK             [64][BS]
  float* sT = sAq + LC * BS;            // T = (I + A)^-1, later dA   [64][BS]
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(sT + LC * BS);
  float* sdc = reinterpret_cast<float*>(sc + 1);   // [64] decay gradient
  float* sdb = sdc + LC;                            // [64] beta gradient

  const int chunk = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / in.rep;
  const int NT_ = in.L / LC;
  const long tok0 = static_cast<long>(b) * in.L + chunk * LC;
  const long row0 = (static_cast<long>(b) * in.Hv + hv) * in.L + chunk * LC;     // rows of the [B, H, L, *] operands
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = (warp & 3) * 16;                  // this warp's 16 output rows in every product

  load_scalars(in, b, hv, chunk, sc);
  load_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  load_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  if (t < LC) { sdc[t] = 0.f; sdb[t] = 0.f; }
  __syncthreads();
  {   // G = (K K^T) E (strictly lower), Aqk = (Q K^T) E (lower): warp tile 16 x 32
    const int n0 = (warp >> 2) * 32;
    float kk[4][4], qk[4][4];
    zero_acc(kk); zero_acc(qk);
    warp_gemm<4, false, false>(sK + m0 * KS, KS, sK + n0 * KS, KS, LK, kk, lane);
    warp_gemm<4, false, false>(sQ + m0 * KS, KS, sK + n0 * KS, KS, LK, qk, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + nt * 8 + 2 * tq + (e & 1);
        const float ex = (j <= i && sc->seg[i] == sc->seg[j]) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
        sG[i * BS + j] = (j < i) ? kk[nt][e] * ex : 0.f;
        sAq[i * BS + j] = qk[nt][e] * ex;
      }
  }
  __syncthreads();
  // ---- T = (I + A)^-1, one column per thread (threads 0..63): x_c = 1, x_i = -beta_i sum_{m < i} G_im x_m
  if (t < LC) {
    float x[LC];
#pragma unroll
    for (int i = 0; i < LC; ++i) x[i] = (i == t) ? 1.f : 0.f;
#pragma unroll
    for (int i = 1; i < LC; ++i) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int m = 0; m + 1 < i; m += 2) { a0 += sG[i * BS + m] * x[m]; a1 += sG[i * BS + m + 1] * x[m + 1]; }
      if (i & 1) a0 += sG[i * BS + i - 1] * x[i - 1];
      x[i] -= sc->beta[i] * (a0 + a1);
    }
#pragma unroll
    for (int i = 0; i < LC; ++i) sT[i * BS + t] = x[i];
  }
  __syncthreads();

  constexpr int COLS = DV + LK;
  constexpr int NP = DV / 128;      // one partial sum per 128-wide value slice of the state pass
  float* sDX = sQ;      // the q tile is not needed again until the outputs; it is reloaded there
  // ---- dAqk = dO v_new^T over the value dimension, 128 columns at a time (warp tile 16 x 32), kept in registers
  float dAq[4][4];
  zero_acc(dAq);
#pragma unroll 1
  for (int vb = 0; vb < DV / 128; ++vb) {
    for (int idx = t; idx < LC * 16; idx += 256) {
      const int row = idx >> 4, c8 = (idx & 15) * 8;
      float fa[8], fb[8];
      load8(gr.dO + ((tok0 + row) * in.Hv + hv) * DV + vb * 128 + c8, fa);
      load8(gr.Vnew + (row0 + row) * DV + vb * 128 + c8, fb);
      *reinterpret_cast<float4*>(sDR + row * KS + c8) = make_float4(fa[0], fa[1], fa[2], fa[3]);
      *reinterpret_cast<float4*>(sDR + row * KS + c8 + 4) = make_float4(fa[4], fa[5], fa[6], fa[7]);
      *reinterpret_cast<float4*>(sX + row * KS + c8) = make_float4(fb[0], fb[1], fb[2], fb[3]);
      *reinterpret_cast<float4*>(sX + row * KS + c8 + 4) = make_float4(fb[4], fb[5], fb[6], fb[7]);
    }
    __syncthreads();
    warp_gemm<4, false, false>(sDR + m0 * KS, KS, sX + (warp >> 2) * 32 * KS, KS, 128, dAq, lane);
    __syncthreads();
  }
  // ---- per block of 128 columns of [U | W]: dR = T^T dX (warp tile 16 x 64), dA += dR X^T (warp tile 16 x 32)
  float dA[4][4];
  zero_acc(dA);
#pragma unroll 1
  for (int blk = 0; blk < COLS / 128; ++blk) {
    const bool is_u = blk * 128 < DV;
    const int c0 = is_u ? blk * 128 : 0;
    const __nv_bfloat16* xx = is_u ? gr.U + row0 * DV + c0 : gr.W + row0 * LK;
    const int ld = is_u ? DV : LK;
    for (int idx = t; idx < LC * 16; idx += 256) {          // 64 rows x 16 vectors of 8
      const int row = idx >> 4, c8 = (idx & 15) * 8;
      float fa[8], fb[8];
      load8(xx + static_cast<long>(row) * ld + c8, fb);
      if (is_u) load8(gr.dU + (row0 + row) * DV + c0 + c8, fa);
      else sum8<NP>(gr.dWp + (row0 + row) * LK + c8, gr.part_stride, fa);
      *reinterpret_cast<float4*>(sDX + row * KS + c8) = make_float4(fa[0], fa[1], fa[2], fa[3]);
      *reinterpret_cast<float4*>(sDX + row * KS + c8 + 4) = make_float4(fa[4], fa[5], fa[6], fa[7]);
      *reinterpret_cast<float4*>(sX + row * KS + c8) = make_float4(fb[0], fb[1], fb[2], fb[3]);
      *reinterpret_cast<float4*>(sX + row * KS + c8 + 4) = make_float4(fb[4], fb[5], fb[6], fb[7]);
    }
    __syncthreads();
    {
      const int n0 = (warp >> 2) * 64;
      float dr[8][4];
      zero_acc(dr);
      warp_gemm<8, true, true>(sT + m0, BS, sDX + n0, KS, LC, dr, lane);      // A(i, j) = T[j][i], B(j, col) = dX[j][col]
      // dv = beta dR_u ; dbeta += dR_u . v ; stage dR
      float pb0 = 0.f, pb1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = m0 + g + (e >> 1) * 8, col = n0 + nt * 8 + 2 * tq + (e & 1);
          const float v = dr[nt][e];
          sDR[i * KS + col] = v;
          if (is_u) {
            const long vidx = (tok0 + i) * in.v_tok + static_cast<long>(hv) * DV + c0 + col;
            const float pv = v * __bfloat162float(in.v[vidx]);
            if (e >> 1) pb1 += pv; else pb0 += pv;
            gr.dv[(tok0 + i) * gr.dv_tok + static_cast<long>(hv) * DV + c0 + col] = __float2bfloat16(sc->beta[i] * v);
          }
        }
      if (is_u) {      // reduce over the 4 lanes that share a row, then one shared atomic per row per warp
        pb0 += __shfl_xor_sync(0xffffffffu, pb0, 1); pb0 += __shfl_xor_sync(0xffffffffu, pb0, 2);
        pb1 += __shfl_xor_sync(0xffffffffu, pb1, 1); pb1 += __shfl_xor_sync(0xffffffffu, pb1, 2);
        if (tq == 0) { atomicAdd(&sdb[m0 + g], pb0); atomicAdd(&sdb[m0 + g + 8], pb1); }
      }
    }
    __syncthreads();
    warp_gemm<4, false, false>(sDR + m0 * KS, KS, sX + (warp >> 2) * 32 * KS, KS, 128, dA, lane);   // dR X^T
    __syncthreads();
  }
  // sDR / sX now hold the W columns: dR_w [i][kk] and W [i][kk]. Reload q (its buffer staged dX).
  load_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);

  // ---- score matrices: beta / decay gradients; then sT <- dKK (lower), sAq <- dQK
  {
    const int n0 = (warp >> 2) * 32;
    float dKKv[4][4], dQKv[4][4];
    float rb[2] = {0.f, 0.f}, rc[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + nt * 8 + 2 * tq + (e & 1);
        const bool same = sc->seg[i] == sc->seg[j];
        const float ex = (j <= i && same) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
        const float G = sG[i * BS + j];
        const float da = (j < i && same) ? -dA[nt][e] : 0.f;
        const float dG = da * sc->beta[i];
        const float t1 = dG * G;
        const float dq_ij = (j <= i && same) ? dAq[nt][e] : 0.f;
        const float t2 = dq_ij * sAq[i * BS + j];
        rb[e >> 1] += da * G;
        rc[e >> 1] += t1 + t2;
        atomicAdd(&sdc[j], -(t1 + t2));
        dKKv[nt][e] = dG * ex;
        dQKv[nt][e] = dq_ij * ex;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rb[h] += __shfl_xor_sync(0xffffffffu, rb[h], 1); rb[h] += __shfl_xor_sync(0xffffffffu, rb[h], 2);
      rc[h] += __shfl_xor_sync(0xffffffffu, rc[h], 1); rc[h] += __shfl_xor_sync(0xffffffffu, rc[h], 2);
      if (tq == 0) { atomicAdd(&sdb[m0 + g + 8 * h], rb[h]); atomicAdd(&sdc[m0 + g + 8 * h], rc[h]); }
    }
    __syncthreads();     // every reader of sG / sAq / sT (old contents) is done
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = m0 + g + (e >> 1) * 8, j = n0 + nt * 8 + 2 * tq + (e & 1);
        sT[i * BS + j] = dKKv[nt][e];
        sAq[i * BS + j] = dQKv[nt][e];
      }
  }
  __syncthreads();
  for (int idx = t; idx < LC * LC; idx += 256) {      // S = dKK + dKK^T (dKK is strictly lower)
    const int i = idx >> 6, j = idx & 63;
    sG[i * BS + j] = sT[i * BS + j] + sT[j * BS + i];
  }
  __syncthreads();

  // ---- outputs: dk = S K + dQK^T Q + diagonal terms ; dq = dQK K + diagonal term (warp tile 16 x 64)
  {
    const int n0 = (warp >> 2) * 64;
    float dk[8][4], dq[8][4];
    zero_acc(dk); zero_acc(dq);
    float2 pq[2][8], pk[2][8];          // the state pass's dq_in / dk_out, fetched ahead of the products that hide their latency
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const long at = (row0 + m0 + g + 8 * h) * LK + n0 + nt * 8 + 2 * tq;
        pq[h][nt] = sum2<NP>(gr.dQp + at, gr.part_stride);
        pk[h][nt] = sum2<NP>(gr.dKp + at, gr.part_stride);
      }
    warp_gemm<8, false, true>(sG + m0 * BS, BS, sK + n0, KS, LC, dk, lane);       // S K
    warp_gemm<8, true, true>(sAq + m0, BS, sQ + n0, KS, LC, dk, lane);           // dQK^T Q : A(r, i) = dQK[i][r]
    warp_gemm<8, false, true>(sAq + m0 * BS, BS, sK + n0, KS, LC, dq, lane);      // dQK K
    float dots[2][3] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = m0 + g + 8 * h;
      const float fq = sc->seg[r] == 0 ? sc->gamma[r] : 0.f;                       // q_in = q fq ; W rhs = beta fq k
      const float fk = sc->seg[r] == sc->last_seg ? sc->to_end[r] : 0.f;           // k_out = k fk
      const float br = sc->beta[r];
      float* dqo = gr.dq16 ? nullptr : gr.dq + ((tok0 + r) * in.Hv + hv) * LK;
      float* dko = gr.dq16 ? nullptr : gr.dk + ((tok0 + r) * in.Hv + hv) * LK;
      __nv_bfloat16* dqh = gr.dq16 ? gr.dq16 + (tok0 + r) * gr.qk_tok + static_cast<long>(hv) * LK : nullptr;
      __nv_bfloat16* dkh = gr.dq16 ? gr.dk16 + (tok0 + r) * gr.qk_tok + static_cast<long>(hv) * LK : nullptr;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int kk = n0 + nt * 8 + 2 * tq;
        const float2 drw = *reinterpret_cast<const float2*>(sDR + r * KS + kk);
        const float2 kre = *reinterpret_cast<const float2*>(sK + r * KS + kk);
        const float2 qre = *reinterpret_cast<const float2*>(sQ + r * KS + kk);
        const float2 dqi = pq[h][nt], dkv = pk[h][nt];
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

// ================================================================================================ backward, bf16 tiles
// Same function as gdn_local_bwd_kernel on bf16 shared-memory tiles: operands that are bf16 in memory (K, Q, U, W, dU,
// dO, v_new) are copied as they are and fed to mma.sync m16n8k16 through ldmatrix (plain or transposed, so no tile is
// ever stored twice); T = (I + A)^-1 comes from a blocked inverse (16 x 16 diagonal blocks by substitution, then two
// merge levels of small tf32 products, the form ced/kernels/gdn_triton.py:133-325 uses) and enters its products as a
// bf16 pair (value + residual). Shared memory 107 KB and at most 128 registers: two CTAs per SM.
constexpr int TS = 136;         // row stride (elements) of the 64 x 128 bf16 tiles: 272 bytes, conflict-free for ldmatrix
constexpr int MS = 72;          // row stride (elements) of the 64 x 64 bf16 matrices

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

struct Bwd2Smem {
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
gdn_local_bwd2_kernel(LocalIn in, LocalGrads gr) {
  extern __shared__ __align__(16) unsigned char smb[];
  using S = Bwd2Smem;
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

constexpr size_t LOCAL_BWD_SMEM = (4 * LC * KS + 3 * LC * BS + 2 * LC) * sizeof(float) + sizeof(ChunkScalars) + 64;

int gdn_local_bwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, const void* U, const void* W, const void* dU,
                  const float* dWp, const float* dQp, const float* dKp, int n_part, const void* dO, const void* Vnew, const float* dcarry,
                  float* dq, float* dk, void* dq16, void* dk16, long qk_tok, void* dvv, long dv_tok, float* dg, float* dbeta, cudaStream_t st) {
  if (L % LC || (dv != 128 && dv != 256) || Hv % Hk || n_part != dv / 128) return 1;
  if (dq16 ? (Hv != Hk || !dk16 || qk_tok % 2) : (!dq || !dk)) return 1;
  LocalIn in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), q_tok, k_tok, v_tok,
             g, beta, start, L, Hv, Hv / Hk};
  LocalGrads gr{static_cast<const __nv_bfloat16*>(U), static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(dU), dWp, dQp, dKp,
                static_cast<long>(B) * Hv * L * LK, n_part, static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(Vnew), dcarry,
                dq, dk, static_cast<__nv_bfloat16*>(dq16), static_cast<__nv_bfloat16*>(dk16), qk_tok, static_cast<__nv_bfloat16*>(dvv), dv_tok, dg, dbeta};
  dim3 grid(L / LC, Hv, B);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_local_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_BWD_SMEM));
    cudaFuncSetAttribute(gdn_local_bwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_BWD_SMEM));
    attr = true;
  }
  static int version = 0;
  if (!version) { const char* e = getenv("GHB_GDN_LOCAL"); version = (e && e[0] == '1') ? 1 : 2; }
  if (version == 2) {
    static bool attr2 = false;
    if (!attr2) {
      cudaFuncSetAttribute(gdn_local_bwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Bwd2Smem::TOTAL));
      cudaFuncSetAttribute(gdn_local_bwd2_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Bwd2Smem::TOTAL));
      cudaFuncSetAttribute(gdn_local_bwd2_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      cudaFuncSetAttribute(gdn_local_bwd2_kernel<256>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      attr2 = true;
    }
    if (dv == 128) gdn_local_bwd2_kernel<128><<<grid, 256, Bwd2Smem::TOTAL, st>>>(in, gr);
    else gdn_local_bwd2_kernel<256><<<grid, 256, Bwd2Smem::TOTAL, st>>>(in, gr);
    return cudaGetLastError() == cudaSuccess ? 0 : 4;
  }
  if (dv == 128) gdn_local_bwd_kernel<128><<<grid, 256, LOCAL_BWD_SMEM, st>>>(in, gr);
  else gdn_local_bwd_kernel<256><<<grid, 256, LOCAL_BWD_SMEM, st>>>(in, gr);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
