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
// Gradients of the chunk-local stage, one CTA per (batch row, value head, chunk). Inputs: the forward inputs and the
// gradients of U, W, q_in, k_out, Aqk, carry handed back by the state pass. The forward quantities are recomputed.
//   solve:   X = (I + A)^-1 R (as forward), dR = (I + A)^-T dX by back substitution (column per thread, registers);
//            dA_ij = -sum_col dR_i X_j, accumulated by a tiled product over staged column blocks;
//   scores:  A_ij = beta_i G_ij, G_ij = (k_i.k_j) E_ij  ->  dbeta, dc (decay), dKK = dG E;  Aqk likewise -> dQK, dc;
//   outputs: dk = (dKK + dKK^T) K + dQK^T Q + diagonal terms, dq = dQK K + diagonal term, dv = beta dR_u,
//            dg = reverse cumulative sum of dc, dbeta.
namespace ghb {

struct LocalGrads {
  const __nv_bfloat16* U; const __nv_bfloat16* W;       // the forward's outputs (X = [U | W])
  const __nv_bfloat16* dU; const __nv_bfloat16* dW; const __nv_bfloat16* dQin; const __nv_bfloat16* dKout; const __nv_bfloat16* dAqk;
  const float* dcarry;
  float* dq; float* dk;            // [B, L, Hv, 128] fp32 (per value head; heads sharing a key head are summed by the caller)
  __nv_bfloat16* dv;               // [B, L, Hv, DV]
  float* dg; float* dbeta;         // [B, L, Hv]
};

__device__ __forceinline__ void tile_dot_acc(const float* X, const float* Y, int ty, int tx, float (&acc)[4][4]) {
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
__global__ void __launch_bounds__(256, 1)
gdn_local_bwd_kernel(LocalIn in, LocalGrads gr) {
  extern __shared__ __align__(16) float sm[];
  float* sK = sm;
  float* sQ = sK + LC * KS;
  float* sDR = sQ + LC * KS;            // staged dR columns [64][KS]
  float* sX = sDR + LC * KS;            // staged X columns  [64][KS]
  float* sG = sX + LC * KS;             // G, later dKK      [64][AS]
  float* sAq = sG + LC * AS;            // Aqk, later dQK    [64][AS]
  float* sT = sAq + LC * AS;            // T = (I + A)^-1    [64][AS]
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(sT + LC * AS);
  float* sdc = reinterpret_cast<float*>(sc + 1);   // [64] decay gradient
  float* sdb = sdc + LC;                            // [64] beta gradient

  const int chunk = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / in.rep;
  const int NT = in.L / LC;
  const long tok0 = static_cast<long>(b) * in.L + chunk * LC;
  const long row0 = (static_cast<long>(b) * in.Hv + hv) * in.L + chunk * LC;     // rows of the [B, H, L, *] operands
  const int t = threadIdx.x, lane = t & 31;
  const int ty = t >> 4, tx = t & 15;

  load_scalars(in, b, hv, chunk, sc);
  load_tile(in.k + tok0 * in.k_tok + hk * LK, in.k_tok, sK);
  load_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  if (t < LC) { sdc[t] = 0.f; sdb[t] = 0.f; }
  __syncthreads();
  {
    float kk[4][4], qk[4][4];
    tile_dot(sK, sK, ty, tx, kk);
    tile_dot(sQ, sK, ty, tx, qk);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int i = ty + 16 * ii, j = tx + 16 * jj;
        const float e = (j <= i && sc->seg[i] == sc->seg[j]) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
        sG[i * AS + j] = (j < i) ? kk[ii][jj] * e : 0.f;
        sAq[i * AS + j] = qk[ii][jj] * e;
      }
  }
  __syncthreads();

  // ---- T = (I + A)^-1, one column per thread (threads 0..63): x_c = 1, x_i = -sum_{m < i} A_im x_m
  if (t < LC) {
    float x[LC];
#pragma unroll
    for (int i = 0; i < LC; ++i) x[i] = (i == t) ? 1.f : 0.f;
#pragma unroll
    for (int i = 1; i < LC; ++i) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int m = 0; m + 1 < i; m += 2) { a0 += sG[i * AS + m] * x[m]; a1 += sG[i * AS + m + 1] * x[m + 1]; }
      if (i & 1) a0 += sG[i * AS + i - 1] * x[i - 1];
      x[i] -= sc->beta[i] * (a0 + a1);
    }
#pragma unroll
    for (int i = 0; i < LC; ++i) sT[i * AS + t] = x[i];
  }
  __syncthreads();

  // ---- per block of 128 columns of [U | W]: X from the forward's outputs, dR = T^T dX, dA -= dR X^T
  float dA[4][4];
#pragma unroll
  for (int ii = 0; ii < 4; ++ii)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) dA[ii][jj] = 0.f;
  constexpr int COLS = DV + LK;
  float* sDX = sQ;      // the q tile is not needed again until the outputs; it is reloaded there
#pragma unroll 1
  for (int blk = 0; blk < COLS / 128; ++blk) {
    const bool is_u = blk * 128 < DV;
    const int c0 = is_u ? blk * 128 : 0;
    const __nv_bfloat16* gx = is_u ? gr.dU + row0 * DV + c0 : gr.dW + row0 * LK;
    const __nv_bfloat16* xx = is_u ? gr.U + row0 * DV + c0 : gr.W + row0 * LK;
    const int ld = is_u ? DV : LK;
    for (int idx = t; idx < LC * 16; idx += 256) {          // 64 rows x 16 vectors of 8
      const int row = idx >> 4, c8 = (idx & 15) * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(gx + static_cast<long>(row) * ld + c8);
      const uint4 bq = *reinterpret_cast<const uint4*>(xx + static_cast<long>(row) * ld + c8);
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wa[e]));
        const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wb[e]));
        sDX[row * KS + c8 + 2 * e] = fa.x; sDX[row * KS + c8 + 2 * e + 1] = fa.y;
        sX[row * KS + c8 + 2 * e] = fb.x; sX[row * KS + c8 + 2 * e + 1] = fb.y;
      }
    }
    __syncthreads();
    {
      const int col = t & 127, i0 = (t >> 7) * 32;          // 32 rows of one column per thread
      float acc[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] = 0.f;
      for (int j = i0; j < LC; ++j) {                          // dR_i = sum_{j >= i} T_ji dX_j
        const float d = sDX[j * KS + col];
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[e] += sT[j * AS + i0 + e] * d;
      }
      if (is_u) {      // dv = beta dR_u ; dbeta += dR_u . v
        const __nv_bfloat16* vp = in.v + tok0 * in.v_tok + static_cast<long>(hv) * DV + c0 + col;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int i = i0 + e;
          gr.dv[(tok0 + i) * in.Hv * DV + static_cast<long>(hv) * DV + c0 + col] = __float2bfloat16(sc->beta[i] * acc[e]);
          float p = acc[e] * __bfloat162float(vp[i * in.v_tok]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
          if (lane == 0) atomicAdd(&sdb[i], p);
        }
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) sDR[(i0 + e) * KS + col] = acc[e];
    }
    __syncthreads();
    tile_dot_acc(sDR, sX, ty, tx, dA);
    __syncthreads();
  }
  load_tile(in.q + tok0 * in.q_tok + hk * LK, in.q_tok, sQ);
  __syncthreads();   // sDR / sX now hold the W columns: dR_w [i][kk] and W [i][kk]

  // ---- score matrices: beta / decay gradients, then overwrite sG <- dKK, sAq <- dQK
  {
    float dGs[4][4], dQs[4][4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int i = ty + 16 * ii;
      float rb = 0.f, rc = 0.f;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = tx + 16 * jj;
        const bool same = sc->seg[i] == sc->seg[j];
        const float e = (j <= i && same) ? __expf(sc->c[i] - sc->c[j]) : 0.f;
        const float G = sG[i * AS + j];
        const float da = (j < i && same) ? -dA[ii][jj] : 0.f;
        rb += da * G;
        const float dG = da * sc->beta[i];
        const float t1 = dG * G;
        const float dq_ij = (j <= i && same) ? __bfloat162float(gr.dAqk[(row0 + i) * LC + j]) : 0.f;
        const float t2 = dq_ij * sAq[i * AS + j];
        rc += t1 + t2;
        atomicAdd(&sdc[j], -(t1 + t2));
        dGs[ii][jj] = dG * e;
        dQs[ii][jj] = dq_ij * e;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) { rb += __shfl_xor_sync(0xffffffffu, rb, o); rc += __shfl_xor_sync(0xffffffffu, rc, o); }
      if (tx == 0) { atomicAdd(&sdb[i], rb); atomicAdd(&sdc[i], rc); }
    }
    __syncthreads();
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int i = ty + 16 * ii, j = tx + 16 * jj;
        sG[i * AS + j] = dGs[ii][jj];
        sAq[i * AS + j] = dQs[ii][jj];
      }
  }
  __syncthreads();

  // ---- outputs: thread owns row r and 32 consecutive key channels
  {
    const int r = t >> 2, k0 = (t & 3) * 32;
    float dk[32], dq[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) { dk[e] = 0.f; dq[e] = 0.f; }
    for (int i = 0; i < LC; ++i) {
      const float s_ri = i < r ? sG[r * AS + i] : (i > r ? sG[i * AS + r] : 0.f);      // (dKK + dKK^T)[r][i]
      const float qk_ir = i >= r ? sAq[i * AS + r] : 0.f;                                // dQK[i][r]
      const float qk_ri = i <= r ? sAq[r * AS + i] : 0.f;                                // dQK[r][i]
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(sK + i * KS + k0 + e);
        const float4 qv = *reinterpret_cast<const float4*>(sQ + i * KS + k0 + e);
        dk[e] += s_ri * kv.x + qk_ir * qv.x; dk[e + 1] += s_ri * kv.y + qk_ir * qv.y;
        dk[e + 2] += s_ri * kv.z + qk_ir * qv.z; dk[e + 3] += s_ri * kv.w + qk_ir * qv.w;
        dq[e] += qk_ri * kv.x; dq[e + 1] += qk_ri * kv.y; dq[e + 2] += qk_ri * kv.z; dq[e + 3] += qk_ri * kv.w;
      }
    }
    const float fq = sc->seg[r] == 0 ? sc->gamma[r] : 0.f;                       // q_in = q fq ; W rhs = beta fq k
    const float fk = sc->seg[r] == sc->last_seg ? sc->to_end[r] : 0.f;           // k_out = k fk
    const float br = sc->beta[r];
    float dot_w = 0.f, dot_q = 0.f, dot_k = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float kre = sK[r * KS + k0 + e], qre = sQ[r * KS + k0 + e];
      const float drw = sDR[r * KS + k0 + e];
      const float dqi = __bfloat162float(gr.dQin[(row0 + r) * LK + k0 + e]);
      const float dko = __bfloat162float(gr.dKout[(row0 + r) * LK + k0 + e]);
      dk[e] += br * fq * drw + fk * dko;
      dq[e] += fq * dqi;
      dot_w += drw * kre; dot_q += dqi * qre; dot_k += dko * kre;
    }
#pragma unroll
    for (int o = 2; o > 0; o >>= 1) {
      dot_w += __shfl_xor_sync(0xffffffffu, dot_w, o); dot_q += __shfl_xor_sync(0xffffffffu, dot_q, o); dot_k += __shfl_xor_sync(0xffffffffu, dot_k, o);
    }
    if ((t & 3) == 0) {
      atomicAdd(&sdb[r], fq * dot_w);
      atomicAdd(&sdc[r], br * fq * dot_w + fq * dot_q - fk * dot_k);
      atomicAdd(&sdc[LC - 1], fk * dot_k);
    }
    float* dqo = gr.dq + ((tok0 + r) * in.Hv + hv) * LK + k0;
    float* dko_ = gr.dk + ((tok0 + r) * in.Hv + hv) * LK + k0;
#pragma unroll
    for (int e = 0; e < 32; e += 4) {
      *reinterpret_cast<float4*>(dqo + e) = make_float4(dq[e], dq[e + 1], dq[e + 2], dq[e + 3]);
      *reinterpret_cast<float4*>(dko_ + e) = make_float4(dk[e], dk[e + 1], dk[e + 2], dk[e + 3]);
    }
  }
  __syncthreads();
  if (t == 0) {
    sdc[LC - 1] += sc->carry * gr.dcarry[(static_cast<long>(b) * in.Hv + hv) * NT + chunk];
    float acc = 0.f;
    for (int i = LC - 1; i >= 0; --i) { acc += sdc[i]; sdc[i] = acc; }      // dg_m = sum_{i >= m} dc_i
  }
  __syncthreads();
  if (t < LC) {
    gr.dg[(tok0 + t) * in.Hv + hv] = sdc[t];
    gr.dbeta[(tok0 + t) * in.Hv + hv] = sdb[t];
  }
}

constexpr size_t LOCAL_BWD_SMEM = (4 * LC * KS + 3 * LC * AS + 2 * LC) * sizeof(float) + sizeof(ChunkScalars) + 64;

int gdn_local_bwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, const void* U, const void* W, const void* dU, const void* dW, const void* dQin,
                  const void* dKout, const void* dAqk, const float* dcarry, float* dq, float* dk, void* dvv, float* dg, float* dbeta,
                  cudaStream_t st) {
  if (L % LC || (dv != 128 && dv != 256) || Hv % Hk) return 1;
  LocalIn in{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), q_tok, k_tok, v_tok,
             g, beta, start, L, Hv, Hv / Hk};
  LocalGrads gr{static_cast<const __nv_bfloat16*>(U), static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(dU), static_cast<const __nv_bfloat16*>(dW), static_cast<const __nv_bfloat16*>(dQin),
                static_cast<const __nv_bfloat16*>(dKout), static_cast<const __nv_bfloat16*>(dAqk), dcarry, dq, dk,
                static_cast<__nv_bfloat16*>(dvv), dg, dbeta};
  dim3 grid(L / LC, Hv, B);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_local_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_BWD_SMEM));
    cudaFuncSetAttribute(gdn_local_bwd_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(LOCAL_BWD_SMEM));
    attr = true;
  }
  if (dv == 128) gdn_local_bwd_kernel<128><<<grid, 256, LOCAL_BWD_SMEM, st>>>(in, gr);
  else gdn_local_bwd_kernel<256><<<grid, 256, LOCAL_BWD_SMEM, st>>>(in, gr);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
