// Fused model-specific kernels: GDN input preparation (causal document-masked conv + SiLU + L2 norm), the depth-mix
// softmax combine over finished blocks, and the cross-entropy gradient of one chunk of logits.
//
// Reference behaviour: ced/model/gdn.py:218-258, 692-699 (conv taps of another document contribute nothing; q, k
// L2-normalised with eps 1e-6, q scaled by dk^-0.5); ced/model/attn_res.py:457-482 (logit = (v . w(1+g)) rsqrt(mean
// v^2 + eps), softmax over sources, weighted sum, >= fp32); ced/train/fused_head.py:56-110 (online LSE over the
// vocabulary; logits overwritten by softmax * (a + 2 b lse) - a onehot).
#include "kernels.h"
#include <cuda_bf16.h>

namespace ghb {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Special-function instructions in their flush-to-zero forms: one issue slot each (the default forms add denormal
// scaling around them, and a full-precision division costs an order of magnitude more; the elementwise kernels here are
// issue-bound). Relative error of a few ulp; ex2 of a large argument gives inf and rcp(inf) = 0, so sigm saturates.
__device__ __forceinline__ float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fast_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fast_rsqrt(float x) { float y; asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float sigm(float x) { return fast_rcp(1.f + fast_ex2(-1.4426950408889634f * x)); }
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t; t.x = *reinterpret_cast<uint32_t*>(&a); t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// ================================================================================================ GDN input prep
// Channels come in groups of 128 (a q head, a k head, or a 128-wide slice of v). K = 4 taps. doc == nullptr means every
// row is a single document (only t - j >= 0 is checked). Channels [0, nq) are q (norm + scale), [nq, 2nq) are k (norm),
// the rest v (no norm). dk must be 128.
constexpr int PREP_K = 4;

// Both kernels work on tiles of PREP_TOK tokens x 128 channels: the CTA first issues every load of the tile (inputs with
// the K - 1 rows before it, 16 bytes per thread and load, all in flight together) into shared memory, then half-warps
// take tokens (8 channels per lane, 16-byte stores); the L2 norm of a q or k head is a reduction over the 16 lanes.
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) { __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]); w[e] = *reinterpret_cast<uint32_t*>(&h); }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float hsum16(float v) {       // sum over the 16 lanes of a half-warp
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int PREP_TOK = 64;

struct PrepTile {        // the tile's place: 128-channel group, first row, and rows of the tensor
  int grp; long r0, r1;
};

// Rows [r_lo, r_lo + n) of one 128-channel group into shared memory (row-major, 128 bf16 per row); rows outside
// [0, rows) are zero-filled.
__device__ __forceinline__ void prep_load_rows(const __nv_bfloat16* __restrict__ g, __nv_bfloat16* sm, long r_lo, int n, long rows, int C, int c0) {
  for (int i = threadIdx.x; i < n * 16; i += blockDim.x) {
    const long r = r_lo + (i >> 4);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r >= 0 && r < rows) v = *reinterpret_cast<const uint4*>(g + r * C + c0 + (i & 15) * 8);
    reinterpret_cast<uint4*>(sm)[i] = v;
  }
}
__device__ __forceinline__ void lds8(const __nv_bfloat16* p, float (&v)[8]) { ld8(p, v); }

// Valid taps of every token of a tile, formed once per CTA (the lanes then compare one small integer per tap):
// back[i]: how many of u[s], u[s-1], ... token s = r0 + i reads (same row, same document); fwd[i]: how many of the tokens
// s, s+1, ... read u[s]. sdoc: document ids of rows r_lo .. r_lo + n - 1 (zeros without ids), r_lo = r0 - (K - 1).
__device__ __forceinline__ void prep_tap_counts(const int* sdoc, bool has_doc, long r0, int n_tok, long rows, int L, unsigned char* back, unsigned char* fwd) {
  for (int i = threadIdx.x; i < n_tok; i += blockDim.x) {
    const long s = r0 + i;
    int nb = 0, nf = 0;
    if (s < rows) {
      const int t = static_cast<int>(s % L);
      const int d = sdoc[i + PREP_K - 1];
      for (int j = 0; j < PREP_K; ++j) {
        if (t - j < 0 || (has_doc && sdoc[i + PREP_K - 1 - j] != d)) break;
        ++nb;
      }
      if (fwd && i < PREP_TOK) {               // only the tile's own tokens are written; later rows' documents are not staged
        for (int j = 0; j < PREP_K; ++j) {
          if (t + j >= L || s + j >= rows || (has_doc && sdoc[i + PREP_K - 1 + j] != d)) break;
          ++nf;
        }
      }
    }
    back[i] = static_cast<unsigned char>(nb);
    if (fwd) fwd[i] = static_cast<unsigned char>(nf);
  }
}

__global__ void __launch_bounds__(256) gdn_prep_fwd_kernel(const __nv_bfloat16* __restrict__ u, const int* __restrict__ doc, const float* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, long rows, int L, int C, int nq, float qscale) {
  __shared__ __align__(16) __nv_bfloat16 su[(PREP_TOK + PREP_K - 1) * 128];
  __shared__ int sdoc[PREP_TOK + PREP_K - 1];
  __shared__ unsigned char sback[PREP_TOK];
  const int groups = C / 128;
  const int grp = blockIdx.x % groups;
  const long r0 = static_cast<long>(blockIdx.x / groups) * PREP_TOK, r1 = min(rows, r0 + PREP_TOK);
  const int c0 = grp * 128, l = threadIdx.x & 15, hw = threadIdx.x >> 4;
  prep_load_rows(u, su, r0 - (PREP_K - 1), PREP_TOK + PREP_K - 1, rows, C, c0);
  if (threadIdx.x < PREP_TOK + PREP_K - 1) {
    const long r = r0 - (PREP_K - 1) + threadIdx.x;
    sdoc[threadIdx.x] = (doc && r >= 0 && r < rows) ? doc[r] : 0;
  }
  float wt[8][PREP_K];
#pragma unroll
  for (int e = 0; e < 8; ++e) { const float4 q = *reinterpret_cast<const float4*>(w + static_cast<long>(c0 + l * 8 + e) * PREP_K); wt[e][0] = q.x; wt[e][1] = q.y; wt[e][2] = q.z; wt[e][3] = q.w; }
  const bool normed = c0 < 2 * nq;
  const float s_norm = c0 < nq ? qscale : 1.f;
  __syncthreads();
  prep_tap_counts(sdoc, doc != nullptr, r0, PREP_TOK, rows, L, sback, nullptr);
  __syncthreads();
#pragma unroll 1
  for (int i = hw; i < PREP_TOK; i += 16) {      // every half-warp runs the same trip count: the shuffles need all lanes
    const long s = r0 + i;
    const bool on = s < r1;
    const int taps = sback[i];
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < PREP_K; ++j) {
      if (j < taps) {
        float x[8];
        lds8(su + (i + PREP_K - 1 - j) * 128 + l * 8, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += x[e] * wt[e][PREP_K - 1 - j];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { a[e] = a[e] * sigm(a[e]); ss += a[e] * a[e]; }
    if (normed) {
      ss = hsum16(ss);
      const float r = fast_rsqrt(ss + 1e-6f) * s_norm;
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] *= r;
    }
    if (on) st8(out + s * C + c0 + l * 8, a);
  }
}

// Backward, one pass per tile: dconv of the tile's tokens and of the K - 1 tokens after it (their taps reach back into
// the tile; they are recomputed, not read) is formed from the staged inputs and output gradients and kept in shared
// memory in fp32; then du[s] = sum_j dconv[s + j] w[K-1-j]. The conv-weight gradient is summed per thread over the
// CTA's tiles (a thread keeps its 8 channels), across the CTA's half-warps in shared memory, then one atomic per entry.
constexpr int PREP_BROWS = PREP_TOK + 2 * (PREP_K - 1);      // input rows a backward tile reads
constexpr int PREP_DROWS = PREP_TOK + PREP_K - 1;            // rows of dout read / of dconv formed
constexpr int PREP_BWD_SMEM = PREP_BROWS * 256 + PREP_DROWS * 256 + PREP_DROWS * 512 + PREP_BROWS * 4 + 2 * PREP_DROWS + 2;

__global__ void __launch_bounds__(256, 2) gdn_prep_bwd_kernel(const __nv_bfloat16* __restrict__ u, const int* __restrict__ doc, const float* __restrict__ w,
                                                              const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ du, float* __restrict__ dw,
                                                              long rows, int L, int C, int nq, float qscale, int tiles_per_cta) {
  extern __shared__ __align__(16) unsigned char prep_smem[];
  __nv_bfloat16* su = reinterpret_cast<__nv_bfloat16*>(prep_smem);                       // [PREP_BROWS][128], row 0 = r0 - (K-1)
  __nv_bfloat16* sdy = su + PREP_BROWS * 128;                                             // [PREP_DROWS][128], row 0 = r0
  float* sdc = reinterpret_cast<float*>(sdy + PREP_DROWS * 128);                          // [PREP_DROWS][128]: lane l's channels at l*4 and 64 + l*4
  int* sdoc = reinterpret_cast<int*>(sdc + PREP_DROWS * 128);                             // [PREP_BROWS]
  unsigned char* sback = reinterpret_cast<unsigned char*>(sdoc + PREP_BROWS);             // [PREP_DROWS]
  unsigned char* sfwd = sback + PREP_DROWS;                                               // [PREP_DROWS]
  const int groups = C / 128;
  const int grp = blockIdx.x % groups;
  const long tile0 = static_cast<long>(blockIdx.x / groups) * tiles_per_cta;
  const int c0 = grp * 128, l = threadIdx.x & 15, hw = threadIdx.x >> 4;
  float wt[8][PREP_K], acc[8][PREP_K];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float4 q = *reinterpret_cast<const float4*>(w + static_cast<long>(c0 + l * 8 + e) * PREP_K);
    wt[e][0] = q.x; wt[e][1] = q.y; wt[e][2] = q.z; wt[e][3] = q.w;
#pragma unroll
    for (int j = 0; j < PREP_K; ++j) acc[e][j] = 0.f;
  }
  const bool normed = c0 < 2 * nq;
  const float s_norm = c0 < nq ? qscale : 1.f;
  for (int tile = 0; tile < tiles_per_cta; ++tile) {
    const long r0 = (tile0 + tile) * PREP_TOK;
    if (r0 >= rows) break;                      // uniform over the CTA
    const long r1 = min(rows, r0 + PREP_TOK);
    __syncthreads();                            // the previous tile's readers are done
    prep_load_rows(u, su, r0 - (PREP_K - 1), PREP_BROWS, rows, C, c0);
    prep_load_rows(dout, sdy, r0, PREP_DROWS, rows, C, c0);
    if (threadIdx.x < PREP_BROWS) {
      const long r = r0 - (PREP_K - 1) + threadIdx.x;
      sdoc[threadIdx.x] = (doc && r >= 0 && r < rows) ? doc[r] : 0;
    }
    __syncthreads();
    prep_tap_counts(sdoc, doc != nullptr, r0, PREP_DROWS, rows, L, sback, sfwd);
    __syncthreads();
    // ---- dconv of tokens r0 .. r0 + PREP_DROWS - 1 (token index i: input row i + K - 1 of su)
#pragma unroll 1
    for (int round = 0; round < (PREP_DROWS + 15) / 16; ++round) {      // the same trip count for every half-warp (shuffles below)
      const int i = hw + 16 * round;
      const bool on = i < PREP_DROWS && r0 + i < rows;
      const int taps = on ? sback[i] : 0;
      float pre[8], a[8], dy[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) { pre[e] = 0.f; dy[e] = 0.f; }
      if (on) lds8(sdy + i * 128 + l * 8, dy);
#pragma unroll
      for (int j = 0; j < PREP_K; ++j) {
        if (j < taps) {
          float x[8];
          lds8(su + (i + PREP_K - 1 - j) * 128 + l * 8, x);
#pragma unroll
          for (int e = 0; e < 8; ++e) pre[e] += x[e] * wt[e][PREP_K - 1 - j];
        }
      }
      float sg[8], ss = 0.f, ady = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) { sg[e] = sigm(pre[e]); a[e] = pre[e] * sg[e]; ss += a[e] * a[e]; ady += a[e] * dy[e]; }
      if (normed) { ss = hsum16(ss); ady = hsum16(ady); }
      if (on) {
        float dc[8];
        const float r = fast_rsqrt(ss + 1e-6f);
        const float k1 = s_norm * r, k2 = r * r * ady;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float da = normed ? k1 * (dy[e] - a[e] * k2) : dy[e];
          dc[e] = da * (sg[e] + a[e] * (1.f - sg[e]));          // d silu = sg (1 + pre (1 - sg))
        }
        *reinterpret_cast<float4*>(sdc + i * 128 + l * 4) = make_float4(dc[0], dc[1], dc[2], dc[3]);
        *reinterpret_cast<float4*>(sdc + i * 128 + 64 + l * 4) = make_float4(dc[4], dc[5], dc[6], dc[7]);
        if (i < PREP_TOK) {
#pragma unroll
          for (int j = 0; j < PREP_K; ++j) {
            if (j < taps) {
              float x[8];
              lds8(su + (i + PREP_K - 1 - j) * 128 + l * 8, x);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[e][PREP_K - 1 - j] += dc[e] * x[e];
            }
          }
        }
      }
    }
    __syncthreads();
    // ---- du of the tile's tokens
#pragma unroll 1
    for (int i = hw; i < PREP_TOK; i += 16) {
      const long tr = r0 + i;
      if (tr >= r1) break;
      const int nf = sfwd[i];
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < PREP_K; ++j) {       // token tr + j reads tr through tap j
        if (j < nf) {
          const float4 d0 = *reinterpret_cast<const float4*>(sdc + (i + j) * 128 + l * 4), d1 = *reinterpret_cast<const float4*>(sdc + (i + j) * 128 + 64 + l * 4);
          const float dcv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] += dcv[e] * wt[e][PREP_K - 1 - j];
        }
      }
      st8(du + tr * C + c0 + l * 8, g);
    }
  }
  // ---- conv-weight gradient: sum the 16 half-warps in shared memory (the dconv buffer is free now), one atomic per entry
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 8; ++e)
#pragma unroll
    for (int j = 0; j < PREP_K; ++j) sdc[hw * 512 + (l * 8 + e) * PREP_K + j] = acc[e][j];
  __syncthreads();
  for (int i = threadIdx.x; i < 512; i += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int h = 0; h < 16; ++h) t += sdc[h * 512 + i];
    atomicAdd(dw + static_cast<long>(c0) * PREP_K + i, t);
  }
}

int gdn_prep_fwd(const void* u, const int* doc, const float* w, void* out, long rows, int L, int C, int nq, float qscale, cudaStream_t st) {
  if (C % 128 || nq % 128) return 1;
  const long tiles = (rows + PREP_TOK - 1) / PREP_TOK;
  gdn_prep_fwd_kernel<<<static_cast<unsigned>(tiles * (C / 128)), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(u), doc, w, static_cast<__nv_bfloat16*>(out), rows, L, C, nq, qscale);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int gdn_prep_bwd(const void* u, const int* doc, const float* w, const void* dout, void* du, float* dw, long rows, int L, int C,
                 int nq, float qscale, cudaStream_t st) {
  if (C % 128 || nq % 128) return 1;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_prep_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_BWD_SMEM) != cudaSuccess) return 4;
    cudaFuncSetAttribute(gdn_prep_bwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(gdn_prep_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    attr = true;
  }
  const long tiles = (rows + PREP_TOK - 1) / PREP_TOK;
  const int per = tiles >= 64 ? 4 : 1;          // several tiles per CTA: fewer conv-weight atomics
  const long ctas = (tiles + per - 1) / per;
  gdn_prep_bwd_kernel<<<static_cast<unsigned>(ctas * (C / 128)), 256, PREP_BWD_SMEM, st>>>(
      static_cast<const __nv_bfloat16*>(u), doc, w, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(du), dw, rows, L, C, nq, qscale, per);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ depth mix
// One CTA of 128 threads per row; thread holds VPT float4 of every source (d = 512 * VPT). Sources fp32.
constexpr int MIX_MAX = 8;
struct MixPtrs { const float* src[MIX_MAX]; float* dsrc[MIX_MAX]; };

__device__ __forceinline__ float block_sum_128(float v, float* sh) {
  v = wsum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = sh[0] + sh[1] + sh[2] + sh[3];
  __syncthreads();
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(128) depth_mix_fwd_kernel(MixPtrs p, int n, const float* __restrict__ ueff, float* __restrict__ out,
                                                            float* __restrict__ alpha, float* __restrict__ rnorm, int d, float eps) {
  __shared__ float sh[4];
  const long row = blockIdx.x;
  float4 v[MIX_MAX][VPT];
  float logit[MIX_MAX];
  float4 uq[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) uq[k] = reinterpret_cast<const float4*>(ueff)[k * 128 + threadIdx.x];
#pragma unroll
  for (int i = 0; i < MIX_MAX; ++i) {
    if (i < n) {
      float dot = 0.f, ss = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        v[i][k] = reinterpret_cast<const float4*>(p.src[i] + row * d)[k * 128 + threadIdx.x];
        dot += v[i][k].x * uq[k].x + v[i][k].y * uq[k].y + v[i][k].z * uq[k].z + v[i][k].w * uq[k].w;
        ss += v[i][k].x * v[i][k].x + v[i][k].y * v[i][k].y + v[i][k].z * v[i][k].z + v[i][k].w * v[i][k].w;
      }
      dot = block_sum_128(dot, sh);
      ss = block_sum_128(ss, sh);
      const float r = rsqrtf(ss / d + eps);
      logit[i] = dot * r;
      if (threadIdx.x == 0) rnorm[row * n + i] = r;
    } else logit[i] = -INFINITY;
  }
  float mx = -INFINITY, den = 0.f;
#pragma unroll
  for (int i = 0; i < MIX_MAX; ++i) mx = fmaxf(mx, logit[i]);
#pragma unroll
  for (int i = 0; i < MIX_MAX; ++i) { logit[i] = i < n ? __expf(logit[i] - mx) : 0.f; den += logit[i]; }
  float4 acc[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < MIX_MAX; ++i) {
    if (i < n) {
      const float a = logit[i] / den;
      if (threadIdx.x == 0) alpha[row * n + i] = a;
#pragma unroll
      for (int k = 0; k < VPT; ++k) { acc[k].x += a * v[i][k].x; acc[k].y += a * v[i][k].y; acc[k].z += a * v[i][k].z; acc[k].w += a * v[i][k].w; }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) reinterpret_cast<float4*>(out + row * d)[k * 128 + threadIdx.x] = acc[k];
}

// dv_i = alpha_i dh + dl_i (u r_i - (v_i . u) r_i^3 v_i / d), dl_i = alpha_i (dh . v_i - sum_j alpha_j dh . v_j);
// du += sum_i dl_i r_i v_i (accumulated per CTA over a grid-stride of rows, then atomics).
template <int VPT>
__global__ void __launch_bounds__(128) depth_mix_bwd_kernel(MixPtrs p, int n, const float* __restrict__ ueff, const float* __restrict__ dh,
                                                            const float* __restrict__ alpha, const float* __restrict__ rnorm,
                                                            float* __restrict__ du, long rows, int d) {
  __shared__ float sh[4];
  float4 uq[VPT], dacc[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) { uq[k] = reinterpret_cast<const float4*>(ueff)[k * 128 + threadIdx.x]; dacc[k] = make_float4(0.f, 0.f, 0.f, 0.f); }
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    float4 g[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) g[k] = reinterpret_cast<const float4*>(dh + row * d)[k * 128 + threadIdx.x];
    float da[MIX_MAX], vu[MIX_MAX];
    float mean = 0.f;
#pragma unroll
    for (int i = 0; i < MIX_MAX; ++i) {
      da[i] = 0.f; vu[i] = 0.f;
      if (i < n) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const float4 v = reinterpret_cast<const float4*>(p.src[i] + row * d)[k * 128 + threadIdx.x];
          a += g[k].x * v.x + g[k].y * v.y + g[k].z * v.z + g[k].w * v.w;
          b += uq[k].x * v.x + uq[k].y * v.y + uq[k].z * v.z + uq[k].w * v.w;
        }
        da[i] = block_sum_128(a, sh);
        vu[i] = block_sum_128(b, sh);
        mean += alpha[row * n + i] * da[i];
      }
    }
#pragma unroll
    for (int i = 0; i < MIX_MAX; ++i) {
      if (i < n) {
        const float al = alpha[row * n + i], r = rnorm[row * n + i];
        const float dl = al * (da[i] - mean);
        const float c1 = dl * r, c2 = dl * vu[i] * r * r * r / d;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const float4 v = reinterpret_cast<const float4*>(p.src[i] + row * d)[k * 128 + threadIdx.x];
          float4 o;
          o.x = al * g[k].x + c1 * uq[k].x - c2 * v.x; o.y = al * g[k].y + c1 * uq[k].y - c2 * v.y;
          o.z = al * g[k].z + c1 * uq[k].z - c2 * v.z; o.w = al * g[k].w + c1 * uq[k].w - c2 * v.w;
          reinterpret_cast<float4*>(p.dsrc[i] + row * d)[k * 128 + threadIdx.x] = o;
          dacc[k].x += c1 * v.x; dacc[k].y += c1 * v.y; dacc[k].z += c1 * v.z; dacc[k].w += c1 * v.w;
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    float* o = du + (k * 128 + threadIdx.x) * 4;
    atomicAdd(o, dacc[k].x); atomicAdd(o + 1, dacc[k].y); atomicAdd(o + 2, dacc[k].z); atomicAdd(o + 3, dacc[k].w);
  }
}

int depth_mix_fwd(const float* const* src, int n, const float* ueff, float* out, float* alpha, float* rnorm, long rows, int d, float eps,
                  cudaStream_t st) {
  if (n < 1 || n > MIX_MAX || d % 512 || d > 2048) return 1;
  MixPtrs p{};
  for (int i = 0; i < n; ++i) p.src[i] = src[i];
  switch (d / 512) {
    case 1: depth_mix_fwd_kernel<1><<<static_cast<unsigned>(rows), 128, 0, st>>>(p, n, ueff, out, alpha, rnorm, d, eps); break;
    case 2: depth_mix_fwd_kernel<2><<<static_cast<unsigned>(rows), 128, 0, st>>>(p, n, ueff, out, alpha, rnorm, d, eps); break;
    case 4: depth_mix_fwd_kernel<4><<<static_cast<unsigned>(rows), 128, 0, st>>>(p, n, ueff, out, alpha, rnorm, d, eps); break;
    default: return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int depth_mix_bwd(const float* const* src, float* const* dsrc, int n, const float* ueff, const float* dh, const float* alpha,
                  const float* rnorm, float* du, long rows, int d, int sms, cudaStream_t st) {
  if (n < 1 || n > MIX_MAX || d % 512 || d > 2048) return 1;
  MixPtrs p{};
  for (int i = 0; i < n; ++i) { p.src[i] = src[i]; p.dsrc[i] = dsrc[i]; }
  const unsigned grid = static_cast<unsigned>(rows < sms * 16L ? rows : sms * 16L);
  switch (d / 512) {
    case 1: depth_mix_bwd_kernel<1><<<grid, 128, 0, st>>>(p, n, ueff, dh, alpha, rnorm, du, rows, d); break;
    case 2: depth_mix_bwd_kernel<2><<<grid, 128, 0, st>>>(p, n, ueff, dh, alpha, rnorm, du, rows, d); break;
    case 4: depth_mix_bwd_kernel<4><<<grid, 128, 0, st>>>(p, n, ueff, dh, alpha, rnorm, du, rows, d); break;
    default: return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ---- several readers over the same sources in one pass. The block-entry mix and the write / query mixes of a block's GDN
// layers all read the same finished blocks with different pseudo-queries: the sources are read once for all Q readers,
// and in the backward the Q gradients meet in one write of every source's gradient (instead of Q kernels and Q - 1
// accumulation passes over (rows, d) tensors). Same arithmetic per reader as the single-reader kernels above.
constexpr int MIXQ_MAX = 8;       // readers per launch; NS below: register slots for sources (2, 4 or 8), so few sources cost few registers
struct MultiPtrs { const float* src[MIX_MAX]; float* dsrc[MIX_MAX]; float* out[MIXQ_MAX]; const float* dh[MIXQ_MAX]; };

template <int VPT, int NS>
__global__ void __launch_bounds__(128) depth_mix_multi_fwd_kernel(MultiPtrs p, int n, int Q, const float* __restrict__ ueff, float* __restrict__ alpha,
                                                                  float* __restrict__ rnorm, float* __restrict__ vu, int d, float eps) {
  __shared__ float part[4][MIX_MAX * (MIXQ_MAX + 1)];
  __shared__ float sal[MIXQ_MAX][MIX_MAX];
  const long row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4 v[NS][VPT];
#pragma unroll
  for (int i = 0; i < NS; ++i) {
    if (i < n) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        v[i][k] = reinterpret_cast<const float4*>(p.src[i] + row * d)[k * 128 + threadIdx.x];
        ss += v[i][k].x * v[i][k].x + v[i][k].y * v[i][k].y + v[i][k].z * v[i][k].z + v[i][k].w * v[i][k].w;
      }
      ss = wsum(ss);
      if (lane == 0) part[warp][i] = ss;
    }
  }
  for (int q = 0; q < Q; ++q) {
    float4 uq[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) uq[k] = reinterpret_cast<const float4*>(ueff + static_cast<long>(q) * d)[k * 128 + threadIdx.x];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (i < n) {
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) dot += v[i][k].x * uq[k].x + v[i][k].y * uq[k].y + v[i][k].z * uq[k].z + v[i][k].w * uq[k].w;
        dot = wsum(dot);
        if (lane == 0) part[warp][n + q * n + i] = dot;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < Q * n) {
    const int q = threadIdx.x / n, i = threadIdx.x % n;
    const float ss = part[0][i] + part[1][i] + part[2][i] + part[3][i];
    const int c = n + threadIdx.x;
    const float dot = part[0][c] + part[1][c] + part[2][c] + part[3][c];
    const float r = rsqrtf(ss / d + eps);
    sal[q][i] = dot * r;
    vu[(row * Q + q) * n + i] = dot;
    if (q == 0) rnorm[row * n + i] = r;
  }
  __syncthreads();
  if (threadIdx.x < Q) {
    const int q = threadIdx.x;
    float mx = -INFINITY, den = 0.f;
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, sal[q][i]);
    for (int i = 0; i < n; ++i) { const float e = __expf(sal[q][i] - mx); sal[q][i] = e; den += e; }
    for (int i = 0; i < n; ++i) { const float a = sal[q][i] / den; sal[q][i] = a; alpha[(row * Q + q) * n + i] = a; }
  }
  __syncthreads();
  for (int q = 0; q < Q; ++q) {
    float4 acc[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (i < n) {
        const float a = sal[q][i];
#pragma unroll
        for (int k = 0; k < VPT; ++k) { acc[k].x += a * v[i][k].x; acc[k].y += a * v[i][k].y; acc[k].z += a * v[i][k].z; acc[k].w += a * v[i][k].w; }
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) reinterpret_cast<float4*>(p.out[q] + row * d)[k * 128 + threadIdx.x] = acc[k];
  }
}

// Rows in a grid-stride loop. Per row: the Q products dh_q . v_i (one pass over the readers' gradients), then every
// source's gradient summed over the readers (a second pass over the gradients, which the first left in cache). The
// pseudo-query gradients accumulate per CTA in shared memory (a thread owns its columns), then one atomic per entry.
// TH threads per row (128 or 256): a thread holds VPT float4 of every source, d = 4 VPT TH.
template <int VPT, int NS, int TH>
__global__ void __launch_bounds__(TH) depth_mix_multi_bwd_kernel(MultiPtrs p, int n, int Q, const float* __restrict__ ueff, const float* __restrict__ alpha,
                                                                  const float* __restrict__ rnorm, const float* __restrict__ vu, float* __restrict__ du,
                                                                  long rows, int d) {
  extern __shared__ float sdu[];                       // [Q][d]
  __shared__ float part[TH / 32][MIX_MAX * MIXQ_MAX];
  __shared__ float sda[MIXQ_MAX][MIX_MAX], sal[MIXQ_MAX][MIX_MAX], sc1[MIXQ_MAX][MIX_MAX], sc2[MIXQ_MAX][MIX_MAX];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < Q * d; i += TH) sdu[i] = 0.f;
  __syncthreads();
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    float4 v[NS][VPT];
#pragma unroll
    for (int i = 0; i < NS; ++i)
      if (i < n) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) v[i][k] = reinterpret_cast<const float4*>(p.src[i] + row * d)[k * TH + threadIdx.x];
      }
    for (int q = 0; q < Q; ++q) {
      if (p.dh[q] == nullptr) continue;
      float4 g[VPT];
#pragma unroll
      for (int k = 0; k < VPT; ++k) g[k] = reinterpret_cast<const float4*>(p.dh[q] + row * d)[k * TH + threadIdx.x];
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        if (i < n) {
          float a = 0.f;
#pragma unroll
          for (int k = 0; k < VPT; ++k) a += g[k].x * v[i][k].x + g[k].y * v[i][k].y + g[k].z * v[i][k].z + g[k].w * v[i][k].w;
          a = wsum(a);
          if (lane == 0) part[warp][q * n + i] = a;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < Q * n) {
      const int q = threadIdx.x / n, i = threadIdx.x % n, c = threadIdx.x;
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < TH / 32; ++w) tot += part[w][c];
      sda[q][i] = p.dh[q] ? tot : 0.f;
      sal[q][i] = alpha[(row * Q + q) * n + i];
    }
    __syncthreads();
    if (threadIdx.x < Q * n) {
      const int q = threadIdx.x / n, i = threadIdx.x % n;
      float mean = 0.f;
      for (int j = 0; j < n; ++j) mean += sal[q][j] * sda[q][j];
      const float r = rnorm[row * n + i];
      const float dl = sal[q][i] * (sda[q][i] - mean);
      sc1[q][i] = dl * r;
      sc2[q][i] = dl * vu[(row * Q + q) * n + i] * r * r * r / d;
    }
    __syncthreads();
    float4 acc[NS][VPT];
#pragma unroll
    for (int i = 0; i < NS; ++i)
#pragma unroll
      for (int k = 0; k < VPT; ++k) acc[i][k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < Q; ++q) {
      if (p.dh[q] == nullptr) continue;
      float4 g[VPT], uq[VPT], dq[VPT];
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        g[k] = reinterpret_cast<const float4*>(p.dh[q] + row * d)[k * TH + threadIdx.x];
        uq[k] = reinterpret_cast<const float4*>(ueff + static_cast<long>(q) * d)[k * TH + threadIdx.x];
        dq[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        if (i < n) {
          const float al = sal[q][i], c1 = sc1[q][i], c2 = sc2[q][i];
#pragma unroll
          for (int k = 0; k < VPT; ++k) {
            acc[i][k].x += al * g[k].x + c1 * uq[k].x - c2 * v[i][k].x; acc[i][k].y += al * g[k].y + c1 * uq[k].y - c2 * v[i][k].y;
            acc[i][k].z += al * g[k].z + c1 * uq[k].z - c2 * v[i][k].z; acc[i][k].w += al * g[k].w + c1 * uq[k].w - c2 * v[i][k].w;
            dq[k].x += c1 * v[i][k].x; dq[k].y += c1 * v[i][k].y; dq[k].z += c1 * v[i][k].z; dq[k].w += c1 * v[i][k].w;
          }
        }
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        float4* slot = reinterpret_cast<float4*>(sdu + static_cast<long>(q) * d) + k * TH + threadIdx.x;
        float4 t = *slot;
        t.x += dq[k].x; t.y += dq[k].y; t.z += dq[k].z; t.w += dq[k].w;
        *slot = t;
      }
    }
#pragma unroll
    for (int i = 0; i < NS; ++i)
      if (i < n) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) reinterpret_cast<float4*>(p.dsrc[i] + row * d)[k * TH + threadIdx.x] = acc[i][k];
      }
    __syncthreads();          // the shared per-row scalars are rewritten by the next row
  }
  for (int i = threadIdx.x; i < Q * d; i += TH) atomicAdd(du + i, sdu[i]);
}

int depth_mix_multi_fwd(const float* const* src, int n, float* const* out, int Q, const float* ueff, float* alpha, float* rnorm, float* vu, long rows,
                        int d, float eps, cudaStream_t st) {
  if (n < 1 || n > MIX_MAX || Q < 1 || Q > MIXQ_MAX || d % 512 || d > 2048) return 1;
  MultiPtrs p{};
  for (int i = 0; i < n; ++i) p.src[i] = src[i];
  for (int q = 0; q < Q; ++q) p.out[q] = out[q];
  const unsigned grid = static_cast<unsigned>(rows);
  const int ns = n <= 2 ? 2 : (n <= 4 ? 4 : 8);
#define GHB_MIXF(V, S) depth_mix_multi_fwd_kernel<V, S><<<grid, 128, 0, st>>>(p, n, Q, ueff, alpha, rnorm, vu, d, eps)
#define GHB_MIXF_NS(V) (ns == 2 ? GHB_MIXF(V, 2) : (ns == 4 ? GHB_MIXF(V, 4) : GHB_MIXF(V, 8)))
  switch (d / 512) {
    case 1: GHB_MIXF_NS(1); break;
    case 2: GHB_MIXF_NS(2); break;
    case 4: GHB_MIXF_NS(4); break;
    default: return 1;
  }
#undef GHB_MIXF_NS
#undef GHB_MIXF
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int depth_mix_multi_bwd(const float* const* src, float* const* dsrc, int n, const float* const* dh, int Q, const float* ueff, const float* alpha,
                        const float* rnorm, const float* vu, float* du, long rows, int d, int sms, cudaStream_t st) {
  if (n < 1 || n > MIX_MAX || Q < 1 || Q > MIXQ_MAX || d % 512 || d > 2048) return 1;
  MultiPtrs p{};
  for (int i = 0; i < n; ++i) { p.src[i] = src[i]; p.dsrc[i] = dsrc[i]; }
  for (int q = 0; q < Q; ++q) p.dh[q] = dh[q];
  const size_t smem = static_cast<size_t>(Q) * d * 4;
  const unsigned grid = static_cast<unsigned>(rows < sms * 8L ? rows : sms * 8L);
  const int ns = n <= 2 ? 2 : (n <= 4 ? 4 : 8);
  // 256 threads per row where d allows (d a multiple of 1024): half the registers per thread, more rows in flight per SM
#define GHB_MIXB(V, S, TH)                                                                                                        \
  do {                                                                                                                            \
    static bool attr = false;                                                                                                     \
    if (!attr) { cudaFuncSetAttribute(depth_mix_multi_bwd_kernel<V, S, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, MIXQ_MAX * 2048 * 4); attr = true; } \
    depth_mix_multi_bwd_kernel<V, S, TH><<<grid, TH, smem, st>>>(p, n, Q, ueff, alpha, rnorm, vu, du, rows, d);                    \
  } while (0)
#define GHB_MIXB_NS(V, TH) do { if (ns == 2) GHB_MIXB(V, 2, TH); else if (ns == 4) GHB_MIXB(V, 4, TH); else GHB_MIXB(V, 8, TH); } while (0)
  switch (d / 512) {
    case 1: GHB_MIXB_NS(1, 128); break;
    case 2: GHB_MIXB_NS(1, 256); break;
    case 4: GHB_MIXB_NS(2, 256); break;
    default: return 1;
  }
#undef GHB_MIXB_NS
#undef GHB_MIXB
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ CE gradient
// One CTA per row of fp32 logits (n, V). Pass 1: online max / sum over the row (kept in shared memory when it fits),
// pass 2: grad = softmax * (asum + 2 b lse) written as bf16 in a separate (n, V) buffer, then the s targets subtract
// their weights. ce[row] = sum_k a_k (lse - logit[t_k]); lse[row] saved.
// FIXED: the hard-target cross-entropy without the cancellation of softmax_t - 1 (ced/train/ce_fix.py:1-60): a term's loss is
// softplus(L'), L' = LSE_{j != t}(z_j) - z_t, and its target gradient -sigmoid(L'). Only the row's argmax can have a
// softmax within rounding of 1, so only that column needs the sum of exponentials without it (two more passes over the
// cached row); for any other target L' = (lse - z_t) + log1p(-p_t) has no cancellation (ced/train/ce_fix.py:151-170).
template <bool FIXED>
__global__ void __launch_bounds__(1024) ce_grad_kernel(const float* __restrict__ logits, const long* __restrict__ targets, const float* __restrict__ a,
                                                      const float* __restrict__ b, __nv_bfloat16* __restrict__ grad, float* __restrict__ ce,
                                                      float* __restrict__ lse_out, int V, int s, int cache_row) {
  extern __shared__ float rowbuf[];
  __shared__ float redm[32], reds[32];
  const long row = blockIdx.x;
  const float* lr = logits + row * V;
  float m = -INFINITY, sum = 0.f;
  // Batches of CE_UNROLL float4 per thread: every load of a batch is issued before any of it is used (the row is read
  // once, so the pass is bound by loads in flight), then one max and one sum of exponentials over the registers.
  constexpr int CE_UNROLL = 8;
  for (int i0 = threadIdx.x * 4; i0 < V; i0 += blockDim.x * 4 * CE_UNROLL) {
    float4 t[CE_UNROLL];
#pragma unroll
    for (int u = 0; u < CE_UNROLL; ++u) {
      const int i = i0 + u * blockDim.x * 4;
      t[u] = i < V ? *reinterpret_cast<const float4*>(lr + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float mm = m;
#pragma unroll
    for (int u = 0; u < CE_UNROLL; ++u) {
      const int i = i0 + u * blockDim.x * 4;
      if (cache_row && i < V) *reinterpret_cast<float4*>(rowbuf + i) = t[u];
      mm = fmaxf(mm, fmaxf(fmaxf(t[u].x, t[u].y), fmaxf(t[u].z, t[u].w)));
    }
    if (mm > m) { sum *= __expf(m - mm); m = mm; }       // m == -inf: sum is 0 and exp(-inf) = 0
    if (m > -INFINITY) {
#pragma unroll
      for (int u = 0; u < CE_UNROLL; ++u) sum += __expf(t[u].x - m) + __expf(t[u].y - m) + __expf(t[u].z - m) + __expf(t[u].w - m);
    }
  }
  const float wm = wmax(m);
  sum = (m == -INFINITY) ? 0.f : sum * __expf(m - wm);      // lanes past the row's end (V < 4 x threads) hold no terms
  sum = wsum(sum);
  if ((threadIdx.x & 31) == 0) { redm[threadIdx.x >> 5] = wm; reds[threadIdx.x >> 5] = sum; }
  __syncthreads();
  float gm = -INFINITY, gs = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) gm = fmaxf(gm, redm[i]);
  for (int i = 0; i < nw; ++i) if (redm[i] > -INFINITY) gs += reds[i] * __expf(redm[i] - gm);
  float lse = gm + __logf(gs);
  float s_excl = 0.f;
  int gidx = -1;
  if (FIXED) {
    __shared__ int s_idx;
    __shared__ float red2[32];
    if (threadIdx.x == 0) s_idx = V;
    __syncthreads();
    int mine = V;
    for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) {
      const float4 t = cache_row ? *reinterpret_cast<const float4*>(rowbuf + i) : *reinterpret_cast<const float4*>(lr + i);
      const float v[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int e = 3; e >= 0; --e) if (v[e] == gm) mine = min(mine, i + e);
    }
    if (mine < V) atomicMin(&s_idx, mine);
    __syncthreads();
    gidx = s_idx;
    float se = 0.f;
    for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) {
      const float4 t = cache_row ? *reinterpret_cast<const float4*>(rowbuf + i) : *reinterpret_cast<const float4*>(lr + i);
      const float v[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) if (i + e != gidx) se += __expf(v[e] - gm);
    }
    se = wsum(se);
    if ((threadIdx.x & 31) == 0) red2[threadIdx.x >> 5] = se;
    __syncthreads();
    for (int i = 0; i < nw; ++i) s_excl += red2[i];
    lse = gm + log1pf(s_excl);
  }
  float asum = 0.f;
  for (int k = 0; k < s; ++k) asum += a[row * s + k];
  const float coef = asum + 2.f * b[row] * lse;
  __nv_bfloat16* gr = grad + row * V;
  for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) {
    float4 t = cache_row ? *reinterpret_cast<const float4*>(rowbuf + i) : *reinterpret_cast<const float4*>(lr + i);
    float o[4] = {coef * __expf(t.x - lse), coef * __expf(t.y - lse), coef * __expf(t.z - lse), coef * __expf(t.w - lse)};
    st4(gr + i, o);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float c = 0.f;
    for (int k = 0; k < s; ++k) {
      const float ak = a[row * s + k];
      const long t = targets[row * s + k];
      if (ak != 0.f && t >= 0 && t < V) {
        if (FIXED) {
          const float zt = lr[t], pt = expf(zt - lse);
          const float lp = t == gidx ? logf(s_excl) : (lse - zt) + log1pf(-pt);
          c += ak * (lp > 0.f ? lp + log1pf(expf(-lp)) : log1pf(expf(lp)));
          float aj = 0.f;                          // weight of every term whose target is this column
          for (int k2 = 0; k2 < s; ++k2) if (targets[row * s + k2] == t) aj += a[row * s + k2];
          const float e = expf(-fabsf(lp));
          const float sg = (lp < 0.f ? e : 1.f) / (1.f + e);
          gr[t] = __float2bfloat16((asum - aj + 2.f * b[row] * lse) * pt - aj * sg);
        } else {
          c += ak * (lse - lr[t]);
          float aj = 0.f;
          for (int k2 = 0; k2 < s; ++k2) if (targets[row * s + k2] == t) aj += a[row * s + k2];
          gr[t] = __float2bfloat16(coef * expf(lr[t] - lse) - aj);       // formed in fp32 and rounded once (every term of the column writes the same value)
        }
      }
    }
    ce[row] = c;
    lse_out[row] = lse;
  }
}
int ce_grad(const float* logits, const long* targets, const float* a, const float* b, void* grad, float* ce, float* lse, long rows, int V,
            int s, bool fixed, cudaStream_t st) {
  if (V % 4) return 1;
  const size_t bytes = static_cast<size_t>(V) * 4;
  const int cache = bytes <= 200 * 1024;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(ce_grad_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(ce_grad_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr = true;
  }
  const unsigned threads = V >= 16384 ? 1024 : 512;
  if (fixed) ce_grad_kernel<true><<<static_cast<unsigned>(rows), threads, cache ? bytes : 0, st>>>(logits, targets, a, b, static_cast<__nv_bfloat16*>(grad), ce, lse, V, s, cache);
  else ce_grad_kernel<false><<<static_cast<unsigned>(rows), threads, cache ? bytes : 0, st>>>(logits, targets, a, b, static_cast<__nv_bfloat16*>(grad), ce, lse, V, s, cache);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ input mixes of a GDN layer
// out_a = x + la (ya - x), out_b = x + lb (yb - x) in fp32, rounded to bf16 (the write and query inputs of a GDN layer
// with mixes: ced/model/gdn.py:599-640 forms them as addcmul in fp32 and casts). yb == nullptr: only the first.
// Backward: dx = (1 - la) ga + (1 - lb) gb, dya = la ga, dyb = lb gb, dla = sum ga (ya - x), dlb = sum gb (yb - x).
__global__ void dual_lerp_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ ya, const __nv_bfloat16* __restrict__ yb,
                                     const float* __restrict__ la, const float* __restrict__ lb, __nv_bfloat16* __restrict__ oa,
                                     __nv_bfloat16* __restrict__ ob, long n4) {
  const float a = *la, b = yb ? *lb : 0.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float xv[4], yv[4], o[4];
    ld4(x + i * 4, xv);
    ld4(ya + i * 4, yv);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = fmaf(a, yv[e] - xv[e], xv[e]);
    st4(oa + i * 4, o);
    if (yb) {
      ld4(yb + i * 4, yv);
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = fmaf(b, yv[e] - xv[e], xv[e]);
      st4(ob + i * 4, o);
    }
  }
}
__global__ void dual_lerp_bwd_kernel(const __nv_bfloat16* __restrict__ ga, const __nv_bfloat16* __restrict__ gb, const __nv_bfloat16* __restrict__ x,
                                     const __nv_bfloat16* __restrict__ ya, const __nv_bfloat16* __restrict__ yb, const float* __restrict__ la,
                                     const float* __restrict__ lb, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dya,
                                     __nv_bfloat16* __restrict__ dyb, float* __restrict__ dl, long n4) {
  const float a = *la, b = yb ? *lb : 0.f;
  float sa = 0.f, sb = 0.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float xv[4], yv[4], g[4], d[4], o[4];
    ld4(x + i * 4, xv);
    ld4(ya + i * 4, yv);
    ld4(ga + i * 4, g);
#pragma unroll
    for (int e = 0; e < 4; ++e) { d[e] = (1.f - a) * g[e]; o[e] = a * g[e]; sa += g[e] * (yv[e] - xv[e]); }
    st4(dya + i * 4, o);
    if (yb) {
      ld4(yb + i * 4, yv);
      ld4(gb + i * 4, g);
#pragma unroll
      for (int e = 0; e < 4; ++e) { d[e] += (1.f - b) * g[e]; o[e] = b * g[e]; sb += g[e] * (yv[e] - xv[e]); }
      st4(dyb + i * 4, o);
    }
    st4(dx + i * 4, d);
  }
  __shared__ float red[2][32];
  sa = wsum(sa); sb = wsum(sb);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[0][warp] = sa; red[1][warp] = sb; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    sa = wsum(lane < nw ? red[0][lane] : 0.f);
    sb = wsum(lane < nw ? red[1][lane] : 0.f);
    if (lane == 0) { atomicAdd(dl, sa); if (yb) atomicAdd(dl + 1, sb); }
  }
}
int dual_lerp_fwd(const void* x, const void* ya, const void* yb, const float* la, const float* lb, void* oa, void* ob, long n, int sms, cudaStream_t st) {
  if (n % 4) return 1;
  using T = __nv_bfloat16;
  dual_lerp_fwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(ya), static_cast<const T*>(yb), la, lb, static_cast<T*>(oa),
                                                static_cast<T*>(ob), n / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
// dl: [2] fp32, zeroed by the caller.
int dual_lerp_bwd(const void* ga, const void* gb, const void* x, const void* ya, const void* yb, const float* la, const float* lb, void* dx, void* dya,
                  void* dyb, float* dl, long n, int sms, cudaStream_t st) {
  if (n % 4) return 1;
  using T = __nv_bfloat16;
  dual_lerp_bwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const T*>(ga), static_cast<const T*>(gb), static_cast<const T*>(x), static_cast<const T*>(ya),
                                                static_cast<const T*>(yb), la, lb, static_cast<T*>(dx), static_cast<T*>(dya), static_cast<T*>(dyb), dl, n / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ attention q / k preparation
// Per token and head (head dim 64, two channels per lane, one warp per token walking its heads): zero-centred RMSNorm,
// then the partial NeoX rotation at the token's position, and under the distance cap a second copy of the query
// rotated by the cap itself and the unrotated normed key (ced/model/attention.py:836-935, ced/model/rope.py:14-58 do
// this as separate norm, table and rotate ops). cos / sin: [tokens, R2] fp32 tables (R2 = rotary pairs, a power of two
// <= 32, or 0 for a position-free layer); cos_c / sin_c: [R2] tables of the cap rotation or null.
struct PrepQK {
  const __nv_bfloat16* q; long q_ts; int q_hs;      // raw queries: token stride, head stride (the gate may be interleaved)
  const __nv_bfloat16* k; long k_ts;                // raw keys [tokens, Hkv, 64]
  const float* wq; const float* wk;                 // norm gains [64]
  const float* cos; const float* sin; const float* cos_c; const float* sin_c;
  int Hq, Hkv, R2; float eps; long tokens;
};

// Rotation coefficients of one lane: lanes [0, R2 / 2) hold the first halves of the rotary pairs (channels 2 lane,
// 2 lane + 1), lanes [R2 / 2, R2) the second halves; the partner's values come through a shuffle.
struct RotCoef { float c0, c1, s0, s1; bool on; };      // s already signed for this lane's half; on: the lane holds rotary channels

__device__ __forceinline__ RotCoef rot_coef(int lane, int R2, const float* c, const float* s) {
  RotCoef r{1.f, 1.f, 0.f, 0.f, false};
  if (lane < R2) {
    r.on = true;
    const int half = R2 >> 1;
    const bool first = lane < half;
    const int i = (first ? lane : lane - half) * 2;
    r.c0 = c[i]; r.c1 = c[i + 1];
    r.s0 = first ? -s[i] : s[i]; r.s1 = first ? -s[i + 1] : s[i + 1];
  }
  return r;
}
// v' = v c + partner s (forward); the inverse rotation flips the sign of s. Lanes outside the rotary range keep v.
__device__ __forceinline__ void rotate(float& v0, float& v1, int half, const RotCoef& r, bool inverse) {
  const float p0 = __shfl_xor_sync(0xffffffffu, v0, half), p1 = __shfl_xor_sync(0xffffffffu, v1, half);
  if (r.on) {
    v0 = v0 * r.c0 + p0 * (inverse ? -r.s0 : r.s0);
    v1 = v1 * r.c1 + p1 * (inverse ? -r.s1 : r.s1);
  }
}

__global__ void __launch_bounds__(256) attn_prep_fwd_kernel(PrepQK a, __nv_bfloat16* __restrict__ qr, __nv_bfloat16* __restrict__ qf,
                                                            __nv_bfloat16* __restrict__ kr, __nv_bfloat16* __restrict__ kf) {
  const int lane = threadIdx.x & 31;
  const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarp = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const float gq0 = 1.f + a.wq[2 * lane], gq1 = 1.f + a.wq[2 * lane + 1], gk0 = 1.f + a.wk[2 * lane], gk1 = 1.f + a.wk[2 * lane + 1];
  const int half = a.R2 >> 1;
  const RotCoef cap = a.cos_c ? rot_coef(lane, a.R2, a.cos_c, a.sin_c) : RotCoef{1.f, 1.f, 0.f, 0.f, false};
  for (long t = warp; t < a.tokens; t += nwarp) {
    const RotCoef rc = a.R2 ? rot_coef(lane, a.R2, a.cos + t * a.R2, a.sin + t * a.R2) : RotCoef{1.f, 1.f, 0.f, 0.f, false};
    const __nv_bfloat16* qs = a.q + t * a.q_ts;
#pragma unroll 2
    for (int h = 0; h < a.Hq; ++h) {
      const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(qs + static_cast<long>(h) * a.q_hs)[lane]);
      const float r = fast_rsqrt(wsum(x.x * x.x + x.y * x.y) * (1.f / 64.f) + a.eps);
      const float n0 = x.x * r * gq0, n1 = x.y * r * gq1;
      float v0 = n0, v1 = n1;
      if (a.R2) rotate(v0, v1, half, rc, false);
      const long o = (t * a.Hq + h) * 64;
      reinterpret_cast<__nv_bfloat162*>(qr + o)[lane] = __floats2bfloat162_rn(v0, v1);
      if (a.cos_c) {
        float f0 = n0, f1 = n1;
        rotate(f0, f1, half, cap, false);
        reinterpret_cast<__nv_bfloat162*>(qf + o)[lane] = __floats2bfloat162_rn(f0, f1);
      }
    }
    const __nv_bfloat16* ks = a.k + t * a.k_ts;
    for (int h = 0; h < a.Hkv; ++h) {
      const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(ks + static_cast<long>(h) * 64)[lane]);
      const float r = fast_rsqrt(wsum(x.x * x.x + x.y * x.y) * (1.f / 64.f) + a.eps);
      const float n0 = x.x * r * gk0, n1 = x.y * r * gk1;
      float v0 = n0, v1 = n1;
      if (a.R2) rotate(v0, v1, half, rc, false);
      const long o = (t * a.Hkv + h) * 64;
      reinterpret_cast<__nv_bfloat162*>(kr + o)[lane] = __floats2bfloat162_rn(v0, v1);
      if (a.cos_c) reinterpret_cast<__nv_bfloat162*>(kf + o)[lane] = __floats2bfloat162_rn(n0, n1);
    }
  }
}

// Gradients w.r.t. the raw q / k and the two gains. dqraw is written with the raw queries' strides (the interleaved gate
// half is left untouched); dw: [2][64] fp32, zeroed by the caller.
__device__ __forceinline__ void prep_bwd_head(float2 x, float d0, float d1, float g0, float g1, float eps, float& acc0, float& acc1, __nv_bfloat16* dst, int lane) {
  const float r = fast_rsqrt(wsum(x.x * x.x + x.y * x.y) * (1.f / 64.f) + eps);
  const float h0 = x.x * r, h1 = x.y * r;
  acc0 += d0 * h0; acc1 += d1 * h1;
  const float e0 = d0 * g0, e1 = d1 * g1;
  const float dot = wsum(e0 * h0 + e1 * h1) * (1.f / 64.f);
  reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(r * (e0 - h0 * dot), r * (e1 - h1 * dot));
}

__global__ void __launch_bounds__(256) attn_prep_bwd_kernel(PrepQK a, const __nv_bfloat16* __restrict__ dqr, const __nv_bfloat16* __restrict__ dqf,
                                                            const __nv_bfloat16* __restrict__ dkr, const __nv_bfloat16* __restrict__ dkf,
                                                            __nv_bfloat16* __restrict__ dqraw, __nv_bfloat16* __restrict__ dkraw, float* __restrict__ dw) {
  __shared__ float red[8][4][32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarp = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const float gq0 = 1.f + a.wq[2 * lane], gq1 = 1.f + a.wq[2 * lane + 1], gk0 = 1.f + a.wk[2 * lane], gk1 = 1.f + a.wk[2 * lane + 1];
  const int half = a.R2 >> 1;
  const RotCoef cap = a.cos_c ? rot_coef(lane, a.R2, a.cos_c, a.sin_c) : RotCoef{1.f, 1.f, 0.f, 0.f, false};
  float acc[4] = {0.f, 0.f, 0.f, 0.f};      // dwq (2 channels), dwk (2 channels)
  for (long t = warp; t < a.tokens; t += nwarp) {
    const RotCoef rc = a.R2 ? rot_coef(lane, a.R2, a.cos + t * a.R2, a.sin + t * a.R2) : RotCoef{1.f, 1.f, 0.f, 0.f, false};
#pragma unroll 2
    for (int h = 0; h < a.Hq; ++h) {
      const long o = (t * a.Hq + h) * 64, so = t * a.q_ts + static_cast<long>(h) * a.q_hs;
      const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(a.q + so)[lane]);
      const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dqr + o)[lane]);
      float d0 = g.x, d1 = g.y;
      if (a.R2) rotate(d0, d1, half, rc, true);
      if (a.cos_c) {
        const float2 gf = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dqf + o)[lane]);
        float f0 = gf.x, f1 = gf.y;
        rotate(f0, f1, half, cap, true);
        d0 += f0; d1 += f1;
      }
      prep_bwd_head(x, d0, d1, gq0, gq1, a.eps, acc[0], acc[1], dqraw + so, lane);
    }
    for (int h = 0; h < a.Hkv; ++h) {
      const long o = (t * a.Hkv + h) * 64, so = t * a.k_ts + static_cast<long>(h) * 64;
      const float2 x = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(a.k + so)[lane]);
      const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dkr + o)[lane]);
      float d0 = g.x, d1 = g.y;
      if (a.R2) rotate(d0, d1, half, rc, true);
      if (a.cos_c) {
        const float2 gf = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dkf + o)[lane]);
        d0 += gf.x; d1 += gf.y;
      }
      prep_bwd_head(x, d0, d1, gk0, gk1, a.eps, acc[2], acc[3], dkraw + so, lane);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) red[wib][e][lane] = acc[e];
  __syncthreads();
  if (wib == 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float s = 0.f;
      for (int w = 0; w < 8; ++w) s += red[w][e][lane];
      atomicAdd(dw + (e >> 1) * 64 + 2 * lane + (e & 1), s);
    }
  }
}

static int prep_check(const PrepQK& a) {
  if (a.R2 < 0 || a.R2 > 32 || (a.R2 & (a.R2 - 1)) || a.R2 == 1 || a.q_hs % 2 || a.q_ts % 2 || a.k_ts % 2) return 1;
  if (a.cos_c && !a.R2) return 1;
  return 0;
}
int attn_prep_fwd(const void* q, long q_ts, int q_hs, const void* k, long k_ts, const float* wq, const float* wk, const float* cos, const float* sin,
                  const float* cos_c, const float* sin_c, int Hq, int Hkv, int R2, float eps, long tokens, void* qr, void* qf, void* kr, void* kf,
                  int sms, cudaStream_t st) {
  PrepQK a{static_cast<const __nv_bfloat16*>(q), q_ts, q_hs, static_cast<const __nv_bfloat16*>(k), k_ts, wq, wk, cos, sin, cos_c, sin_c, Hq, Hkv, R2, eps, tokens};
  if (prep_check(a)) return 1;
  attn_prep_fwd_kernel<<<sms * 8, 256, 0, st>>>(a, static_cast<__nv_bfloat16*>(qr), static_cast<__nv_bfloat16*>(qf), static_cast<__nv_bfloat16*>(kr),
                                                static_cast<__nv_bfloat16*>(kf));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int attn_prep_bwd(const void* q, long q_ts, int q_hs, const void* k, long k_ts, const float* wq, const float* wk, const float* cos, const float* sin,
                  const float* cos_c, const float* sin_c, int Hq, int Hkv, int R2, float eps, long tokens, const void* dqr, const void* dqf,
                  const void* dkr, const void* dkf, void* dqraw, void* dkraw, float* dw, int sms, cudaStream_t st) {
  PrepQK a{static_cast<const __nv_bfloat16*>(q), q_ts, q_hs, static_cast<const __nv_bfloat16*>(k), k_ts, wq, wk, cos, sin, cos_c, sin_c, Hq, Hkv, R2, eps, tokens};
  if (prep_check(a)) return 1;
  attn_prep_bwd_kernel<<<sms * 4, 256, 0, st>>>(a, static_cast<const __nv_bfloat16*>(dqr), static_cast<const __nv_bfloat16*>(dqf),
                                                static_cast<const __nv_bfloat16*>(dkr), static_cast<const __nv_bfloat16*>(dkf),
                                                static_cast<__nv_bfloat16*>(dqraw), static_cast<__nv_bfloat16*>(dkraw), dw);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ attention output gate
// y = o * sigmoid(gate) with the gate interleaved in the query projection's output: per token and head the 128
// channels are [q (64) | gate (64)]. Backward writes do and the gate half of the projection's gradient buffer.
__global__ void gate_out_fwd_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ qg, __nv_bfloat16* __restrict__ y, long n4) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long unit = i >> 4; const int c = static_cast<int>(i & 15) * 4;      // (token, head), channel
    float ov[4], gv[4], out[4];
    ld4(o + unit * 64 + c, ov);
    ld4(qg + unit * 128 + 64 + c, gv);
#pragma unroll
    for (int e = 0; e < 4; ++e) out[e] = ov[e] * sigm(gv[e]);
    st4(y + unit * 64 + c, out);
  }
}
__global__ void gate_out_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ qg,
                                    __nv_bfloat16* __restrict__ dO, __nv_bfloat16* __restrict__ dqg, long n4) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long unit = i >> 4; const int c = static_cast<int>(i & 15) * 4;
    float dv[4], ov[4], gv[4], a[4], b[4];
    ld4(dy + unit * 64 + c, dv);
    ld4(o + unit * 64 + c, ov);
    ld4(qg + unit * 128 + 64 + c, gv);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float s = sigm(gv[e]); a[e] = dv[e] * s; b[e] = dv[e] * ov[e] * s * (1.f - s); }
    st4(dO + unit * 64 + c, a);
    st4(dqg + unit * 128 + 64 + c, b);
  }
}
int gate_out_fwd(const void* o, const void* qg, void* y, long units, int sms, cudaStream_t st) {
  using T = __nv_bfloat16;
  gate_out_fwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const T*>(o), static_cast<const T*>(qg), static_cast<T*>(y), units * 16);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int gate_out_bwd(const void* dy, const void* o, const void* qg, void* dO, void* dqg, long units, int sms, cudaStream_t st) {
  using T = __nv_bfloat16;
  gate_out_bwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(o), static_cast<const T*>(qg), static_cast<T*>(dO),
                                               static_cast<T*>(dqg), units * 16);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ GDN decode step
// One token of the gated delta rule per (row, value head), in place on the fp32 state S [B, Hv, 128, dv]:
//   S <- 0 at a document start;  S <- S e^g;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// (ced/model/gdn.py:1153-1189 per token). A thread owns one column of S in registers, so the state is read once and
// written once (the tensor-op form makes five passes over it). q, k: [B, Hk, 128] fp32; v, o: [B, Hv, dv] fp32; g, beta:
// [B, Hv]; value head j reads key head j / (Hv / Hk). Grid (dv / 128, Hv, B), 256 threads (two per column).
__global__ void __launch_bounds__(256) gdn_step_kernel(float* __restrict__ S, const float* __restrict__ q, const float* __restrict__ k,
                                                       const float* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                                                       const unsigned char* __restrict__ start, float* __restrict__ o, int Hk, int Hv, int dv) {
  constexpr int DK = 128, HALF = 64;          // threads 0-127 hold rows 0-63 of their column, threads 128-255 rows 64-127
  __shared__ float sq[DK], sk[DK], part[2][128];
  const int b = blockIdx.z, hv = blockIdx.y, c = threadIdx.x & 127, half = threadIdx.x >> 7, col = blockIdx.x * 128 + c;
  const int hk = hv / (Hv / Hk);
  if (threadIdx.x < DK) sq[threadIdx.x] = q[(static_cast<long>(b) * Hk + hk) * DK + threadIdx.x];
  else sk[threadIdx.x - DK] = k[(static_cast<long>(b) * Hk + hk) * DK + threadIdx.x - DK];
  __syncthreads();
  const long bh = static_cast<long>(b) * Hv + hv;
  float* Sp = S + bh * DK * dv + static_cast<long>(half) * HALF * dv + col;
  const float* kk = sk + half * HALF;
  const float* qq = sq + half * HALF;
  const bool fresh = start != nullptr && start[b] != 0;
  const float decay = __expf(g[bh]);
  float s[HALF];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < HALF; ++i) {
    s[i] = fresh ? 0.f : Sp[static_cast<long>(i) * dv] * decay;
    dot += s[i] * kk[i];
  }
  part[half][c] = dot;
  __syncthreads();
  const float u = beta[bh] * (v[bh * dv + col] - (part[0][c] + part[1][c]));
  float out = 0.f;
#pragma unroll
  for (int i = 0; i < HALF; ++i) {
    s[i] += kk[i] * u;
    out += s[i] * qq[i];
    Sp[static_cast<long>(i) * dv] = s[i];
  }
  __syncthreads();
  part[half][c] = out;
  __syncthreads();
  if (half == 0) o[bh * dv + col] = part[0][c] + part[1][c];
}
int gdn_step(float* S, const float* q, const float* k, const float* v, const float* g, const float* beta, const unsigned char* start, float* o,
             int B, int Hk, int Hv, int dk, int dv, cudaStream_t st) {
  if (dk != 128 || dv % 128 || Hv % Hk) return 1;
  gdn_step_kernel<<<dim3(dv / 128, Hv, B), 256, 0, st>>>(S, q, k, v, g, beta, start, o, Hk, Hv, dv);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
