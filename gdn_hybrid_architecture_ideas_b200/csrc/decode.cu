// Single-token decode attention over a static KV cache (flash-decoding: split the cached positions over CTAs, merge
// the partial softmax statistics), with the rotary distance cap applied through the relative-rotation identity
//   R(p_q) q . R(p_k) k = q . R(-(p_q - p_k)) k     and, beyond the cap C,   R(C) q . k = q . R(-C) k,
// so the cache holds ONE copy of the keys (normed, unrotated) and the kernel rotates by min(distance, C) while it
// scores; the reference keeps a rotated and an unrotated copy and scores near and far keys in two partial attentions
// merged by log-sum-exp (ced/infer/engine.py:391-457). Batched (the reference engine is batch 1), any query/KV head
// grouping; memory-bound by design: every cached key and value byte is read once per step.
#include "kernels.h"
#include <cuda_bf16.h>

namespace ghb {

constexpr int DH = 64;          // head dimension
constexpr int DTILE = 32;       // positions per warp tile
constexpr int DWARPS = 4;
constexpr int MAXG = 16;        // query heads per KV head

struct DecodeArgs {
  const float* q;               // [B, Hq, 64] normed, temperature-scaled, unrotated queries
  const __nv_bfloat16* k;       // [B, T, Hkv, 64] normed, unrotated keys
  const __nv_bfloat16* v;       // [B, T, Hkv, 64]
  const int* lens;              // [B] cached positions including the current token
  const int* doc_start;         // [B] first position of the current document (earlier positions are masked), or null
  const float* cos_t; const float* sin_t;   // [n_angles, r/2] rotation tables indexed by min(distance, cap)
  float* part_o; float* part_ml;             // [B, Hq, splits, 64], [B, Hq, splits, 2]
  int T, Hq, Hkv, rot, cap, n_angles, splits;
  float scale;
};

template <int G>
__global__ void __launch_bounds__(DWARPS * 32, G <= 4 ? 4 : 1)
decode_attn_partial_kernel(DecodeArgs a) {
  __shared__ float sq[MAXG][DH];
  __shared__ float sp[DWARPS][DTILE][MAXG];
  __shared__ float s_m[DWARPS][MAXG], s_l[DWARPS][MAXG], s_o[DWARPS][MAXG][DH];
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < G * DH; i += blockDim.x) sq[i / DH][i % DH] = a.q[(static_cast<long>(b) * a.Hq + hk * G + i / DH) * DH + i % DH] * a.scale;
  __syncthreads();
  const int len = a.lens[b];
  const int first = a.doc_start ? a.doc_start[b] : 0;
  const int per = (len - first + a.splits - 1) / a.splits;
  const int lo = first + split * per, hi = min(len, lo + per);
  const int qpos = len - 1;
  const int half = a.rot / 2;
  // P V: a lane holds 8 output dimensions (vc .. vc + 7) and every fourth key of a tile (vr, vr + 4, ...), so a tile's values
  // arrive as 8 independent 16-byte loads per lane (4 key rows per warp instruction); the four lane groups meet at the end.
  const int vr = lane >> 3, vc = (lane & 7) * 8;
  float m[G], l[G], o[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[g][e] = 0.f;
  }
  for (int t0 = lo + warp * DTILE; t0 < hi; t0 += DWARPS * DTILE) {
    const int t = t0 + lane;
    float logit[G];
#pragma unroll
    for (int g = 0; g < G; ++g) logit[g] = -INFINITY;
    if (t < hi) {
      const __nv_bfloat16* kp = a.k + ((static_cast<long>(b) * a.T + t) * a.Hkv + hk) * DH;
      float kf[DH];
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        const uint4 pk = reinterpret_cast<const uint4*>(kp)[c];
        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])); kf[c * 8 + 2 * e] = f.x; kf[c * 8 + 2 * e + 1] = f.y; }
      }
      if (half > 0) {       // rotate the key by -(min(distance, cap)): k'_i = k_i cos + k_{i+half} sin ; k'_{i+half} = k_{i+half} cos - k_i sin
        int d = qpos - t;
        if (a.cap >= 0 && d > a.cap) d = a.cap;
        d = min(d, a.n_angles - 1);
        // half is one of 8 / 16 / 32 in practice; static indices keep the key row in registers
#define GHB_ROT(HALF)                                                                   \
        _Pragma("unroll") for (int i = 0; i < HALF; ++i) {                              \
          const float c = a.cos_t[d * HALF + i], s = a.sin_t[d * HALF + i];              \
          const float x1 = kf[i], x2 = kf[i + HALF];                                     \
          kf[i] = x1 * c + x2 * s;                                                       \
          kf[i + HALF] = x2 * c - x1 * s;                                                \
        }
        if (half == 8) { GHB_ROT(8) } else if (half == 16) { GHB_ROT(16) } else if (half == 32) { GHB_ROT(32) } else if (half == 4) { GHB_ROT(4) }
#undef GHB_ROT
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int dd = 0; dd < DH; ++dd) acc += sq[g][dd] * kf[dd];
        logit[g] = acc;
      }
    }
    // tile softmax statistics per head, then P V with lanes over dimensions
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = logit[g];
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      const float m_new = fmaxf(m[g], mx);
      const float p = (logit[g] == -INFINITY) ? 0.f : __expf(logit[g] - m_new);
      float ps = p;
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, s);
      const float alpha = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
      l[g] = l[g] * alpha + ps;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[g][e] *= alpha;
      m[g] = m_new;
      sp[warp][lane][g] = p;          // 0 for the lanes past the end of the split
    }
    __syncwarp();
    uint4 vv[DTILE / 4];
#pragma unroll
    for (int i = 0; i < DTILE / 4; ++i) {
      const int j = 4 * i + vr;
      vv[i] = (t0 + j < hi) ? *reinterpret_cast<const uint4*>(a.v + ((static_cast<long>(b) * a.T + t0 + j) * a.Hkv + hk) * DH + vc) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < DTILE / 4; ++i) {
      const int j = 4 * i + vr;
      const uint32_t w[4] = {vv[i].x, vv[i].y, vv[i].z, vv[i].w};
      float vf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])); vf[2 * e] = f.x; vf[2 * e + 1] = f.y; }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = sp[warp][j][g];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[g][e] += p * vf[e];
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[g][e] += __shfl_xor_sync(0xffffffffu, o[g][e], 8);
      o[g][e] += __shfl_xor_sync(0xffffffffu, o[g][e], 16);
    }
  // merge the warps of this CTA, write the split's partial result
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
    if (vr == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) s_o[warp][g][vc + e] = o[g][e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * DH; idx += blockDim.x) {
    const int g = idx / DH, d = idx % DH;
    float mm = -INFINITY;
    for (int w = 0; w < DWARPS; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < DWARPS; ++w) {
      const float sc = (s_m[w][g] == -INFINITY) ? 0.f : __expf(s_m[w][g] - mm);
      ll += s_l[w][g] * sc; oo += s_o[w][g][d] * sc;
    }
    const long base = (static_cast<long>(b) * a.Hq + hk * G + g) * a.splits + split;
    a.part_o[base * DH + d] = oo;
    if (d == 0) { a.part_ml[base * 2] = mm; a.part_ml[base * 2 + 1] = ll; }
  }
}

__global__ void decode_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                                         int splits) {
  const long bh = blockIdx.x;           // (b, query head)
  const int d = threadIdx.x;            // 64 threads
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(bh * splits + s) * 2]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(bh * splits + s) * 2];
    const float sc = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += part_ml[(bh * splits + s) * 2 + 1] * sc;
    oo += part_o[(bh * splits + s) * DH + d] * sc;
  }
  out[bh * DH + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
}

// q: [B, Hq, 64] fp32; k, v: [B, T, Hkv, 64] bf16; out: [B, Hq, 64] bf16; part_o / part_ml: scratch of
// B*Hq*splits*64 and B*Hq*splits*2 floats. cap < 0: no distance cap. rot: rotary dimensions (0: position-free).
int decode_attention(const float* q, const void* k, const void* v, const int* lens, const int* doc_start, const float* cos_t, const float* sin_t,
                     void* out, float* part_o, float* part_ml, int B, int T, int Hq, int Hkv, int rot, int cap, int n_angles, int splits,
                     float scale, cudaStream_t st) {
  if (Hq % Hkv || Hq / Hkv > MAXG || (rot != 0 && rot != 8 && rot != 16 && rot != 32 && rot != 64) || splits < 1) return 1;
  DecodeArgs a{q, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), lens, doc_start, cos_t, sin_t, part_o, part_ml,
               T, Hq, Hkv, rot, cap, n_angles, splits, scale};
  const dim3 grid(splits, Hkv, B);
  switch (Hq / Hkv) {
    case 1: decode_attn_partial_kernel<1><<<grid, DWARPS * 32, 0, st>>>(a); break;
    case 2: decode_attn_partial_kernel<2><<<grid, DWARPS * 32, 0, st>>>(a); break;
    case 4: decode_attn_partial_kernel<4><<<grid, DWARPS * 32, 0, st>>>(a); break;
    case 8: decode_attn_partial_kernel<8><<<grid, DWARPS * 32, 0, st>>>(a); break;
    case 16: decode_attn_partial_kernel<16><<<grid, DWARPS * 32, 0, st>>>(a); break;
    default: return 1;
  }
  decode_attn_merge_kernel<<<B * Hq, DH, 0, st>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), splits);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ grid KV sharing
// Grid-shared keys and values (4 row components and 4 column components of 32 channels; head (i, j) reads
// [row_i ; col_j]) scored straight from the RAW cached components, so the cache holds 256 channels per token like
// grouped attention with 4 KV heads instead of the 16 assembled heads (reference cache: ced/model/attention.py:943-1030).
// The key norm runs over the assembled 64-channel head, so it cannot be cached per component; it factors as
//   k_(i,j) = [g_r * row_i ; g_c * col_j] * rsqrt((|row_i|^2 + |col_j|^2) / 64 + eps)
// and the kernel forms the two sums of squares from the cached values, applies the gain, rotates the row part by
// min(distance, cap) (the rotary channels are the head's first ones) and scales each head's score by its factor.
// One CTA per (split of the cached positions, batch row): a tile of 32 positions is staged in shared memory once
// (512 bytes of keys and of values per position), warp i scores and accumulates the four heads of grid row i.
constexpr int GR = 4, GCO = 4, GD = 32;            // grid rows, columns, channels per component
constexpr int GW = (GR + GCO) * GD;                // 256 cached channels per token
constexpr int GROW = GW * 2 + 16;                  // shared-memory bytes per cached token (16 bytes of padding: conflict-free 16-byte reads)

struct GridDecodeArgs {
  const float* q;               // [B, 16, 64] normed, temperature-scaled, unrotated queries
  const __nv_bfloat16* k;       // [B, T, 256] raw key components
  const __nv_bfloat16* v;       // [B, T, 256] raw value components
  const int* lens; const int* doc_start;
  const float* cos_t; const float* sin_t;
  const float* gain;            // [64] key-norm gain, or null (no key norm)
  float* part_o; float* part_ml;
  int T, rot, cap, n_angles, splits;
  float scale, eps;
};

__device__ __forceinline__ void unpack8(const uint4 pk, float* f) {
  const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}

__global__ void __launch_bounds__(GR * 32, 4)
decode_attn_grid_kernel(GridDecodeArgs a) {
  __shared__ float sq[GR * GCO][DH];
  __shared__ float sg[DH];
  __shared__ __align__(16) uint8_t sk[DTILE * GROW];
  __shared__ __align__(16) uint8_t sv[DTILE * GROW];
  __shared__ float sp[GR][DTILE][GCO];
  const int split = blockIdx.x, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;      // warp = grid row
  for (int i = threadIdx.x; i < GR * GCO * DH; i += blockDim.x) sq[i / DH][i % DH] = a.q[static_cast<long>(b) * GR * GCO * DH + i] * a.scale;
  if (threadIdx.x < DH) sg[threadIdx.x] = a.gain ? a.gain[threadIdx.x] : 1.f;
  __syncthreads();
  const int len = a.lens[b];
  const int first = a.doc_start ? a.doc_start[b] : 0;
  const int per = (len - first + a.splits - 1) / a.splits;
  const int lo = first + split * per, hi = min(len, lo + per);
  const int qpos = len - 1;
  const int half = a.rot / 2;
  const int vr = lane >> 3, vc8 = lane & 7;
  float m[GCO], l[GCO], o[GCO][8];
#pragma unroll
  for (int j = 0; j < GCO; ++j) {
    m[j] = -INFINITY; l[j] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[j][e] = 0.f;
  }
  for (int t0 = lo; t0 < hi; t0 += DTILE) {
    __syncthreads();      // the tile before is consumed
    // ---- stage 32 positions x 512 bytes of keys and of values (16 bytes per thread and pass, coalesced)
    {
      uint4 kk[8], vv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = i * 128 + threadIdx.x;          // 16-byte piece of the tile
        const int tok = idx >> 5, piece = idx & 31;
        const bool in = t0 + tok < hi;
        const long off = (static_cast<long>(b) * a.T + t0 + tok) * GW + piece * 8;
        kk[i] = in ? *reinterpret_cast<const uint4*>(a.k + off) : make_uint4(0u, 0u, 0u, 0u);
        vv[i] = in ? *reinterpret_cast<const uint4*>(a.v + off) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = i * 128 + threadIdx.x;
        const int tok = idx >> 5, piece = idx & 31;
        *reinterpret_cast<uint4*>(sk + tok * GROW + piece * 16) = kk[i];
        *reinterpret_cast<uint4*>(sv + tok * GROW + piece * 16) = vv[i];
      }
    }
    __syncthreads();
    // ---- scores of heads (warp, 0..3) for position t0 + lane
    const int t = t0 + lane;
    float logit[GCO];
#pragma unroll
    for (int j = 0; j < GCO; ++j) logit[j] = -INFINITY;
    if (t < hi) {
      float x[GD];
      const uint8_t* base = sk + lane * GROW;
#pragma unroll
      for (int c = 0; c < GD / 8; ++c) unpack8(*reinterpret_cast<const uint4*>(base + warp * (GD * 2) + c * 16), x + c * 8);
      float ss_r = 0.f;
#pragma unroll
      for (int i = 0; i < GD; ++i) { ss_r += x[i] * x[i]; x[i] *= sg[i]; }
      if (half > 0) {
        int d = qpos - t;
        if (a.cap >= 0 && d > a.cap) d = a.cap;
        d = min(d, a.n_angles - 1);
#define GHB_GROT(HALF)                                                                  \
        _Pragma("unroll") for (int i = 0; i < HALF; ++i) {                              \
          const float c = a.cos_t[d * HALF + i], s = a.sin_t[d * HALF + i];              \
          const float x1 = x[i], x2 = x[i + HALF];                                       \
          x[i] = x1 * c + x2 * s;                                                        \
          x[i + HALF] = x2 * c - x1 * s;                                                 \
        }
        if (half == 8) { GHB_GROT(8) } else if (half == 16) { GHB_GROT(16) } else if (half == 4) { GHB_GROT(4) }
#undef GHB_GROT
      }
      float acc[GCO];
#pragma unroll
      for (int j = 0; j < GCO; ++j) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < GD; ++i) s += sq[warp * GCO + j][i] * x[i];
        acc[j] = s;
      }
#pragma unroll
      for (int j = 0; j < GCO; ++j) {
#pragma unroll
        for (int c = 0; c < GD / 8; ++c) unpack8(*reinterpret_cast<const uint4*>(base + (GR + j) * (GD * 2) + c * 16), x + c * 8);
        float ss_c = 0.f, s = 0.f;
#pragma unroll
        for (int i = 0; i < GD; ++i) { ss_c += x[i] * x[i]; s += sq[warp * GCO + j][GD + i] * (x[i] * sg[GD + i]); }
        const float factor = a.gain ? rsqrtf((ss_r + ss_c) * (1.f / DH) + a.eps) : 1.f;
        logit[j] = (acc[j] + s) * factor;
      }
    }
#pragma unroll
    for (int j = 0; j < GCO; ++j) {
      float mx = logit[j];
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      const float m_new = fmaxf(m[j], mx);
      const float p = (logit[j] == -INFINITY) ? 0.f : __expf(logit[j] - m_new);
      float ps = p;
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, s);
      const float alpha = (m[j] == -INFINITY) ? 0.f : __expf(m[j] - m_new);
      l[j] = l[j] * alpha + ps;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[j][e] *= alpha;
      m[j] = m_new;
      sp[warp][lane][j] = p;
    }
    __syncwarp();
    // ---- P V: a lane holds 8 channels of the head's output and every fourth position; channels 0..31 come from value
    // row component `warp` (shared by the four heads), channels 32..63 from column component j
#pragma unroll
    for (int i = 0; i < DTILE / 4; ++i) {
      const int jt = 4 * i + vr;
      const uint8_t* base = sv + jt * GROW;
      float vf[8];
      if (vc8 < 4) {
        unpack8(*reinterpret_cast<const uint4*>(base + warp * (GD * 2) + vc8 * 16), vf);
#pragma unroll
        for (int j = 0; j < GCO; ++j) {
          const float p = sp[warp][jt][j];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[j][e] += p * vf[e];
        }
      } else {
#pragma unroll
        for (int j = 0; j < GCO; ++j) {
          unpack8(*reinterpret_cast<const uint4*>(base + (GR + j) * (GD * 2) + (vc8 - 4) * 16), vf);
          const float p = sp[warp][jt][j];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[j][e] += p * vf[e];
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < GCO; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[j][e] += __shfl_xor_sync(0xffffffffu, o[j][e], 8);
      o[j][e] += __shfl_xor_sync(0xffffffffu, o[j][e], 16);
    }
  // every warp owns its four heads: the split's partial result leaves without a merge across warps
#pragma unroll
  for (int j = 0; j < GCO; ++j) {
    const long base = (static_cast<long>(b) * GR * GCO + warp * GCO + j) * a.splits + split;
    if (vr == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) a.part_o[base * DH + vc8 * 8 + e] = o[j][e];
    }
    if (lane == 0) { a.part_ml[base * 2] = m[j]; a.part_ml[base * 2 + 1] = l[j]; }
  }
}

// q [B, 16, 64] fp32; k, v [B, T, 256] bf16 raw components of a 4 x 4 grid with 32-channel components; gain [64] or null.
int decode_attention_grid(const float* q, const void* k, const void* v, const int* lens, const int* doc_start, const float* cos_t,
                          const float* sin_t, const float* gain, void* out, float* part_o, float* part_ml, int B, int T, int rot, int cap,
                          int n_angles, int splits, float scale, float eps, cudaStream_t st) {
  if ((rot != 0 && rot != 8 && rot != 16 && rot != 32) || rot > GD || splits < 1) return 1;
  GridDecodeArgs a{q, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), lens, doc_start, cos_t, sin_t, gain, part_o, part_ml,
                   T, rot, cap, n_angles, splits, scale, eps};
  decode_attn_grid_kernel<<<dim3(splits, 1, B), GR * 32, 0, st>>>(a);
  decode_attn_merge_kernel<<<B * GR * GCO, DH, 0, st>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), splits);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb

// ================================================================================================ allocation-free entry
// See noalloc.h for who needs this and the contract. The scratch is a file-scope device array: in host code its name
// is only a handle for the runtime, so the device address is resolved once per device with cudaGetSymbolAddress.
#include "noalloc.h"
#include <mutex>
#include <stdio.h>

namespace {
constexpr size_t NOALLOC_FLOATS = GHB_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_scratch_addr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_scratch_mutex;

int fail(int code, char* buf, int len, const char* msg) {
  if (buf && len > 0) snprintf(buf, static_cast<size_t>(len), "%s", msg);
  return code;
}
}  // namespace

extern "C" int ghb_decode_attention_noalloc(const float* q, const void* k, const void* v, const int* lens, const int* doc_start,
                                            const float* cos_t, const float* sin_t, void* out, int B, int T, int Hq, int Hkv, int rot,
                                            int cap, int n_angles, int splits, float scale, void* stream, char* errbuf, int errlen) {
  if (B < 1 || T < 1 || Hq < 1 || Hkv < 1 || splits < 1)
    return fail(1, errbuf, errlen, "ghb_decode_attention_noalloc: B, T, Hq, Hkv and splits must be positive");
  if (!q || !k || !v || !lens || !out)
    return fail(1, errbuf, errlen, "ghb_decode_attention_noalloc: q, k, v, lens and out must be device pointers");
  if (rot < 0 || (rot > 0 && (n_angles < 1 || !cos_t || !sin_t)))
    return fail(1, errbuf, errlen, "ghb_decode_attention_noalloc: a rotary width above 0 needs cos/sin tables with at least one angle row");
  const size_t need = static_cast<size_t>(B) * Hq * splits * 66;
  if (need > NOALLOC_FLOATS) {
    char msg[200];
    snprintf(msg, sizeof msg, "ghb_decode_attention_noalloc: B*Hq*splits*66 = %zu floats exceeds the built-in scratch of %zu floats; use fewer splits or the regular entry",
             need, static_cast<size_t>(NOALLOC_FLOATS));
    return fail(1, errbuf, errlen, msg);
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
    return fail(2, errbuf, errlen, "ghb_decode_attention_noalloc: no current device (or more than 64 devices)");
  float* scratch;
  {
    std::lock_guard<std::mutex> hold(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {     // first call on this device: resolve the array's device address (before any stream capture)
      void* p = nullptr;
      const cudaError_t rc = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (rc != cudaSuccess || !p) {
        char msg[200];
        snprintf(msg, sizeof msg, "ghb_decode_attention_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(rc));
        return fail(2, errbuf, errlen, msg);
      }
      g_scratch_addr[dev] = static_cast<float*>(p);
    }
    scratch = g_scratch_addr[dev];
  }
  float* part_o = scratch;
  float* part_ml = scratch + static_cast<size_t>(B) * Hq * splits * 64;
  const int rc = ghb::decode_attention(q, k, v, lens, doc_start, cos_t, sin_t, out, part_o, part_ml, B, T, Hq, Hkv, rot, cap, n_angles, splits,
                                       scale, static_cast<cudaStream_t>(stream));
  if (rc == 1) return fail(1, errbuf, errlen, "ghb_decode_attention_noalloc: unsupported head grouping (Hq/Hkv in 1,2,4,8,16) or rotary width (0,8,16,32,64)");
  if (rc != 0) return fail(4, errbuf, errlen, "ghb_decode_attention_noalloc: kernel launch refused by the runtime");
  return 0;
}
