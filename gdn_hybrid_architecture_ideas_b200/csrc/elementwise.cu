// Bandwidth-bound kernels: RMSNorm family (plain, gated, residual-add), SwiGLU activation, fused AdamW, reductions.
// Each reads its inputs once and writes its outputs once; statistics are fp32; vectors are 8-16 bytes per lane.
//
// Reference behaviour: ced/model/norms.py:51-94 (zero-centred gain, >= fp32 maths), ced/model/mlp.py:20-36,
// ced/train/muon.py:112-128 (AdamW branch). The reference leaves these to Inductor-fused elementwise graphs.
#include "kernels.h"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace ghb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// ex2.approx.ftz and rcp.approx.ftz: one issue slot each, relative error of a few ulp (the default forms add denormal
// scaling, a full-precision division an order of magnitude more; the elementwise kernels are issue-bound). Saturates
// correctly: ex2 of a large argument is inf and rcp(inf) = 0.
__device__ __forceinline__ float sigmoidf_(float x) {
  float e, y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(1.f + e));
  return y;
}

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t; t.x = *reinterpret_cast<uint32_t*>(&a); t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

// ------------------------------------------------------------------------------------------------ RMSNorm forward
// One warp per row; lane handles 4 consecutive channels per iteration (ITERS * 128 >= d).
// y = [resid +] scale * x * rstd * (1 + w) [* act(z)], rstd = rsqrt(mean x^2 + eps) saved for the backward.
template <typename TI, typename TO, int ITERS, int GATE>
__global__ void rmsnorm_fwd_kernel(const TI* __restrict__ x, const float* __restrict__ w, int w_scalar, const __nv_bfloat16* __restrict__ z,
                                   const float* __restrict__ resid, TO* __restrict__ y, float* __restrict__ rstd, long rows, int d,
                                   float eps, float scale) {
  const int lane = threadIdx.x & 31;
  const long row = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const TI* xr = x + row * d;
  float v[ITERS][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < d) { Vec4<TI>::load(xr + c, v[i]); ss += v[i][0] * v[i][0] + v[i][1] * v[i][1] + v[i][2] * v[i][2] + v[i][3] * v[i][3]; }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / d + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < d) {
      float g[4], o[4];
      if (w_scalar) { g[0] = g[1] = g[2] = g[3] = 1.f + w[0]; }
      else { float4 t = *reinterpret_cast<const float4*>(w + c); g[0] = 1.f + t.x; g[1] = 1.f + t.y; g[2] = 1.f + t.z; g[3] = 1.f + t.w; }
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = v[i][e] * r * g[e] * scale;
      if (GATE) {
        float zz[4]; Vec4<__nv_bfloat16>::load(z + row * d + c, zz);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float s = sigmoidf_(zz[e]); o[e] *= (GATE == 1 ? zz[e] * s : s); }
      }
      if (resid) { float rr[4]; Vec4<float>::load(resid + row * d + c, rr);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] += rr[e]; }
      Vec4<TO>::store(y + row * d + c, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------ RMSNorm backward
// g = scale * dy * [act(z)] * (1 + w); dx = rstd * (g - xhat * mean(g * xhat)) [+ dres]; dw += scale * dy * [act] * xhat;
// dz = dy * scale * xhat * (1 + w) * act'(z). WPR warps share a row (each lane covers 4 * ITERS of its warp's
// d / WPR channels), so a wide row costs few registers per thread and many warps stay resident; the row's dot
// product crosses warps through shared memory. Blocks walk rows with a grid stride (the same trip count for every
// warp of a block) and keep their dw partial in registers; partials meet in shared memory, then one atomicAdd per
// channel per block.
constexpr int NORM_BWD_WARPS = 8;

template <typename TI, typename TG, int ITERS, int WPR, int GATE>
__global__ void __launch_bounds__(NORM_BWD_WARPS * 32)
rmsnorm_bwd_kernel(const TG* __restrict__ dy, const TI* __restrict__ x, const float* __restrict__ w, int w_scalar,
                   const __nv_bfloat16* __restrict__ z, const float* __restrict__ rstd, const float* __restrict__ dres,
                   TI* __restrict__ dx, __nv_bfloat16* __restrict__ dz, float* __restrict__ dw, long rows, int d, float scale) {
  extern __shared__ float red[];   // d floats, then 2 x NORM_BWD_WARPS exchange slots
  float* xch = red + d;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int RPB = NORM_BWD_WARPS / WPR;            // rows per block per trip
  const int rsub = warp / WPR, wsub = warp % WPR;
  for (int c = threadIdx.x; c < d; c += blockDim.x) red[c] = 0.f;
  __syncthreads();
  float acc[ITERS][4];
#pragma unroll
  for (int i = 0; i < ITERS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const float g_scalar = w_scalar ? 1.f + w[0] : 0.f;
  int par = 0;
  for (long base = static_cast<long>(blockIdx.x) * RPB; base < rows; base += static_cast<long>(gridDim.x) * RPB) {
    const long row = base + rsub;
    const bool live = row < rows;
    const float r = live ? rstd[row] : 0.f;
    float xh[ITERS][4], gg[ITERS][4];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = ((wsub * ITERS + i) * 32 + lane) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) { xh[i][e] = 0.f; gg[i][e] = 0.f; }
      if (live && c < d) {
        float xv[4], dv[4], g1[4];
        Vec4<TI>::load(x + row * d + c, xv);
        Vec4<TG>::load(dy + row * d + c, dv);
        if (w_scalar) { g1[0] = g1[1] = g1[2] = g1[3] = g_scalar; }
        else { const float4 t = __ldg(reinterpret_cast<const float4*>(w + c)); g1[0] = 1.f + t.x; g1[1] = 1.f + t.y; g1[2] = 1.f + t.z; g1[3] = 1.f + t.w; }
        float zz[4] = {0.f, 0.f, 0.f, 0.f};
        if (GATE) Vec4<__nv_bfloat16>::load(z + row * d + c, zz);
        float dzv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xh[i][e] = xv[e] * r;
          float dn = dv[e] * scale;        // gradient w.r.t. the normalised, gained value (before the gate)
          if (GATE) {
            const float s = sigmoidf_(zz[e]);
            const float act = GATE == 1 ? zz[e] * s : s;
            const float dact = GATE == 1 ? s * (1.f + zz[e] * (1.f - s)) : s * (1.f - s);
            dzv[e] = dn * xh[i][e] * g1[e] * dact;
            dn *= act;
          }
          acc[i][e] += dn * xh[i][e];
          gg[i][e] = dn * g1[e];
          dot += gg[i][e] * xh[i][e];
        }
        if (GATE) Vec4<__nv_bfloat16>::store(dz + row * d + c, dzv);
      }
    }
    dot = warp_sum(dot);
    if (WPR > 1) {                     // two alternating slot sets: a warp may run one trip ahead of its row partners
      if (lane == 0) xch[par * NORM_BWD_WARPS + warp] = dot;
      __syncthreads();
      dot = 0.f;
#pragma unroll
      for (int k = 0; k < WPR; ++k) dot += xch[par * NORM_BWD_WARPS + rsub * WPR + k];
      par ^= 1;
    }
    dot /= d;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = ((wsub * ITERS + i) * 32 + lane) * 4;
      if (live && c < d) {
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = r * (gg[i][e] - xh[i][e] * dot);
        if (dres) { float rr[4]; Vec4<float>::load(dres + row * d + c, rr);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] += rr[e]; }
        Vec4<TI>::store(dx + row * d + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = ((wsub * ITERS + i) * 32 + lane) * 4;
    if (c < d) {
#pragma unroll
      for (int e = 0; e < 4; ++e) atomicAdd(&red[c + e], acc[i][e]);
    }
  }
  __syncthreads();
  if (w_scalar) {
    float t = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) t += red[c];
    t = warp_sum(t);
    if (lane == 0) atomicAdd(dw, t);
  } else {
    for (int c = threadIdx.x; c < d; c += blockDim.x) atomicAdd(dw + c, red[c]);
  }
}

template <typename TI, typename TO, int GATE>
static int norm_fwd_t(const void* x, const float* w, int ws, const void* z, const float* resid, void* y, float* rstd, long rows, int d,
                      float eps, float scale, cudaStream_t st) {
  const int warps = 4;
  dim3 grid(static_cast<unsigned>((rows + warps - 1) / warps)), block(warps * 32);
#define GHB_LAUNCH(IT) rmsnorm_fwd_kernel<TI, TO, IT, GATE><<<grid, block, 0, st>>>(static_cast<const TI*>(x), w, ws, static_cast<const __nv_bfloat16*>(z), resid, static_cast<TO*>(y), rstd, rows, d, eps, scale)
  if (d <= 128) GHB_LAUNCH(1); else if (d <= 256) GHB_LAUNCH(2); else if (d <= 512) GHB_LAUNCH(4); else if (d <= 1024) GHB_LAUNCH(8);
  else if (d <= 2048) GHB_LAUNCH(16); else return 1;
#undef GHB_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// in_dtype / out_dtype: 0 fp32, 1 bf16. gate: 0 none, 1 SiLU, 2 sigmoid.
int rmsnorm_fwd(const void* x, int in_bf16, const float* w, int w_scalar, const void* z, int gate, const float* resid, void* y,
                int out_bf16, float* rstd, long rows, int d, float eps, float scale, cudaStream_t st) {
  if (d % 4) return 1;
#define GHB_G(TI, TO)                                                                                          \
  (gate == 0 ? norm_fwd_t<TI, TO, 0>(x, w, w_scalar, z, resid, y, rstd, rows, d, eps, scale, st)                 \
             : (gate == 1 ? norm_fwd_t<TI, TO, 1>(x, w, w_scalar, z, resid, y, rstd, rows, d, eps, scale, st)    \
                          : norm_fwd_t<TI, TO, 2>(x, w, w_scalar, z, resid, y, rstd, rows, d, eps, scale, st)))
  if (in_bf16 && out_bf16) return GHB_G(__nv_bfloat16, __nv_bfloat16);
  if (in_bf16) return GHB_G(__nv_bfloat16, float);
  if (out_bf16) return GHB_G(float, __nv_bfloat16);
  return GHB_G(float, float);
#undef GHB_G
}

template <typename TI, typename TG, int ITERS, int WPR, int GATE>
static int norm_bwd_launch(const void* dy, const void* x, const float* w, int ws, const void* z, const float* rstd, const float* dres, void* dx,
                           void* dz, float* dw, long rows, int d, float scale, int sms, cudaStream_t st) {
  auto kern = rmsnorm_bwd_kernel<TI, TG, ITERS, WPR, GATE>;
  const size_t sh = (d + 2 * NORM_BWD_WARPS) * sizeof(float);
  int resident = 0;                  // blocks that fit one SM: the grid is one full wave, so no tail wave runs part-empty
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NORM_BWD_WARPS * 32, sh) != cudaSuccess || resident < 1) resident = 1;
  constexpr int RPB = NORM_BWD_WARPS / WPR;
  const long want = (rows + RPB - 1) / RPB;
  const long cap = static_cast<long>(sms) * resident;
  kern<<<static_cast<unsigned>(want < cap ? want : cap), NORM_BWD_WARPS * 32, sh, st>>>(
      static_cast<const TG*>(dy), static_cast<const TI*>(x), w, ws, static_cast<const __nv_bfloat16*>(z), rstd, dres, static_cast<TI*>(dx),
      static_cast<__nv_bfloat16*>(dz), dw, rows, d, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <typename TI, typename TG, int GATE>
static int norm_bwd_t(const void* dy, const void* x, const float* w, int ws, const void* z, const float* rstd, const float* dres, void* dx,
                      void* dz, float* dw, long rows, int d, float scale, int sms, cudaStream_t st) {
#define GHB_LAUNCH(IT, WPR) return norm_bwd_launch<TI, TG, IT, WPR, GATE>(dy, x, w, ws, z, rstd, dres, dx, dz, dw, rows, d, scale, sms, st)
  if (d <= 128) GHB_LAUNCH(1, 1);
  if (d <= 256) GHB_LAUNCH(2, 1);
  if (d <= 512) GHB_LAUNCH(4, 1);
  if (d <= 1024) GHB_LAUNCH(4, 2);
  if (d <= 2048) GHB_LAUNCH(4, 4);
#undef GHB_LAUNCH
  return 1;
}

// x_bf16: dtype of x and dx; dy_bf16: dtype of dy. dw must be zeroed (or hold a running sum) by the caller.
int rmsnorm_bwd(const void* dy, int dy_bf16, const void* x, int x_bf16, const float* w, int w_scalar, const void* z, int gate,
                const float* rstd, const float* dres, void* dx, void* dz, float* dw, long rows, int d, float scale, int sms, cudaStream_t st) {
  if (d % 4) return 1;
#define GHB_G(TI, TG)                                                                                                    \
  (gate == 0 ? norm_bwd_t<TI, TG, 0>(dy, x, w, w_scalar, z, rstd, dres, dx, dz, dw, rows, d, scale, sms, st)               \
             : (gate == 1 ? norm_bwd_t<TI, TG, 1>(dy, x, w, w_scalar, z, rstd, dres, dx, dz, dw, rows, d, scale, sms, st)  \
                          : norm_bwd_t<TI, TG, 2>(dy, x, w, w_scalar, z, rstd, dres, dx, dz, dw, rows, d, scale, sms, st)))
  if (x_bf16 && dy_bf16) return GHB_G(__nv_bfloat16, __nv_bfloat16);
  if (x_bf16) return GHB_G(__nv_bfloat16, float);
  if (dy_bf16) return GHB_G(float, __nv_bfloat16);
  return GHB_G(float, float);
#undef GHB_G
}

// ------------------------------------------------------------------------------------------------ SwiGLU activation
// h = silu(g) * u on bf16; g and u are column blocks of one [rows, ld] buffer (the fused gate_up GEMM output).
__global__ void silu_mul_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u, long ld,
                                    __nv_bfloat16* __restrict__ h, long rows, int f) {
  const long n4 = rows * (f / 4);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long row = i / (f / 4); const int c = static_cast<int>(i % (f / 4)) * 4;
    float a[4], b[4], o[4];
    Vec4<__nv_bfloat16>::load(g + row * ld + c, a);
    Vec4<__nv_bfloat16>::load(u + row * ld + c, b);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = a[e] * sigmoidf_(a[e]) * b[e];
    Vec4<__nv_bfloat16>::store(h + row * f + c, o);
  }
}
__global__ void silu_mul_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                    long ld, __nv_bfloat16* __restrict__ dg, __nv_bfloat16* __restrict__ du, long rows, int f) {
  const long n4 = rows * (f / 4);
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long row = i / (f / 4); const int c = static_cast<int>(i % (f / 4)) * 4;
    float a[4], b[4], d[4], og[4], ou[4];
    Vec4<__nv_bfloat16>::load(g + row * ld + c, a);
    Vec4<__nv_bfloat16>::load(u + row * ld + c, b);
    Vec4<__nv_bfloat16>::load(dh + row * f + c, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float s = sigmoidf_(a[e]);
      ou[e] = d[e] * a[e] * s;
      og[e] = d[e] * b[e] * s * (1.f + a[e] * (1.f - s));
    }
    Vec4<__nv_bfloat16>::store(dg + row * ld + c, og);
    Vec4<__nv_bfloat16>::store(du + row * ld + c, ou);
  }
}
int silu_mul_fwd(const void* g, const void* u, long ld, void* h, long rows, int f, int sms, cudaStream_t st) {
  if (f % 4 || ld % 4) return 1;
  silu_mul_fwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u), ld, static_cast<__nv_bfloat16*>(h), rows, f);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int silu_mul_bwd(const void* dh, const void* g, const void* u, long ld, void* dg, void* du, long rows, int f, int sms, cudaStream_t st) {
  if (f % 4 || ld % 4) return 1;
  silu_mul_bwd_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dh), static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u), ld,
                                               static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(du), rows, f);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ------------------------------------------------------------------------------------------------ AdamW, reductions
// Decoupled weight decay, bias corrections c1 = 1 - b1^t, c2 = 1 - b2^t passed in; the gradient is multiplied by
// *grad_scale (device scalar: the clip coefficient) when the pointer is given, else by scale_host. Writes the bf16
// compute copy in the same pass.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ lp, long n, float lr, float b1, float b2, float eps, float wd, float c1, float c2,
                             const float* __restrict__ grad_scale, float scale_host) {
  const float gs = grad_scale ? *grad_scale : scale_host;
  const long n4 = n / 4;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float pv[4], gv[4], mv[4], vv[4];
    Vec4<float>::load(p + i * 4, pv); Vec4<float>::load(g + i * 4, gv); Vec4<float>::load(m + i * 4, mv); Vec4<float>::load(v + i * 4, vv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float gr = gv[e] * gs;
      mv[e] = b1 * mv[e] + (1.f - b1) * gr;
      vv[e] = b2 * vv[e] + (1.f - b2) * gr * gr;
      pv[e] = pv[e] * (1.f - lr * wd) - (lr / c1) * mv[e] / (sqrtf(vv[e] / c2) + eps);
    }
    Vec4<float>::store(p + i * 4, pv); Vec4<float>::store(m + i * 4, mv); Vec4<float>::store(v + i * 4, vv);
    if (lp) Vec4<__nv_bfloat16>::store(lp + i * 4, pv);
  }
}
int adamw(float* p, const float* g, float* m, float* v, void* lp, long n, float lr, float b1, float b2, float eps, float wd, float c1,
          float c2, const float* grad_scale, float scale_host, int sms, cudaStream_t st) {
  if (n % 4) return 1;
  adamw_kernel<<<sms * 8, 256, 0, st>>>(p, g, m, v, static_cast<__nv_bfloat16*>(lp), n, lr, b1, b2, eps, wd, c1, c2, grad_scale, scale_host);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// partial[b] = sum of squares of block b's grid-stride share (deterministic: fixed grid, fixed order inside a block).
__global__ void sumsq_kernel(const float* __restrict__ x, long n, float* __restrict__ partial) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long n4 = n / 4;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 t = reinterpret_cast<const float4*>(x)[i];
    acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  for (long i = n4 * 4 + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) acc += x[i] * x[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}
int sumsq_partials(const float* x, long n, float* partial, int blocks, cudaStream_t st) {
  sumsq_kernel<<<blocks, 256, 0, st>>>(x, n, partial);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// y = bf16(x) for a flat fp32 buffer (refreshing the compute copy after a collective wrote master weights).
__global__ void cast_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long n) {
  const long n4 = n / 4;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float v[4]; Vec4<float>::load(x + i * 4, v); Vec4<__nv_bfloat16>::store(y + i * 4, v);
  }
}
int cast_bf16(const float* x, void* y, long n, int sms, cudaStream_t st) {
  if (n % 4) return 1;
  cast_bf16_kernel<<<sms * 8, 256, 0, st>>>(x, static_cast<__nv_bfloat16*>(y), n);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ embedding
// out[n] = mean over the s ids of row n of table[id] (s = 1: a plain gather; s > 1: token-superposition bags;
// ced/model/control.py:436-455). Backward: table_grad[id] += g[n] / s for every id of the row, through vector
// reductions in L2 (`red.global.add.v4.f32`): no sort and no (N, s, d) intermediate; the summation order is not fixed.
// One warp per row, fp32 table and rows, d a multiple of 4.
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out, long n, int s, int d) {
  const int lane = threadIdx.x & 31;
  const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarp = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const float inv = 1.f / s;
  for (long r = warp; r < n; r += nwarp) {
    for (int c = lane * 4; c < d; c += 128) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < s; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(table + ids[r * s + k] * d + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (s > 1) { acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv; }
      *reinterpret_cast<float4*>(out + r * d + c) = acc;
    }
  }
}
__global__ void embedding_bwd_kernel(const long* __restrict__ ids, const float* __restrict__ g, float* __restrict__ table_grad, long n, int s, int d) {
  const int lane = threadIdx.x & 31;
  const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarp = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const float inv = 1.f / s;
  for (long r = warp; r < n; r += nwarp) {
    for (int c = lane * 4; c < d; c += 128) {
      float4 v = *reinterpret_cast<const float4*>(g + r * d + c);
      if (s > 1) { v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv; }
      for (int k = 0; k < s; ++k) {
        float* dst = table_grad + ids[r * s + k] * d + c;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
      }
    }
  }
}
int embedding_fwd(const long* ids, const float* table, float* out, long n, int s, int d, int sms, cudaStream_t st) {
  if (d % 4 || s < 1) return 1;
  embedding_fwd_kernel<<<sms * 8, 256, 0, st>>>(ids, table, out, n, s, d);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int embedding_bwd(const long* ids, const float* g, float* table_grad, long n, int s, int d, int sms, cudaStream_t st) {
  if (d % 4 || s < 1) return 1;
  embedding_bwd_kernel<<<sms * 8, 256, 0, st>>>(ids, g, table_grad, n, s, d);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// ================================================================================================ MXFP8 fake quantisation
// Blocks of 32 along one dimension of a [rows, n] matrix: E8M0 exponent of amax / 448 rounded up to a power of two, elements
// scaled, clamped to +-448 and rounded to E4M3 (nearest even), then multiplied back: the values a block-scaled GEMM
// would see, written as bf16 (exact: 3 mantissa bits times a power of two). A block with a non-finite element becomes NaN
// with exponent code 255; a NaN does not count toward amax (ced/model/mxfp8.py:86-188). One read of the input.
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int mx_exponent(float amax) {
  const int bits = __float_as_int(amax * (1.0f / 448.0f));
  const int e = (bits >> 23) & 0xFF, m = bits & 0x7FFFFF;
  if (e == 255) return m == 0 ? 254 : 255;
  const bool bump = m > 0 && e != 254 && (e != 0 || m > 0x400000);
  return e + (bump ? 1 : 0);
}
__device__ __forceinline__ float mx_round_trip(float x, int b, bool bad) {
  if (bad) return __int_as_float(0x7FFFFFFF);
  const float inv = __int_as_float(b == 254 ? 0x00400000 : (254 - b) << 23);
  const float scale = __int_as_float(b == 0 ? 0x00400000 : b << 23);
  const float y = fminf(fmaxf(x * inv, -448.f), 448.f);
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3))) * scale;
}
template <typename T>
__global__ void mx_fake_last_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, long rows, long n) {
  const int lane = threadIdx.x & 31;
  const long per_row = (n + 31) / 32, blocks = rows * per_row;
  const long warp = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarp = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long blk = warp; blk < blocks; blk += nwarp) {
    const long r = blk / per_row, c = (blk % per_row) * 32 + lane;
    const bool in = c < n;
    const float v = in ? to_float(x[r * n + c]) : 0.f;
    const bool fin = isfinite(v);
    const float amax = wmax(isnan(v) ? 0.f : fabsf(v));
    const bool bad = __any_sync(0xffffffffu, !fin);
    const int b = mx_exponent(amax);
    if (in) out[r * n + c] = __float2bfloat16(mx_round_trip(v, b, bad));
  }
}
// Blocks of 32 consecutive rows of one column; a thread owns a column of a row block, threads run along the columns.
template <typename T>
__global__ void mx_fake_first_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, long rows, long n) {
  const long row_blocks = (rows + 31) / 32, units = row_blocks * n;
  for (long u = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += static_cast<long>(gridDim.x) * blockDim.x) {
    const long rb = u / n, c = u % n;
    const long r0 = rb * 32, r1 = min(rows, r0 + 32);
    float amax = 0.f; bool bad = false;
    for (long r = r0; r < r1; ++r) {
      const float v = to_float(x[r * n + c]);
      bad |= !isfinite(v);
      amax = fmaxf(amax, isnan(v) ? 0.f : fabsf(v));
    }
    const int b = mx_exponent(amax);
    for (long r = r0; r < r1; ++r) out[r * n + c] = __float2bfloat16(mx_round_trip(to_float(x[r * n + c]), b, bad));
  }
}
int mx_fake(const void* x, bool x_bf16, void* out, long rows, long n, bool along_rows, int sms, cudaStream_t st) {
  auto* o = static_cast<__nv_bfloat16*>(out);
  if (along_rows) {
    if (x_bf16) mx_fake_first_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), o, rows, n);
    else mx_fake_first_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const float*>(x), o, rows, n);
  } else {
    if (x_bf16) mx_fake_last_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), o, rows, n);
    else mx_fake_last_kernel<<<sms * 8, 256, 0, st>>>(static_cast<const float*>(x), o, rows, n);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
