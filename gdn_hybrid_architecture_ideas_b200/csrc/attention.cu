// Causal, document-masked attention with grouped KV heads and the rotary distance cap, on tcgen05 tensor cores.
//
// Forward: one CTA per (128-query tile, query head, batch row). Per 128-key tile: S = Q K^T (tcgen05.mma into tensor
// memory), online softmax by 128 threads (one query row each, reading S with tcgen05.ld), P written to shared memory
// as a swizzled bf16 operand, O_tile = P V (tcgen05.mma), accumulated in registers with the usual rescale.
// Distance cap C: a pair with i - j > C is scored with (Q_far, K_far) — the query rotated by C against the unrotated
// key — instead of (Q, K). A key tile whose pairs are all near or all far costs one pass; a tile straddling the cap is
// processed as two passes with complementary masks (online softmax accepts any partition of the keys), so the cap
// needs no second score matrix and no second kernel launch (the reference runs two flex-attention calls and merges by
// log-sum-exp: ced/model/fast_attention.py:464-573; ground truth ced/model/attention.py:526-551).
// Backward: one CTA per (128-key tile, KV head, batch row), looping over the query heads of the group and the query
// tiles at or after it; dK, dK_far, dV accumulate in tensor memory, dQ / dQ_far tiles are reduced into fp32 global
// buffers. Every wait is bounded and reports through the status word.
#include "kernels.h"
#include "sm100.cuh"

namespace ghb {
using namespace sm100;

constexpr int AT = 128;        // tile edge (queries and keys)
constexpr int HD = 64;         // head dimension
constexpr uint32_t TILE_BYTES = AT * HD * 2;   // 16 KB: one [128][64] bf16 tile = one 128-byte-swizzled box

struct AttnMaps {
  CUtensorMap q, qf, k, kf, v, dO;
};

__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// Write 128 bf16 of one operand row (two 64-wide K blocks of 16 KB each) with the 128-byte swizzle: 16-byte chunk c of
// row r in a block lands at chunk (c ^ (r & 7)).
__device__ __forceinline__ void store_row_chunk(uint8_t* base, int row, int col0, const float* v8) {
  // col0: multiple of 8 in [0,128)
  const int kb = col0 >> 6, c = (col0 & 63) >> 3;
  uint4 pk;
  __nv_bfloat162 a = __floats2bfloat162_rn(v8[0], v8[1]), b = __floats2bfloat162_rn(v8[2], v8[3]);
  __nv_bfloat162 cc = __floats2bfloat162_rn(v8[4], v8[5]), d = __floats2bfloat162_rn(v8[6], v8[7]);
  pk.x = *reinterpret_cast<uint32_t*>(&a); pk.y = *reinterpret_cast<uint32_t*>(&b);
  pk.z = *reinterpret_cast<uint32_t*>(&cc); pk.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(base + kb * TILE_BYTES + row * 128 + ((c ^ (row & 7)) << 4)) = pk;
}

// A pass over one key tile: which operands score it and which side of the cap its mask keeps.
struct Pass { int kt; int far; int split; };   // split: the tile straddles the cap, so the mask also tests the distance

__device__ __forceinline__ int passes_for_tile(int q0, int k0, int cap, bool capped, Pass* out, int kt) {
  if (!capped) { out[0] = {kt, 0, 0}; return 1; }
  const int dmax = q0 + AT - 1 - k0, dmin = q0 - (k0 + AT - 1);
  if (dmax <= cap) { out[0] = {kt, 0, 0}; return 1; }
  if (dmin > cap) { out[0] = {kt, 1, 0}; return 1; }
  out[0] = {kt, 0, 1}; out[1] = {kt, 1, 1};
  return 2;
}

struct PassIter {
  int q0, cap, kt, kt_hi, sub, n; bool capped; Pass cur[2];
  __device__ void init(int q0_, int cap_, bool capped_, int kt_lo, int kt_hi_) {
    q0 = q0_; cap = cap_; capped = capped_; kt = kt_lo; kt_hi = kt_hi_; sub = 0;
    n = kt <= kt_hi ? passes_for_tile(q0, kt * AT, cap, capped, cur, kt) : 0;
  }
  __device__ bool valid() const { return kt <= kt_hi; }
  __device__ Pass get() const { return sub ? cur[1] : cur[0]; }
  __device__ void next() {
    if (!valid()) return;
    if (++sub >= n) { ++kt; sub = 0; if (kt <= kt_hi) n = passes_for_tile(q0, kt * AT, cap, capped, cur, kt); }
  }
};

// ================================================================================================ forward
// Keys a query row may see inside one key tile form one interval of tile columns [e_lo, e_lo + w]: causality and the
// end of the tile bound it above, the row's document start and (in a split pass) the cap bound it on one side.
struct RowMask { int e_lo; uint32_t w; };
__device__ __forceinline__ RowMask row_mask(bool row_ok, int i, int lo_i, int k0, int cap, const Pass& p) {
  int lo = max(0, lo_i - k0), hi = row_ok ? min(AT - 1, i - k0) : -1;
  if (p.split) { if (p.far) hi = min(hi, i - cap - 1 - k0); else lo = max(lo, i - cap - k0); }
  RowMask m;
  if (hi < lo) { m.e_lo = 1 << 20; m.w = 0; } else { m.e_lo = lo; m.w = static_cast<uint32_t>(hi - lo); }
  return m;
}

// Row maximum of one score row (128 columns of tensor memory), the loads running one chunk ahead of the arithmetic.
template <bool MASKED>
__device__ __forceinline__ float score_row_max(uint32_t taddr, RowMask rm) {
  uint32_t sv[2][16];
  float mx0 = -INFINITY, mx1 = -INFINITY;
  tmem_ld_x16(taddr, sv[0]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < AT / 16; ++c) {
    if (c + 1 < AT / 16) tmem_ld_x16(taddr + (c + 1) * 16, sv[(c + 1) & 1]);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float x = __uint_as_float(sv[c & 1][e]);
      if (MASKED) x = (static_cast<uint32_t>(c * 16 + e - rm.e_lo) <= rm.w) ? x : -INFINITY;
      if (e & 1) mx1 = fmaxf(mx1, x); else mx0 = fmaxf(mx0, x);
    }
    if (c + 1 < AT / 16) tmem_ld_wait();
  }
  return fmaxf(mx0, mx1);
}

// Probabilities of one score row against the reference maximum, written as the bf16 A operand of P V; returns the row sum.
template <bool MASKED>
__device__ __forceinline__ float score_row_probs(uint32_t taddr, RowMask rm, float scale_log2, float m_use, uint8_t* sP, int r) {
  uint32_t sv[2][16];
  float rs0 = 0.f, rs1 = 0.f;
  tmem_ld_x16(taddr, sv[0]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < AT / 16; ++c) {
    if (c + 1 < AT / 16) tmem_ld_x16(taddr + (c + 1) * 16, sv[(c + 1) & 1]);
    float pv[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float pe = exp2f(fmaf(__uint_as_float(sv[c & 1][e]), scale_log2, -m_use));
      if (MASKED) pe = (static_cast<uint32_t>(c * 16 + e - rm.e_lo) <= rm.w) ? pe : 0.f;
      pv[e] = pe;
      if (e & 1) rs1 += pe; else rs0 += pe;
    }
#pragma unroll
    for (int g = 0; g < 2; ++g) store_row_chunk(sP, r, c * 16 + g * 8, pv + g * 8);
    if (c + 1 < AT / 16) tmem_ld_wait();
  }
  return rs0 + rs1;
}

// Shared memory: Q, Q_far, one K stage, two V stages, P (7 tiles of 16 KB) so that two CTAs share an SM: while one CTA
// is in its softmax the other's products run. The output accumulates in tensor memory across key tiles; the softmax
// threads rescale it only when a row's maximum has grown by more than 2^8 since the reference maximum was set (the
// probabilities then stay below 2^8 relative to it, well inside bf16 / fp32 range), so most tiles touch the
// accumulator from the tensor pipe alone.
constexpr float RESCALE_STEP = 8.f;

template <bool CAPPED>
__global__ void __launch_bounds__(160, 2)
attn_fwd_kernel(const __grid_constant__ AttnMaps maps, __nv_bfloat16* __restrict__ O, float* __restrict__ LSE,
                const int* __restrict__ doc, const int* __restrict__ pos, int L, int Hq, int Hkv, int cap, float scale_log2,
                int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;                         // 16 KB
  uint8_t* sQf = sQ + TILE_BYTES;             // 16 KB
  uint8_t* sK = sQf + TILE_BYTES;             // 16 KB (K or K_far of the pass)
  uint8_t* sV = sK + TILE_BYTES;              // 2 stages x 16 KB
  uint8_t* sP = sV + 2 * TILE_BYTES;          // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * TILE_BYTES);
  uint64_t* bar_q = bars; uint64_t* k_full = bars + 1; uint64_t* k_free = bars + 2; uint64_t* v_full = bars + 3; uint64_t* v_free = bars + 5;
  uint64_t* bar_s = bars + 7; uint64_t* bar_p = bars + 8; uint64_t* bar_o = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(err) != 0) return;     // an earlier CTA or launch gave up: do not queue more waits
  if (smem_u32(smem) & 1023u) {               // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(err, 200);
    return;
  }
  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;   // longest rows of tiles first
  const int hk = h / (Hq / Hkv);
  const int q0 = qt * AT;
  const long tok0 = static_cast<long>(b) * L;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1); mbar_init(k_full, 1); mbar_init(k_free, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_free[s], 1); }
    mbar_init(bar_s, 1); mbar_init(bar_p, 128); mbar_init(bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;

  // key tiles: from the tile holding the first query's document start to the diagonal tile
  const int j_lo = doc ? max(0, q0 - pos[tok0 + q0]) : 0;
  const int kt_lo = j_lo / AT, kt_hi = qt;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AT, AT, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(AT, HD, false, true);
      bool ok = true;
      mbar_expect_tx(bar_q, CAPPED ? 2 * TILE_BYTES : TILE_BYTES);
      tma_load_3d(sQ, &maps.q, bar_q, 0, h, static_cast<int>(tok0 + q0));
      if (CAPPED) tma_load_3d(sQf, &maps.qf, bar_q, 0, h, static_cast<int>(tok0 + q0));
      auto load_k = [&](const Pass& p) {
        mbar_expect_tx(k_full, TILE_BYTES);
        tma_load_3d(sK, p.far ? &maps.kf : &maps.k, k_full, 0, hk, static_cast<int>(tok0 + p.kt * AT));
      };
      auto load_v = [&](const Pass& p, int s) {
        mbar_expect_tx(&v_full[s], TILE_BYTES);
        tma_load_3d(sV + s * TILE_BYTES, &maps.v, &v_full[s], 0, hk, static_cast<int>(tok0 + p.kt * AT));
      };
      auto issue_s = [&](const Pass& p) {
        const uint32_t qa = smem_u32(p.far ? sQf : sQ), ka = smem_u32(sK);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(tS, umma_desc_sw128(qa + k * 32, 16, 1024), umma_desc_sw128(ka + k * 32, 16, 1024), idesc_s, k != 0);
        umma_commit(bar_s);
        umma_commit(k_free);
      };
      // iterators: `cur` is the pass whose P V runs this iteration, n1 / n2 the passes one and two ahead
      PassIter cur, n1, n2;
      cur.init(q0, cap, CAPPED, kt_lo, kt_hi);
      n1 = cur; n1.next();
      n2 = n1; n2.next();
      uint32_t ph_kfull = 0, ph_kfree = 0, ph_vfull[2] = {0, 0}, ph_vfree[2] = {0, 0}, ph_p = 0;
      load_k(cur.get());
      load_v(cur.get(), 0);
      if (n1.valid()) load_v(n1.get(), 1);
      do {
        if (!mbar_wait(bar_q, 0)) { atomicExch(err, 203); ok = false; break; }
        if (!mbar_wait(k_full, ph_kfull)) { atomicExch(err, 202); ok = false; break; }
        ph_kfull ^= 1;
        tc_fence_after();
        issue_s(cur.get());
        if (n1.valid()) {
          if (!mbar_wait(k_free, ph_kfree)) { atomicExch(err, 201); ok = false; break; }
          ph_kfree ^= 1;
          load_k(n1.get());
        }
      } while (false);
      for (int it = 0; cur.valid() && ok; ++it, cur.next(), n1.next(), n2.next()) {
        const int s = it & 1;
        if (!mbar_wait(bar_p, ph_p)) { atomicExch(err, 204); ok = false; break; }      // P(it) written, S drained
        ph_p ^= 1;
        tc_fence_after();
        if (n1.valid()) {                       // scores of the next pass first: its softmax overlaps P V of this one
          if (!mbar_wait(k_full, ph_kfull)) { atomicExch(err, 202); ok = false; break; }
          ph_kfull ^= 1;
          tc_fence_after();
          issue_s(n1.get());
        }
        if (!mbar_wait(&v_full[s], ph_vfull[s])) { atomicExch(err, 205); ok = false; break; }
        ph_vfull[s] ^= 1;
        tc_fence_after();
        const uint32_t va = smem_u32(sV + s * TILE_BYTES), pa = smem_u32(sP);
#pragma unroll
        for (int k = 0; k < AT / 16; ++k)
          umma_bf16(tO, umma_desc_sw128(pa + (k >> 2) * TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_desc_sw128(va + k * 16 * 128, TILE_BYTES, 1024), idesc_o, it != 0 || k != 0);
        umma_commit(bar_o);
        umma_commit(&v_free[s]);
        if (n2.valid()) {
          if (!mbar_wait(k_free, ph_kfree)) { atomicExch(err, 201); ok = false; break; }     // S of the next pass has read K
          ph_kfree ^= 1;
          load_k(n2.get());
          if (!mbar_wait(&v_free[s], ph_vfree[s])) { atomicExch(err, 206); ok = false; break; }   // P V of this pass has read V
          ph_vfree[s] ^= 1;
          load_v(n2.get(), s);
        }
      }
      if (!ok) __nanosleep(100000);
    }
  } else {
    const int r = threadIdx.x;                 // query row of this thread = TMEM lane
    const int i = q0 + r;
    const bool row_ok = i < L;
    const int lo_i = (doc && row_ok) ? i - pos[tok0 + i] : 0;
    // the latest document start among the tile's rows: a key tile at or after it, below the diagonal, needs no mask
    const int lo_last = doc ? min(q0 + AT, L) - 1 - pos[tok0 + min(q0 + AT, L) - 1] : 0;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;              // reference maximum (log2 units, scaled) and the row sum against it
    uint32_t ph_s = 0, ph_o = 0;
    bool ok = true;
    int it = 0;
    for (int kt = kt_lo; kt <= kt_hi && ok; ++kt) {
      Pass ps[2];
      const int np = passes_for_tile(q0, kt * AT, cap, CAPPED, ps, kt);
      const int k0 = kt * AT;
      for (int sp = 0; sp < np && ok; ++sp, ++it) {
        const Pass p = sp ? ps[1] : ps[0];
        const bool masked = p.split || k0 + AT - 1 > q0 || q0 + AT > L || lo_last > k0;     // uniform over the CTA
        const RowMask rm = row_mask(row_ok, i, lo_i, k0, cap, p);
        if (!mbar_wait(bar_s, ph_s)) { if (lane == 0) atomicExch(err, 207); ok = false; break; }
        ph_s ^= 1;
        tc_fence_after();
        const float mx = (masked ? score_row_max<true>(tS + lane_off, rm) : score_row_max<false>(tS + lane_off, rm)) * scale_log2;
        const bool grow = mx > m + RESCALE_STEP || (m == -INFINITY && mx > -INFINITY);
        bool o_waited = false;
        if (it > 0 && __any_sync(0xffffffffu, grow)) {      // rescale the accumulator rows of this warp (warp-collective)
          if (!mbar_wait(bar_o, ph_o)) { if (lane == 0) atomicExch(err, 208); ok = false; break; }
          ph_o ^= 1; o_waited = true;
          tc_fence_after();
          const float alpha = grow ? exp2f(m - mx) : 1.f;    // m = -inf: every earlier probability of the row was 0
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_x32(tO + lane_off + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            tmem_st_x32(tO + lane_off + c * 32, ov);
          }
          tmem_st_wait();
          l *= alpha;
        }
        if (grow) m = mx;
        const float m_use = (m == -INFINITY) ? 0.f : m;
        if (it > 0 && !o_waited) {               // P V of the previous pass still reads the P buffer
          if (!mbar_wait(bar_o, ph_o)) { if (lane == 0) atomicExch(err, 208); ok = false; break; }
          ph_o ^= 1;
        }
        l += masked ? score_row_probs<true>(tS + lane_off, rm, scale_log2, m_use, sP, r)
                    : score_row_probs<false>(tS + lane_off, rm, scale_log2, m_use, sP, r);
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_p);
      }
    }
    if (ok && !mbar_wait(bar_o, ph_o)) { if (lane == 0) atomicExch(err, 209); ok = false; }
    tc_fence_after();
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = O + ((tok0 + min(i, L - 1)) * Hq + h) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ov[32];
        tmem_ld_x32(tO + lane_off + c * 32, ov);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(ov[v * 8 + 2 * e]) * inv, __uint_as_float(ov[v * 8 + 2 * e + 1]) * inv);
              pk[e] = *reinterpret_cast<uint32_t*>(&t);
            }
            reinterpret_cast<uint4*>(op + c * 32)[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
      if (row_ok) LSE[(static_cast<long>(b) * Hq + h) * L + i] = (m + log2f(l)) * 0.6931471805599453f;   // natural-log units, scaled scores
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// ================================================================================================ backward
// Preprocess: D[b,h,i] = sum_d dO[b,i,h,d] * O[b,i,h,d].
__global__ void attn_bwd_dot_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ D,
                                    long tokens, int Hq, int L) {
  const long idx = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (token, head)
  if (idx >= tokens * Hq) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162*>(O + idx * HD)[lane];
  const __nv_bfloat162 g = reinterpret_cast<const __nv_bfloat162*>(dO + idx * HD)[lane];
  float s = __bfloat162float(a.x) * __bfloat162float(g.x) + __bfloat162float(a.y) * __bfloat162float(g.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const long tok = idx / Hq; const int h = static_cast<int>(idx % Hq);
    D[((tok / L) * Hq + h) * L + tok % L] = s;
  }
}

// The passes of one backward CTA: query heads of the group x query tiles kt..qt_end x (one or two) passes per tile.
struct BwdIter {
  int g, qt, sub, n, kt, qt_end, G, cap; bool capped; Pass cur[2];
  __device__ void load() { if (g < G) n = passes_for_tile(qt * AT, kt * AT, cap, capped, cur, kt); }
  __device__ void init(int kt_, int qt_end_, int G_, int cap_, bool capped_) {
    g = 0; qt = kt_; sub = 0; kt = kt_; qt_end = qt_end_; G = G_; cap = cap_; capped = capped_; n = 0;
    load();
  }
  __device__ bool valid() const { return g < G; }
  __device__ Pass get() const { return sub ? cur[1] : cur[0]; }
  __device__ void next() {
    if (!valid()) return;
    if (++sub >= n) { sub = 0; if (++qt > qt_end) { qt = kt; ++g; } load(); }
  }
};

// One query row of a pass: P = exp(S scale - lse), dS = P (dP - D) (the score scale is applied to dQ and dK when they
// leave tensor memory), written as bf16 operand rows. Tensor-memory loads run one 16-column chunk ahead.
template <bool MASKED>
__device__ __forceinline__ void bwd_row(uint32_t tS, uint32_t tdP, RowMask rm, float scale_log2, float lse2, float Di, uint8_t* sP, uint8_t* sdS, int r) {
  uint32_t sv[2][16], dv[2][16];
  tmem_ld_x16(tS, sv[0]);
  tmem_ld_x16(tdP, dv[0]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < AT / 16; ++c) {
    if (c + 1 < AT / 16) { tmem_ld_x16(tS + (c + 1) * 16, sv[(c + 1) & 1]); tmem_ld_x16(tdP + (c + 1) * 16, dv[(c + 1) & 1]); }
    float pv[16], gs[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float pe = exp2f(fmaf(__uint_as_float(sv[c & 1][e]), scale_log2, -lse2));
      if (MASKED) pe = (static_cast<uint32_t>(c * 16 + e - rm.e_lo) <= rm.w) ? pe : 0.f;
      pv[e] = pe;
      gs[e] = pe * (__uint_as_float(dv[c & 1][e]) - Di);
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) { store_row_chunk(sP, r, c * 16 + q * 8, pv + q * 8); store_row_chunk(sdS, r, c * 16 + q * 8, gs + q * 8); }
    if (c + 1 < AT / 16) tmem_ld_wait();
  }
}

// One CTA per (key tile, KV head, batch row). Thread r of the four softmax warps owns query row q0 + r during the
// passes and key row k0 + r in the epilogue. Per pass n the tensor pipe runs, in this order, dQ(n) = dS K,
// dV += P^T dO and dK += dS^T Q, then S(n+1) = Q K^T and dP(n+1) = dO V^T from the other Q / dO stage, while the
// softmax threads drain dQ(n) into the global accumulator and then turn S(n+1), dP(n+1) into P, dS.
template <bool CAPPED>
__global__ void __launch_bounds__(160, 1)
attn_bwd_kernel(const __grid_constant__ AttnMaps maps, const float* __restrict__ LSE, const float* __restrict__ Dsum,
                float* __restrict__ dQ, float* __restrict__ dQf, __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dKf,
                __nv_bfloat16* __restrict__ dV, const int* __restrict__ pos, int L, int Hq, int Hkv, int cap, float scale,
                int* __restrict__ err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;                          // K tile
  uint8_t* sKf = sK + TILE_BYTES;              // K_far tile
  uint8_t* sV = sKf + TILE_BYTES;              // V tile
  uint8_t* sQ = sV + TILE_BYTES;               // 2 stages: Q or Q_far of the pass
  uint8_t* sdO = sQ + 2 * TILE_BYTES;          // 2 stages: dO tile
  uint8_t* sP = sdO + 2 * TILE_BYTES;          // P  [q rows][key columns] (32 KB)
  uint8_t* sdS = sP + 2 * TILE_BYTES;          // dS (32 KB)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * TILE_BYTES);
  uint64_t* bar_kv = bars; uint64_t* qdo_full = bars + 1; uint64_t* bar_s = bars + 3; uint64_t* bar_p = bars + 4;
  uint64_t* bar_dq = bars + 5; uint64_t* bar_c = bars + 6; uint64_t* bar_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(err, 210);
    return;
  }
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int k0 = kt * AT;
  const long tok0 = static_cast<long>(b) * L;
  const int n_qt = (L + AT - 1) / AT;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1); mbar_init(&qdo_full[0], 1); mbar_init(&qdo_full[1], 1); mbar_init(bar_s, 1); mbar_init(bar_p, 128);
    mbar_init(bar_dq, 1); mbar_init(bar_c, 1); mbar_init(bar_done, 1);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256, tdV = tmem + 320, tdK = tmem + 384, tdKf = tmem + 448;
  // the last query tile that can see this key tile: documents are contiguous, so it is the last tile whose first row's
  // document starts at or before the tile's last key
  int qt_end = kt;
  if (pos) { while (qt_end + 1 < n_qt && (qt_end + 1) * AT - pos[tok0 + (qt_end + 1) * AT] <= k0 + AT - 1) ++qt_end; }
  else qt_end = n_qt - 1;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AT, AT, false, false);       // S = Q K^T, dP = dO V^T
      constexpr uint32_t idesc_dq = umma_idesc_bf16(AT, HD, false, true);       // dQ = dS K (B MN-major)
      constexpr uint32_t idesc_kv = umma_idesc_bf16(AT, HD, true, true);        // dV += P^T dO, dK += dS^T Q (A read MN-major)
      bool ok = true;
      mbar_expect_tx(bar_kv, CAPPED ? 3 * TILE_BYTES : 2 * TILE_BYTES);
      tma_load_3d(sK, &maps.k, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      tma_load_3d(sV, &maps.v, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      if (CAPPED) tma_load_3d(sKf, &maps.kf, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      auto load_qdo = [&](const BwdIter& itr, int st) {
        const Pass p = itr.get();
        const int h = hk * G + itr.g;
        mbar_expect_tx(&qdo_full[st], 2 * TILE_BYTES);
        tma_load_3d(sQ + st * TILE_BYTES, p.far ? &maps.qf : &maps.q, &qdo_full[st], 0, h, static_cast<int>(tok0 + itr.qt * AT));
        tma_load_3d(sdO + st * TILE_BYTES, &maps.dO, &qdo_full[st], 0, h, static_cast<int>(tok0 + itr.qt * AT));
      };
      auto issue_scores = [&](const Pass& p, int st) {
        const uint32_t ka = smem_u32(p.far ? sKf : sK), va = smem_u32(sV), qa = smem_u32(sQ + st * TILE_BYTES), da = smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          umma_bf16(tS, umma_desc_sw128(qa + k * 32, 16, 1024), umma_desc_sw128(ka + k * 32, 16, 1024), idesc_s, k != 0);
          umma_bf16(tdP, umma_desc_sw128(da + k * 32, 16, 1024), umma_desc_sw128(va + k * 32, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(bar_s);
      };
      BwdIter cur, n1, n2;
      cur.init(kt, qt_end, G, cap, CAPPED);
      n1 = cur; n1.next();
      n2 = n1; n2.next();
      uint32_t ph_full[2] = {0, 0}, ph_p = 0, ph_c = 0;
      bool first_v = true, first_k = true, first_kf = true;
      load_qdo(cur, 0);
      if (n1.valid()) load_qdo(n1, 1);
      do {
        if (!mbar_wait(bar_kv, 0)) { atomicExch(err, 212); ok = false; break; }
        if (!mbar_wait(&qdo_full[0], ph_full[0])) { atomicExch(err, 213); ok = false; break; }
        ph_full[0] ^= 1;
        tc_fence_after();
        issue_scores(cur.get(), 0);
      } while (false);
      for (int n = 0; cur.valid() && ok; ++n, cur.next(), n1.next(), n2.next()) {
        const Pass p = cur.get();
        const int st = n & 1;
        if (!mbar_wait(bar_p, ph_p)) { atomicExch(err, 214); ok = false; break; }     // P, dS written; S, dP and dQ drained
        ph_p ^= 1;
        tc_fence_after();
        const uint32_t ka = smem_u32(p.far ? sKf : sK), qa = smem_u32(sQ + st * TILE_BYTES), da = smem_u32(sdO + st * TILE_BYTES);
        const uint32_t pa = smem_u32(sP), sa = smem_u32(sdS);
#pragma unroll
        for (int k = 0; k < AT / 16; ++k)       // dQ [q x hd] = dS K: A = dS K-major, B = K tile [key rows][hd] MN-major
          umma_bf16(tdQ, umma_desc_sw128(sa + (k >> 2) * TILE_BYTES + (k & 3) * 32, 16, 1024), umma_desc_sw128(ka + k * 16 * 128, TILE_BYTES, 1024), idesc_dq, k != 0);
        umma_commit(bar_dq);
        const uint32_t tk = p.far ? tdKf : tdK;
        bool& fk = p.far ? first_kf : first_k;
#pragma unroll
        for (int k = 0; k < AT / 16; ++k) {     // A = P / dS stored [q rows][key columns] read MN-major (M = keys), B = dO / Q [q rows][hd] MN-major
          umma_bf16(tdV, umma_desc_sw128(pa + k * 16 * 128, TILE_BYTES, 1024), umma_desc_sw128(da + k * 16 * 128, TILE_BYTES, 1024), idesc_kv, !(first_v && k == 0));
          umma_bf16(tk, umma_desc_sw128(sa + k * 16 * 128, TILE_BYTES, 1024), umma_desc_sw128(qa + k * 16 * 128, TILE_BYTES, 1024), idesc_kv, !(fk && k == 0));
        }
        umma_commit(bar_c);
        first_v = false; fk = false;
        if (n1.valid()) {
          if (!mbar_wait(&qdo_full[st ^ 1], ph_full[st ^ 1])) { atomicExch(err, 213); ok = false; break; }
          ph_full[st ^ 1] ^= 1;
          tc_fence_after();
          issue_scores(n1.get(), st ^ 1);
        }
        if (!mbar_wait(bar_c, ph_c)) { atomicExch(err, 211); ok = false; break; }       // this pass's products have read Q / dO
        ph_c ^= 1;
        if (n2.valid()) load_qdo(n2, st);
      }
      if (ok) umma_commit(bar_done);
      else __nanosleep(100000);
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const float scale_log2 = scale * 1.4426950408889634f;
    uint32_t ph_s = 0, ph_q = 0;
    bool ok = true, any_far = false, any_near = false;
    for (int g = 0; g < G && ok; ++g) {
      const int h = hk * G + g;
      const float* lse_row = LSE + (static_cast<long>(b) * Hq + h) * L;
      const float* d_row = Dsum + (static_cast<long>(b) * Hq + h) * L;
      for (int qt = kt; qt <= qt_end && ok; ++qt) {
        const int q0 = qt * AT, i = q0 + r;
        const bool row_ok = i < L;
        const int lo_i = (pos && row_ok) ? i - pos[tok0 + i] : 0;
        const int i_last = min(q0 + AT, L) - 1;
        const int lo_last = pos ? i_last - pos[tok0 + i_last] : 0;
        const float lse2 = row_ok ? lse_row[i] * 1.4426950408889634f : INFINITY;
        const float Di = row_ok ? d_row[i] : 0.f;
        Pass ps[2];
        const int np = passes_for_tile(q0, k0, cap, CAPPED, ps, kt);
        for (int sp = 0; sp < np && ok; ++sp) {
          const Pass p = sp ? ps[1] : ps[0];
          any_far |= p.far; any_near |= !p.far;
          const bool masked = p.split || k0 + AT - 1 > q0 || q0 + AT > L || lo_last > k0 || k0 + AT > L;
          const RowMask rm = row_mask(row_ok, i, lo_i, k0, cap, p);
          if (!mbar_wait(bar_s, ph_s)) { if (lane == 0) atomicExch(err, 215); ok = false; break; }
          ph_s ^= 1;
          tc_fence_after();
          if (masked) bwd_row<true>(tS + lane_off, tdP + lane_off, rm, scale_log2, lse2, Di, sP, sdS, r);
          else bwd_row<false>(tS + lane_off, tdP + lane_off, rm, scale_log2, lse2, Di, sP, sdS, r);
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(bar_p);
          if (!mbar_wait(bar_dq, ph_q)) { if (lane == 0) atomicExch(err, 216); ok = false; break; }
          ph_q ^= 1;
          tc_fence_after();
          float* dst = (p.far ? dQf : dQ) + ((tok0 + min(i, L - 1)) * Hq + h) * HD;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t qv[32];
            tmem_ld_x32(tdQ + lane_off + c * 32, qv);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int e = 0; e < 32; e += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 32 + e), "f"(__uint_as_float(qv[e]) * scale),
                             "f"(__uint_as_float(qv[e + 1]) * scale), "f"(__uint_as_float(qv[e + 2]) * scale), "f"(__uint_as_float(qv[e + 3]) * scale) : "memory");
            }
          }
          tc_fence_before();
        }
      }
    }
    // epilogue: dV, dK, dK_far of this key tile (complete over the group's query heads). Loads are warp-collective, so
    // every lane issues them; only stores are guarded.
    if (ok && !mbar_wait(bar_done, 0)) { if (lane == 0) atomicExch(err, 217); ok = false; }
    tc_fence_after();
    if (ok) {
      const int j = k0 + r;
      const bool key_ok = j < L;
      const long base = ((tok0 + min(j, L - 1)) * Hkv + hk) * HD;
#pragma unroll 1
      for (int which = 0; which < (CAPPED ? 3 : 2); ++which) {
        const uint32_t t = which == 0 ? tdV : (which == 1 ? tdK : tdKf);
        const float f = which == 0 ? 1.f : ((which == 1 ? any_near : any_far) ? scale : 0.f);
        const bool live = which == 0 || (which == 1 ? any_near : any_far);
        __nv_bfloat16* dst = (which == 0 ? dV : (which == 1 ? dK : dKf)) + base;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t av[32];
          tmem_ld_x32(t + lane_off + c * 32, av);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t pk[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 tt = __floats2bfloat162_rn(live ? __uint_as_float(av[v * 8 + 2 * e]) * f : 0.f, live ? __uint_as_float(av[v * 8 + 2 * e + 1]) * f : 0.f);
                pk[e] = *reinterpret_cast<uint32_t*>(&tt);
              }
              reinterpret_cast<uint4*>(dst + c * 32)[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------ host side
static bool map_heads(CUtensorMap* m, const void* p, long tokens, int H) {
  const uint64_t dims[3] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(H), static_cast<uint64_t>(tokens)};
  const uint64_t strides[2] = {static_cast<uint64_t>(HD) * 2, static_cast<uint64_t>(H) * HD * 2};
  const uint32_t box[3] = {HD, 1, AT};
  return encode_tensor_map_3d(m, p, 2, dims, strides, box, true);
}
constexpr uint32_t FWD_SMEM = 7 * TILE_BYTES + 128;       // 112 KB + barriers: two CTAs per SM
constexpr uint32_t BWD_SMEM = 11 * TILE_BYTES + 128;

// q, qf: [B, L, Hq, 64]; k, kf, v: [B, L, Hkv, 64] bf16 contiguous. qf/kf may be null when cap < 0 (no cap).
// doc, pos: [B, L] int32 or null (every row one document). o: [B, L, Hq, 64] bf16; lse: [B, Hq, L] fp32.
int attention_fwd(const void* q, const void* qf, const void* k, const void* kf, const void* v, void* o, float* lse, const int* doc,
                  const int* pos, int B, int L, int Hq, int Hkv, int cap, float scale, int* err, cudaStream_t st) {
  if (Hq % Hkv) return 1;
  const bool capped = cap >= 0;
  AttnMaps maps;
  const long tokens = static_cast<long>(B) * L;
  if (!map_heads(&maps.q, q, tokens, Hq) || !map_heads(&maps.k, k, tokens, Hkv) || !map_heads(&maps.v, v, tokens, Hkv)) return 2;
  if (capped && (!map_heads(&maps.qf, qf, tokens, Hq) || !map_heads(&maps.kf, kf, tokens, Hkv))) return 2;
  if (!capped) { maps.qf = maps.q; maps.kf = maps.k; }
  maps.dO = maps.q;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return 3;
    if (cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) return 3;
    cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attr = true;
  }
  dim3 grid((L + AT - 1) / AT, Hq, B);
  const float sl2 = scale * 1.4426950408889634f;
  if (capped) attn_fwd_kernel<true><<<grid, 160, FWD_SMEM, st>>>(maps, static_cast<__nv_bfloat16*>(o), lse, doc, pos, L, Hq, Hkv, cap, sl2, err);
  else attn_fwd_kernel<false><<<grid, 160, FWD_SMEM, st>>>(maps, static_cast<__nv_bfloat16*>(o), lse, doc, pos, L, Hq, Hkv, 0, sl2, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// dq, dqf: [B, L, Hq, 64] fp32, zeroed by the caller (reduced into); dk, dkf, dv: [B, L, Hkv, 64] bf16 (written).
// dsum: [B, Hq, L] fp32 scratch. pos: [B, L] int32 position of each token inside its document, or null (one document per row).
int attention_bwd(const void* q, const void* qf, const void* k, const void* kf, const void* v, const void* o, const void* dO,
                  const float* lse, float* dsum, float* dq, float* dqf, void* dk, void* dkf, void* dv, const int* pos, int B, int L, int Hq,
                  int Hkv, int cap, float scale, int* err, cudaStream_t st) {
  if (Hq % Hkv) return 1;
  const bool capped = cap >= 0;
  AttnMaps maps;
  const long tokens = static_cast<long>(B) * L;
  if (!map_heads(&maps.q, q, tokens, Hq) || !map_heads(&maps.k, k, tokens, Hkv) || !map_heads(&maps.v, v, tokens, Hkv) ||
      !map_heads(&maps.dO, dO, tokens, Hq)) return 2;
  if (capped && (!map_heads(&maps.qf, qf, tokens, Hq) || !map_heads(&maps.kf, kf, tokens, Hkv))) return 2;
  if (!capped) { maps.qf = maps.q; maps.kf = maps.k; }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return 3;
    if (cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return 3;
    attr = true;
  }
  const long units = tokens * Hq;
  attn_bwd_dot_kernel<<<static_cast<unsigned>((units + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dO), dsum, tokens, Hq, L);
  dim3 grid((L + AT - 1) / AT, Hkv, B);
  if (capped) attn_bwd_kernel<true><<<grid, 160, BWD_SMEM, st>>>(maps, lse, dsum, dq, dqf, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dkf),
                                                                 static_cast<__nv_bfloat16*>(dv), pos, L, Hq, Hkv, cap, scale, err);
  else attn_bwd_kernel<false><<<grid, 160, BWD_SMEM, st>>>(maps, lse, dsum, dq, dqf, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dkf),
                                                           static_cast<__nv_bfloat16*>(dv), pos, L, Hq, Hkv, 0, scale, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
