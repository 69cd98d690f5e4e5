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
  __device__ Pass get() const { return cur[sub]; }
  __device__ void next() {
    if (!valid()) return;
    if (++sub >= n) { ++kt; sub = 0; if (kt <= kt_hi) n = passes_for_tile(q0, kt * AT, cap, capped, cur, kt); }
  }
};

// ================================================================================================ forward
template <bool CAPPED>
__global__ void __launch_bounds__(160, 1)
attn_fwd_kernel(const __grid_constant__ AttnMaps maps, __nv_bfloat16* __restrict__ O, float* __restrict__ LSE,
                const int* __restrict__ doc, const int* __restrict__ pos, int L, int Hq, int Hkv, int cap, float scale_log2,
                int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                         // 16 KB
  uint8_t* sQf = sQ + TILE_BYTES;             // 16 KB
  uint8_t* sK = sQf + TILE_BYTES;             // 2 stages x 16 KB (holds K or K_far of the pass)
  uint8_t* sV = sK + 2 * TILE_BYTES;          // 2 stages x 16 KB
  uint8_t* sP = sV + 2 * TILE_BYTES;          // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * TILE_BYTES);
  uint64_t* bar_q = bars; uint64_t* kv_full = bars + 1; uint64_t* kv_empty = bars + 3;
  uint64_t* bar_s = bars + 5; uint64_t* bar_p = bars + 6; uint64_t* bar_o = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;   // longest rows of tiles first
  const int hk = h / (Hq / Hkv);
  const int q0 = qt * AT;
  const long tok0 = static_cast<long>(b) * L;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
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
      PassIter cur, ahead;
      cur.init(q0, cap, CAPPED, kt_lo, kt_hi);
      ahead = cur;
      ahead.next();
      auto load_pass = [&](const Pass& p, int s) {
        mbar_expect_tx(&kv_full[s], 2 * TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, p.far ? &maps.kf : &maps.k, &kv_full[s], 0, hk, static_cast<int>(tok0 + p.kt * AT));
        tma_load_3d(sV + s * TILE_BYTES, &maps.v, &kv_full[s], 0, hk, static_cast<int>(tok0 + p.kt * AT));
      };
      load_pass(cur.get(), 0);
      uint32_t ph_full[2] = {0, 0}, ph_empty[2] = {0, 0}, ph_p = 0;
      for (int it = 0; cur.valid() && ok; ++it, cur.next(), ahead.next()) {
        const Pass p = cur.get();
        const int s = it & 1;
        if (ahead.valid()) {   // prefetch the next pass into the other stage once its previous user (pass it-1) is done
          if (it >= 1) { if (!mbar_wait(&kv_empty[s ^ 1], ph_empty[s ^ 1])) { atomicExch(err, 201); ok = false; break; } ph_empty[s ^ 1] ^= 1; }
          load_pass(ahead.get(), s ^ 1);
        }
        if (!mbar_wait(&kv_full[s], ph_full[s])) { atomicExch(err, 202); ok = false; break; }
        ph_full[s] ^= 1;
        if (it == 0 && !mbar_wait(bar_q, 0)) { atomicExch(err, 203); ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(p.far ? sQf : sQ), ka = smem_u32(sK + s * TILE_BYTES), va = smem_u32(sV + s * TILE_BYTES), pa = smem_u32(sP);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(tS, umma_desc_sw128(qa + k * 32, 16, 1024), umma_desc_sw128(ka + k * 32, 16, 1024), idesc_s, k != 0);
        umma_commit(bar_s);
        if (!mbar_wait(bar_p, ph_p)) { atomicExch(err, 204); ok = false; break; }
        ph_p ^= 1;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT / 16; ++k)
          umma_bf16(tO, umma_desc_sw128(pa + (k >> 2) * TILE_BYTES + (k & 3) * 32, 16, 1024),
                    umma_desc_sw128(va + k * 16 * 128, TILE_BYTES, 1024), idesc_o, k != 0);
        umma_commit(bar_o);
        umma_commit(&kv_empty[s]);
      }
      if (!ok) __nanosleep(100000);
    }
  } else {
    const int r = threadIdx.x;                 // query row of this thread = TMEM lane
    const int i = q0 + r;
    const bool row_ok = i < L;
    const int my_doc = (doc && row_ok) ? doc[tok0 + i] : 0;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o[HD];
#pragma unroll
    for (int e = 0; e < HD; ++e) o[e] = 0.f;
    uint32_t ph_s = 0, ph_o = 0;
    bool ok = true;
    for (int kt = kt_lo; kt <= kt_hi && ok; ++kt) {
      Pass ps[2];
      const int np = passes_for_tile(q0, kt * AT, cap, CAPPED, ps, kt);
      const int k0 = kt * AT;
      for (int sp = 0; sp < np && ok; ++sp) {
        const Pass p = ps[sp];
        if (!mbar_wait(bar_s, ph_s)) { if (lane == 0) atomicExch(err, 205); ok = false; break; }
        ph_s ^= 1;
        tc_fence_after();
        // pass 1: row maximum over allowed keys
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < AT / 32; ++c) {
          uint32_t sv[32];
          tmem_ld_x32(tS + lane_off + c * 32, sv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int j = k0 + c * 32 + e;
            bool allow = row_ok && j <= i;
            if (doc) allow = allow && (j < L) && (__ldg(doc + tok0 + j) == my_doc);
            if (CAPPED && p.split) allow = allow && (p.far ? (i - j > cap) : (i - j <= cap));
            if (allow) mx = fmaxf(mx, __uint_as_float(sv[e]));
          }
        }
        const float m_new = fmaxf(m, mx * scale_log2);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
        float rs = 0.f;
        // pass 2: probabilities -> bf16 operand rows
#pragma unroll 1
        for (int c = 0; c < AT / 32; ++c) {
          uint32_t sv[32];
          tmem_ld_x32(tS + lane_off + c * 32, sv);
          tmem_ld_wait();
          float pv[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int j = k0 + c * 32 + e;
            bool allow = row_ok && j <= i;
            if (doc) allow = allow && (j < L) && (__ldg(doc + tok0 + j) == my_doc);
            if (CAPPED && p.split) allow = allow && (p.far ? (i - j > cap) : (i - j <= cap));
            const float pe = allow ? exp2f(__uint_as_float(sv[e]) * scale_log2 - m_use) : 0.f;
            pv[e] = pe; rs += pe;
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) store_row_chunk(sP, r, c * 32 + g * 8, pv + g * 8);
        }
        l = l * alpha + rs;
        m = m_new;
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(bar_p);
        if (!mbar_wait(bar_o, ph_o)) { if (lane == 0) atomicExch(err, 206); ok = false; break; }
        ph_o ^= 1;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_x32(tO + lane_off + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[c * 32 + e] = o[c * 32 + e] * alpha + __uint_as_float(ov[e]);
        }
        tc_fence_before();
      }
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = O + ((tok0 + i) * Hq + h) * HD;
#pragma unroll
      for (int v = 0; v < HD / 8; ++v) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 t = __floats2bfloat162_rn(o[v * 8 + 2 * e] * inv, o[v * 8 + 2 * e + 1] * inv);
          pk[e] = *reinterpret_cast<uint32_t*>(&t);
        }
        reinterpret_cast<uint4*>(op)[v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      LSE[(static_cast<long>(b) * Hq + h) * L + i] = (m + log2f(l)) * 0.6931471805599453f;   // natural-log units, scaled scores
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

template <bool CAPPED>
__global__ void __launch_bounds__(160, 1)
attn_bwd_kernel(const __grid_constant__ AttnMaps maps, const float* __restrict__ LSE, const float* __restrict__ Dsum,
                float* __restrict__ dQ, float* __restrict__ dQf, __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dKf,
                __nv_bfloat16* __restrict__ dV, const int* __restrict__ doc, int L, int Hq, int Hkv, int cap, float scale,
                int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                          // K tile
  uint8_t* sKf = sK + TILE_BYTES;              // K_far tile
  uint8_t* sV = sKf + TILE_BYTES;              // V tile
  uint8_t* sQ = sV + TILE_BYTES;               // Q or Q_far of the pass
  uint8_t* sdO = sQ + TILE_BYTES;              // dO tile
  uint8_t* sP = sdO + TILE_BYTES;              // P^T  (32 KB)
  uint8_t* sdS = sP + 2 * TILE_BYTES;          // dS^T (32 KB)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * TILE_BYTES);
  uint64_t* bar_kv = bars; uint64_t* bar_q = bars + 1; uint64_t* bar_s = bars + 2; uint64_t* bar_p = bars + 3;
  uint64_t* bar_acc = bars + 4; uint64_t* bar_dq_read = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int k0 = kt * AT;
  const long tok0 = static_cast<long>(b) * L;
  const int n_qt = (L + AT - 1) / AT;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1); mbar_init(bar_q, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 128); mbar_init(bar_acc, 1); mbar_init(bar_dq_read, 128);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 320, tdKf = tmem + 384, tdQ = tmem + 448;
  // the last query tile that can see this key tile: with documents, stop once a query tile starts in a later document
  const int last_kdoc = doc ? doc[tok0 + min(k0 + AT - 1, L - 1)] : 0;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AT, AT, false, false);       // S^T = K Q^T, dP^T = V dO^T
      constexpr uint32_t idesc_kv = umma_idesc_bf16(AT, HD, false, true);       // dV += P^T dO, dK += dS^T Q  (B MN-major)
      constexpr uint32_t idesc_dq = umma_idesc_bf16(AT, HD, true, true);        // dQ = dS K (A = dS^T read MN-major)
      bool ok = true;
      mbar_expect_tx(bar_kv, CAPPED ? 3 * TILE_BYTES : 2 * TILE_BYTES);
      tma_load_3d(sK, &maps.k, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      tma_load_3d(sV, &maps.v, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      if (CAPPED) tma_load_3d(sKf, &maps.kf, bar_kv, 0, hk, static_cast<int>(tok0 + k0));
      uint32_t ph_q = 0, ph_p = 0, ph_r = 0;
      bool first_v = true, first_k = true, first_kf = true, first = true;
      int npass = 0;
      for (int g = 0; g < G && ok; ++g) {
        const int h = hk * G + g;
        for (int qt = kt; qt < n_qt && ok; ++qt) {
          const int q0 = qt * AT;
          if (doc && doc[tok0 + q0] > last_kdoc) break;
          Pass ps[2];
          const int np = passes_for_tile(q0, k0, cap, CAPPED, ps, kt);
          for (int sp = 0; sp < np && ok; ++sp) {
            const Pass p = ps[sp];
            // wait until the softmax threads have drained the previous pass's dQ tile and operand buffers
            if (npass > 0) { if (!mbar_wait(bar_dq_read, ph_r)) { atomicExch(err, 211); ok = false; break; } ph_r ^= 1; }
            mbar_expect_tx(bar_q, 2 * TILE_BYTES);
            tma_load_3d(sQ, p.far ? &maps.qf : &maps.q, bar_q, 0, h, static_cast<int>(tok0 + q0));
            tma_load_3d(sdO, &maps.dO, bar_q, 0, h, static_cast<int>(tok0 + q0));
            if (first) { if (!mbar_wait(bar_kv, 0)) { atomicExch(err, 212); ok = false; break; } first = false; }
            if (!mbar_wait(bar_q, ph_q)) { atomicExch(err, 213); ok = false; break; }
            ph_q ^= 1;
            tc_fence_after();
            const uint32_t ka = smem_u32(p.far ? sKf : sK), va = smem_u32(sV), qa = smem_u32(sQ), da = smem_u32(sdO);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              umma_bf16(tS, umma_desc_sw128(ka + k * 32, 16, 1024), umma_desc_sw128(qa + k * 32, 16, 1024), idesc_s, k != 0);
              umma_bf16(tdP, umma_desc_sw128(va + k * 32, 16, 1024), umma_desc_sw128(da + k * 32, 16, 1024), idesc_s, k != 0);
            }
            umma_commit(bar_s);
            if (!mbar_wait(bar_p, ph_p)) { atomicExch(err, 214); ok = false; break; }
            ph_p ^= 1;
            tc_fence_after();
            const uint32_t pa = smem_u32(sP), sa = smem_u32(sdS);
            const uint32_t tk = p.far ? tdKf : tdK;
            bool& fk = p.far ? first_kf : first_k;
#pragma unroll
            for (int k = 0; k < AT / 16; ++k) {
              const uint32_t koff = (k >> 2) * TILE_BYTES + (k & 3) * 32;
              umma_bf16(tdV, umma_desc_sw128(pa + koff, 16, 1024), umma_desc_sw128(da + k * 16 * 128, TILE_BYTES, 1024), idesc_kv, !(first_v && k == 0));
              umma_bf16(tk, umma_desc_sw128(sa + koff, 16, 1024), umma_desc_sw128(qa + k * 16 * 128, TILE_BYTES, 1024), idesc_kv, !(fk && k == 0));
            }
            first_v = false; fk = false;
            // dQ tile [q x hd] = dS K: A = dS^T buffer read as MN-major ([kv rows][q], two 64-wide boxes), B = K tile MN-major
#pragma unroll
            for (int k = 0; k < AT / 16; ++k)
              umma_bf16(tdQ, umma_desc_sw128(sa + k * 16 * 128, TILE_BYTES, 1024), umma_desc_sw128(ka + k * 16 * 128, TILE_BYTES, 1024), idesc_dq, k != 0);
            umma_commit(bar_acc);
            ++npass;
          }
        }
      }
      if (!ok) __nanosleep(100000);
    }
  } else {
    const int r = threadIdx.x;                   // key row of this thread = TMEM lane
    const int j = k0 + r;
    const bool key_ok = j < L;
    const int my_doc = (doc && key_ok) ? doc[tok0 + j] : 0;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t ph_s = 0, ph_a = 0;
    bool ok = true, any_far = false, any_near = false;
    int npass = 0;
    for (int g = 0; g < G && ok; ++g) {
      const int h = hk * G + g;
      for (int qt = kt; qt < n_qt && ok; ++qt) {
        const int q0 = qt * AT;
        if (doc && doc[tok0 + q0] > last_kdoc) break;
        Pass ps[2];
        const int np = passes_for_tile(q0, k0, cap, CAPPED, ps, kt);
        for (int sp = 0; sp < np && ok; ++sp) {
          const Pass p = ps[sp];
          const float* lse_row = LSE + (static_cast<long>(b) * Hq + h) * L;
          const float* d_row = Dsum + (static_cast<long>(b) * Hq + h) * L;
          any_far |= p.far; any_near |= !p.far;
          if (!mbar_wait(bar_s, ph_s)) { if (lane == 0) atomicExch(err, 215); ok = false; break; }
          ph_s ^= 1;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < AT / 32; ++c) {
            uint32_t sv[32], dv[32];
            tmem_ld_x32(tS + lane_off + c * 32, sv);
            tmem_ld_x32(tdP + lane_off + c * 32, dv);
            tmem_ld_wait();
            float pv[32], gs[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int i = q0 + c * 32 + e;
              bool allow = key_ok && i < L && j <= i;
              if (doc) allow = allow && (__ldg(doc + tok0 + min(i, L - 1)) == my_doc);
              if (CAPPED && p.split) allow = allow && (p.far ? (i - j > cap) : (i - j <= cap));
              const int ic = min(i, L - 1);
              const float pe = allow ? __expf(__uint_as_float(sv[e]) * scale - __ldg(lse_row + ic)) : 0.f;
              pv[e] = pe;
              gs[e] = pe * (__uint_as_float(dv[e]) - __ldg(d_row + ic)) * scale;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) { store_row_chunk(sP, r, c * 32 + q * 8, pv + q * 8); store_row_chunk(sdS, r, c * 32 + q * 8, gs + q * 8); }
          }
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(bar_p);
          // dQ tile of this pass: thread r now plays query row q0 + r
          if (!mbar_wait(bar_acc, ph_a)) { if (lane == 0) atomicExch(err, 216); ok = false; break; }
          ph_a ^= 1;
          tc_fence_after();
          {
            const int i = q0 + r;
            float* dst = (p.far ? dQf : dQ) + ((tok0 + i) * Hq + h) * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t qv[32];
              tmem_ld_x32(tdQ + lane_off + c * 32, qv);
              tmem_ld_wait();
              if (i < L) {
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 32 + e), "f"(__uint_as_float(qv[e])),
                               "f"(__uint_as_float(qv[e + 1])), "f"(__uint_as_float(qv[e + 2])), "f"(__uint_as_float(qv[e + 3])) : "memory");
              }
            }
          }
          tc_fence_before();
          mbar_arrive(bar_dq_read);
          ++npass;
        }
      }
    }
    // epilogue: dV, dK, dK_far of this key tile (complete over the group's query heads). The accumulating MMAs of the
    // last pass completed with bar_acc. Loads are warp-collective, so every lane issues them; only stores are guarded.
    if (ok) {
      const long base = ((tok0 + min(j, L - 1)) * Hkv + hk) * HD;
#pragma unroll 1
      for (int which = 0; which < (CAPPED ? 3 : 2); ++which) {
        const uint32_t t = which == 0 ? tdV : (which == 1 ? tdK : tdKf);
        const bool live = npass > 0 && (which == 0 ? true : (which == 1 ? any_near : any_far));
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
                __nv_bfloat162 tt = __floats2bfloat162_rn(live ? __uint_as_float(av[v * 8 + 2 * e]) : 0.f, live ? __uint_as_float(av[v * 8 + 2 * e + 1]) : 0.f);
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
constexpr uint32_t FWD_SMEM = 8 * TILE_BYTES + 128 + 1024;
constexpr uint32_t BWD_SMEM = 9 * TILE_BYTES + 128 + 1024;

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
    attr = true;
  }
  dim3 grid((L + AT - 1) / AT, Hq, B);
  const float sl2 = scale * 1.4426950408889634f;
  if (capped) attn_fwd_kernel<true><<<grid, 160, FWD_SMEM, st>>>(maps, static_cast<__nv_bfloat16*>(o), lse, doc, pos, L, Hq, Hkv, cap, sl2, err);
  else attn_fwd_kernel<false><<<grid, 160, FWD_SMEM, st>>>(maps, static_cast<__nv_bfloat16*>(o), lse, doc, pos, L, Hq, Hkv, 0, sl2, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// dq, dqf: [B, L, Hq, 64] fp32, zeroed by the caller (reduced into); dk, dkf, dv: [B, L, Hkv, 64] bf16 (written).
// dsum: [B, Hq, L] fp32 scratch.
int attention_bwd(const void* q, const void* qf, const void* k, const void* kf, const void* v, const void* o, const void* dO,
                  const float* lse, float* dsum, float* dq, float* dqf, void* dk, void* dkf, void* dv, const int* doc, int B, int L, int Hq,
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
                                                                 static_cast<__nv_bfloat16*>(dv), doc, L, Hq, Hkv, cap, scale, err);
  else attn_bwd_kernel<false><<<grid, 160, BWD_SMEM, st>>>(maps, lse, dsum, dq, dqf, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dkf),
                                                           static_cast<__nv_bfloat16*>(dv), doc, L, Hq, Hkv, 0, scale, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace ghb
