// Tensor-parallel GEMMs fused with their sequence-parallel collectives over NVLink peer memory / NVSwitch multicast.
//
//   AG (all-gather -> GEMM): one operand is the concatenation over ranks of token shards ("gathered" buffer, rows
//     [r Ts, (r+1) Ts) owned by rank r). A few CTAs of the launch push this rank's shard into every peer's gathered
//     buffer, 128 rows at a time, and raise one flag per 128-row chunk on every destination. With a multicast mapping
//     of the buffer the push is ONE `multimem.st` per 16 bytes that the switch delivers to all ranks (the shard leaves
//     this GPU once instead of W - 1 times); without one, plain 16-byte peer stores rank by rank. The GEMM CTAs of the
//     same launch walk their tiles starting at the local shard and, before the TMA loads of a tile whose chunk came
//     from a peer, wait (bounded) for that chunk's flag: the transfer of later shards overlaps the math on earlier
//     ones. The gathered operand can be the row operand (forward, dgrad: chunks index the M tiles) or lie along the
//     reduction (wgrad: chunks index the k-blocks).
//   RS (GEMM -> reduce-scatter): the product is a partial sum over ranks whose rows are owned rank by rank. Every rank
//     writes its partial tiles (bf16, TMA tile stores) into its OWN symmetric buffer, walking the owners' row ranges
//     starting with the next rank's, and raises "my partial rows for owner d are complete" on d as soon as they are.
//     The same launch then reduces: each CTA, done with its tiles, waits (bounded) for every rank's flag for THIS
//     rank's rows and sums them: one `multimem.ld_reduce` per 16 bytes when the buffer has a multicast mapping (the
//     switch adds the W partial values in fp32 and returns the sum, so a row crosses this GPU's links once), else W
//     peer loads summed in fp32. bf16 on the wire either way, a fixed summation order per path.
//
// Buffers are reused in rings; a writer never overwrites a slot before its readers are done: readers publish
// "released up to call n" counters (`tp_signal`, and the tail of the RS launch) and writers wait (bounded) for them.
// All flags are call sequence numbers written with system-scope release stores and read with acquire loads; a wait
// that runs out writes a status code and the kernel drains and returns. No TMA load here uses cluster multicast
// (`multimem.*` is the switch's multicast, a different mechanism).
// The reference has no tensor parallelism; its sequence of NCCL calls for the same math would be all_gather_into_tensor
// + matmul and matmul + reduce_scatter_tensor.
#include "kernels.h"
#include "sm100.cuh"
#include "gemm_epilogue.cuh"
#include <algorithm>
#include <cstring>

namespace ghb {
using namespace sm100;

namespace tp {
constexpr int BM = 128, BK = 64, UK = 16, BN = 256;
constexpr int THREADS = 192;
constexpr int STAGES = 4;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr uint32_t SMEM = STAGES * (A_BYTES + B_BYTES) + EPI_SMEM_BYTES + 256 + 1024;      // operand ring, RS output slabs, barriers
constexpr uint32_t TMEM_COLS = 2 * BN;
constexpr int MAXR = 8;
constexpr unsigned long long WAIT_NS = 2000000000ull;
constexpr int CHUNK = 128;           // rows per gather chunk = BM

// Pad layout (uint32 words) of each rank's symmetric signal pad.
constexpr int PAD_AG_DONE = 0;       // [MAXR]  AG_DONE[j]: rank j has released every gather slot use <= value
constexpr int PAD_RS_READY = 8;      // [MAXR]  RS_READY[j]: rank j's partial tiles of call <= value have landed here
constexpr int PAD_RS_DONE = 16;      // [MAXR]  RS_DONE[j]: rank j has reduced every staging slot use <= value
constexpr int PAD_WORDS = 32;

struct Args {
  // --- gather
  __nv_bfloat16* xg[MAXR];           // every rank's gathered buffer for this call's slot
  unsigned int* chunk[MAXR];         // every rank's chunk flags for this slot: [rows / CHUNK]
  unsigned int* pad[MAXR];           // every rank's signal pad
  int rank, world;
  int mode;                          // 0: AG, 1: RS, 2: plain
  int push;                          // AG: this launch pushes the local shard (first consumer of the gather)
  int axis;                          // AG: 0 = gathered rows are A's rows (M tiles); 1 = gathered rows lie along K
  long shard_rows;                   // Ts
  long row_elems;                    // elements per gathered row
  long ld;                           // row stride (elements) of the gathered buffers
  unsigned int seq;                  // sequence number of the gather (AG) or of the scatter (RS)
  unsigned int need;                 // peers must have released uses <= need of the slot before it is overwritten
  int n_push;                        // CTAs [0, n_push) push, the rest multiply
  // --- scatter
  __nv_bfloat16* stage[MAXR];        // every rank's partial-product buffer for this call's slot: [T][N]
  unsigned int* done_counter;        // local, zero between launches
  unsigned int* owner_counters;      // local [MAXR], zero between launches: tiles of each owner's rows stored so far
  // --- multicast views (null: peer loads / stores)
  __nv_bfloat16* xg_mc;              // the gather slot on every rank at once
  __nv_bfloat16* stage_mc;           // the partial-product slot of every rank at once
  // --- scatter output
  void* out;                         // [Ts][N] this rank's reduced rows
  int out_f32;
  int tma;                           // bit 0: a scatter's partial tiles are tile-stored into their owner's slot and summed there
                                     // from local memory, and tiles / k-blocks are walked chunk-major over the shards;
                                     // bit 1: a gather's push CTAs drive tile loads and tile stores (else threads copy)
};

// One tensor map per rank over the same buffer on every GPU. AG: the gather slot [T][row_elems] (boxes of PUSH_ROWS x
// PUSH_COLS, unswizzled; this rank's own entry is the source of its pushes). RS: rank d's entry covers the rows that
// THIS rank's partial products occupy in d's staging slot, [Ts][N] at source index `rank` (64-column swizzled slabs).
struct PeerMaps {
  CUtensorMap m[MAXR];
};
constexpr int PUSH_ROWS = CHUNK, PUSH_COLS = 128, PUSH_STAGES = 6;
constexpr uint32_t PUSH_TILE_BYTES = PUSH_ROWS * PUSH_COLS * 2;

__device__ __forceinline__ void mc_st16(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
               "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
// Sum over every rank's copy of 8 bf16 values, added in fp32 inside the switch, returned as bf16.
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int seq) {
  if (static_cast<int>(ld_acquire_sys(p) - seq) >= 0) return true;
  const unsigned long long t0 = now_ns();
  while (static_cast<int>(ld_acquire_sys(p) - seq) < 0) {
    if (now_ns() - t0 > WAIT_NS) return false;
    __nanosleep(100);
  }
  return true;
}
}  // namespace tp

// The scatter's second half, run by every CTA of a launch: wait (bounded) until every rank's partial rows for THIS
// rank's row range are flagged, sum them and write the reduced rows; the last CTA publishes "this rank has read the
// slot" to every rank. Sources: with a.tma the partials lie in this rank's own slot, source after source (local loads, a
// fixed order); else each rank's partial rows are read from that rank's buffer (through the switch's multicast
// reduction when mapped).
__device__ void tp_scatter_tail(const tp::Args& a, int N, int* __restrict__ err, bool wait_own) {
  using namespace tp;
  {
    // RS, second half: this rank's rows. Every rank's partial rows for them are flagged as they complete; sum them (in the
    // switch when the buffer is multicast-mapped) and write the reduced rows.
    __shared__ int go_reduce;
    if (threadIdx.x == 0) {
      go_reduce = (*reinterpret_cast<volatile int*>(err) == 0) ? 1 : 0;
      for (int j = 0; j < a.world && go_reduce; ++j)      // this rank's own rows may be complete by stream order instead
        if (wait_own || j != a.rank) go_reduce = wait_flag(a.pad[a.rank] + PAD_RS_READY + j, a.seq) ? 1 : 0;
      if (!go_reduce && *reinterpret_cast<volatile int*>(err) == 0) atomicExch(err, 508);
    }
    __syncthreads();
    if (go_reduce) {
      // 16-byte items, several in flight per thread: a load over NVLink (or through the switch) takes microseconds, and the
      // reduction is bound by how many of them are outstanding, not by arithmetic
      constexpr int RU = 8;
      const long n8 = a.shard_rows * N / 8;
      const long base = static_cast<long>(a.rank) * a.shard_rows * N;
      const long stride = static_cast<long>(gridDim.x) * blockDim.x;
      auto put = [&](long i, const float* sum) {
        if (a.out_f32) {
          float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + i * 8);
          o[0] = make_float4(sum[0], sum[1], sum[2], sum[3]); o[1] = make_float4(sum[4], sum[5], sum[6], sum[7]);
        } else {
          uint32_t p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) { __nv_bfloat162 h = __floats2bfloat162_rn(sum[2 * e], sum[2 * e + 1]); p[e] = *reinterpret_cast<uint32_t*>(&h); }
          reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + i * 8)[0] = make_uint4(p[0], p[1], p[2], p[3]);
        }
      };
      auto widen = [](const uint4 v, float* f, bool add) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
          f[2 * e] = (add ? f[2 * e] : 0.f) + t.x; f[2 * e + 1] = (add ? f[2 * e + 1] : 0.f) + t.y;
        }
      };
      for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < n8; i0 += stride * RU) {
        if (a.tma & 1) {       // every rank's partial rows already lie in this rank's slot, source after source: local loads, fixed order
          float sum[RU][8];
          for (int j = 0; j < a.world; ++j) {
            uint4 v[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) v[u] = reinterpret_cast<const uint4*>(a.stage[a.rank] + j * a.shard_rows * N)[i]; }
#pragma unroll
            for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) widen(v[u], sum[u], j != 0); }
          }
#pragma unroll
          for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) put(i, sum[u]); }
        } else if (a.stage_mc) {
          uint4 v[RU];
#pragma unroll
          for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) v[u] = mc_ld_reduce_bf16x8(a.stage_mc + base + i * 8); }
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const long i = i0 + u * stride;
            if (i < n8) { float sum[8]; widen(v[u], sum, false); put(i, sum); }
          }
        } else {
          float sum[RU][8];
          for (int q = 0; q < a.world; ++q) {
            const int j = (a.rank + q) % a.world;
            uint4 v[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) v[u] = reinterpret_cast<const uint4*>(a.stage[j] + base)[i]; }
#pragma unroll
            for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) widen(v[u], sum[u], q != 0); }
          }
#pragma unroll
          for (int u = 0; u < RU; ++u) { const long i = i0 + u * stride; if (i < n8) put(i, sum[u]); }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {      // the last CTA to finish publishes "this rank has read every rank's buffer slot of this call"
      __threadfence_system();
      const unsigned int arrived = atomicAdd(a.done_counter, 1u);
      if (arrived == gridDim.x - 1) {
        if (go_reduce) for (int p = 0; p < a.world; ++p) st_release_sys(a.pad[p] + PAD_RS_DONE + a.rank, a.seq);
        *a.done_counter = 0u;
      }
    }
  }
}

// out: 0 bf16, 1 fp32, 2 fp32 accumulate (modes AG and plain); RS writes bf16 staging tiles.
template <bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(tp::THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const __grid_constant__ CUtensorMap tma_c,
               void* __restrict__ Cout, long ldc, int M, int N, int K, const __grid_constant__ tp::Args a,
               const __grid_constant__ tp::PeerMaps pm, int splits, int* __restrict__ err) {
  using namespace tp;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (*reinterpret_cast<volatile int*>(err) != 0) return;

  // ------------------------------------------------------------------ push CTAs (AG): local shard -> every peer
  if (a.mode == 0 && static_cast<int>(blockIdx.x) < a.n_push) {
    if (!a.push) return;
    __shared__ int go;
    const long chunks_per_shard = a.shard_rows / CHUNK;
    const long vec_per_row = a.row_elems / 8;                 // 16-byte vectors
    const __nv_bfloat16* src = a.xg[a.rank] + a.rank * a.shard_rows * a.ld;
    constexpr int UNROLL = 8;                                  // loads in flight per thread: the copy is latency-bound otherwise
    if (a.tma & 2) {
      // One thread drives the bulk-copy engine: a PUSH_ROWS x PUSH_COLS box of the local shard comes into shared memory
      // (tile load) and leaves once per peer (tile stores into the same rows of that peer's buffer). Loads run
      // PUSH_STAGES - 1 boxes ahead of the stores; a chunk's flag is raised on every peer once all of its stores are done.
      if (threadIdx.x != 0) return;
      uint8_t* ring = smem;
      uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PUSH_STAGES * PUSH_TILE_BYTES);
      for (int d = 0; d < a.world; ++d)
        if (d != a.rank && !wait_flag(a.pad[a.rank] + PAD_AG_DONE + d, a.need)) { atomicExch(err, 501); return; }
      for (int i = 0; i < PUSH_STAGES; ++i) mbar_init(&bars[i], 1);
      mbar_fence_init();
      for (int d = 0; d < a.world; ++d) tma_prefetch_desc(&pm.m[d]);
      const long cols = (a.row_elems + PUSH_COLS - 1) / PUSH_COLS;
      const long my_chunks = blockIdx.x < chunks_per_shard ? (chunks_per_shard - blockIdx.x + a.n_push - 1) / a.n_push : 0;
      const long total = my_chunks * cols;
      const long row_base = a.rank * a.shard_rows;
      auto load = [&](long n) {
        const int s = static_cast<int>(n % PUSH_STAGES);
        const long c = blockIdx.x + (n / cols) * a.n_push;
        mbar_expect_tx(&bars[s], PUSH_TILE_BYTES);
        tma_load_2d(ring + s * PUSH_TILE_BYTES, &pm.m[a.rank], &bars[s], static_cast<int>((n % cols) * PUSH_COLS), static_cast<int>(row_base + c * CHUNK));
      };
      for (long n = 0; n < total && n < PUSH_STAGES - 1; ++n) load(n);
      for (long n = 0; n < total; ++n) {
        const int s = static_cast<int>(n % PUSH_STAGES);
        const long c = blockIdx.x + (n / cols) * a.n_push;
        if (!mbar_wait(&bars[s], static_cast<uint32_t>((n / PUSH_STAGES) & 1))) { atomicExch(err, 509); break; }
        for (int q = 1; q < a.world; ++q) {
          const int d = (a.rank - q + a.world) % a.world;
          tma_store_2d(&pm.m[d], ring + s * PUSH_TILE_BYTES, static_cast<int>((n % cols) * PUSH_COLS), static_cast<int>(row_base + c * CHUNK));
        }
        tma_store_commit();
        if (n + PUSH_STAGES - 1 < total) {
          tma_store_wait_read<1>();          // the box stored one trip ago has left shared memory: its buffer takes the next load
          load(n + PUSH_STAGES - 1);
        }
        if (n % cols == cols - 1) {          // the chunk's last box
          tma_store_wait<0>();
          asm volatile("fence.proxy.async.global;" ::: "memory");
          __threadfence_system();
          for (int d = 0; d < a.world; ++d)
            if (d != a.rank) st_release_sys(a.chunk[d] + a.rank * chunks_per_shard + c, a.seq);
        }
      }
      tma_store_wait<0>();
      return;
    }
    if (a.xg_mc) {
      // one store per 16 bytes reaches every rank through the switch: wait until every destination has released the slot
      if (threadIdx.x == 0) {
        go = 1;
        for (int d = 0; d < a.world && go; ++d)
          if (d != a.rank) go = wait_flag(a.pad[a.rank] + PAD_AG_DONE + d, a.need) ? 1 : 0;
        if (!go) atomicExch(err, 501);
      }
      __syncthreads();
      if (!go) return;
      __nv_bfloat16* dst = a.xg_mc + a.rank * a.shard_rows * a.ld;
      for (long c = blockIdx.x; c < chunks_per_shard; c += a.n_push) {
        const long total = CHUNK * vec_per_row;
        for (long i0 = threadIdx.x; i0 < total; i0 += static_cast<long>(blockDim.x) * UNROLL) {
          uint4 v[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long i = i0 + static_cast<long>(u) * blockDim.x;
            if (i < total) v[u] = reinterpret_cast<const uint4*>(src + (c * CHUNK + i / vec_per_row) * a.ld)[i % vec_per_row];
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long i = i0 + static_cast<long>(u) * blockDim.x;
            if (i < total) mc_st16(dst + (c * CHUNK + i / vec_per_row) * a.ld + (i % vec_per_row) * 8, v[u]);
          }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence_system();
          for (int d = 0; d < a.world; ++d)
            if (d != a.rank) st_release_sys(a.chunk[d] + a.rank * chunks_per_shard + c, a.seq);
        }
        __syncthreads();
      }
      return;
    }
    for (int q = 1; q < a.world; ++q) {
      const int d = (a.rank - q + a.world) % a.world;         // destination d reads shard d + q as its q-th shard
      if (threadIdx.x == 0) {
        go = wait_flag(a.pad[a.rank] + PAD_AG_DONE + d, a.need) ? 1 : 0;
        if (!go) atomicExch(err, 501);
      }
      __syncthreads();
      if (!go) return;
      __nv_bfloat16* dst = a.xg[d] + a.rank * a.shard_rows * a.ld;
      for (long c = blockIdx.x; c < chunks_per_shard; c += a.n_push) {
        const long total = CHUNK * vec_per_row;
        for (long i0 = threadIdx.x; i0 < total; i0 += static_cast<long>(blockDim.x) * UNROLL) {
          uint4 v[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long i = i0 + static_cast<long>(u) * blockDim.x;
            if (i < total) v[u] = reinterpret_cast<const uint4*>(src + (c * CHUNK + i / vec_per_row) * a.ld)[i % vec_per_row];
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long i = i0 + static_cast<long>(u) * blockDim.x;
            if (i < total) reinterpret_cast<uint4*>(dst + (c * CHUNK + i / vec_per_row) * a.ld)[i % vec_per_row] = v[u];
          }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence_system();
          st_release_sys(a.chunk[d] + a.rank * chunks_per_shard + c, a.seq);
        }
      }
      __syncthreads();
    }
    return;
  }

  // ------------------------------------------------------------------ GEMM CTAs
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* slabs = smem + STAGES * (A_BYTES + B_BYTES);              // RS output staging (1024-byte aligned)
  uint64_t* full = reinterpret_cast<uint64_t*>(slabs + EPI_SMEM_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int first = a.mode == 0 ? a.n_push : 0;
  const int cta = static_cast<int>(blockIdx.x) - first, n_cta = static_cast<int>(gridDim.x) - first;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  // ring order: AG starts at the local shard, RS at the next rank's rows (its own rows last)
  const int tiles_per_shard = a.mode == 2 ? 0 : static_cast<int>(a.shard_rows / BM);
  const int m_rot = a.mode == 0 ? (a.axis == 0 ? a.rank * tiles_per_shard : 0) : (a.mode == 1 ? ((a.rank + 1) % a.world) * tiles_per_shard : 0);
  const int kb_rot = (a.mode == 0 && a.axis == 1) ? static_cast<int>(a.rank * (a.shard_rows / BK)) : 0;
  const bool k_interleave = (a.tma & 1) && a.mode == 0 && a.axis == 1;
  const int chunks_in_shard = a.mode == 2 ? 1 : static_cast<int>(a.shard_rows / CHUNK);
  auto kb_of = [&](int pos) -> int {      // position in this rank's reduction order -> k-block
    if (!k_interleave) return (pos + kb_rot) % num_kb;
    constexpr int PER = CHUNK / BK;       // chunk-major over the shards, own shard first (the order the pushed chunks arrive)
    const int q = pos / PER, b = pos % PER, c = q / a.world, j = q % a.world;
    return (((a.rank + j) % a.world) * chunks_in_shard + c) * PER + b;
  };
  // A work unit is (output tile, slice of the reduction); slices > 1 only where the gathered rows lie along K (weight
  // gradients: few output tiles, K = all tokens). Units are ordered slice-major and the k-blocks are rotated to start at
  // the local shard, so the first units need no peer's data; slices meet in the fp32 output through reductions in L2.
  const int units = tiles * splits;
  const int kbs = (num_kb + splits - 1) / splits;
  auto tile_of = [&](int u, int& tm, int& tn, int& k_lo, int& k_hi) {     // column tiles of one row tile are consecutive: they share its chunk
    const int t = u % tiles, sp = u / tiles;
    if ((a.tma & 1) && ((a.mode == 0 && a.axis == 0) || a.mode == 1)) {
      // chunk-major over the shards: row tile c of every shard, then row tile c + 1 (AG: the order in which the pushed
      // chunks arrive, own shard first; RS: every owner's link carries partial tiles during the whole product, own rows last)
      const int i = t / tiles_n, c = i / a.world, j = i % a.world;
      tm = ((a.rank + j + (a.mode == 1 ? 1 : 0)) % a.world) * tiles_per_shard + c;
    } else {
      tm = (t / tiles_n + m_rot) % tiles_m;
    }
    tn = t % tiles_n;
    k_lo = sp * kbs;
    k_hi = k_lo + kbs < num_kb ? k_lo + kbs : num_kb;
  };

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (a.mode == 1) tma_prefetch_desc(&tma_c);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      const long chunks_per_shard = a.mode == 0 ? a.shard_rows / CHUNK : 1;
      auto chunk_ready = [&](long chunk) -> bool {        // chunks of the local shard never wait
        if (chunk / chunks_per_shard == a.rank) return true;
        if (!wait_flag(a.chunk[a.rank] + chunk, a.seq)) { atomicExch(err, 502); return false; }
        asm volatile("fence.proxy.async.global;" ::: "memory");   // peer stores (generic proxy) before TMA reads (async proxy)
        return true;
      };
      for (int t = cta; t < units && ok; t += n_cta) {
        int tm, tn, k_lo, k_hi; tile_of(t, tm, tn, k_lo, k_hi);
        const int m0 = tm * BM, n0 = tn * BN;
        if (a.mode == 0 && a.axis == 0 && !chunk_ready(tm)) { ok = false; break; }
        for (int kk = k_lo; kk < k_hi; ++kk) {
          const int kb = kb_of(kk);
          if (a.mode == 0 && a.axis == 1 && ((kb & 1) == 0 || kk == k_lo) && !chunk_ready(kb / 2)) { ok = false; break; }
          if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 503); ok = false; break; }
          mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
          uint8_t* pa = sA + s * A_BYTES; uint8_t* pb = sB + s * B_BYTES;
          if (!A_MN) tma_load_2d(pa, &tma_a, &full[s], kb * BK, m0);
          else for (int j = 0; j < BM / 64; ++j) tma_load_2d(pa + j * (BK * 128), &tma_a, &full[s], m0 + j * 64, kb * BK);
          if (!B_MN) tma_load_2d(pb, &tma_b, &full[s], kb * BK, n0);
          else for (int j = 0; j < BN / 64; ++j) tma_load_2d(pb + j * (BK * 128), &tma_b, &full[s], n0 + j * 64, kb * BK);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) __nanosleep(100000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0; uint32_t ph = 0; int it = 0; bool ok = true;
      for (int t = cta; t < units && ok; t += n_cta, ++it) {
        const int acc = it & 1; const uint32_t aph = (it >> 1) & 1;
        int tm_, tn_, k_lo, k_hi; tile_of(t, tm_, tn_, k_lo, k_hi);
        if (!mbar_wait(&tempty[acc], aph ^ 1)) { atomicExch(err, 504); ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kk = k_lo; kk < k_hi; ++kk) {
          if (!mbar_wait(&full[s], ph)) { atomicExch(err, 505); ok = false; break; }
          tc_fence_after();
          const uint32_t pa = smem_u32(sA + s * A_BYTES), pb = smem_u32(sB + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(pa + k * UK * 128, BK * 128, 1024) : umma_desc_sw128(pa + k * UK * 2, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(pb + k * UK * 128, BK * 128, 1024) : umma_desc_sw128(pb + k * UK * 2, 16, 1024);
            umma_bf16(d, da, db, idesc, kk != k_lo || k != 0);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int quad = warp & 3;
    int it = 0; bool ok = true;
    unsigned int dest_ok = 0;                 // RS: owners known to have finished reading this rank's buffer slot
    uint32_t slab_count = 0;
    int pending_owner = -1;                   // RS over the copy engine: owner of the tile whose stores may still be in flight
    auto publish = [&](int owner) {           // one more tile of `owner`'s rows is complete in its staging slot
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence_system();
      const unsigned int total = static_cast<unsigned int>(tiles_per_shard) * static_cast<unsigned int>(tiles_n);
      if (atomicAdd(a.owner_counters + owner, 1u) + 1u == total) {
        __threadfence_system();
        st_release_sys(a.pad[owner] + PAD_RS_READY + a.rank, a.seq);
        a.owner_counters[owner] = 0u;
      }
    };
    for (int t = cta; t < units && ok; t += n_cta, ++it) {
      const int acc = it & 1; const uint32_t aph = (it >> 1) & 1;
      int tm, tn, k_lo_, k_hi_; tile_of(t, tm, tn, k_lo_, k_hi_);
      if (!mbar_wait(&tfull[acc], aph)) { if (lane == 0) atomicExch(err, 506); ok = false; break; }
      tc_fence_after();
      const long row = static_cast<long>(tm) * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (a.mode == 1) {
        const int d = static_cast<int>((static_cast<long>(tm) * BM) / a.shard_rows);
        if (!((dest_ok >> d) & 1u)) {
          int good = 1;
          if (lane == 0 && d != a.rank) good = wait_flag(a.pad[a.rank] + PAD_RS_DONE + d, a.need) ? 1 : 0;
          good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) { if (lane == 0) atomicExch(err, 507); ok = false; }
          dest_ok |= 1u << d;
        }
      }
      if (a.mode == 1) {
        // RS: the partial tile goes to THIS rank's buffer (TMA tile stores through the swizzled slabs); once every tile of an
        // owner's row range is stored, the owner is told
        const int d = static_cast<int>((static_cast<long>(tm) * BM) / a.shard_rows);
        if (ok && (a.tma & 1)) {
          // the tile goes straight into owner d's staging slot, at this rank's source index: the bulk-copy engine writes
          // it over NVLink while the next tile is multiplied. A tile is counted for its owner one tile later, once its
          // stores are complete (at most the newest tile's stores stay in flight)
          epilogue_store_bf16<BN>(taddr, slabs, &pm.m[d], tm * BM - d * static_cast<int>(a.shard_rows), n0, N, quad, lane, slab_count, &tempty[acc]);
          if (quad == 0 && lane == 0) {
            const bool whole = n0 + BN <= N;               // BN / 64 store groups were committed for this tile
            if (whole) tma_store_wait<BN / 64>(); else tma_store_wait<0>();
            if (pending_owner >= 0) publish(pending_owner);
            pending_owner = d;
            if (!whole) { publish(d); pending_owner = -1; }
          }
          continue;
        }
        if (ok) {
          epilogue_store_bf16<BN>(taddr, slabs, &tma_c, tm * BM, n0, N, quad, lane, slab_count, &tempty[acc]);
          if (quad == 0 && lane == 0) {
            tma_store_wait<0>();                       // the tile's stores are complete, not merely read out of shared memory
            __threadfence_system();
            const unsigned int total = static_cast<unsigned int>(tiles_per_shard) * static_cast<unsigned int>(tiles_n);
            if (atomicAdd(a.owner_counters + d, 1u) + 1u == total) {
              __threadfence_system();
              st_release_sys(a.pad[d] + PAD_RS_READY + a.rank, a.seq);
              a.owner_counters[d] = 0u;
            }
          }
          continue;
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (ok && row < M && col < N) {
          if (OUT == 0) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(Cout) + row * ldc + col;
            if (col + 32 <= N) {
              uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]), __uint_as_float(r[v * 8 + 2 * e + 1]));
                  p[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                o4[v] = make_uint4(p[0], p[1], p[2], p[3]);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) if (col + e < N) out[e] = __float2bfloat16(__uint_as_float(r[e]));
            }
          } else {
            float* out = reinterpret_cast<float*>(Cout) + row * ldc + col;
            if (splits > 1) {
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
                float4 x = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (a.mode == 1 && quad == 0 && lane == 0) {
      tma_store_wait<0>();
      if (pending_owner >= 0) publish(pending_owner);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (a.mode == 1) tp_scatter_tail(a, N, err, true);
}

// The scatter's reduction as a launch of its own (partials delivered by the copy engines).
__global__ void __launch_bounds__(tp::THREADS)
tp_reduce_kernel(const __grid_constant__ tp::Args a, int N, int* __restrict__ err) {
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  tp_scatter_tail(a, N, err, false);
}

// Publishes "this rank has released gather-slot uses <= seq" to every rank (stream-ordered after the slot's readers).
// With wait_word >= 0 it then waits (bounded) until every peer has published a.need in that word: what a push that no
// kernel carries out (copy-engine copies queued behind this launch) must know before it overwrites the peers' slot.
__global__ void tp_signal_kernel(tp::Args a, int word, int wait_word, int* err) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (a.seq) for (int p = 0; p < a.world; ++p) tp::st_release_sys(a.pad[p] + word + a.rank, a.seq);
    if (wait_word >= 0 && a.need)
      for (int d = 0; d < a.world; ++d)
        if (d != a.rank && !tp::wait_flag(a.pad[a.rank] + wait_word + d, a.need)) { atomicExch(err, 501); break; }
  }
}

// ------------------------------------------------------------------------------------------------ host side
static bool tp_encode(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, bool mn_major, int block_mn) {
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (!mn_major) { dims[0] = cols; dims[1] = rows; box[0] = tp::BK; box[1] = block_mn; }
  else { dims[0] = rows; dims[1] = cols; box[0] = 64; box[1] = tp::BK; }
  strides[0] = static_cast<uint64_t>(ld) * 2;
  return encode_tensor_map_2d(map, ptr, 2, dims, strides, box, true);
}

size_t tp_args_bytes() { return sizeof(tp::Args); }
int tp_pad_words() { return tp::PAD_WORDS; }

template <bool A_MN, bool B_MN, int OUT>
static int tp_launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, long ldc, int M, int N, int K, const tp::Args& a,
                     const tp::PeerMaps& pm, int splits, int* err, int sms, cudaStream_t st) {
  auto kern = gemm_tp_kernel<A_MN, B_MN, OUT>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp::SMEM) != cudaSuccess) return 3;
    attr = true;
  }
  const int tiles = ((M + tp::BM - 1) / tp::BM) * ((N + tp::BN - 1) / tp::BN);
  const int first = a.mode == 0 ? a.n_push : 0;
  const int units = tiles * splits;
  const int grid = first + (units < sms - first ? units : sms - first);       // every CTA co-resident: one per SM
  kern<<<grid, tp::THREADS, tp::SMEM, st>>>(ta, tb, tc, C, ldc, M, N, K, a, pm, splits, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// D = A B^T on this rank's operands; `args` is a host copy of tp::Args (tp_args_bytes() bytes). mode AG: the gathered
// operand is whichever of A (axis 0: its rows; axis 1 with a_gathered) or B (axis 1) lives in args.xg[rank].
// out: 0 bf16, 1 fp32, 2 fp32 accumulate (ignored in mode RS, whose tiles go to the staging buffers as bf16).
int gemm_tp(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc, bool a_mn, bool b_mn, int out,
            const void* args, int* err, int sms, cudaStream_t st) {
  tp::Args a;
  memcpy(&a, args, sizeof(a));       // the table arrives in a byte buffer of unknown alignment
  if (M <= 0 || N <= 0 || K <= 0) return 1;
  if (lda % 8 || ldb % 8) return 11;
  if (a.mode != 1 && (ldc % (out == 0 ? 8 : 4))) return 13;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return 14;
  if (a.world > tp::MAXR || a.world < 1) return 1;
  if (a.mode != 2) {
    if (a.shard_rows % tp::CHUNK) return 17;
    if (a.mode == 0 && (a.row_elems % 8 || a.ld % 8 || a.n_push < (a.push ? 1 : 0) || a.n_push >= sms)) return 18;
    if (a.mode == 0 && a.axis == 0 && static_cast<long>(M) != a.shard_rows * a.world) return 19;
    if (a.mode == 0 && a.axis == 1 && static_cast<long>(K) != a.shard_rows * a.world) return 19;
    if (a.mode == 1 && (static_cast<long>(M) != a.shard_rows * a.world || N % 8)) return 19;
  }
  CUtensorMap ta, tb, tc;
  if (!tp_encode(&ta, A, M, K, lda, a_mn, tp::BM)) return 21;
  if (!tp_encode(&tb, B, N, K, ldb, b_mn, tp::BN)) return 22;
  tc = ta;
  if (a.mode == 1) {      // the partial product [M, N] (bf16) in this rank's own buffer, stored as 64-column slabs
    if (!a.stage[a.rank] || !a.out || !a.owner_counters) return 20;
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)}, strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, tp::BM};
    if (!encode_tensor_map_2d(&tc, a.stage[a.rank], 2, dims, strides, box, true)) return 23;
  }
  // the same buffer on every GPU, one map per rank (pushes of a gather; partial tiles of a scatter)
  static_assert(tp::PUSH_STAGES * tp::PUSH_TILE_BYTES + 256 <= tp::SMEM - 1024, "the push ring fits the kernel's shared memory");
  tp::PeerMaps pm;
  memset(&pm, 0, sizeof(pm));
  if ((a.tma & 2) && a.mode == 0 && a.push) {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.row_elems), static_cast<uint64_t>(a.shard_rows * a.world)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.ld) * 2};
    const uint32_t box[2] = {tp::PUSH_COLS, tp::PUSH_ROWS};
    for (int d = 0; d < a.world; ++d)
      if (!a.xg[d] || !encode_tensor_map_2d(&pm.m[d], a.xg[d], 2, dims, strides, box, false)) return 24;
  }
  if ((a.tma & 1) && a.mode == 1) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(a.shard_rows)}, strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, tp::BM};
    for (int d = 0; d < a.world; ++d)
      if (!a.stage[d] || !encode_tensor_map_2d(&pm.m[d], a.stage[d] + static_cast<long>(a.rank) * a.shard_rows * N, 2, dims, strides, box, true)) return 25;
  }
  // gathered rows along K with an fp32 output: slice the reduction so that the units fill the SMs the pushes leave
  int splits = 1;
  if (a.mode == 0 && a.axis == 1 && out != 0) {
    const int tiles = ((M + tp::BM - 1) / tp::BM) * ((N + tp::BN - 1) / tp::BN), num_kb = (K + tp::BK - 1) / tp::BK;
    const int free_sms = sms - (a.push ? a.n_push : 0);
    // about four units per SM: the units of a slice run while the next slices' chunks are still arriving, and the
    // last wave is short
    splits = std::max(1, std::min(std::min((4 * free_sms + tiles / 2) / tiles, num_kb / 16), 32));
    while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
    if (splits > 1 && out == 1 && cudaMemset2DAsync(C, ldc * 4, 0, static_cast<size_t>(N) * 4, M, st) != cudaSuccess) return 5;
  }
#define GHB_TP(AM, BMN)                                                                              \
  switch (a.mode == 1 ? 0 : out) {                                                                   \
    case 0: return tp_launch<AM, BMN, 0>(ta, tb, tc, C, ldc, M, N, K, a, pm, 1, err, sms, st);       \
    case 1: return tp_launch<AM, BMN, 1>(ta, tb, tc, C, ldc, M, N, K, a, pm, splits, err, sms, st);  \
    default: return tp_launch<AM, BMN, 2>(ta, tb, tc, C, ldc, M, N, K, a, pm, splits, err, sms, st); \
  }
  if (!a_mn && !b_mn) { GHB_TP(false, false) }
  if (!a_mn && b_mn) { GHB_TP(false, true) }
  if (a_mn && !b_mn) { GHB_TP(true, false) }
  GHB_TP(true, true)
#undef GHB_TP
}

int tp_signal(const void* args, int word, int wait_word, int* err, cudaStream_t st) {
  tp::Args a;
  memcpy(&a, args, sizeof(a));
  tp_signal_kernel<<<1, 32, 0, st>>>(a, word, wait_word, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// The gather's push by the copy engines: this rank's shard (already in its own slot) goes into the same rows of every
// peer's slot, `pieces` row ranges per peer; behind each piece a second small copy writes the call's sequence number
// into the peer's flags of the piece's chunks (`seq_src`: device words holding a.seq, at least shard_rows / CHUNK of
// them). The peer at distance q (rank - q) is served by streams[q - 1]: copies of one stream run in order, so a flag
// lands after its data, and the streams' copies run side by side on different engines (one peer-to-peer copy alone was
// measured at about half of what the link carries). No SM is used; the consuming GEMM polls the flags chunk by chunk.
int tp_push_copies(const void* args, const void* seq_src, int pieces, const cudaStream_t* streams, int n_streams) {
  tp::Args a;
  memcpy(&a, args, sizeof(a));
  if (a.world < 1 || a.world > tp::MAXR || a.shard_rows % tp::CHUNK || a.ld != a.row_elems || pieces < 1 || n_streams < a.world - 1) return 1;
  const long cps = a.shard_rows / tp::CHUNK;
  if (pieces > cps) pieces = static_cast<int>(cps);
  for (int p = 0; p < pieces; ++p) {
    const long c0 = p * cps / pieces, c1 = (p + 1) * cps / pieces;
    const long off = (a.rank * a.shard_rows + c0 * tp::CHUNK) * a.ld;
    const size_t bytes = static_cast<size_t>((c1 - c0) * tp::CHUNK * a.ld) * 2;
    for (int q = 1; q < a.world; ++q) {
      const int d = (a.rank - q + a.world) % a.world;
      cudaStream_t st = streams[q - 1];
      if (!a.xg[d] || !a.chunk[d]) return 2;
      if (cudaMemcpyAsync(a.xg[d] + off, a.xg[a.rank] + off, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return 5;
      if (cudaMemcpyAsync(a.chunk[d] + a.rank * cps + c0, seq_src, static_cast<size_t>(c1 - c0) * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return 5;
    }
  }
  return 0;
}

// Reduction of a scatter whose partials the copy engines delivered: args as for mode RS (stage[rank], pad, seq, out).
int tp_reduce(const void* args, int N, int* err, int sms, cudaStream_t st) {
  tp::Args a;
  memcpy(&a, args, sizeof(a));
  if (a.world < 1 || a.world > tp::MAXR || !a.stage[a.rank] || !a.out || !a.done_counter || N % 8 || !(a.tma & 1)) return 1;
  tp_reduce_kernel<<<2 * sms, tp::THREADS, 0, st>>>(a, N, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// One copy-engine delivery: `bytes` from src to dst (this GPU's or a peer's memory), then a 4-byte copy of *flag_src to
// flag_dst on the same stream (so the word lands after the data).
int tp_copy_flagged(void* dst, const void* src, size_t bytes, void* flag_dst, const void* flag_src, cudaStream_t st) {
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return 5;
  if (cudaMemcpyAsync(flag_dst, flag_src, 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return 5;
  return 0;
}

}  // namespace ghb
