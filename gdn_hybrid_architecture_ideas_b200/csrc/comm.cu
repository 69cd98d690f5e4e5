// Data-parallel gradient reduce-scatter fused with the sharded AdamW update and the parameter all-gather, over
// NVLink peer memory (plain peer loads / stores, or NVSwitch multimem reductions and broadcasts when a multicast
// mapping of the buffers exists). The flat buffers are cut into buckets (contiguous ranges whose gradients finish
// together during the backward); every rank owns one slice of every bucket. Per bucket, on a stream of their own:
//
//   reduce:  every rank signals "my gradients of this bucket are final", waits (bounded) for all peers' signals, then
//            sums the W copies of ITS slice straight out of the peers' gradient buffers (or one multimem.ld_reduce per
//            vector) into a local fp32 shard buffer. Launched while the backward of earlier layers is still running,
//            on a small grid; the last bucket's launch also publishes the rank's sum of squares to all peers;
//   update:  (first bucket: waits, bounded, for all W partial norms and forms the clip coefficient) applies AdamW to
//            its slice of the fp32 master weights and writes the new bf16 values into EVERY rank's compute-weight
//            buffer, plus the fp32 values where a tensor is read in fp32 (norm gains, gates, the embedding: marked in
//            a bitmap; matrices that are only read as bf16 keep their fp32 master on the owner alone: 2 bytes per
//            parameter on the wire instead of 6), then signals "my slice of this bucket is written";
//   settle:  waits (bounded) until every peer's slice of the bucket has landed; the next forward's first reader of the
//            bucket is ordered after it by an event, so the parameter all-gather of later layers hides behind the
//            forward of earlier ones.
//
// The reference does this as NCCL all-reduce / reduce-scatter, a separate clip, a separate optimizer step and an
// all-gather (ced/train/data_parallel.py:476-479, ced/train/zero1.py:250-264, 293-337). Flags are monotonically
// increasing step numbers in each rank's signal pad, written with system-scope release stores and read with acquire
// loads. A wait that exceeds its limit writes a status code and the kernel returns; nothing spins forever.
#include "kernels.h"
#include <cuda_bf16.h>

namespace ghb {

constexpr int MAX_RANKS = 8;
constexpr unsigned long long COMM_WAIT_NS = 2000000000ull;

constexpr int MAX_GROUPS = 6;
struct GroupTable { long start[MAX_GROUPS]; float wd[MAX_GROUPS]; float lr[MAX_GROUPS]; int count; };

struct CommPeers {
  float* grads[MAX_RANKS];            // each rank's full flat gradient buffer
  float* params[MAX_RANKS];           // each rank's full flat fp32 parameter buffer
  __nv_bfloat16* lp[MAX_RANKS];       // each rank's full flat bf16 parameter buffer (may be null)
  unsigned int* flags[MAX_RANKS];     // each rank's signal pad: [3][MAX_RANKS] step counters
  float* norms[MAX_RANKS];            // each rank's [MAX_RANKS] partial sums of squares
  float* mc_grads;                    // multicast views (null: peer loads / stores)
  float* mc_params;
  __nv_bfloat16* mc_lp;
};

__device__ __forceinline__ unsigned long long timer_ns() {
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
// Wait until flag[p] >= seq for every rank p; false on timeout.
__device__ __forceinline__ bool wait_all(const unsigned int* flag, int world, unsigned int seq) {
  const unsigned long long t0 = timer_ns();
  for (int p = 0; p < world; ++p) {
    while (static_cast<int>(ld_acquire_sys(flag + p) - seq) < 0) {
      if (timer_ns() - t0 > COMM_WAIT_NS) return false;
      __nanosleep(200);
    }
  }
  return true;
}
__device__ __forceinline__ float4 mc_ld_reduce(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(float* p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ------------------------------------------------------------------------------------------------ reduce
// ticket: this launch's number in the job-wide sequence of reduce launches (every rank launches the same sequence), the
// value of the "gradients final" flag. publish_seq != 0: this is the step's last bucket; publish the accumulated sum of
// squares and raise the norm flag to publish_seq.
__global__ void comm_reduce_kernel(CommPeers peers, int rank, int world, long lo, long n, float* __restrict__ shard, unsigned int ticket,
                                   unsigned int publish_seq, float* __restrict__ block_acc, unsigned int* __restrict__ done_counter,
                                   int* __restrict__ err) {
  __shared__ float red[32];
  __shared__ int go;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {   // gradients of this bucket were completed by earlier work this stream waited for
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 0 * MAX_RANKS + rank, ticket);
    }
    go = wait_all(peers.flags[rank] + 0 * MAX_RANKS, world, ticket) ? 1 : 0;
    if (!go) atomicExch(err, 401);
  }
  __syncthreads();
  float acc = 0.f;
  if (go) {
    const long n4 = n / 4;
    for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
      float4 s;
      if (peers.mc_grads) {
        s = mc_ld_reduce(peers.mc_grads + lo + i * 4);
      } else {
        s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < world; ++q) {
          const int p = (rank + q) % world;   // start at self, spread the link load
          const float4 t = reinterpret_cast<const float4*>(peers.grads[p] + lo)[i];
          s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
        }
      }
      reinterpret_cast<float4*>(shard)[i] = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(block_acc, t);
    __threadfence();
    const unsigned int arrived = atomicAdd(done_counter, 1u);
    if (arrived == gridDim.x - 1) {   // last block of this launch
      if (publish_seq) {              // last bucket of the step: this rank's partial norm to every peer, then the flag
        const float total = atomicAdd(block_acc, 0.f);
        for (int p = 0; p < world; ++p) peers.norms[p][rank] = total;
        __threadfence_system();
        for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 1 * MAX_RANKS + rank, publish_seq);
        *block_acc = 0.f;
      }
      *done_counter = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------------------ update + gather
// first != 0: the step's first update launch; waits for the norms, forms (norm, clip coefficient) and leaves them in
// `coef_buf` for the step's later launches (stream-ordered after this one). fp32_map: one bit per 64 elements of the
// flat buffers, set where the fp32 value must reach every rank (null: everywhere). ticket: this launch's number in the
// job-wide sequence of update launches, the value of the "slice written" flag.
__global__ void comm_update_kernel(CommPeers peers, int rank, int world, long lo, long n, const float* __restrict__ shard,
                                   float* __restrict__ m, float* __restrict__ v, GroupTable groups,
                                   float b1, float b2, float eps, float c1, float c2, float max_norm, unsigned int seq, int first,
                                   float* __restrict__ coef_buf, const unsigned int* __restrict__ fp32_map, unsigned int ticket,
                                   unsigned int* __restrict__ done_counter, int* __restrict__ err) {
  __shared__ float coef_s;
  __shared__ int go;
  if (threadIdx.x == 0) {
    if (first) {
      go = wait_all(peers.flags[rank] + 1 * MAX_RANKS, world, seq) ? 1 : 0;
      if (!go) atomicExch(err, 402);
      float total = 0.f;
      for (int p = 0; p < world; ++p) total += peers.norms[rank][p];
      const float norm = sqrtf(total);
      coef_s = (max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
      if (blockIdx.x == 0) { coef_buf[0] = norm; coef_buf[1] = coef_s; }
    } else {
      go = 1;
      coef_s = coef_buf[1];
    }
  }
  __syncthreads();
  if (go) {
    const float coef = coef_s;
    __nv_bfloat16* const lp_mine = peers.lp[rank];
    float* const params_mine = peers.params[rank];
    // optimizer groups are contiguous 64-aligned ranges of the flat buffers, so an 8-vector lies inside one group (and
    // inside one 64-element cell of the fp32 bitmap)
    for (long at = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; at < n; at += static_cast<long>(gridDim.x) * blockDim.x * 8) {
      const long e0 = lo + at;
      int seg = 0;
#pragma unroll
      for (int s2 = 1; s2 < MAX_GROUPS; ++s2) if (s2 < groups.count && e0 >= groups.start[s2]) seg = s2;
      const float wd = groups.wd[seg], lr = groups.lr[seg];
      if (lr == 0.f) continue;       // a group this optimizer does not own (matrix optimizer groups)
      float g[8], mm[8], vv[8], pp[8];
      *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(shard + at);
      *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(shard + at + 4);
      *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + at);
      *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + at + 4);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + at);
      *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + at + 4);
      *reinterpret_cast<float4*>(pp) = *reinterpret_cast<const float4*>(params_mine + e0);
      *reinterpret_cast<float4*>(pp + 4) = *reinterpret_cast<const float4*>(params_mine + e0 + 4);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float gr = g[e] * coef;
        mm[e] = b1 * mm[e] + (1.f - b1) * gr;
        vv[e] = b2 * vv[e] + (1.f - b2) * gr * gr;
        pp[e] = pp[e] * (1.f - lr * wd) - (lr / c1) * mm[e] / (sqrtf(vv[e] / c2) + eps);
      }
      *reinterpret_cast<float4*>(m + at) = *reinterpret_cast<float4*>(mm);
      *reinterpret_cast<float4*>(m + at + 4) = *reinterpret_cast<float4*>(mm + 4);
      *reinterpret_cast<float4*>(v + at) = *reinterpret_cast<float4*>(vv);
      *reinterpret_cast<float4*>(v + at + 4) = *reinterpret_cast<float4*>(vv + 4);
      const float4 p_lo = *reinterpret_cast<float4*>(pp), p_hi = *reinterpret_cast<float4*>(pp + 4);
      const bool everywhere = !fp32_map || ((fp32_map[e0 >> 11] >> ((e0 >> 6) & 31)) & 1u);
      if (!everywhere) {
        *reinterpret_cast<float4*>(params_mine + e0) = p_lo;
        *reinterpret_cast<float4*>(params_mine + e0 + 4) = p_hi;
      } else if (peers.mc_params) {
        mc_st(peers.mc_params + e0, p_lo);
        mc_st(peers.mc_params + e0 + 4, p_hi);
      } else {
        for (int q = 0; q < world; ++q) {
          float* dst = peers.params[(rank + q) % world] + e0;
          *reinterpret_cast<float4*>(dst) = p_lo;
          *reinterpret_cast<float4*>(dst + 4) = p_hi;
        }
      }
      if (lp_mine) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(pp[2 * e], pp[2 * e + 1]);
        const float4 bits = *reinterpret_cast<float4*>(h);      // eight bf16 values moved as 16 opaque bytes
        if (peers.mc_lp) {
          mc_st(reinterpret_cast<float*>(peers.mc_lp + e0), bits);
        } else {
          for (int q = 0; q < world; ++q) *reinterpret_cast<float4*>(peers.lp[(rank + q) % world] + e0) = bits;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int arrived = atomicAdd(done_counter, 1u);
    if (arrived == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 2 * MAX_RANKS + rank, ticket);
      *done_counter = 0u;
    }
  }
}

__global__ void comm_settle_kernel(CommPeers peers, int rank, int world, unsigned int ticket, int* __restrict__ err) {
  if (threadIdx.x == 0 && !wait_all(peers.flags[rank] + 2 * MAX_RANKS, world, ticket)) atomicExch(err, 403);
}

// Waits on one flag slot that nothing sets: exercises the bounded-wait path (status 404 after `limit_ns`).
__global__ void comm_wait_probe_kernel(const unsigned int* flag, unsigned int seq, unsigned long long limit_ns, int* __restrict__ err) {
  const unsigned long long t0 = timer_ns();
  while (static_cast<int>(ld_acquire_sys(flag) - seq) < 0) {
    if (timer_ns() - t0 > limit_ns) { atomicExch(err, 404); return; }
    __nanosleep(200);
  }
}

int comm_reduce(const void* peers, int rank, int world, long lo, long n, float* shard, unsigned int ticket, unsigned int publish_seq,
                float* block_acc, unsigned int* done_counter, int* err, int ctas, cudaStream_t st) {
  if (world > MAX_RANKS || n % 4 || lo % 4 || ctas < 1) return 1;
  comm_reduce_kernel<<<ctas, 512, 0, st>>>(*static_cast<const CommPeers*>(peers), rank, world, lo, n, shard, ticket, publish_seq, block_acc,
                                           done_counter, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int comm_update(const void* peers, int rank, int world, long lo, long n, const float* shard, float* m, float* v, int n_groups,
                const long* group_start, const float* group_wd, const float* group_lr, float b1, float b2, float eps, float c1, float c2,
                float max_norm, unsigned int seq, int first, float* coef_buf, const unsigned int* fp32_map, unsigned int ticket,
                unsigned int* done_counter, int* err, int ctas, cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || lo % 8 || n_groups > MAX_GROUPS || n_groups < 1 || ctas < 1) return 1;
  const CommPeers* p = static_cast<const CommPeers*>(peers);
  GroupTable g{};
  g.count = n_groups;
  for (int i = 0; i < n_groups; ++i) { g.start[i] = group_start[i]; g.wd[i] = group_wd[i]; g.lr[i] = group_lr[i]; }
  comm_update_kernel<<<ctas, 256, 0, st>>>(*p, rank, world, lo, n, shard, m, v, g, b1, b2, eps, c1, c2, max_norm, seq, first, coef_buf,
                                           fp32_map, ticket, done_counter, err);
  comm_settle_kernel<<<1, 32, 0, st>>>(*p, rank, world, ticket, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int comm_wait_probe(const unsigned int* flag, unsigned int seq, unsigned long long limit_ns, int* err, cudaStream_t st) {
  comm_wait_probe_kernel<<<1, 1, 0, st>>>(flag, seq, limit_ns, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
size_t comm_peers_bytes() { return sizeof(CommPeers); }

}  // namespace ghb
