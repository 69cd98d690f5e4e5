// Data-parallel gradient reduce-scatter fused with the sharded AdamW update and the parameter all-gather, over
// NVLink peer memory (plain peer loads / stores, or NVSwitch multimem reductions and broadcasts when a multicast
// mapping of the buffers exists). Three launches per step on one stream:
//
//   reduce:  every rank signals "my gradients are final", waits (bounded) for all peers' signals, then sums the W
//            copies of ITS element range straight out of the peers' gradient buffers (or one multimem.ld_reduce per
//            vector), keeps the fp32 sum in a local shard buffer and publishes the shard's sum of squares to all peers;
//   update:  waits (bounded) for all W partial norms, forms the clip coefficient, applies AdamW to its range of the
//            fp32 master weights and writes the new fp32 and bf16 values into EVERY rank's parameter buffers
//            (peer stores or multimem.st), then signals "my range is written";
//   settle:  waits (bounded) until every peer's range has landed, so the next forward reads complete parameters.
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
__global__ void comm_reduce_kernel(CommPeers peers, int rank, int world, long lo, long n, float* __restrict__ shard, unsigned int seq,
                                   float* __restrict__ block_acc, unsigned int* __restrict__ done_counter, int* __restrict__ err) {
  __shared__ float red[32];
  __shared__ int go;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {   // gradients of this rank were completed by earlier work on this stream
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 0 * MAX_RANKS + rank, seq);
    }
    go = wait_all(peers.flags[rank] + 0 * MAX_RANKS, world, seq) ? 1 : 0;
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
    const unsigned int ticket = atomicAdd(done_counter, 1u);
    if (ticket == gridDim.x - 1) {   // last block: publish this rank's partial norm to every peer, then the flag
      const float total = atomicAdd(block_acc, 0.f);
      for (int p = 0; p < world; ++p) peers.norms[p][rank] = total;
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 1 * MAX_RANKS + rank, seq);
      *block_acc = 0.f;
      *done_counter = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------------------ update + gather
__global__ void comm_update_kernel(CommPeers peers, int rank, int world, long lo, long n, const float* __restrict__ shard,
                                   float* __restrict__ m, float* __restrict__ v, GroupTable groups,
                                   float b1, float b2, float eps, float c1, float c2, float max_norm, unsigned int seq,
                                   float* __restrict__ norm_out, unsigned int* __restrict__ done_counter, int* __restrict__ err) {
  __shared__ float coef_s;
  __shared__ int go;
  if (threadIdx.x == 0) {
    go = wait_all(peers.flags[rank] + 1 * MAX_RANKS, world, seq) ? 1 : 0;
    if (!go) atomicExch(err, 402);
    float total = 0.f;
    for (int p = 0; p < world; ++p) total += peers.norms[rank][p];
    const float norm = sqrtf(total);
    coef_s = (max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    if (blockIdx.x == 0) *norm_out = norm;
  }
  __syncthreads();
  if (go) {
    const float coef = coef_s;
    // optimizer groups are contiguous 64-aligned ranges of the flat buffers, so a 4-vector lies inside one group
    {
      for (long at = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; at < n; at += static_cast<long>(gridDim.x) * blockDim.x * 4) {
        int seg = 0;
#pragma unroll
        for (int s2 = 1; s2 < MAX_GROUPS; ++s2) if (s2 < groups.count && lo + at >= groups.start[s2]) seg = s2;
        const float wd = groups.wd[seg], lr = groups.lr[seg];
        if (lr == 0.f) continue;       // a group this optimizer does not own (matrix optimizer groups)
        const float4 g4 = *reinterpret_cast<const float4*>(shard + at);
        float4 m4 = *reinterpret_cast<float4*>(m + at), v4 = *reinterpret_cast<float4*>(v + at);
        float4 p4 = *reinterpret_cast<const float4*>(peers.params[rank] + lo + at);
        float* gp = const_cast<float*>(&g4.x); float* mp = &m4.x; float* vp = &v4.x; float* pp = &p4.x;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float gr = gp[e] * coef;
          mp[e] = b1 * mp[e] + (1.f - b1) * gr;
          vp[e] = b2 * vp[e] + (1.f - b2) * gr * gr;
          pp[e] = pp[e] * (1.f - lr * wd) - (lr / c1) * mp[e] / (sqrtf(vp[e] / c2) + eps);
        }
        *reinterpret_cast<float4*>(m + at) = m4;
        *reinterpret_cast<float4*>(v + at) = v4;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(p4.x, p4.y), h1 = __floats2bfloat162_rn(p4.z, p4.w);
        uint2 hp; hp.x = *reinterpret_cast<uint32_t*>(&h0); hp.y = *reinterpret_cast<uint32_t*>(&h1);
        if (peers.mc_params) {
          mc_st(peers.mc_params + lo + at, p4);
        } else {
          for (int q = 0; q < world; ++q) *reinterpret_cast<float4*>(peers.params[(rank + q) % world] + lo + at) = p4;
        }
        if (peers.lp[rank]) {
          for (int q = 0; q < world; ++q) *reinterpret_cast<uint2*>(peers.lp[(rank + q) % world] + lo + at) = hp;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int ticket = atomicAdd(done_counter, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence_system();
      for (int p = 0; p < world; ++p) st_release_sys(peers.flags[p] + 2 * MAX_RANKS + rank, seq);
      *done_counter = 0u;
    }
  }
}

__global__ void comm_settle_kernel(CommPeers peers, int rank, int world, unsigned int seq, int* __restrict__ err) {
  if (threadIdx.x == 0 && !wait_all(peers.flags[rank] + 2 * MAX_RANKS, world, seq)) atomicExch(err, 403);
}

// Waits on one flag slot that nothing sets: exercises the bounded-wait path (status 404 after `limit_ns`).
__global__ void comm_wait_probe_kernel(const unsigned int* flag, unsigned int seq, unsigned long long limit_ns, int* __restrict__ err) {
  const unsigned long long t0 = timer_ns();
  while (static_cast<int>(ld_acquire_sys(flag) - seq) < 0) {
    if (timer_ns() - t0 > limit_ns) { atomicExch(err, 404); return; }
    __nanosleep(200);
  }
}

int comm_reduce(const void* peers, int rank, int world, long lo, long n, float* shard, unsigned int seq, float* block_acc,
                unsigned int* done_counter, int* err, int sms, cudaStream_t st) {
  if (world > MAX_RANKS || n % 4 || lo % 4) return 1;
  comm_reduce_kernel<<<sms * 2, 512, 0, st>>>(*static_cast<const CommPeers*>(peers), rank, world, lo, n, shard, seq, block_acc, done_counter, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int comm_update(const void* peers, int rank, int world, long lo, long n, const float* shard, float* m, float* v, int n_groups,
                const long* group_start, const float* group_wd, const float* group_lr, float b1, float b2, float eps, float c1, float c2,
                float max_norm, unsigned int seq, float* norm_out, unsigned int* done_counter, int* err, int sms, cudaStream_t st) {
  if (world > MAX_RANKS || n % 4 || lo % 4 || n_groups > MAX_GROUPS || n_groups < 1) return 1;
  const CommPeers* p = static_cast<const CommPeers*>(peers);
  GroupTable g{};
  g.count = n_groups;
  for (int i = 0; i < n_groups; ++i) { g.start[i] = group_start[i]; g.wd[i] = group_wd[i]; g.lr[i] = group_lr[i]; }
  comm_update_kernel<<<sms * 2, 256, 0, st>>>(*p, rank, world, lo, n, shard, m, v, g, b1, b2, eps, c1, c2, max_norm, seq, norm_out,
                                              done_counter, err);
  comm_settle_kernel<<<1, 32, 0, st>>>(*p, rank, world, seq, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
int comm_wait_probe(const unsigned int* flag, unsigned int seq, unsigned long long limit_ns, int* err, cudaStream_t st) {
  comm_wait_probe_kernel<<<1, 1, 0, st>>>(flag, seq, limit_ns, err);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
size_t comm_peers_bytes() { return sizeof(CommPeers); }

}  // namespace ghb
