// Allocation-free C entry point of the decode attention kernel.
//
// This entry point has no counterpart in the reference implementation. It exists for callers that are not allowed to
// allocate device memory at the point where they need attention over a static KV cache: code running inside a
// serving loop whose memory plan is frozen after start-up (every byte of the device is already assigned to weights
// and caches, so a cudaMalloc could fail or fragment the plan), plug-ins that are handed raw device pointers by a host
// runtime that owns the allocator, and latency-critical paths where an allocator call (which may synchronise the
// device) is forbidden. Such callers pass inputs and the output; the split-softmax scratch that the regular entry
// takes from the caller lives in a fixed array inside the library instead.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the library holds per device, in bytes (a file-scope device array; every GPU that loads the
// library keeps it until the process exits). A call needs B * Hq * splits * 66 floats and is refused beyond this.
#define GHB_NOALLOC_SCRATCH_BYTES (4u << 20)

// Single-token attention of q [B, Hq, 64] (fp32, normed, unrotated) over cached k, v [B, T, Hkv, 64] (bf16), rows
// limited by lens [B] (and doc_start [B] when not null), rotation tables cos_t / sin_t [n_angles, rot / 2], output
// out [B, Hq, 64] (bf16). Same arithmetic as the regular decode attention entry. `stream` is a cudaStream_t.
//
// Returns 0 on success. On failure returns a nonzero code and, when errbuf is not null, writes a message of at most
// errlen bytes: 1 = a size beyond the limits above, a null input / output pointer, a rotary width above 0 without angle
// tables (n_angles < 1 or a null table), or an unsupported head grouping / rotary width; 2 = the device
// address of the scratch array could not be obtained, 4 = the launch was refused by the runtime.
//
// The first call on each device resolves the device address of the scratch array (cudaGetSymbolAddress) with that
// device current; make that first call before any stream capture begins. No call allocates or frees memory.
// All calls on a device share the one scratch array and it keeps the previous call's contents: calls that may
// overlap on the GPU (different streams, no ordering) race on it, so order them. Nothing in it has to start at
// zero; every slot a call reads is written by that call first.
int ghb_decode_attention_noalloc(const float* q, const void* k, const void* v, const int* lens, const int* doc_start,
                                 const float* cos_t, const float* sin_t, void* out, int B, int T, int Hq, int Hkv, int rot,
                                 int cap, int n_angles, int splits, float scale, void* stream, char* errbuf, int errlen);

#ifdef __cplusplus
}
#endif
