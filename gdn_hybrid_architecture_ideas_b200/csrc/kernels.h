// Host-callable launchers of the sm_100a kernels (raw pointers + stream; no framework types), and the TMA descriptor
// helper shared by the kernels that use tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ghb {

// Encodes a 2-D tiled tensor map through the driver entry point resolved at run time (no link dependency on libcuda).
// dims/box: innermost first; strides: bytes of dimension 1. Returns false if the driver refuses the descriptor.
bool encode_tensor_map_2d(CUtensorMap* map, const void* ptr, int elem_bytes, const uint64_t dims[2], const uint64_t strides[1],
                          const uint32_t box[2], bool swizzle128);

int last_encode_error();
bool encode_tensor_map_3d(CUtensorMap* map, const void* ptr, int elem_bytes, const uint64_t dims[3], const uint64_t strides[2],
                          const uint32_t box[3], bool swizzle128);

int gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc, bool a_mn, bool b_mn,
              int out, int* err, int sms, cudaStream_t stream);

int rmsnorm_fwd(const void* x, int in_bf16, const float* w, int w_scalar, const void* z, int gate, const float* resid, void* y,
                int out_bf16, float* rstd, long rows, int d, float eps, float scale, cudaStream_t st);
int rmsnorm_bwd(const void* dy, int dy_bf16, const void* x, int x_bf16, const float* w, int w_scalar, const void* z, int gate,
                const float* rstd, const float* dres, void* dx, void* dz, float* dw, long rows, int d, float scale, int sms, cudaStream_t st);
int silu_mul_fwd(const void* g, const void* u, long ld, void* h, long rows, int f, int sms, cudaStream_t st);
int silu_mul_bwd(const void* dh, const void* g, const void* u, long ld, void* dg, void* du, long rows, int f, int sms, cudaStream_t st);
int adamw(float* p, const float* g, float* m, float* v, void* lp, long n, float lr, float b1, float b2, float eps, float wd, float c1,
          float c2, const float* grad_scale, float scale_host, int sms, cudaStream_t st);
int sumsq_partials(const float* x, long n, float* partial, int blocks, cudaStream_t st);
int cast_bf16(const float* x, void* y, long n, int sms, cudaStream_t st);

int gdn_prep_fwd(const void* u, const int* doc, const float* w, void* out, long rows, int L, int C, int nq, float qscale, cudaStream_t st);
int gdn_prep_bwd(const void* u, const int* doc, const float* w, const void* dout, void* du, float* dw, long rows, int L, int C,
                 int nq, float qscale, cudaStream_t st);
int depth_mix_multi_fwd(const float* const* src, int n, float* const* out, int Q, const float* ueff, float* alpha, float* rnorm, float* vu, long rows,
                        int d, float eps, cudaStream_t st);
int depth_mix_multi_bwd(const float* const* src, float* const* dsrc, int n, const float* const* dh, int Q, const float* ueff, const float* alpha,
                        const float* rnorm, const float* vu, float* du, long rows, int d, int sms, cudaStream_t st);
int depth_mix_fwd(const float* const* src, int n, const float* ueff, float* out, float* alpha, float* rnorm, long rows, int d, float eps,
                  cudaStream_t st);
int depth_mix_bwd(const float* const* src, float* const* dsrc, int n, const float* ueff, const float* dh, const float* alpha,
                  const float* rnorm, float* du, long rows, int d, int sms, cudaStream_t st);
int gdn_step(float* S, const float* q, const float* k, const float* v, const float* g, const float* beta, const unsigned char* start, float* o,
             int B, int Hk, int Hv, int dk, int dv, cudaStream_t st);
int mx_fake(const void* x, bool x_bf16, void* out, long rows, long n, bool along_rows, int sms, cudaStream_t st);
// MXFP8 on the tensor cores (csrc/gemm_mx.cu): quantiser to E4M3 + E8M0 scale cells (either or both block orientations
// in one read) and the block-scaled GEMM D = A B^T over K-major E4M3 operands. out: 0 bf16, 1 fp32, 2 fp32 accumulate.
long mx_scale_bytes(long rows, long k);
int mx_quantize(const void* x, bool x_bf16, long R, long C, long ld, void* q_row, void* sf_row, void* q_col, void* sf_col, int sms,
                cudaStream_t st);
int gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long ldc, int out, int* err,
               int sms, cudaStream_t stream);
int embedding_fwd(const long* ids, const float* table, float* out, long n, int s, int d, int sms, cudaStream_t st);
int embedding_bwd(const long* ids, const float* g, float* table_grad, long n, int s, int d, int sms, cudaStream_t st);
int ce_grad(const float* logits, const long* targets, const float* a, const float* b, void* grad, float* ce, float* lse, long rows, int V,
            int s, bool fixed, cudaStream_t st);

int dual_lerp_fwd(const void* x, const void* ya, const void* yb, const float* la, const float* lb, void* oa, void* ob, long n, int sms, cudaStream_t st);
int dual_lerp_bwd(const void* ga, const void* gb, const void* x, const void* ya, const void* yb, const float* la, const float* lb, void* dx, void* dya,
                  void* dyb, float* dl, long n, int sms, cudaStream_t st);

int attn_prep_fwd(const void* q, long q_ts, int q_hs, const void* k, long k_ts, const float* wq, const float* wk, const float* cos, const float* sin,
                  const float* cos_c, const float* sin_c, int Hq, int Hkv, int R2, float eps, long tokens, void* qr, void* qf, void* kr, void* kf,
                  int sms, cudaStream_t st);
int attn_prep_bwd(const void* q, long q_ts, int q_hs, const void* k, long k_ts, const float* wq, const float* wk, const float* cos, const float* sin,
                  const float* cos_c, const float* sin_c, int Hq, int Hkv, int R2, float eps, long tokens, const void* dqr, const void* dqf,
                  const void* dkr, const void* dkf, void* dqraw, void* dkraw, float* dw, int sms, cudaStream_t st);

int gate_out_fwd(const void* o, const void* qg, void* y, long units, int sms, cudaStream_t st);
int gate_out_bwd(const void* dy, const void* o, const void* qg, void* dO, void* dqg, long units, int sms, cudaStream_t st);

int attention_fwd(const void* q, const void* qf, const void* k, const void* kf, const void* v, void* o, float* lse, const int* doc,
                  const int* pos, int B, int L, int Hq, int Hkv, int cap, float scale, int* err, cudaStream_t st);
int attention_bwd(const void* q, const void* qf, const void* k, const void* kf, const void* v, const void* o, const void* dO,
                  const float* lse, float* dsum, float* dq, float* dqf, void* dk, void* dkf, void* dv, const int* pos, int B, int L, int Hq,
                  int Hkv, int cap, float scale, int* err, cudaStream_t st);

int gdn_scan_fwd(const void* W, const void* Qin, const void* Kout, const void* Aqk, const void* U, const float* carry, const float* S0,
                 void* O, float* Sfinal, void* Hsave, void* Vnew, int B, int H, int L, int dv, int* err, cudaStream_t st);
int gdn_scan_bwd(const void* W, const void* Qin, const void* Kout, const void* Aqk, const void* Hsave, const void* Vnew, const void* dO,
                 const float* carry, const float* dSfinal, void* dU, float* dWp, float* dQp, float* dKp, float* dcarry, float* dS0, int B, int H,
                 int L, int dv, int* err, cudaStream_t st);

int gdn_local_fwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, void* U, void* W, void* Aqk, void* Qin, void* Kout,
                  float* carry, cudaStream_t st);
int gdn_local_bwd(const void* q, const void* k, const void* v, long q_tok, long k_tok, long v_tok, const float* g, const float* beta,
                  const unsigned char* start, int B, int L, int Hv, int Hk, int dv, const void* U, const void* W, const void* dU,
                  const float* dWp, const float* dQp, const float* dKp, int n_part, const void* dO, const void* Vnew, const float* dcarry,
                  float* dq, float* dk, void* dq16, void* dk16, long qk_tok, void* dvv, long dv_tok, float* dg, float* dbeta, cudaStream_t st);

int decode_attention(const float* q, const void* k, const void* v, const int* lens, const int* doc_start, const float* cos_t, const float* sin_t,
                     void* out, float* part_o, float* part_ml, int B, int T, int Hq, int Hkv, int rot, int cap, int n_angles, int splits,
                     float scale, cudaStream_t st);

// The same over the raw components of a 4 x 4 grid-shared cache (k, v [B, T, 256]; 16 query heads); gain: key-norm gain or null.
int decode_attention_grid(const float* q, const void* k, const void* v, const int* lens, const int* doc_start, const float* cos_t,
                          const float* sin_t, const float* gain, void* out, float* part_o, float* part_ml, int B, int T, int rot, int cap,
                          int n_angles, int splits, float scale, float eps, cudaStream_t st);

// Fused data-parallel step over peer memory (csrc/comm.cu). `peers` points at a host copy of the CommPeers table
// (comm_peers_bytes() bytes: 5 arrays of 8 device pointers, then 3 multicast pointers).
size_t comm_peers_bytes();
// `ctas`: grid size (a few CTAs for a launch that overlaps the backward, every SM for one that is exposed).
int comm_reduce(const void* peers, int rank, int world, long lo, long n, float* shard, unsigned int ticket, unsigned int publish_seq,
                float* block_acc, unsigned int* done_counter, int* err, int ctas, cudaStream_t st);
int comm_update(const void* peers, int rank, int world, long lo, long n, const float* shard, float* m, float* v, int n_groups,
                const long* group_start, const float* group_wd, const float* group_lr, float b1, float b2, float eps, float c1, float c2,
                float max_norm, unsigned int seq, int first, float* coef_buf, const unsigned int* fp32_map, unsigned int ticket,
                unsigned int* done_counter, int* err, int ctas, cudaStream_t st);
int comm_wait_probe(const unsigned int* flag, unsigned int seq, unsigned long long limit_ns, int* err, cudaStream_t st);

// Tensor-parallel GEMMs fused with the sequence-parallel all-gather / reduce-scatter (csrc/gemm_tp.cu). `args` points at a
// host copy of the kernel's argument table (tp_args_bytes() bytes; layout in parallel/tensor_parallel.py).
size_t tp_args_bytes();
int tp_pad_words();
int gemm_tp(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc, bool a_mn, bool b_mn, int out,
            const void* args, int* err, int sms, cudaStream_t st);
int tp_signal(const void* args, int word, int wait_word, int* err, cudaStream_t st);
int tp_reduce(const void* args, int N, int* err, int sms, cudaStream_t st);
int tp_copy_flagged(void* dst, const void* src, size_t bytes, void* flag_dst, const void* flag_src, cudaStream_t st);
int tp_push_copies(const void* args, const void* seq_src, int pieces, const cudaStream_t* streams, int n_streams);

}  // namespace ghb
