// C entry points of the native library. Every function enqueues work on `stream` and returns 0 on
// success or a negative code when the arguments cannot be served (the Python layer raises). None
// of them synchronises. Pointers are device pointers unless stated otherwise. `status` (may be
// null) is a device int that a kernel sets to a non-zero fmb::ERR_* code when one of its bounded
// waits ran out.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dtype codes used across the API
#define FMB_BF16 0
#define FMB_F32 1
// ranks of one NVSwitch domain that the peer-memory kernels address
#define FMB_MAX_PEERS 8

// ---- GEMM (gemm_sm100.cu)
int fmb_gemm_bf16(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int a_mn, int b_mn,
                  long long lda, long long ldb, long long ldd, long long ldc, int d_f32, int c_f32, float alpha,
                  float beta, const float* alpha_ptr, int allow_split, int* status, int force_bn,
                  cudaStream_t stream);

// ---- normalisation / elementwise (elementwise.cu)
int fmb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int d, float eps, int dtype,
                    int w_dtype, cudaStream_t stream);
int fmb_add_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* xn, void* y, float* rstd,
                        long long rows, int d, float eps, int dtype, int w_dtype, cudaStream_t stream);
// dx = norm backward (+ dres when given); dw_partial is [nblocks, d] fp32 scratch, dw receives its column sum.
int fmb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw_partial, float* dw, int dw_accumulate, long long rows, int d, int dtype, int w_dtype,
                    int nblocks, cudaStream_t stream);
int fmb_rmsnorm_bwd_blocks(long long rows, int d);
// `row_limit` (device int, may be null): process only the first min(rows, *row_limit) rows
int fmb_swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int h, long long ld_in, int dtype,
                   const int* row_limit, cudaStream_t stream);
int fmb_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, long long rows, int h,
                   long long ld_in, int dtype, const int* row_limit, cudaStream_t stream);
// Half-split rotary embedding of the first n_rot_heads heads of each row of
// src[rows, n_heads_total * hd] into dst (dst may be src; otherwise the other heads are copied);
// position = row % T; sign = +1 forward, -1 backward.
int fmb_rope(const void* src, void* dst, const float* cos, const float* sin, long long rows, int T, int n_rot_heads,
             int heads_total, int hd, float sign, int dtype, const float* q32, int n_q32, cudaStream_t stream);
int fmb_qk_norm_rope_fwd(const void* x, const void* w, const float* cos, const float* sin, void* y, float* rstd,
                         long long rows, int T, int H, int hd, float eps, int dtype, int w_dtype, cudaStream_t stream);
int fmb_qk_norm_rope_bwd(const void* dy, const void* x, const void* w, const float* cos, const float* sin,
                         const float* rstd, void* dx, float* dw_partial, float* dw, long long rows, int T, int H, int hd,
                         int dtype, int w_dtype, int nblocks, cudaStream_t stream);
int fmb_softmax_fwd(const void* x, void* y, long long rows, int n, int dtype, cudaStream_t stream);
int fmb_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int n, int dtype, cudaStream_t stream);
int fmb_topk(const void* x, void* values, long long* indices, long long rows, int n, int k, int dtype,
             cudaStream_t stream);

// ---- losses (loss.cu)
// In place: logits[rows, V] (bf16) become dlogits = (softmax - onehot) * grad_scale; per-row loss
// (lse - logit[label], 0 for ignored rows) goes to row_loss.
int fmb_ce_fwd_bwd(void* logits, const long long* labels, float* row_loss, long long rows, int V, long long ld,
                   float grad_scale, const float* grad_scale_ptr, long long ignore_index, int write_grad,
                   cudaStream_t stream);
int fmb_kl_fwd_bwd(const void* student, const void* teacher, float* row_loss, void* grad, long long rows, int V,
                   float grad_scale, int dtype, int write_grad, cudaStream_t stream);
int fmb_sum_f32(const float* x, float* out, long long n, float scale, int accumulate, cudaStream_t stream);

// ---- router (moe.cu)
int fmb_router_blocks(long long rows);
int fmb_router_fwd(const void* logits, long long ld, int dtype, float* probs, float* weights, int* idx, float* lse,
                   float* psum_partial, int* counts, long long rows, int E, int k, int nblocks, cudaStream_t stream);
int fmb_router_bwd(const float* probs, const int* idx, const float* weights, const float* lse, const float* dweights,
                   const float* aux_grad, const float* zc, void* dlogits, long long ld, int dtype, long long rows, int E,
                   int k, cudaStream_t stream);
int fmb_moe_plan(const int* idx, int* chunk_counts, int* region, int* meta, int* slot_of_entry, int* token_of_slot,
                 long long entries, int E, int k, int align, int cap, int mode, cudaStream_t stream);
int fmb_moe_tile_groups(const int* region, int* tile_group, int n_tiles, int E, cudaStream_t stream);
int fmb_moe_combine_bwd(const void* dout, const void* ys, const int* slot_of_entry, const float* w, void* dys, float* dw,
                        long long entries, int k, int d, cudaStream_t stream);
int fmb_moe_gather(const void* x, const int* token_of_slot, void* out, long long slots, int d, cudaStream_t stream);
int fmb_moe_combine(const void* ys, const int* slot_of_entry, const float* w, void* out, long long tokens, int k,
                    int d, cudaStream_t stream);

// ---- optimizer (optim.cu)
// Flat AdamW over n fp32 elements. `ctl` points to {float clip_coef, int ok}; when ok == 0 the
// kernel leaves everything untouched. shadow (bf16, may be null) receives the updated weights.
int fmb_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow, long long n, float lr, float beta1,
                   float beta2, float eps, float wd, float bc1, float bc2, const float* ctl, cudaStream_t stream);
// sum of squares of n floats; `partial` must hold at least 1024 floats
int fmb_sqnorm_f32_scratch(const float* x, float* partial, float* out, long long n, int accumulate, cudaStream_t stream);
int fmb_scale_cast(const void* src, void* dst, long long n, float scale, int src_dtype, int dst_dtype,
                   cudaStream_t stream);
int fmb_ns_axpby(const void* x, const void* y, void* out, long long n, float a, float b, int dtype,
                 cudaStream_t stream);

// ---- attention (attention_sm100.cu)
int fmb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq, int Hkv,
                 int hd, long long q_stride_t, long long kv_stride_t, long long o_stride_t, float scale, int causal,
                 int* status, cudaStream_t stream);
int fmb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                 void* dq, void* dk, void* dv, float* delta, float* dq_acc, int B, int T, int Hq, int Hkv, int hd,
                 long long q_stride_t, long long kv_stride_t, long long o_stride_t, long long dq_stride_t,
                 long long dkv_stride_t, float scale, int causal, int delta_ready, int* status, cudaStream_t stream);

// grouped products (rows partitioned into expert regions): see the comment at the definition
int fmb_gemm_bf16_grouped(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int a_mn, int b_mn,
                          long long lda, long long ldb, long long ldd, long long ldc, int d_f32, int c_f32, float alpha,
                          float beta, int mode, int n_groups, const int* tile_group, const int* region,
                          long long group_stride_b, long long group_stride_d, int* status, cudaStream_t stream);

// bf16 product with a fused epilogue: epi 1 SwiGLU forward (B = stacked gate|up weight [2h, K], D = gate|up
// [M, 2h], aux_out = activation [M, h]); 2 SwiGLU backward (accumulator = d(act) [M, h], aux_in = gate|up,
// D = d(gate)|d(up) [M, 2h]); 3 also writes aux_out[row, col / seg] = sum over seg columns of D * aux_in.
int fmb_gemm_bf16_epi(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn, long long lda,
                      long long ldb, long long ldd, int d_f32, float alpha, int epi, int h, int seg,
                      const void* aux_in, long long ld_aux_in, void* aux_out, long long ld_aux_out, int* status,
                      cudaStream_t stream);

// ---- 8-bit GEMMs and their quantisers (gemm8_sm100.cu)
int fmb_gemm8(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
              int d_f32, int kind, const float* sa, const float* sb, int sa_ld, int sb_ld, int* status,
              cudaStream_t stream);
int fmb_quant_rows(const void* x, void* q, float* scale, long long rows, int cols, long long ldx, int dtype, int kind,
                   int block, cudaStream_t stream);
int fmb_quant_tiles_fp8(const void* x, void* q, float* scale, int rows, int cols, long long ldx, int dtype,
                        cudaStream_t stream);

// ---- expert parallelism over peer memory (moe_ep.cu); see the comment at the top of that file
int fmb_ep_collect_idx(const void* const* idx_ptrs, int* out, long long n, int world, int rank, int e_local,
                       const unsigned* flags, int slot, unsigned epoch, unsigned long long timeout_ns, int* status,
                       cudaStream_t stream);
// region [n, 3] = {start, used, padded} rows per expert, last row = first row past the live ones: cut to `rows`
// buffer rows in place; `code` goes to the status word when the plan needed more.
int fmb_ep_clamp_plan(int* region, int n, int rows, int* status, int code, cudaStream_t stream);
int fmb_ep_gather(const void* const* x_ptrs, const int* token_of_slot, const int* limit_ptr, void* out,
                  long long max_slots, int d, long long tokens_per_rank, int world, const unsigned* flags, int slot,
                  unsigned epoch, unsigned long long timeout_ns, int* status, cudaStream_t stream);
int fmb_ep_combine(const void* const* ys_ptrs, const void* const* slot_ptrs, const int* idx, const float* w, void* out,
                   long long tokens, int k, int d, int e_local, int rank, int world, const unsigned* flags, int slot,
                   unsigned epoch, unsigned long long timeout_ns, int* status, cudaStream_t stream);
int fmb_ep_combine_bwd(const void* const* dout_ptrs, const void* const* w_ptrs, const void* const* drw_ptrs,
                       const void* ys, const int* entry_of_slot, const int* limit_ptr, void* dys, long long max_slots,
                       long long n, int k, int d, int world, const unsigned* flags, int slot, unsigned epoch,
                       unsigned long long timeout_ns, int* status, cudaStream_t stream);

// ---- collectives over peer memory, fused with what follows them (comm.cu)
// `*_ptrs` are HOST arrays of `world` device pointers: the same symmetric buffer as mapped for each
// rank. Flags are uint32 epochs, FMB_MAX_PEERS per slot, zero before first use; `epoch` must grow by
// one per use of a slot on every rank. A wait that exceeds `timeout_ns` sets *status to ERR_WAIT_PEER.
int fmb_comm_rs_reduce(const void* const* grad_ptrs, long long lo, long long n, float scale, float* dst, float* partial,
                       int n_partial, const void* const* flag_ptrs, int slot, unsigned epoch, int rank, int world,
                       unsigned long long timeout_ns, int* status, cudaStream_t stream);
int fmb_comm_step_reduce(const float* partial, int n_partial, const float* extra_sq, const float* loss,
                         const void* const* xchg_ptrs, const void* const* flag_ptrs, int slot, unsigned epoch,
                         int rank, int world, float max_norm, int skip_nonfinite, float* stats, float* ctl,
                         unsigned long long timeout_ns, int* status, cudaStream_t stream);
int fmb_comm_adamw_push(float* master, const float* grad, float* m, float* v, const void* const* shadow_ptrs,
                        int world, const long long* off, const long long* soff, const int* len, const float* wd,
                        int n_chunks, float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                        const float* ctl, int grad_compact, cudaStream_t stream);
// fp32 master ranges (chunk table off/len on the device, len a multiple of 8) -> bf16 at the same offsets of every
// rank's working-weight buffer.
int fmb_comm_push_cast(const float* master, const void* const* shadow_ptrs, int world, const long long* off,
                       const int* len, int n_chunks, cudaStream_t stream);
int fmb_comm_adam_chunk(void);
// Debug build (-DFMB_DEBUG_BOUNDS): 1, and fmb_debug_register_extent() adds a buffer to the table that every checked
// peer access is validated against (outside it: access skipped, ERR_BOUNDS = 7 in *status). Normal build: 0 / no-op.
int fmb_debug_bounds_enabled(void);
int fmb_debug_register_extent(const void* base, unsigned long long bytes, int* status);
int fmb_comm_signal(const void* const* flag_ptrs, int slot, unsigned epoch, int rank, int world, cudaStream_t stream);
// Product whose operands / output are spread over the ranks (gemm_sm100.cu): see the comment at the definition.
int fmb_gemm_bf16_peer(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn, long long lda,
                       long long ldb, long long ldd, int d_f32, float alpha, int accumulate, int rank, int world,
                       int gather, const void* const* gather_ptrs, int* ready, void* const* d_ptrs,
                       const unsigned* flags, int slot, unsigned epoch, unsigned long long timeout_ns, int* status,
                       cudaStream_t stream);
// out[rows, cols] (bf16) = sum over the `world` slices of staging[world, rows, cols] (bf16) (+ residual)
int fmb_comm_sum_partials(const void* staging, const void* residual, void* out, long long rows, int cols, int world,
                          cudaStream_t stream);
int fmb_comm_barrier(const void* const* flag_ptrs, int slot, unsigned epoch, int rank, int world,
                     unsigned long long timeout_ns, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
