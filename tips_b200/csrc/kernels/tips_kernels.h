/* extern "C" launchers of the sm_100a kernel library (libtips_kernels.so).
 *
 * Conventions: pointers are device pointers unless a parameter is named host_*;
 * dtype arguments use the tips Datatype codes (0 fp32, 1 fp64, 2 int32, 3 int64,
 * 4 int8, 5 uint8, 6 bf16, 7 fp16); `stream` is a cudaStream_t; the return value
 * is 0 on success and negative on failure, with the message available from
 * tipsk_last_error() on the calling thread.  None of the reference's code has a
 * GPU path (its AllreduceGpu is declared and never defined,
 * tips/core/collective/utils.h:136-137), so nothing here has a counterpart there.
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* tipsk_last_error(void);

/* ---- optimizers on flat slabs (elementwise.cu) ---- */
int tipsk_sgd_momentum_flat(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* momentum_buf,
                            int64_t n, float lr, float momentum, float dampening, float weight_decay, int nesterov,
                            float grad_scale, int first_step, void* stream);
int tipsk_adam_flat(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* exp_avg,
                    float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay,
                    int64_t step, float grad_scale, int decoupled, void* stream);
int tipsk_adam_flat_devstep(float* p32, void* p16, int p16_dtype, const void* grad, int grad_dtype, float* exp_avg,
                            float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps,
                            float weight_decay, int64_t step, const int64_t* step_dev, float grad_scale, int decoupled,
                            void* stream);
/* host arrays of device pointers / element offsets / element counts */
int tipsk_pack(const void* const* host_srcs, const int64_t* host_offsets, const int64_t* host_numels, int ntensors,
               int src_dtype, void* flat, int flat_dtype, float scale, int accumulate, void* stream);
int tipsk_unpack(const void* flat, int flat_dtype, void* const* host_dsts, const int64_t* host_offsets,
                 const int64_t* host_numels, int ntensors, int dst_dtype, float scale, void* stream);
/* Strided 4-D copy with contiguous rows (byte strides for the three outer axes; everything 16-byte aligned). */
int tipsk_copy4d(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t row_bytes,
                 const int64_t* src_strides, const int64_t* dst_strides, void* stream);
int tipsk_scale_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, float scale, void* stream);

/* ---- normalisation (norm.cu) ---- */
/* NHWC batch norm on [M, C] rows (M = N*H*W). Training forward: batch statistics
 * (written to save_mean / save_invstd, running stats updated when non-null), then
 * y = relu?(gamma * (x - mean) * invstd + beta + residual?). `workspace` holds
 * 2*C*partials floats (partials = tipsk_bn_partials(M, C)). */
int tipsk_bn_partials(int64_t m, int c);
int tipsk_bn_fwd_train(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                       float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                       float* workspace, int64_t m, int c, float eps, float momentum, int relu, int dtype, void* stream);
/* Same, with the column sums already known: stats = fp32 [2, C] (sums, sums of squares). */
int tipsk_bn_fwd_train_stats(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                             float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                             const float* stats, int64_t m, int c, float eps, float momentum, int relu, int dtype,
                             void* stream);
int tipsk_bn_fwd_eval(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                      const float* running_mean, const float* running_var, int64_t m, int c, float eps, int relu,
                      int dtype, void* stream);
/* Backward of the fused op; y is the forward output (needed for the ReLU mask).
 * dresidual may be null. dgamma/dbeta are fp32 [C]. */
int tipsk_bn_bwd(const void* dy, const void* x, const void* y, const float* gamma, const float* save_mean,
                 const float* save_invstd, void* dx, void* dresidual, float* dgamma, float* dbeta, float* workspace,
                 int64_t m, int c, int relu, int dtype, void* stream);
/* Forward that also writes one ReLU bit per element (uint8 [M*C/8]) and the backward that reads those bits instead
 * of the forward output; `stats` may be null (then `workspace` is used for the reduction). */
int tipsk_bn_fwd_train_mask(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                            float* workspace, const float* stats, void* relu_mask, int64_t m, int c, float eps,
                            float momentum, int relu, int dtype, void* stream);
int tipsk_bn_bwd_bitmask(const void* dy, const void* x, const void* relu_mask, const float* gamma,
                         const float* save_mean, const float* save_invstd, void* dx, void* dresidual, float* dgamma,
                         float* dbeta, float* workspace, int64_t m, int c, int dtype, void* stream);
/* BN + ReLU without residual: the mask is rebuilt from x and the saved statistics, the forward output is not read. */
int tipsk_bn_bwd_relu_recompute(const void* dy, const void* x, const float* gamma, const float* beta,
                                const float* save_mean, const float* save_invstd, void* dx, float* dgamma, float* dbeta,
                                float* workspace, int64_t m, int c, int dtype, void* stream);
/* Layer norm over the last dimension of [rows, cols]. */
int tipsk_ln_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int64_t rows,
                 int cols, float eps, int dtype, void* stream);
/* y = LN(x + residual); sum_out receives x + residual (what the backward pass differentiates through). */
int tipsk_ln_fwd_residual(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                          void* sum_out, float* mean, float* rstd, int64_t rows, int cols, float eps, int dtype,
                          void* stream);
int tipsk_ln_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                 float* dgamma_partial, float* dbeta_partial, int partial_rows, int64_t rows, int cols, int dtype,
                 void* stream);
int tipsk_ln_bwd_partials(int64_t rows, int cols);
int tipsk_ln_reduce_partials(const float* dgamma_partial, const float* dbeta_partial, int partial_rows, int cols,
                             void* dgamma, void* dbeta, int dtype, void* stream);

/* ---- pointwise epilogues and losses (epilogue.cu) ---- */
/* act: 0 none, 1 relu, 2 gelu (erf). y = act(x + bias[col]) on [rows, cols]. */
int tipsk_bias_act_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols, int act, int dtype,
                       void* stream);
/* dx = dy * act'(x + bias); dbias (fp32 [cols]) = column sums of dx, when non-null. */
int tipsk_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, float* dbias, int64_t rows, int cols,
                       int act, int dtype, void* stream);
/* Binary cross entropy with logits: loss_sum (fp32 scalar, accumulated) and dlogits = (sigmoid(z) - t) * scale. */
/* One-unit output layer fused with the sigmoid cross-entropy loss (forward keeps dz for the backward pass). */
int tipsk_dot_sigmoid_bce_fwd(const void* x, const void* w, const void* bias, const float* targets, float* loss_sum,
                              float* dz, float* logits, int64_t rows, int k, int64_t ldx, float scale, int dtype,
                              void* stream);
int tipsk_dot_sigmoid_bce_bwd(const void* x, const void* w, const float* dz, const float* dloss, void* dx, float* dw,
                              float* db, int64_t rows, int k, int64_t ldx, int dtype, void* stream);
/* Encoder input embedding: token row + position row + type row, and its backward (epilogue.cu). */
int tipsk_embed_sum_fwd(const int64_t* ids, const void* tok, const void* pos, const void* typ, void* x, int64_t tokens,
                        int seq, int hidden, int64_t vocab, int dtype, void* stream);
int tipsk_embed_sum_bwd(const int64_t* ids, const void* dx, void* dtok, void* dpos, void* dtyp, int64_t tokens, int seq,
                        int hidden, int64_t vocab, int dtype, void* stream);
int tipsk_sigmoid_bce(const void* logits, const float* targets, float* loss_sum, void* dlogits, int64_t n,
                      float grad_scale, int dtype, void* stream);
/* Softmax cross entropy over [rows, cols] with int64 labels (ignore_index skipped):
 * loss_sum / count accumulated into fp32 scalars, dlogits = (softmax - onehot) * scale. */
int tipsk_softmax_xent(const void* logits, const int64_t* labels, float* loss_sum, float* count, void* dlogits,
                       int64_t rows, int cols, int64_t ignore_index, float grad_scale, int dtype, void* stream);

/* ---- NVLink collectives (comm.cu, comm_executor.cu) ----
 * A "window" is a buffer of identical size on every rank, mapped into every process
 * (peer_windows[r] = address of rank r's window here; multicast_window = NVLS multicast
 * mapping or NULL).  Layout: [64 KiB signal flags][staging area][caller-managed space].
 * With `emulated` non-zero all windows live on the current device and one launch runs
 * every rank (cooperative launch); used to test the multi-rank algorithms on one GPU. */
int tipsk_comm_init(int rank, int nranks, void* const* peer_windows, void* multicast_window, uint64_t window_bytes,
                    uint64_t staging_bytes, int wait_budget_ms, int blocks, uint64_t one_shot_bytes, int use_multimem,
                    int emulated);
int tipsk_comm_shutdown(void);
int tipsk_comm_ready(void);
uint64_t tipsk_comm_staging_offset(void);
uint64_t tipsk_comm_launches(void);
void* tipsk_comm_stream(int channel);
int tipsk_comm_uses_multimem(void);
int tipsk_comm_set_budget_ms(int ms);
int tipsk_comm_status(int slot, int32_t* out7, int clear);
int tipsk_comm_reset(void);
int tipsk_allreduce(const void* const* host_srcs, void* const* host_dsts, int64_t win_off, uint64_t nbytes, int dtype,
                    int op, float prescale, float postscale, int channel, void* stream);
int tipsk_allgatherv(const void* const* host_srcs, void* const* host_dsts, const uint64_t* bytes_per_rank, int channel,
                     void* stream);
int tipsk_broadcast(const void* const* host_srcs, void* const* host_dsts, uint64_t nbytes, int root, int channel,
                    void* stream);
int tipsk_comm_wait_never(int channel, void* stream);
/* Device collectives of a sub-group of ranks (see comm.cu): the group owns kFlagBytes + stage_bytes bytes at `area_off`
 * of every rank's window. */
int tipsk_comm_group_create(int64_t id, const int32_t* members, int n, uint64_t area_off, uint64_t stage_bytes);
int tipsk_comm_group_destroy(int64_t id);
int tipsk_group_allreduce(int64_t id, const void* const* host_srcs, void* const* host_dsts, uint64_t nbytes, int dtype,
                          int op, float prescale, float postscale, void* stream);
int tipsk_group_allgatherv(int64_t id, const void* const* host_srcs, void* const* host_dsts,
                           const uint64_t* bytes_per_member, void* stream);
int tipsk_group_broadcast(int64_t id, const void* const* host_srcs, void* const* host_dsts, uint64_t nbytes, int root,
                          void* stream);
uint64_t tipsk_comm_flag_bytes(void);
int tipsk_comm_set_option(const char* name, uint64_t value);
/* Allreduce fused with the optimizer step on the share of the parameters each rank owns (see comm.cu). */
int tipsk_comm_update_subtile(void);
int64_t tipsk_comm_update_shard_vecs(uint64_t nbytes);
int tipsk_comm_attach_update(int64_t grad_off, uint64_t nbytes, int dtype, int64_t param_off, int kind,
                             void* const* host_master, void* const* host_s0, void* const* host_s1);
int tipsk_comm_detach_update(int64_t grad_off);
int tipsk_comm_update_attached(int64_t grad_off, uint64_t nbytes);
int tipsk_comm_set_update_hyper(int64_t grad_off, const float* h, int nh, int64_t step);
uint64_t tipsk_comm_update_launches(int64_t grad_off);
int tipsk_allreduce_update(int64_t grad_off, float scale, int channel, void* stream);
void* tipsk_event_create(void);
void tipsk_event_recycle(void* ev);
int tipsk_event_record(void* ev, void* stream);
int tipsk_stream_wait_event(void* stream, void* ev);
int tipsk_stream_synchronize(void* stream);
int tipsk_executor_configure(int device, void* my_window, uint64_t window_bytes);
void* tipsk_device_executor_ptr(void);

/* ---- parameter server (ps.cu) ---- */
int tipsk_comm_fence(int channel, void* stream);
int tipsk_table_init(float* shard, int64_t rows_local, int dim, int field, int rank, int nranks, int64_t rows_global,
                     uint64_t seed, float scale, void* stream);
/* Placement of row `id` of `field` under `nranks` ranks (ps_placement.h). */
int tipsk_ps_place(int field, int64_t id, int nranks, int32_t* host_owner, int64_t* host_local_row);
uint64_t tipsk_ps_acc_bytes(uint64_t slots, int dim);
uint64_t tipsk_ps_inbox_bytes(int nranks, uint64_t inbox_cap, int dim);
uint64_t tipsk_ps_ctl_bytes(void);
int tipsk_ps_configure(void* const* host_slabs, void* const* host_inboxes, void* const* host_accs,
                       void* const* host_ulists, void* const* host_ctls, void* const* host_item_slots,
                       void* const* host_caches, int nranks, int nlocal, const int32_t* host_servers, int nservers,
                       const uint64_t* host_field_off, const uint64_t* host_state_off,
                       const int64_t* host_rows_per_shard, int nfields, int dim, uint64_t slots, uint64_t inbox_cap,
                       uint64_t item_cap, uint64_t shadow_base);
int tipsk_ps_traffic(uint64_t* host_out3);
int tipsk_ps_wire_follows_grads(int follow);
int tipsk_ps_phase_timing(int enable);
int tipsk_ps_phase_ms(float* host_out5);
int tipsk_ps_pull_phase_ms(float* host_out4);
int tipsk_ps_status(int32_t* host_error, uint64_t* host_touched);
int tipsk_ps_pull(const int64_t* const* host_ids, void* const* host_outs, int64_t batch, int64_t out_ld,
                  int64_t out_col0, int out_dtype, int fence, int index, void* stream);
int tipsk_ps_push(const int64_t* const* host_ids, const void* const* host_grads, int64_t batch, int64_t grad_ld,
                  int64_t grad_col0, int grad_dtype, float grad_scale, int rule, float lr, float eps, int reuse_index,
                  void* stream);
/* Tables keyed by arbitrary 64-bit ids, rows created (zero) on first pull; see ps.cu. */
int tipsk_hash_pull(void* const* host_keys, void* const* host_rows, int nranks, uint64_t cap, int dim,
                    const int64_t* const* host_ids, void* const* host_outs, int nlocal, int64_t count, int64_t out_ld,
                    int out_dtype, int32_t* error_dev, void* stream);
int tipsk_hash_push(void* const* host_keys, void* const* host_rows, void* const* host_states, int nranks, uint64_t cap,
                    int dim, const int64_t* const* host_ids, const void* const* host_grads, int nlocal, int64_t count,
                    int64_t grad_ld, int grad_dtype, float grad_scale, int rule, float lr, float eps, int32_t* error_dev,
                    unsigned long long* missing_dev, void* stream);
/* Asynchronous push: gradients applied straight to the owner's rows with atomics, no fences (SGD / Adagrad). */
int tipsk_ps_push_async(const int64_t* const* host_ids, const void* const* host_grads, int64_t batch, int64_t grad_ld,
                  int64_t grad_col0, int grad_dtype, float grad_scale, int rule, float lr, float eps, void* stream);

/* ---- tcgen05 GEMM (gemm_tcgen05.cu) ---- */
int tipsk_gemm_supported(int m, int n, int k, int lda, int ldb);
int tipsk_gemm_bf16(const void* a, const void* b, void* c, const void* bias, void* pre, int m, int n, int k, int lda,
                    int ldb, int ldc, int act, void* stream);
/* C[m,n] = A[m,k] * B[k,n] with B row-major [k, n] (contraction over its rows), n >= 64. */
int tipsk_gemm_bf16_nn(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                       int accumulate, void* stream);
int tipsk_gemm_status(void);

/* ---- 3x3 / stride 2 / pad 1 max pooling on NHWC (pool.cu); idx holds the argmax position 0..8 per output ---- */
/* Global average pooling on NHWC (x [n, hw, c] -> y [n, c]) and its backward (pool.cu). */
int tipsk_global_avgpool_fwd(const void* x, void* y, int n, int hw, int c, int dtype, void* stream);
int tipsk_global_avgpool_bwd(const void* dy, void* dx, int n, int hw, int c, int dtype, void* stream);
int tipsk_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int n, int h, int w, int c, int dtype, void* stream);
int tipsk_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int n, int h, int w, int c, int dtype,
                           void* stream);

/* ---- NHWC bf16 convolutions on tcgen05 (conv_tcgen05.cu): 1x1 and 3x3, stride 1 or 2, pad = r/2 ---- */
int tipsk_conv2d_supported(int cin, int cout, int r, int s, int stride, int pad);
int tipsk_conv2d_fwd(const void* x, const void* wgt, void* y, int n, int h, int w, int cin, int cout, int r, int s,
                     int stride, int pad, float* stat_sum, float* stat_sq, void* stream);
int tipsk_conv2d_dgrad(const void* dy, const void* wgt_t, void* dx, int n, int h, int w, int cin, int cout, int r,
                       int s, int stride, int pad, int accumulate, void* stream);
/* The same from the forward weight layout wgt[cout, r, s, cin] (no transposed copy of the weights). */
int tipsk_conv2d_dgrad_ohwi(const void* dy, const void* wgt, void* dx, int n, int h, int w, int cin, int cout, int r,
                            int s, int stride, int pad, int accumulate, void* stream);
int tipsk_conv2d_wgrad(const void* x, const void* dy, float* dw, int n, int h, int w, int cin, int cout, int r, int s,
                       int stride, int pad, void* stream);
int tipsk_conv_status(void);
/* 7x7 / stride 2 / pad 3 stem on 3-channel bf16 images through a zero-padded 8-channel copy xp[n, hp, wp, 8];
 * weights [cout, 7, 8, 8] with the eighth horizontal tap and channels 3..7 zero. */
int tipsk_stem_geometry(int h, int w, int* hp, int* wp, int* ho, int* wo);
int tipsk_stem_pad(const void* x, void* xp, int n, int h, int w, void* stream);
/* The same from an fp32 NCHW image: layout change and cast to bf16 inside the padding copy. */
int tipsk_stem_pad_nchw_f32(const void* x, void* xp, int n, int h, int w, void* stream);
int tipsk_stem_conv_fwd(const void* xp, const void* wgt_p, void* y, int n, int h, int w, int cout, float* stat_sum,
                        float* stat_sq, void* stream);
int tipsk_stem_conv_wgrad(const void* xp, const void* dy, float* dw, int n, int h, int w, int cout, void* stream);

#ifdef __cplusplus
}
#endif
