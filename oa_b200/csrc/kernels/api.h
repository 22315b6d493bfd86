// C ABI of the sm_100a kernel library (liboa_kernels.so).
//
// Every entry point takes raw device pointers and a CUDA stream (as void*), launches
// asynchronously on that stream and returns an OA_* code (0 = launched).  Nothing in
// this library allocates device memory: callers hand in outputs and scratch buffers.
// dtype codes follow the reference's OaScalarType values that appear in checkpoint
// files (Source/Public/Oa/Core/Type.gen.h:17-65): 0 = fp32, 1 = bf16.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { OA_OK = 0, OA_ERR_ARG = 1, OA_ERR_ALIGN = 2, OA_ERR_DRIVER = 3, OA_ERR_LAUNCH = 4, OA_ERR_UNSUPPORTED = 5,
       OA_ERR_TOO_LARGE = 6 };
enum { OA_F32 = 0, OA_BF16 = 1 };
enum { OA_ACT_NONE = 0, OA_ACT_GELU = 1, OA_ACT_RELU = 2, OA_ACT_SILU = 3, OA_ACT_GELU_BWD = 4, OA_ACT_RELU_BWD = 5 };

// unary ops: y = f(x; s0, s1)
enum { OA_U_COPY = 0, OA_U_NEG, OA_U_ABS, OA_U_LOG, OA_U_EXP, OA_U_SQRT, OA_U_SIN, OA_U_COS, OA_U_RECIP, OA_U_SCALE,
       OA_U_ADD_SCALAR, OA_U_POW, OA_U_CLAMP_MAX, OA_U_CLAMP_MIN, OA_U_RELU, OA_U_GELU, OA_U_SILU, OA_U_TANH,
       OA_U_SIGMOID, OA_U_SOFTPLUS, OA_U_LEAKY_RELU, OA_U_ELU, OA_U_MISH, OA_U_SQUARE, OA_U_RSUB_SCALAR,
       OA_U_SIGN, OA_U_COUNT };
// binary ops: y = f(a, b).  The *_BWD ops take a = saved forward input (or output, see elementwise.cu), b = upstream grad.
enum { OA_B_ADD = 0, OA_B_SUB, OA_B_MUL, OA_B_DIV, OA_B_MAX, OA_B_MIN, OA_B_EQ, OA_B_GE, OA_B_RELU_BWD, OA_B_GELU_BWD,
       OA_B_SILU_BWD, OA_B_TANH_BWD, OA_B_SIGMOID_BWD, OA_B_SOFTPLUS_BWD, OA_B_LEAKY_RELU_BWD, OA_B_ELU_BWD,
       OA_B_MISH_BWD, OA_B_ABS_BWD, OA_B_LOG_BWD, OA_B_SQRT_BWD, OA_B_RECIP_BWD, OA_B_SILU_MUL, OA_B_COUNT };
// broadcast modes of the second operand of a binary op
enum { OA_BC_NONE = 0, OA_BC_ROW = 1 /* b is [inner] repeated over rows */, OA_BC_COL = 2 /* b is [rows], one per row of `inner` */,
       OA_BC_SCALAR = 3 };
// row reductions
enum { OA_R_SUM = 0, OA_R_MEAN = 1, OA_R_MAX = 2, OA_R_ARGMAX = 3 };

// ---- GEMM (gemm_tcgen05.cu, gemm_f32.cu)
int oa_gemm_plan_splits(int M, int N, int K, int bn, int sms);
size_t oa_gemm_workspace_bytes(int M, int N, int K);
int oa_gemm_bf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                 int b_mn, const void* bias, const void* residual, int ldr, void* aux_out, const void* aux_in,
                 int ldaux, int act, int out_f32, int accumulate, float alpha, void* workspace,
                 size_t workspace_bytes, int force_bn, int* status, void* stream);
// `batch` independent problems of one shape; s*_batch are element strides between problems (sbias_batch may be 0).
int oa_gemm_bf16_batched(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                         int b_mn, const void* bias, const void* residual, int ldr, void* aux_out, const void* aux_in,
                         int ldaux, int act, int out_f32, int accumulate, float alpha, void* workspace,
                         size_t workspace_bytes, int force_bn, int batch, long long sa_batch, long long sb_batch,
                         long long sc_batch, long long sr_batch, long long saux_batch, long long sbias_batch, int* status,
                         void* stream);
// Grouped (mixture-of-experts) GEMMs; group segments are padded to multiples of 128 rows, `offsets` (int[groups+1]) is on the device.
//   mode 1: out[r,:] = act(A[r,:] * B[g(r)]^T + bias[g(r)]);   mode 2: out[g] = A_g^T * B_g (+ out[g])
int oa_gemm_bf16_grouped(int mode, const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc,
                         int b_mn, const void* bias, int act, void* aux_out, const void* aux_in, int ldaux, int out_f32,
                         int accumulate, int groups, const int* offsets, long long max_rows, long long sb_batch,
                         long long sc_batch, long long sbias_batch, int* status, void* stream);
// fp32 SIMT GEMM with arbitrary element strides and a batch dimension:
//   C[b][m,n] = act(alpha * sum_k A[b][m*sam + k*sak] * B[b][n*sbn + k*sbk] + bias[n]) (+ C if accumulate)
// Tensor-parallel GEMM fused with its collective over peer memory: mode 1 all-gather(rows of A) -> GEMM, mode 2 GEMM ->
// reduce-scatter(rows of out).  bufs / flags: host arrays of `world` device pointers; sync2: device u64[2] of the call site.
int oa_gemm_bf16_tp(int mode, const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc,
                    int b_mn, const void* residual, int ldr, int out_f32, float alpha, const void* src, int ld_src,
                    const void* const* bufs, const void* const* flags, void* sync2, int world, int rank,
                    int comm_ctas, int* status, void* stream);
int oa_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, long long sam, long long sak,
                long long sbn, long long sbk, int ldc, int batch, long long batch_a, long long batch_b,
                long long batch_c, const float* bias, int act, int accumulate, float alpha, void* stream);

// ---- elementwise (elementwise.cu)
int oa_unary(int op, int dtype, const void* x, void* y, long long n, float s0, float s1, void* stream);
int oa_binary(int op, int dtype, const void* a, const void* b, void* y, long long n, long long inner_b, int bcast_mode,
              void* stream);
int oa_cast(int src_dtype, int dst_dtype, const void* x, void* y, long long n, void* stream);
// parts: bf16[terms][n], successive roundings of x (x ~ sum of the parts); terms 1..3
int oa_split_bf16(const float* x, void* parts, long long n, int terms, void* stream);
int oa_fill(int dtype, void* y, long long n, float value, void* stream);
int oa_swiglu_fwd(int dtype, const void* gate_up, void* out, long long rows, int F, void* stream);
int oa_swiglu_bwd(int dtype, const void* gate_up, const void* dout, void* dgate_up, long long rows, int F, void* stream);
int oa_rope(int dtype, void* x, long long rows, int row_stride, int n_heads, int head_dim, int seq_len, int pos_offset,
            float theta, int backward, const int* pos_dev, void* stream);
int oa_embedding_fwd(int dtype, const void* table, const int* ids, void* out, long long n_ids, int dim, int vocab,
                     const void* pos_table, int seq_len, void* stream);
int oa_embedding_bwd(int dtype, const void* dout, const int* ids, float* dtable_f32, long long n_ids, int dim,
                     int vocab, void* stream);
int oa_col_sum(int dtype, const void* x, void* out, int out_dtype, long long rows, int cols, float* scratch,
               int accumulate, void* stream);
int oa_bias_add(int dtype, void* x, const void* bias, long long rows, int cols, void* stream);
int oa_row_reduce(int op, int dtype, const void* x, void* y, long long rows, int cols, void* stream);
int oa_softmax(int dtype, const void* x, void* y, long long rows, int cols, int log_mode, float scale,
               const void* mask, long long mask_rows, void* stream);
int oa_softmax_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int cols, int log_mode,
                   float scale, void* stream);
// `state` (may be null): device u64[2] = {seed, base offset}; when given, the seed comes from it and `offset` is relative to
// its base, so a captured launch draws fresh counters on every replay once oa_philox_state_advance closes the step.
int oa_philox(int dtype, void* y, long long n, unsigned long long seed, unsigned long long offset, int normal,
              float a, float b, const unsigned long long* state, void* stream);
int oa_dropout(int dtype, const void* x, void* y, long long n, float p, unsigned long long seed,
               unsigned long long offset, const unsigned long long* state, void* stream);
int oa_philox_state_advance(unsigned long long* state, unsigned long long delta, void* stream);
int oa_copy_strided(int dtype, const void* x, void* y, int rank, const long long* shape, const long long* src_strides,
                    void* stream);

// ---- norms (norm.cu)
size_t oa_norm_bwd_scratch_bytes(long long rows, int cols);
int oa_rmsnorm_fwd(int dtype, const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                   const void* residual_in, void* residual_out, void* stream);
int oa_rmsnorm_bwd(int dtype, const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw,
                   int dw_dtype, long long rows, int cols, const void* dres, float* scratch, int accumulate_dw,
                   void* stream);
int oa_layernorm_fwd(int dtype, const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                     long long rows, int cols, float eps, void* stream);
int oa_layernorm_bwd(int dtype, const void* x, const void* w, const void* dy, const float* mean, const float* rstd,
                     void* dx, void* dw, void* db, int dw_dtype, long long rows, int cols, float* scratch,
                     int accumulate_dw, void* stream);

// ---- loss (xent.cu)
int oa_xent_fwd_bwd(int dtype, const void* logits, const int* targets, float* row_loss, void* dlogits, long long rows,
                    int vocab, int ld, float grad_scale, int ignore_index, void* stream);
int oa_vp_xent_stats(int dtype, const void* logits, const int* targets, float* stats, long long rows, int vocab, int v0,
                     void* stream);
int oa_vp_xent_finish(int dtype, void* logits, const int* targets, const float* all_stats, float* row_loss, long long rows,
                      int vocab, int v0, int world, float scale, int want_grad, void* stream);
int oa_mean_f32(const float* x, float* out, long long n, float scale, void* stream);

// ---- optimizers (optim.cu)
// state = device float[8] {step, lr, beta1, beta2, eps, weight_decay, grad_scale, unused}; the step lives on the
// device so that a captured graph can be replayed (same idea as Source/Public/Oa/Ml/FnOptim.h:25-53).
int oa_optim_advance(float* state, void* stream);
int oa_adamw(int param_dtype, int grad_dtype, void* param, const void* grad, float* master, float* m, float* v,
             long long n, const float* state, int decoupled, const float* inv_clip, void* stream);
int oa_sgd(int param_dtype, int grad_dtype, void* param, const void* grad, float* master, float* mom, long long n,
           float lr, float momentum, float weight_decay, void* stream);
int oa_sumsq(int dtype, const void* x, long long n, float* partial, float* out, int accumulate, void* stream);
int oa_clip_coef(const float* sumsq, float max_norm, float* coef, void* stream);
int oa_scale_inplace(int dtype, void* x, long long n, const float* coef, void* stream);

// ---- attention (flash_attn.cu)
size_t oa_flash_bwd_scratch_bytes(int batch, int heads, int seq, int head_dim);
int oa_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads, int seq,
                 int head_dim, long long q_row_stride, long long kv_row_stride, long long o_row_stride, float scale,
                 int causal, int* status, void* stream);
int oa_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                 void* dq, void* dk, void* dv, int batch, int heads, int seq, int head_dim, long long q_row_stride,
                 long long kv_row_stride, long long o_row_stride, long long dq_row_stride, long long dkv_row_stride,
                 float scale, int causal, float* scratch, int* status, void* stream);
int oa_attn_f32(const float* q, const float* k, const float* v, float* o, float* lse, int batch, int heads, int seq,
                int head_dim, long long row_stride, long long o_row_stride, float scale, int causal, void* stream);
int oa_attn_f32_bwd(const float* q, const float* k, const float* v, const float* o, const float* dout,
                    const float* lse, float* dq, float* dk, float* dv, int batch, int heads, int seq, int head_dim,
                    long long row_stride, long long o_row_stride, long long d_row_stride, float scale, int causal,
                    void* stream);


// ---- recurrent scans (rnn.cu): gates = 3 (GRU: reset | update | candidate) or 1 (tanh RNN)
int oa_rnn_scan_fwd(int dtype, int gates, const void* gates_i, const void* w_hh, const void* b_hh, const void* h0, void* out,
                    void* hprev, int batch, int seq, int H, void* stream);
int oa_rnn_scan_bwd(int dtype, int gates, const void* gates_i, const void* w_hh, const void* b_hh, const void* hprev,
                    const void* dout, void* dgi, void* dgh, void* dh0, int batch, int seq, int H, void* stream);

// ---- mixture of experts (moe.cu)
int oa_moe_router(int dtype, const void* logits, const float* sel_bias, float* probs, int* topk_idx, float* topk_w,
                  long long tokens, int E, int K, void* stream);
int oa_moe_router_bwd(int dtype, const float* probs, const int* topk_idx, const float* topk_w, const float* dw,
                      const float* dprobs_col, float dprobs_scale, void* dlogits, long long tokens, int E, int K, void* stream);
size_t oa_moe_plan_scratch_bytes(long long routes, int E);
int oa_moe_plan(const int* topk_idx, long long tokens, int K, int E, int* counts, int* offsets, int* packed_token, int* inverse,
                long long max_rows, int* scratch, void* stream);
int oa_moe_gather(const void* x, const int* packed_token, void* packed, const int* offsets, int E, int dim, long long max_rows,
                  void* stream);
int oa_moe_combine(const void* packed, const float* gate, const int* inverse, const void* base, void* out, long long tokens,
                   int K, int dim, void* stream);
int oa_moe_combine_bwd(const void* packed, const float* gate, const int* inverse, const int* packed_token, const void* dout,
                       void* dpacked, float* dgate, const int* offsets, int E, int K, int dim, long long max_rows, void* stream);
int oa_moe_gather_bwd(const void* dpacked, const int* inverse, const void* base, void* dx, long long tokens, int K, int dim,
                      void* stream);

// expert parallelism over peer memory (moe.cu): layout from the exchanged counts, dispatch (push), combine (pull)
int oa_ep_layout(const int* counts_all, const int* topk_idx, const int* inverse, const int* offsets_local, int* route_rank,
                 int* route_row, int* loc_offsets, int* loc_counts, int* counts_global, int* need, long long routes, int E,
                 int world, int rank, void* stream);
int oa_ep_push_rows(const void* x, const void* const* dst_peers, const int* route_rank, const int* route_row, const float* gate,
                    long long routes, int K, int dim, int world, int cap_rows, int* status, void* stream);
int oa_ep_pull_rows(const void* const* src_peers, const int* route_rank, const int* route_row, const float* gate, const void* base,
                    void* out, long long tokens, int K, int dim, int world, void* stream);
int oa_ep_pull_dot(const void* const* src_peers, const int* route_rank, const int* route_row, const void* dout, float* dgate,
                   long long routes, int K, int dim, int world, void* stream);
int oa_ep_zero_pad(void* buf, const int* loc_offsets, const int* loc_counts, int E_loc, int dim, void* stream);

// ---- Mamba-3 SISO selective scan (mamba3.cu): preprocess, chunk-checkpointed scan forward/backward, decode step
int oa_mamba3_pre_fwd(int dtype, const void* proj, long long stride, const float* dt_bias, int rows, int H, int N, int A,
                      int d_inner, float eps, float dt_min, float dt_max, float afloor, float* Bn, float* Cn, float* rstd,
                      float* dt, float* adt, float* trap, float* angle, void* stream);
int oa_mamba3_pre_bwd(int dtype, const void* proj, void* dproj, long long stride, const float* dt_bias, int rows, int H, int N,
                      int A, int d_inner, float eps, float dt_min, float dt_max, float afloor, const float* Bn,
                      const float* Cn, const float* rstd, const float* dBn, const float* dCn, const float* ddt,
                      const float* dadt, const float* dtrap, const float* dangle, float* ddt_bias, void* stream);
int oa_mamba3_scan_fwd(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                       const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb,
                       const float* D, void* y, long long ys, float* Hck, float* Tck, float* Hfinal, float* Tfinal,
                       float* Kfinal, float* Vfinal, int B, int L, int H, int P, int N, int A, int chunk, void* stream);
size_t oa_mamba3_scratch_floats(int B, int H, int P, int N, int chunk);
int oa_mamba3_scan_bwd(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                       const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb,
                       const float* D, const void* dy, long long dys, void* dx, void* dz, long long dxs, float* dCn,
                       float* dBn, float* ddt, float* dadt, float* dtrap, float* dangle, float* dCb, float* dBb, float* dD,
                       const float* Hck, const float* Tck, float* scratch, int B, int L, int H, int P, int N, int A,
                       int chunk, void* stream);
int oa_mamba3_step(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                   const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb, const float* D,
                   void* y, long long ys, float* Hst, float* Vst, const float* Tin, const float* Kin, float* Tout,
                   float* Kout, int B, int H, int P, int N, int A, int first, void* stream);
int oa_gated_norm_fwd(int dtype, const void* y, const void* z, long long zs, const float* w, void* out, float* rstd,
                      long long rows, int H, int P, float eps, void* stream);
int oa_gated_norm_bwd(int dtype, const void* y, const void* z, long long zs, const float* w, const float* rstd, const void* dout,
                      void* dy, void* dz, long long dzs, float* dw, long long rows, int H, int P, void* stream);

// ---- convolution / pooling support (conv.cu); NCHW, columns [N*Ho*Wo, C*kh*kw]
int oa_im2col(int dtype, const void* x, void* cols, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
              int dh, int dw, void* stream);
int oa_col2im(int dtype, const void* cols, void* x, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
              int dh, int dw, void* stream);
int oa_pool2d_fwd(int dtype, int mode, const void* x, void* y, int* idx, int N, int C, int H, int W, int kh, int kw, int sh,
                  int sw, int ph, int pw, void* stream);
int oa_pool2d_bwd(int dtype, int mode, const void* dy, const int* idx, void* dx, int N, int C, int H, int W, int kh, int kw,
                  int sh, int sw, int ph, int pw, void* stream);
int oa_upsample_nearest(int dtype, const void* in, void* out, long long planes, int H, int W, int fy, int fx, int backward,
                        void* stream);

// ---- KV-cache serving (decode.cu)
int oa_kv_append(const void* k_src, const void* v_src, long long src_stride, void* k_cache, void* v_cache, int batch,
                 int s_new, int heads, int head_dim, int pos0, int max_seq, const int* pos_dev, void* stream);
int oa_decode_attn(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out, long long out_stride,
                   int batch, int heads, int head_dim, int len, int max_seq, float scale, const int* pos_dev, void* stream);
size_t oa_decode_attn_stream_scratch_bytes(int batch, int heads, int head_dim, int splits);
int oa_decode_attn_stream(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out, long long out_stride,
                          int batch, int heads, int head_dim, int len, int max_seq, float scale, const int* pos_dev, void* partial,
                          int splits, int* status, void* stream);

// ---- reinforcement learning (rl.cu): vector CartPole, GAE, rollout / replay storage, loss targets, categorical sampling
int oa_rl_cartpole_reset(void* state, void* done, void* steps, void* episode, int envs, unsigned seed_lo, unsigned seed_hi,
                         int only_done, void* stream);
int oa_rl_cartpole_step(const void* action, void* state, void* trans_obs, void* reward, void* terminated, void* truncated,
                        void* done, void* steps, int envs, int max_steps, float gravity, float cart_mass, float pole_mass,
                        float half_len, float force, float dt, float x_limit, float angle_limit, void* stream);
// ---- LunarLander3d (lunar.cu):  cfg_f: 77 host floats, cfg_n: 6 host ints, spawn8: 8 host floats; the rest is device memory.
int oa_rl_lunar_step(const float* cfg_f, const int* cfg_n, const void* terrain, const void* action, const void* external_stop, void* state_f,
                     void* state_u, void* trans_obs, void* obs, void* reward, void* terminated, void* truncated, void* end_reason, int envs,
                     void* stream);
int oa_rl_lunar_reset(const float* cfg_f, const int* cfg_n, const float* spawn8, const void* terrain, void* state_f, void* state_u, void* obs,
                      int envs, unsigned seed_lo, unsigned seed_hi, int only_done, void* stream);
// ---- reinforcement learning, continued (rl.cu)
int oa_rl_gae(const void* reward, const void* value, const void* next_value, const void* terminated, const void* truncated,
              void* adv, void* ret, int T, int E, float gamma, float lambda, void* stream);
int oa_rl_rollout_append(const void* obs, const void* action, const void* reward, const void* value, const void* next_value,
                         const void* logp, const void* term, const void* trunc, void* o_obs, void* o_action, void* o_reward,
                         void* o_value, void* o_next_value, void* o_logp, void* o_term, void* o_trunc, void* o_valid, int envs,
                         int obs_elems, int slot, void* stream);
int oa_rl_replay(int mode, const void* obs, const void* action, const void* next_obs, const void* reward, const void* term,
                 const void* trunc, void* o_obs, void* o_action, void* o_next_obs, void* o_reward, void* o_term, void* o_trunc,
                 void* o_index, int rows, int obs_elems, int act_elems, int capacity, int cursor, int size, unsigned seed_lo,
                 unsigned seed_hi, void* stream);
int oa_rl_ppo_clip(const void* new_lp, const void* old_lp, const void* adv, void* out, int n, float eps, int backward,
                   void* stream);
int oa_rl_dqn_target(const void* reward, const void* next_q, const void* terminated, void* out, int batch, int actions,
                     float discount, void* stream);
int oa_rl_sac_target(const void* reward, const void* q1, const void* q2, const void* logp, const void* terminated, void* out,
                     int batch, float discount, float alpha, void* stream);
int oa_rl_sample_categorical(const void* logits, void* action, int rows, int actions, float temperature, unsigned seed_lo,
                             unsigned seed_hi, int greedy, void* stream);
// ---- rows.cu: row compaction / scatter with a device-resident count, accuracy counters, stochastic rounding, int8 GEMM
size_t oa_rows_scan_scratch_ints(int rows);
int oa_rows_scan(const void* mask, void* position, void* count, void* scratch, int rows, void* stream);
int oa_rows_compact(const void* x, const void* mask, const void* position, void* packed, void* index, int rows, int width, int elem_bytes,
                    void* stream);
int oa_rows_scatter(const void* packed, const void* index, const void* count, void* out, int capacity, int out_rows, int width, int dtype, int add,
                    void* stream);
int oa_rows_gather(const void* src, const void* index, const void* count, void* packed, int capacity, int src_rows, int width, int elem_bytes,
                   void* stream);
int oa_accuracy_count(const void* logits, const void* targets, const void* mask, void* out2, int rows, int vocab, int dtype, void* stream);
int oa_sr_round_bf16(const void* x, void* out, long long n, unsigned seed_lo, unsigned seed_hi, void* stream);
int oa_gemm_int8(const void* a, const void* b, void* c_i32, void* c_f32, const void* row_scale, const void* col_scale, int M, int N, int K,
                 void* stream);

// ---- vector quantisation (vq.cu)
int oa_vq_code_norm(const void* codebook, void* enorm, int K, int D, void* stream);
int oa_vq_argmin_gather(const void* dot, const void* enorm, const void* codebook, void* idx, void* zq, int N, int K, int D,
                        void* stream);
int oa_vq_ema_update(const void* ze, const void* idx, void* embed_sum, void* cluster_size, void* codebook, int N, int D, int K,
                     float decay, float eps, float dead_thresh, unsigned seed, int normalize, void* stream);

// ---- block quantisation (quant.cu): op 0..6 = Q4_0 scales / quantize / dequantize, Q8_0 quantize / dequantize, int8 q / dq
int oa_quantize(int op, const void* in, const void* scale, void* out, long long count, void* stream);

// ---- hashing (hash.cu): batched Keccak-f[1600], SHAKE-128/256 of fixed-length rows, one Merkle level of SHAKE-256 pairs
int oa_keccak_f1600(const void* in, void* out, int n, void* stream);
int oa_shake(int bits, const void* msg, void* out, int n, int msg_len, int msg_stride, int out_len, int out_stride, void* stream);
int oa_merkle_level(const void* in, void* out, int n_in, void* stream);

// ---- chunked Mamba-3 scan glue (mamba3_ssd.cu); chunk layout = [B*H*nC, 128, *]
int oa_ssd_prep_fwd(const void* x, long long ldx, const void* Bn, const void* Cn, const void* Bb, const void* Cb, const void* dt,
                    const void* adt, const void* trap, const void* theta, void* Ct, void* Bt, void* Ce, void* X, void* Xw, void* cum,
                    void* gamma, void* scale, void* w, void* qk, int B, int L, int H, int P, int N, int A, void* stream);
int oa_ssd_mask_fwd(const void* Gm, const void* cum, const void* scale, const void* gamma, const void* qk, const void* Dh, void* M,
                    int G, int H, int nC, void* stream);
int oa_ssd_state_fwd(const void* S, const void* cum, void* Hin, int BH, int nC, int PN, void* stream);
int oa_ssd_state_bwd(const void* T, const void* cum, const void* Hin, void* dHout, void* dcumQ, int BH, int nC, int PN, void* stream);
int oa_ssd_out_fwd(const void* Y, const void* z, long long ldz, void* y, void* yraw, long long ldy, int B, int L, int H, int P,
                   void* stream);
int oa_ssd_dy_prep(const void* dy, const void* yraw, long long ldy, const void* z, long long ldz, void* dz, long long lddz, void* dY,
                   int B, int L, int H, int P, void* stream);
int oa_ssd_mask_bwd(const void* dM, const void* Gm, const void* cum, const void* scale, void* dG, void* row_mm, void* col_mm,
                    void* col_ge, void* diag, int G, void* stream);
int oa_ssd_prep_bwd(const void* dCt, const void* dBt, const void* dCe, const void* Ct, const void* Bt, const void* cum, const void* dqk,
                    const void* theta, void* dCn, void* dBn, void* dCb, void* dBb, void* dtheta, void* dcum_ce, int B, int L, int H,
                    int N, int A, void* stream);
int oa_ssd_theta_fwd(const void* angle, int lda, const void* dt, void* tot, void* theta, int B, int L, int H, int A, void* stream);
int oa_ssd_theta_bwd(const void* dtheta, const void* angle, int lda, const void* dt, void* tot, void* dangle, void* ddt, int B, int L,
                     int H, int A, void* stream);
int oa_ssd_dx_out(const void* dX, const void* dXw, const void* X, const void* w, void* dx, long long lddx, void* dw, int B, int L, int H,
                  int P, void* stream);
// Benchmark-variant options of the Mamba-3 block (mamba3_conv.cu): causal depthwise convolution (width Kw <= 8) + SiLU over
// columns [col0, col0 + C) of x [B*L, ld], in place (`saved` [B*L, C] receives the inputs); its backward overwrites the same
// columns of dy with dx and writes weight-gradient partials float[B * ceil(L/64)][Kw][C]; and the learned-decay fill
// x[row, col0 + h] = exp(a_log[h]) - 1.
int oa_mamba3_conv_fwd(int dtype, void* x, long long ld, int col0, void* saved, const float* w, int B, int L, int C, int Kw,
                       void* stream);
int oa_mamba3_conv_bwd(int dtype, void* dy, long long ld, int col0, const void* saved, const float* w, float* dw_part, void* gbuf,
                       int B, int L, int C, int Kw, void* stream);
int oa_mamba3_alog_fill(int dtype, void* x, long long ld, int col0, const float* a_log, long long rows, int H, void* stream);
// Scalar tail of the chunked-scan backward (three small kernels): [G, Q] inputs -> dadt, ddt, dtrap [B*L, H] and dD [H] (may
// be null); ddt_theta may be null; scratch: float[2 * B*L*H + B*H*L/128].
int oa_ssd_tail(const void* dw, const void* w, const void* col_ge, const void* row_mm, const void* col_mm, const void* dcum_ce,
                const void* diag, const void* qk, const void* cum, const void* dcumQ, const void* dt, const void* trap,
                const void* ddt_theta, void* dadt, void* ddt, void* dtrap, void* dD, void* scratch, int B, int L, int H,
                void* stream);

// ---- audio DSP (audio.cu)
int oa_audio_stft_frame(const void* x, void* frames, int channels, long long samples, int n_frames, int fft, int hop, int win, int kind,
                        int pad, void* stream);
int oa_audio_magnitude(const void* reim, void* spec, long long rows, int bins, void* stream);
int oa_audio_fade(const void* x, void* out, long long count, long long samples, long long fade_in, long long fade_out, void* stream);
int oa_audio_mix(const void* a, const void* b, void* out, long long count, float ga, float gb, void* stream);
int oa_audio_resample(const void* x, void* out, int channels, long long in_samples, long long out_samples, unsigned in_r, unsigned out_r,
                      int half_width, void* stream);
int oa_audio_envelope(const void* x, void* out, int channels, long long samples, int bins, void* stream);

// ---- channel-axis LayerNorm of [B, C, T] tensors (channel_norm.cu)
int oa_channel_norm_fwd(int dtype, const void* x, const void* w, const void* bias, void* y, void* mean, void* rstd, int B, int C, int L, float eps,
                        int relu, void* stream);
int oa_channel_norm_bwd(int dtype, const void* x, const void* w, const void* g, const void* y_relu, const void* mean, const void* rstd, void* dx,
                        void* dw_f32, void* db_f32, int B, int C, int L, void* stream);

// ---- image operations (image.cu)
int oa_image_pointwise(const void* x, void* out, long long n, int op, float p0, float p1, float p2, void* stream);
int oa_image_channels(const void* x, void* out, int batch, int cin, int cout, long long plane, const float* matrix20, const int* sel4,
                      const void* twist, int mode, void* stream);
int oa_image_blend(const void* a, const void* b, const void* mask, void* out, int batch, int channels, int H, int W, int op, float alpha,
                   int mask_channels, int rx, int ry, int rw, int rh, float value, void* stream);
int oa_image_overlay(const void* img, const void* labels, const void* palette, void* out, int batch, int channels, long long plane,
                     int classes, float alpha, void* stream);
int oa_image_noise(const void* x, void* out, long long n, int op, float p0, float p1, float p2, unsigned long long seed, void* stream);
int oa_image_tile_filter(const void* x, void* out, int planes, int H, int W, int kw, int kh, int mode, int border, float border_value,
                         const void* k0, const void* k1, float p0, float p1, float p2, void* stream);
int oa_image_index_map(const void* x, void* out, int planes, int Hi, int Wi, int Ho, int Wo, int op, int a0, int a1, int border,
                       float border_value, void* stream);
int oa_image_resize_bwd(const void* grad_out, void* grad_in, int planes, int Hi, int Wi, int Ho, int Wo, int mode, void* stream);
int oa_image_resize(const void* x, void* out, int planes, int channels, int Hi, int Wi, int Ho, int Wo, int mode, const float* mean3,
                    const float* std3, void* stream);
int oa_image_warp(const void* x, const void* map, void* out, int batch, int channels, int Hi, int Wi, int Ho, int Wo, int op, int map_batch,
                  int interp, int border, float border_value, void* stream);

// ---- detection post-processing and metrics (detection.cu)
int oa_det_box_iou(const void* a, const void* b, void* out, int n, int m, void* stream);
int oa_det_nms(const void* boxes, const void* scores, const void* classes, int n, float iou_thr, float score_thr, int max_det, int agnostic,
               void* indices, void* count, void* alive_scratch, void* stream);
int oa_det_confusion(const void* predicted, const void* target, long long n, int classes, void* out_zeroed, void* stream);
int oa_det_binary_counts(const void* predicted, const void* target, long long n, void* out_zeroed, void* stream);
int oa_det_segmentation_metrics(const void* confusion, int classes, void* per_class, void* mean_iou, void* accuracy, void* stream);
int oa_det_evaluate(const void* pboxes, const void* pscores, const void* pclasses, const void* pimages, const void* order, int P,
                    const void* tboxes, const void* tclasses, const void* timages, int G, const void* thresholds, int T, int classes,
                    float score_thr, void* matched_scratch, void* curve_scratch, void* counts, void* metrics, void* map_by_threshold,
                    void* mean_map, void* stream);

// ---- peer-memory communication (comm.cu): IPC buffers, epoch flags, fused data-parallel step
int oa_ipc_alloc(size_t bytes, void** out);
int oa_ipc_free(void* p);
int oa_ipc_get_handle(void* p, void* handle64);
int oa_ipc_open(const void* handle64, void** out);
int oa_ipc_close(void* p);
int oa_peer_signal(const void* const* flags_peers, void* epoch_local, int rank, int world, void* stream);
int oa_peer_wait(const void* my_flags, const void* epoch_local, int world, int* status, void* stream);
int oa_dp_reduce_adam_gather(const void* const* grad_peers, const void* const* param_peers, float* master, float* m, float* v,
                             long long shard_lo, long long shard_n, const float* state, const float* inv_clip,
                             int decoupled, int rank, int world, const void* my_flags, const void* epoch_local,
                             int* status, int max_blocks, void* stream);
int oa_peer_reduce(int dtype, const void* const* in_peers, void* out, long long lo, long long n, int world, int op,
                   void* stream);
int oa_peer_allreduce_oneshot(const void* const* slots_peers, const void* const* counters_peers, const void* src,
                              const void* residual, void* out, void* sync2, long long n, long long slot_elems, int world,
                              int rank, int max_ctas, int* status, void* stream);
int oa_p2p_attributes(int src, int dst, int* out);
// Bound (milliseconds of wall time) of every device-side wait on a peer flag; the default is 2000.
int oa_set_peer_wait_ms(long long ms);
// Gradient-norm clipping under the fused data-parallel step: sum of squares of this rank's shard of the summed gradient
// (block partials, `oa_dp_sumsq_blocks()` floats, accumulated over calls), publication of the total into slot `rank`
// (16-byte slots) of every rank, and the clip coefficient from the `world` slots (+ `extra[0]`, may be null);
// coef[0] = coefficient, coef[1] = norm.
int oa_dp_sumsq_blocks(void);
int oa_dp_shard_sumsq(const void* const* grad_peers, long long shard_lo, long long shard_n, int rank, int world, float* partial,
                      int accumulate, void* stream);
int oa_dp_sumsq_publish(const float* partial, const void* const* slot_peers, int rank, int world, void* stream);
int oa_dp_clip_finalize(const float* slots, int world, const float* extra, float max_norm, float* coef, void* stream);
int oa_peer_push(const void* const* dst_peers, long long dst_off_bytes, const void* src, long long nbytes, int world,
                 void* stream);

#ifdef __cplusplus
}
#endif
