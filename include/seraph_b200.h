/*
 * seraph_b200.h - C ABI of libseraph_b200.so.
 *
 * Part 1 and 2 are the entry points Seraph's own programs bind for the
 * training path (its headers include/train_cuda.h and
 * include/cuda_train_context.h, implementation src/train_cuda.c and
 * src/cuda_train_context.cu); names, argument meaning and return conventions
 * are theirs, so `seraph-train-cuda` links against this library in place of
 * cuda_train_context.o / train_cuda.o / cuda_profiler.o.  Part 3 is the
 * profiler ABI (include/cuda_profiler.h).  Part 4 are additions that have no
 * counterpart in the reference.
 *
 * Everything runs on an NVIDIA B200 (sm_100a).  There is no CPU path: without
 * a device cuda_train_init() returns NULL and nothing else may be called.
 * All tensors are FP32, row-major, token-major: activations [T, dim] with
 * heads contiguous inside a row, weights [out_dim, in_dim]; packed batches
 * are concatenated sequences with seq_starts[B+1] prefix sums (uint32 on the
 * device, int on the host side of the step functions).
 */
#ifndef SERAPH_B200_H
#define SERAPH_B200_H

#include "seraph_b200_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ===== 1. step-level API (reference: include/train_cuda.h:12-64) ========== */

/* src/cuda_train_context.cu:2246.  NULL when no sm_100 device can be used. */
cuda_train_context_t* cuda_train_init(int device_id);
/* src/cuda_train_context.cu:2404 */
void cuda_train_free(cuda_train_context_t* ctx);
/* src/cuda_train_context.cu:2559 */
void cuda_train_sync(cuda_train_context_t* ctx);
/* src/cuda_train_context.cu:2387 */
void cuda_train_get_gpu_info(cuda_train_context_t* ctx, char* name, int name_len, float* memory_gb);

/* One full-weight step on one sequence: forward, loss, backward, AdamW when the
 * accumulation count is reached.  Returns the mean loss, -1.0f on bad
 * arguments or allocation failure, 0.0f when nothing is predicted.
 * src/train_cuda.c:597 */
float cuda_train_step_gpu_full(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx);
/* Packed batch of `batch_size` sequences.  src/train_cuda.c:1966 */
float cuda_train_step_gpu_full_batch(train_state_t* state, int* tokens_packed, int total_tokens,
                                     int* seq_starts, int batch_size, cuda_train_context_t* ctx);
/* LoRA steps: frozen base, adapter gradients by the complete chain rule of the
 * reference's Vulkan LoRA step (src/train.c:5847, backward :6287-6615).  The
 * frozen base is taken from state->full_weights.  src/train_cuda.c:1599, :2332 */
float cuda_train_step_gpu_lora(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx);
float cuda_train_step_gpu_lora_batch(train_state_t* state, int* tokens_packed, int total_tokens,
                                     int* seq_starts, int batch_size, cuda_train_context_t* ctx);
/* src/train_cuda.c:1244 (weights and Adam moments) and :1317 (gradients) back into state->full_weights */
void cuda_download_full_weights(cuda_train_context_t* ctx, train_state_t* state);
void cuda_download_gpu_gradients(cuda_train_context_t* ctx, train_state_t* state);
/* src/train_cuda.c:2677 and :2812 */
float cuda_eval_forward(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx);
float cuda_evaluate(train_state_t* state, int* val_tokens, int num_val_tokens, int* offsets, int num_samples,
                    int max_seq_len, int max_eval_samples, cuda_train_context_t* ctx, float* out_perplexity);

/* ===== 2. op-level API (reference: include/cuda_train_context.h:239-325) === */

/* buffers: src/cuda_train_context.cu:2568-2640 */
cuda_buffer_t* cuda_train_buffer_create(cuda_train_context_t* ctx, size_t size);
void cuda_train_buffer_free(cuda_train_context_t* ctx, cuda_buffer_t* buf);
void cuda_train_buffer_upload(cuda_train_context_t* ctx, cuda_buffer_t* buf, const float* data, size_t count);
void cuda_train_buffer_upload_u32(cuda_train_context_t* ctx, cuda_buffer_t* buf, const uint32_t* data, size_t count);
void cuda_train_buffer_download(cuda_train_context_t* ctx, cuda_buffer_t* buf, float* data, size_t count);
void cuda_train_buffer_download_bytes(cuda_train_context_t* ctx, cuda_buffer_t* buf, void* data, size_t bytes);
void cuda_train_fill_buffer(cuda_train_context_t* ctx, cuda_buffer_t* buf, uint32_t value, size_t bytes);
void cuda_train_fill_buffer_range(cuda_train_context_t* ctx, cuda_buffer_t* buf, size_t offset, uint32_t value, size_t bytes);
void cuda_train_copy_buffer(cuda_train_context_t* ctx, cuda_buffer_t* src, cuda_buffer_t* dst, size_t bytes);

/* forward ops */
void cuda_train_matmul(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, int M, int N, int K);                 /* :2697 */
void cuda_train_matmul_transpose(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, int M, int N, int K,
                                 int transpose_A, int transpose_B, int accumulate);                                                             /* :2702 */
void cuda_train_silu(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* output, size_t count);                                     /* :2711 */
void cuda_train_rmsnorm(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* scale, cuda_buffer_t* output, int rows, int cols, float eps);
void cuda_train_softmax(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* output, int rows, int cols);
void cuda_train_rope(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, int seq_len, int num_heads, int head_dim, float rope_theta);
void cuda_train_add(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, size_t count);
void cuda_train_mul(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, size_t count);
void cuda_train_scale(cuda_train_context_t* ctx, cuda_buffer_t* A, size_t count, float alpha);
void cuda_train_batch_attention(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V, cuda_buffer_t* out,
                                cuda_buffer_t* lse_out, int seq_len, int num_heads, int kv_heads, int head_dim);
void cuda_train_batch_attention_packed(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V, cuda_buffer_t* out,
                                       cuda_buffer_t* lse_out, cuda_buffer_t* seq_starts, int total_tokens, int batch_size,
                                       int num_heads, int kv_heads, int head_dim, int max_seq_in_batch);
void cuda_train_embed_lookup(cuda_train_context_t* ctx, cuda_buffer_t* tokens_u32, cuda_buffer_t* embed_weight, cuda_buffer_t* out_hidden,
                             int seq_len, int hidden_size, int vocab_size);
void cuda_train_rope_packed(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, cuda_buffer_t* seq_starts,
                            int total_tokens, int batch_size, int num_heads, int head_dim, float rope_theta);

/* loss + backward ops */
void cuda_train_cross_entropy_grad(cuda_train_context_t* ctx, cuda_buffer_t* logits, cuda_buffer_t* targets_u32, cuda_buffer_t* grad_logits,
                                   cuda_buffer_t* loss_rows, int rows, int cols);                                                               /* :2941, kernel :1566 */
void cuda_train_cross_entropy_grad_packed(cuda_train_context_t* ctx, cuda_buffer_t* logits, cuda_buffer_t* targets_u32,
                                          cuda_buffer_t* grad_logits, cuda_buffer_t* loss_rows, cuda_buffer_t* seq_starts,
                                          int total_tokens, int batch_size, int vocab_size, int num_valid_predictions);                        /* :3171, kernel :1657 */
void cuda_train_reduce_sum(cuda_train_context_t* ctx, cuda_buffer_t* in_buf, cuda_buffer_t* out_buf, size_t count);                             /* :2966 */
void cuda_train_silu_backward(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* grad_output, cuda_buffer_t* grad_input, size_t count);   /* :2978 */
void cuda_train_elementwise_mul_backward(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* grad_C,
                                         cuda_buffer_t* grad_A, cuda_buffer_t* grad_B, size_t count);                                           /* :2989 */
void cuda_train_rmsnorm_backward_batch(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* scale, cuda_buffer_t* grad_output,
                                       cuda_buffer_t* grad_input, cuda_buffer_t* grad_scale, int rows, int cols, float eps);                    /* :3001, kernel :1767 */
void cuda_train_rope_backward(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, int seq_len, int num_heads, int head_dim, float rope_theta);
void cuda_train_rope_backward_packed(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, cuda_buffer_t* seq_starts,
                                     int total_tokens, int batch_size, int num_heads, int head_dim, float rope_theta);                          /* kernel :679 */
void cuda_train_batch_attention_backward(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V,
                                         cuda_buffer_t* attn_out, cuda_buffer_t* lse, cuda_buffer_t* grad_out,
                                         cuda_buffer_t* grad_Q, cuda_buffer_t* grad_K, cuda_buffer_t* grad_V,
                                         int seq_len, int num_heads, int kv_heads, int head_dim);                                               /* :3041 */
void cuda_train_batch_attention_backward_packed(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V,
                                                cuda_buffer_t* attn_out, cuda_buffer_t* lse, cuda_buffer_t* grad_out,
                                                cuda_buffer_t* grad_Q, cuda_buffer_t* grad_K, cuda_buffer_t* grad_V,
                                                cuda_buffer_t* seq_starts, int total_tokens, int batch_size,
                                                int num_heads, int kv_heads, int head_dim, int max_seq_in_batch);                               /* :3107, kernels :1013/:2012 */
void cuda_train_embedding_backward(cuda_train_context_t* ctx, cuda_buffer_t* tokens_u32, cuda_buffer_t* grad_hidden, cuda_buffer_t* grad_embed,
                                   int seq_len, int hidden_size, int vocab_size);                                                               /* :3192, kernel :2175 */
void cuda_train_adamw_update(cuda_train_context_t* ctx, cuda_buffer_t* weight, cuda_buffer_t* grad, cuda_buffer_t* m, cuda_buffer_t* v,
                             float lr, float beta1, float beta2, float weight_decay, float eps, int step, size_t size,
                             const char* tensor_name, int rows, int cols);                                                                      /* :3203, kernel :2187 */
void cuda_train_nan_check(cuda_train_context_t* ctx, cuda_buffer_t* input, size_t count_floats, cuda_buffer_t* flags_u32, uint32_t flag_index);
void cuda_train_set_profiler(cuda_train_context_t* ctx, cuda_profiler_t* prof);

/* LoRA: src/cuda_train_context.cu:3240-3394 */
void cuda_train_lora_backward(cuda_train_context_t* ctx, cuda_buffer_t* grad_output, cuda_buffer_t* input, cuda_buffer_t* A, cuda_buffer_t* B,
                              cuda_buffer_t* gA, cuda_buffer_t* gB, cuda_buffer_t* hidden_tmp,
                              int seq_len, int in_dim, int out_dim, int rank, float scale);
void cuda_train_zero_lora_grads(cuda_train_context_t* ctx);
void cuda_download_lora_weights(cuda_train_context_t* ctx, void* lora /* lora_model_t* */);

/* ===== 3. profiler (reference: include/cuda_profiler.h:53-82) ============== */
cuda_profiler_t* cuda_profiler_create(void);
void cuda_profiler_destroy(cuda_profiler_t* prof);
void cuda_profiler_enable(cuda_profiler_t* prof);
void cuda_profiler_disable(cuda_profiler_t* prof);
void cuda_profiler_reset(cuda_profiler_t* prof);
int  cuda_profiler_begin_op(cuda_profiler_t* prof, const char* name, void* stream);
void cuda_profiler_end_op(cuda_profiler_t* prof, int op_idx, void* stream);
void cuda_profiler_set_launch(cuda_profiler_t* prof, int op_idx, int gx, int gy, int gz, int bx, int by, int bz, size_t shared_mem);
void cuda_profiler_set_flops(cuda_profiler_t* prof, int op_idx, size_t flops);
void cuda_profiler_set_bytes(cuda_profiler_t* prof, int op_idx, size_t bytes);
void cuda_profiler_sync_and_analyze(cuda_profiler_t* prof, void* stream);
void cuda_profiler_print(cuda_profiler_t* prof);
void cuda_profiler_print_top(cuda_profiler_t* prof, int top_n);
void cuda_profiler_set_log(cuda_profiler_t* prof, void* file_ptr);

/* ===== 4. additions (no counterpart in the reference) ====================== */

/* Status of the calls since the last query: 0 ok, 1 bad argument, 2 CUDA error,
 * 3 out of memory, 4 token id outside the vocabulary reached a kernel, 5 a
 * bounded wait ran out, 6 NCCL error, 7 size beyond a fixed capacity.
 * Synchronises the stream, reads the device status word, clears both. */
int seraph_b200_last_status(cuda_train_context_t* ctx);
/* GEMM arithmetic.  4 (default) = FP32-accurate on tensor cores: plain products
 * from two FP16 parts per operand (power-of-two scale per operand, three
 * kind::f16 passes), attention's products and small or unaligned shapes from
 * a TF32 hi/lo split (three kind::tf32 passes); 0 = the TF32 split everywhere;
 * 1 = single-pass TF32; 2 = reduced precision as selected by ctx->use_bf16
 * (runs the single-pass kernel); 3 = FP32 FMA on CUDA cores. */
int seraph_b200_set_gemm_mode(cuda_train_context_t* ctx, int mode);
/* 1 (default): tensor-core GEMMs of plain matrices run on pairs of CTAs that
 * share one 256-row MMA (half of each B tile per CTA); 0: one CTA per tile. */
int seraph_b200_set_gemm_pair(cuda_train_context_t* ctx, int on);
/* 1 (default): the tiles of a GEMM's last, partly filled wave are cut into
 * pieces of the k range that fill the machine and are added in a fixed order;
 * 0: whole tiles only. */
int seraph_b200_set_gemm_tail_split(cuda_train_context_t* ctx, int on);
/* 1 (default; SERAPH_B200_PARTS_CACHE=0 turns it off): inside one training or evaluation call the FP16 parts of the
 * weights and of the activations saved for the backward pass are made at their first use and shared by every later
 * product of the call that reads the same tensor (arena of 4 bytes per element, taken only while an eighth of the
 * device stays free); 0: every product or run of products prepares its own operands.  Results are identical. */
int seraph_b200_set_parts_cache(cuda_train_context_t* ctx, int on);
/* Q/K normalisation over the whole token row (all heads), in place: y = x / max(sqrt(mean(x^2)), eps).  Replaces
 * vulkan_qk_norm (include/vulkan_backend.h:600, shaders/qk_norm.comp:30-76; called on Q and K after RoPE,
 * src/train.c:4688-4689); the reference's CUDA backend has no such kernel.  use_qk_norm == 0: no-op, as there.
 * rms_out (may be NULL): sqrt(mean(x^2)) of every row before the clamp, [seq_len] floats, for the backward call. */
void seraph_b200_qk_norm(cuda_train_context_t* ctx, cuda_buffer_t* qk, cuda_buffer_t* rms_out, int seq_len, int num_heads, int head_dim,
                         int use_qk_norm, float eps);
/* Backward of the above (the reference has none: its training passes the gradient through unchanged).
 * rms > eps: grad_in = (grad_out - y * mean(grad_out o y)) / rms; clamp active: grad_in = grad_out / eps.
 * qk_out and rms are what the forward call left; grad_in may be grad_out. */
void seraph_b200_qk_norm_backward(cuda_train_context_t* ctx, cuda_buffer_t* qk_out, cuda_buffer_t* rms, cuda_buffer_t* grad_out,
                                  cuda_buffer_t* grad_in, int seq_len, int num_heads, int head_dim, int use_qk_norm, float eps);
/* The resident FP32 weights as a BF16 safetensors file: byte for byte what trainable_weights_save_to_safetensors
 * (src/train.c:433-569) writes from the host copies after cuda_download_full_weights (same header, tensor order and
 * FP32 -> BF16 truncation), but converted on the GPU (2 bytes per parameter cross to the host, in chunks, while the
 * previous chunk is written).  The host copies in `state` are not touched.  Returns SB_OK or an SB_ERR_* code. */
int seraph_b200_save_safetensors(cuda_train_context_t* ctx, train_state_t* state, const char* path);
/* trainable_weights_load_from_safetensors (src/train.c:571-629) into the device: the tensors are read in saved order
 * (the header is skipped, as there), cross to the GPU as BF16 in chunks and are widened into the resident FP32 weights
 * (uploading the model from `state` first if it is not resident yet).  Adam moments and the host copies are left as they
 * are; cuda_download_full_weights refreshes the host side.  Returns SB_OK or an SB_ERR_* code. */
int seraph_b200_load_safetensors(cuda_train_context_t* ctx, train_state_t* state, const char* path);
/* save_checkpoint (src/train.c:7760-7804) for a full-weight state whose weights are resident on the GPU: the
 * safetensors file as above plus "<path>.state" (current_epoch, current_step, current_loss, optimizer_step).
 * SB_ERR_ARG for a LoRA state (those go through cuda_download_lora_weights and the reference's lora_save). */
int seraph_b200_save_checkpoint(cuda_train_context_t* ctx, train_state_t* state, const char* path);
/* Model options beyond the reference's training step (its trainable_weights_t has no tensors for them, include/train.h:75-90),
 * so that Qwen3- and Mistral-shaped models run as their configurations state them:
 *   per_head_qk_norm  q and k pass through a learned RMSNorm over each head before RoPE (scales q_norm [hd], k_norm [hd] per layer);
 *   untied_lm_head    logits come from a separate lm_head [V,d] instead of the embedding matrix.
 * `flat` holds the parameters (per layer q_norm then k_norm; then lm_head), n their count; both options off takes NULL, 0.
 * The call drops the resident model; the next step uploads everything again.  Full-weight steps train the extra parameters
 * with the same AdamW (and reduce their gradients across data-parallel ranks); LoRA steps keep them frozen.  They are not part
 * of the reference's checkpoint formats: read them with seraph_b200_get_model_extras (which: 0 parameters, 1 gradients,
 * 2 Adam m, 3 Adam v).  Distinct from config->use_qk_norm, the reference's unweighted whole-row form. */
int seraph_b200_set_model_extras(cuda_train_context_t* ctx, int per_head_qk_norm, int untied_lm_head, const float* flat, size_t n);
int seraph_b200_get_model_extras(cuda_train_context_t* ctx, int which, float* out, size_t n);
/* LoRA adapter files.  version 2 is the reference's format, byte for byte (lora_save, src/lora.c:441-494): the Q and V
 * adapters only, which is all that format holds.  version 3 is an extension that keeps every adapter the model trains
 * (k, o, gate, up, down too, which the reference trains and then drops on save) and, with with_moments != 0, the Adam
 * moments and the optimizer step, so that a LoRA run can resume.  Saving first downloads the resident adapters
 * (cuda_download_lora_weights).  seraph_b200_lora_load reads either version into the adapters `state` already holds (same
 * rank and shapes, as lora_load of src/lora.c:496-560 would create them) and makes the next LoRA step upload them. */
int seraph_b200_lora_save(cuda_train_context_t* ctx, train_state_t* state, const char* path, int version, int with_moments);
int seraph_b200_lora_load(cuda_train_context_t* ctx, train_state_t* state, const char* path);
/* cuda_evaluate (include/train_cuda.h:60-64 of the reference, src/train_cuda.c:2812-2846) runs one forward pass per
 * validation sample there; here it packs samples into passes of up to `tokens` tokens (default 8192, at least
 * max_seq_len, at most 256 samples; SERAPH_B200_EVAL_BATCH_TOKENS sets the default) and takes every sample's mean loss
 * from the per-token losses of the pass.  0 = one pass per sample. */
int seraph_b200_set_eval_batch_tokens(cuda_train_context_t* ctx, int tokens);
/* Attention of 128-wide heads in the default GEMM mode.  0 = score product, row softmax and value product as separate
 * launches over a score scratch.  Otherwise the forward is one kernel per call that keeps the scores in tensor memory and the
 * probabilities in shared memory (online softmax, no score-sized scratch), and the backward is
 *   1  (default) and 3  one kernel that keeps dK and dV on chip (P^T and dS^T return to tensor memory as operands) plus one
 *      product for dQ,
 *   2  the scores in one kernel per sequence and head group, written as FP16 parts for three long products.
 * SERAPH_B200_ATTN_FLASH sets the default. */
int seraph_b200_set_attn_flash(cuda_train_context_t* ctx, int on);
/* Attention backward on the tensor cores: 0 (default) P and dS are made by a
 * streaming kernel from the stored scores; 1: by the epilogues of the two score
 * products (fewer bytes, but measured slower: the epilogue is what bounds the
 * short products). */
int seraph_b200_set_attn_fused(cuda_train_context_t* ctx, int on);
/* 0 (default): LoRA steps leave the adapters' own term out of dX, as the
 * reference does; 1: full chain rule, dX += s (dY B) A. */
int seraph_b200_set_lora_exact(cuda_train_context_t* ctx, int exact);
/* Global-norm gradient clipping before AdamW; 0 switches it off (default: the
 * reference clips nothing). */
int seraph_b200_set_grad_clip(cuda_train_context_t* ctx, float max_norm);
/* NaN guard of the training step (state->debug_nan_check, src/train_cuda.c:626-645 and :1086-1187): the flags the last
 * guarded step left in ctx->debug_nan_flags, copied to `out` (at most max_words words); returns the words written.
 * Index layout as in the reference: [0..9] fixed buffers, [10 + l] hidden after layer l, [10 + L + 5 l + k] grad_attn /
 * grad_q / grad_k / grad_v of layer l, [10 + 6 L + l] grad_hidden after layer l's backward, [10 + 7 L] embedding weights. */
int seraph_b200_nan_flags(cuda_train_context_t* ctx, uint32_t* out, int max_words);
/* Category totals (ms) of a cuda_profiler_t after cuda_profiler_sync_and_analyze: step, matmul, attention, attention_bwd,
 * rmsnorm, rmsnorm_bwd, cross_entropy, adamw, copy, other; returns the number of recorded ops.  With a profiler attached
 * (cuda_train_set_profiler, include/cuda_train_context.h:298) the training step's own launches are recorded, one op per
 * launch under its class name, as well as the calls of the per-op ABI. */
int seraph_b200_profiler_totals(cuda_profiler_t* profiler, float* out10);
/* Self-test of the bounded waits inside the tensor-core kernels: a one-warp kernel waits at most limit_cycles (<= 2e9) clock
 * cycles on a barrier that nothing completes, gives up, and leaves status 5 (bounded wait ran out) for
 * seraph_b200_last_status; the kernel returns normally and the context stays usable.  *waited_cycles_out: cycles it waited. */
int seraph_b200_selftest_bounded_wait(cuda_train_context_t* ctx, long long limit_cycles, long long* waited_cycles_out);
/* Kernels launched by this library on ctx since the last reset. */
unsigned long long seraph_b200_launch_count(cuda_train_context_t* ctx, int reset);
/* Integer tables of the last cuda_train_embedding_backward(seq_len=T, vocab=V):
 * occurring rows in ascending order, their token counts, and the token
 * positions sorted by (row, position).  Returns the number of rows or -1. */
int seraph_b200_embedding_segments(cuda_train_context_t* ctx, int T, int V, int* rows_out, int* counts_out, int* sorted_pos_out);
/* C = op(A) op(B) like cuda_train_matmul_transpose without accumulation, plus the largest |C| that the tensor-core kernel's
 * epilogue leaves behind for the next operand split inside a training step (test surface).  1: *amax_out set; 0: the shape
 * does not run on that kernel (C is computed all the same); -1: bad arguments. */
int seraph_b200_matmul_amax(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, int M, int N, int K,
                            int transpose_A, int transpose_B, float* amax_out);
/* Fused SwiGLU: out = silu(gate)*up; backward gives dgate and dup from gate, up, dout. */
void seraph_b200_swiglu(cuda_train_context_t* ctx, cuda_buffer_t* gate, cuda_buffer_t* up, cuda_buffer_t* out, size_t count);
void seraph_b200_swiglu_backward(cuda_train_context_t* ctx, cuda_buffer_t* gate, cuda_buffer_t* up, cuda_buffer_t* grad_out,
                                 cuda_buffer_t* grad_gate, cuda_buffer_t* grad_up, size_t count);
/* CUDA-event timer on the context's stream: start, then stop returns milliseconds. */
void seraph_b200_timer_start(cuda_train_context_t* ctx);
float seraph_b200_timer_stop(cuda_train_context_t* ctx);
/* Forget the resident weights, adapters and optimizer state: the next step uploads them again from
 * the host state (like the reference, a context otherwise uploads once and then only downloads). */
int seraph_b200_reset_model(cuda_train_context_t* ctx);
/* Repeat the full-weight step on the batch the previous step call left on the device: nothing is
 * copied between host and device and the call does not wait for the GPU.  The mean loss of the
 * last step can be read (with a synchronisation) through seraph_b200_last_loss. */
int seraph_b200_step_full_resident(train_state_t* state, cuda_train_context_t* ctx);
/* the same for either kind of step: full != 0 the full-weight step, 0 the LoRA step */
int seraph_b200_step_resident(train_state_t* state, cuda_train_context_t* ctx, int full);
float seraph_b200_last_loss(cuda_train_context_t* ctx);
/* Per-class kernel timing with CUDA events on the context's stream.  read() fills
 * out[class*4 + {0 ms, 1 algorithmic FLOPs, 2 algorithmic bytes, 3 launches}] and resets. */
int seraph_b200_timing_enable(cuda_train_context_t* ctx, int on);
int seraph_b200_timing_classes(void);
const char* seraph_b200_timing_class_name(int cls);
int seraph_b200_timing_read(cuda_train_context_t* ctx, double* out);
/* Logits [T, vocab] of the last step or evaluation, copied to host memory. */
int seraph_b200_download_logits(cuda_train_context_t* ctx, float* out, int T);

/* RMSNorm backward that never allocates.  No counterpart in the reference.
 * For hosts that cannot call the CUDA allocator when they need this op (a stream
 * capture open elsewhere in the process, a framework or real-time loop that bans
 * cudaMalloc after start-up, an embedder that owns all device memory): the
 * partial sums of the scale gradient go to a fixed array inside the library
 * image (296 x 8192 floats, 9.7 MB, held by every GPU that loads the library
 * until the process ends) instead of grow-on-demand scratch.
 *   - all pointers are device pointers; grad_scale is accumulated into, grad_input
 *     is written, exactly as cuda_train_rmsnorm_backward_batch does;
 *   - cols must be <= 8192: larger rows return 7 (size beyond capacity) and print why;
 *   - `stream` is a cudaStream_t (NULL = default stream); work is only enqueued;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) and the SM count, so make that first call with the
 *     device current and before any stream capture begins;
 *   - all calls on a device share the one array: calls that may overlap on the GPU
 *     (different streams without ordering) race on it and give wrong grad_scale;
 *     nothing has to be cleared between calls, each call overwrites what it reads.
 * Returns 0, or 1 bad argument / 2 CUDA error / 7 size. */
int seraph_b200_rmsnorm_backward_static(const float* input, const float* scale, const float* grad_output,
                                        float* grad_input, float* grad_scale, int rows, int cols, float eps, void* stream);

/* Data parallel over NCCL: rank 0 makes the 128-byte id, every rank calls init
 * with it before its first step; steps then all-reduce gradient buckets while
 * backward still runs and AdamW applies the mean.  wait() is a host-side wait
 * with a time limit that aborts the communicator instead of hanging. */
int seraph_dp_get_unique_id(void* id_out_128);
int seraph_dp_init(cuda_train_context_t* ctx, int rank, int world, const void* nccl_unique_id);
void seraph_dp_finalize(cuda_train_context_t* ctx);
int seraph_dp_wait(cuda_train_context_t* ctx, int timeout_ms);
int seraph_dp_world(cuda_train_context_t* ctx);
/* For a command-line trainer run as one process per GPU (the reference's tools/seraph_train_cuda.c runs a single process):
 * env: rank and world from SERAPH_DP_RANK / SERAPH_DP_WORLD, else RANK / WORLD_SIZE (0, 1 when unset); returns 0 or 1 (inconsistent).
 * init_from_env: seraph_dp_init for that rank, the communicator id carried from rank 0 through the file SERAPH_DP_ID_FILE
 *   (default /tmp/seraph_dp_id.<MASTER_PORT>); the other ranks wait up to two minutes for it.
 * shard_samples: this rank's contiguous share (num_samples / world samples) of what train_load_data left in the state
 *   (src/train.c:812), moved to the front of sample_offsets, num_train_tokens set to the share's end; returns the first
 *   sample's original index or -1.
 * all_min: the smallest value any rank passed; with 1 = "I have a batch" a trainer stops all ranks together. */
int seraph_dp_env(int* rank, int* world);
int seraph_dp_init_from_env(cuda_train_context_t* ctx);
int seraph_dp_shard_samples(int* sample_offsets, int* num_samples, int* num_train_tokens, int rank, int world);
int seraph_dp_all_min(cuda_train_context_t* ctx, int value);

/* A train_state_t built in memory from flat float arrays, for callers that hold
 * the weights already (the reference only builds one from a model directory,
 * src/train.c:7854).  Flat parameter order: embed [V,d], final_norm [d], then
 * per layer q, k, v, o, gate, up, down, in_norm, post_norm.  `which`: 0
 * weights, 1 gradients, 2 Adam m, 3 Adam v.  LoRA mask bits: 0 q, 1 k, 2 v,
 * 3 o, 4 gate, 5 up, 6 down; flat LoRA order: per layer, per selected adapter,
 * A [r,in] then B [out,r]. */
train_state_t* seraph_b200_state_create(int V, int d, int L, int Hq, int Hkv, int hd, int F, float theta, float lr, int accum);
/* weights only on the host: gradients and Adam moments live on the device alone */
train_state_t* seraph_b200_state_create_lean(int V, int d, int L, int Hq, int Hkv, int hd, int F, float theta, float lr, int accum);
void seraph_b200_state_free(train_state_t* st);
size_t seraph_b200_state_param_count(train_state_t* st);
void seraph_b200_state_set(train_state_t* st, int which, const float* flat);
void seraph_b200_state_get(train_state_t* st, int which, float* flat);
void seraph_b200_state_set_counters(train_state_t* st, int optimizer_step, int accumulation_counter);
void seraph_b200_state_get_counters(train_state_t* st, int* optimizer_step, int* accumulation_counter);
void seraph_b200_state_set_lr(train_state_t* st, float lr, int accum);
/* the state's trainable_weights_t (host FP32 master copies), e.g. for the reference's own checkpoint writer */
void* seraph_b200_state_weights(train_state_t* st);
/* config->use_qk_norm of a state built by seraph_b200_state_create (the reference sets it for --video, src/train.c:7867-7868) */
void seraph_b200_state_set_qk_norm(train_state_t* st, int on);
/* state->debug_nan_check (tools/seraph_train_cuda.c --debug-nan) and state->nan_detected */
void seraph_b200_state_set_debug_nan(train_state_t* st, int on);
int seraph_b200_state_nan_detected(train_state_t* st);
/* Turns the state into what the reference's train_init builds for LoRA training (src/train.c:7900-7909): full_weights = NULL
 * and state->model = the safetensors file at `path`, memory-mapped; the frozen base is then read from its BF16 tensors by
 * their Hugging Face names, as ensure_cuda_lora_base_weights does (src/train_cuda.c:1376-1460).  Returns 0 on success. */
int seraph_b200_state_attach_model_file(train_state_t* st, const char* path);
size_t seraph_b200_state_lora_count(train_state_t* st, int rank, int mask);
int seraph_b200_state_attach_lora(train_state_t* st, int rank, float alpha, int mask, const float* flat);
void seraph_b200_state_lora_get(train_state_t* st, int which, float* flat);

#ifdef __cplusplus
}
#endif
#endif
