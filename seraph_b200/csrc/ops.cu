// ops.cu - the per-op C ABI of the reference (include/cuda_train_context.h:262-325),
// implemented over this library's kernels.  Same names, argument meaning and
// error behaviour: functions are void, print CUDA failures to stderr and
// return (src/cuda_train_context.cu:90-106); seraph_b200_last_status() adds a
// queryable code.  All work is ordered on ctx->stream.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include "sb_internal.h"

extern "C" {

int sb_embedding_segments(sb_ctx_t* c, int T, int V, int* rows_out, int* counts_out, int* sorted_pos_out);

// grow-only per-token index buffers shared by the packed ops and the step
int sb_ensure_tokens(sb_ctx_t* c, int T, int B) {
    if (T > c->seq_cap || !c->tokens) {
        cudaStreamSynchronize((cudaStream_t)c->pub.stream);
        if (c->tokens) cudaFree(c->tokens);
        int cap = T < 1024 ? 1024 : T;
        void* p = NULL;
        if (sb_check(c, cudaMalloc(&p, (size_t)cap * 4 * sizeof(uint32_t)), "token buffers")) { c->tokens = NULL; c->seq_cap = 0; return 1; }
        c->tokens = (uint32_t*)p; c->targets = c->tokens + cap; c->pos_ids = c->targets + cap; c->seq_ids = c->pos_ids + cap;
        c->seq_cap = cap;
    }
    static const int kMinB = 64;
    size_t need = (size_t)(B + 1 < kMinB ? kMinB : B + 1);
    if (!c->seq_starts || (size_t)c->seq_starts_cap < need) {
        cudaStreamSynchronize((cudaStream_t)c->pub.stream);
        if (c->seq_starts) cudaFree(c->seq_starts);
        void* p = NULL;
        if (sb_check(c, cudaMalloc(&p, need * sizeof(uint32_t)), "seq_starts")) { c->seq_starts = NULL; return 1; }
        c->seq_starts = (uint32_t*)p;
        c->seq_starts_cap = (int)need;
    }
    return 0;
}

int sb_set_host_seq(sb_ctx_t* c, const int* starts, int B) {
    if (B + 1 > c->h_seq_cap) {
        int cap = B + 1 < 64 ? 64 : B + 1;
        int* p = (int*)realloc(c->h_seq, sizeof(int) * cap);
        if (!p) { c->h_seq_n = 0; return 1; }
        c->h_seq = p; c->h_seq_cap = cap;
    }
    for (int b = 0; b <= B; b++) c->h_seq[b] = starts[b];
    for (int b = 0; b < B; b++) if (starts[b + 1] < starts[b]) { c->h_seq_n = 0; return 1; }
    c->h_seq_n = B;
    return 0;
}

// index tables for one packed batch described by a device seq_starts array; the boundaries are also read back
// to the host (small synchronous copy) because the tensor-core attention builds its tile maps per sequence
static int index_from_device_starts(sb_ctx_t* c, const uint32_t* d_starts, int B, int T) {
    if (sb_ensure_tokens(c, T, B)) return 1;
    sb_seq_index(c, d_starts, B, T, c->pos_ids, c->seq_ids);
    c->h_seq_n = 0;
    if (B > 0 && B < (1 << 20)) {
        int* tmp = (int*)malloc(sizeof(int) * (size_t)(B + 1));
        if (tmp) {
            cudaStreamSynchronize((cudaStream_t)c->pub.stream);
            if (cudaMemcpy(tmp, d_starts, sizeof(int) * (size_t)(B + 1), cudaMemcpyDeviceToHost) == cudaSuccess && tmp[0] == 0 && tmp[B] == T)
                sb_set_host_seq(c, tmp, B);
            free(tmp);
        }
    }
    return 0;
}
// single sequence of `len` rows (len may exceed T so that no row counts as "last")
static int index_single(sb_ctx_t* c, int T, int len) {
    if (sb_ensure_tokens(c, T, 1)) return 1;
    uint32_t h[2] = {0u, (uint32_t)len};
    if (sb_check(c, cudaMemcpyAsync(c->seq_starts, h, sizeof h, cudaMemcpyHostToDevice, (cudaStream_t)c->pub.stream), "seq_starts upload")) return 1;
    sb_seq_index(c, c->seq_starts, 1, T, c->pos_ids, c->seq_ids);
    if (len == T) { int hs[2] = {0, T}; sb_set_host_seq(c, hs, 1); } else c->h_seq_n = 0;
    return 0;
}

#define CTX_OR_RETURN(ctx) sb_ctx_t* c = sb_priv(ctx); if (!c) { fprintf(stderr, "seraph_b200: invalid context\n"); return; }
#define NEED(...) do { const void* ptrs_[] = {__VA_ARGS__}; for (size_t i_ = 0; i_ < sizeof(ptrs_) / sizeof(ptrs_[0]); i_++) \
        if (!ptrs_[i_]) { sb_set_status(c, SB_ERR_ARG); return; } } while (0)

// ---------------------------------------------------------------------------
// GEMM dispatch
// ---------------------------------------------------------------------------
void sb_gemm(sb_ctx_t* c, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc) {
    if (M <= 0 || N <= 0 || K < 0) return;
    int mode = c->pub.use_bf16 ? SB_GEMM_BF16 : c->gemm_mode;
    sb_amax_forget(c, C);                 /* a maximum left for C by an earlier writer is void; the tensor-core launch leaves a new one when asked */
    if (mode != SB_GEMM_SIMT && sb_gemm_tc(c, A, B, C, M, N, K, tA, tB, acc, mode) == 0) return;
    int t = sb_tick_begin(c, SB_CLS_GEMM);
    sb_gemm_simt(c, A, B, C, M, N, K, tA, tB, acc);
    sb_tick_end(c, t, 2.0 * M * N * K, 4.0 * ((double)M * K + (double)N * K + (double)M * N * (acc ? 2 : 1)));
}

// reference: cuda_train_matmul, src/cuda_train_context.cu:2697
void cuda_train_matmul(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, int M, int N, int K) {
    CTX_OR_RETURN(ctx); NEED(A, B, C);
    int op = sb_prof_begin(c, "matmul");
    sb_gemm(c, A->data, B->data, C->data, M, N, K, 0, 0, 0);
    sb_prof_end(c, op, (size_t)2 * M * N * K, ((size_t)M * K + (size_t)K * N + (size_t)M * N) * 4);
}
// reference: cuda_train_matmul_transpose, src/cuda_train_context.cu:2702
void cuda_train_matmul_transpose(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C,
                                 int M, int N, int K, int transpose_A, int transpose_B, int accumulate) {
    CTX_OR_RETURN(ctx); NEED(A, B, C);
    int op = sb_prof_begin(c, (transpose_A && !transpose_B) ? "matmul_At" : (!transpose_A && transpose_B) ? "matmul_Bt" : "matmul");
    sb_gemm(c, A->data, B->data, C->data, M, N, K, transpose_A, transpose_B, accumulate);
    sb_prof_end(c, op, (size_t)2 * M * N * K, ((size_t)M * K + (size_t)K * N + (size_t)M * N * (accumulate ? 2 : 1)) * 4);
}

// ---------------------------------------------------------------------------
// Forward ops (src/cuda_train_context.cu:2709-2960)
// ---------------------------------------------------------------------------
void cuda_train_silu(cuda_train_context_t* ctx, cuda_buffer_t* in, cuda_buffer_t* out, size_t count) {
    CTX_OR_RETURN(ctx); NEED(in, out);
    int op = sb_prof_begin(c, "silu"); sb_silu(c, in->data, out->data, count); sb_prof_end(c, op, 0, count * 8);
}
void cuda_train_rmsnorm(cuda_train_context_t* ctx, cuda_buffer_t* in, cuda_buffer_t* scale, cuda_buffer_t* out, int rows, int cols, float eps) {
    CTX_OR_RETURN(ctx); NEED(in, scale, out);
    int op = sb_prof_begin(c, "rmsnorm"); sb_rmsnorm(c, in->data, scale->data, out->data, rows, cols, eps);
    sb_prof_end(c, op, 0, (size_t)rows * cols * 8);
}
void cuda_train_softmax(cuda_train_context_t* ctx, cuda_buffer_t* in, cuda_buffer_t* out, int rows, int cols) {
    CTX_OR_RETURN(ctx); NEED(in, out);
    int op = sb_prof_begin(c, "softmax"); sb_softmax(c, in->data, out->data, rows, cols); sb_prof_end(c, op, 0, (size_t)rows * cols * 8);
}
void cuda_train_add(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, size_t count) {
    CTX_OR_RETURN(ctx); NEED(A, B, C);
    int op = sb_prof_begin(c, "add"); sb_add(c, A->data, B->data, C->data, count); sb_prof_end(c, op, 0, count * 12);
}
void cuda_train_mul(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, size_t count) {
    CTX_OR_RETURN(ctx); NEED(A, B, C);
    int op = sb_prof_begin(c, "mul"); sb_mul(c, A->data, B->data, C->data, count); sb_prof_end(c, op, 0, count * 12);
}
void cuda_train_scale(cuda_train_context_t* ctx, cuda_buffer_t* A, size_t count, float alpha) {
    CTX_OR_RETURN(ctx); NEED(A);
    int op = sb_prof_begin(c, "scale"); sb_scale(c, A->data, count, alpha); sb_prof_end(c, op, 0, count * 8);
}
void cuda_train_embed_lookup(cuda_train_context_t* ctx, cuda_buffer_t* tokens_u32, cuda_buffer_t* embed, cuda_buffer_t* out,
                             int seq_len, int hidden_size, int vocab_size) {
    CTX_OR_RETURN(ctx); NEED(tokens_u32, embed, out);
    int op = sb_prof_begin(c, "embed_lookup");
    sb_embed_lookup(c, (const uint32_t*)tokens_u32->data, embed->data, out->data, seq_len, hidden_size, vocab_size);
    sb_prof_end(c, op, 0, (size_t)seq_len * hidden_size * 8);
}

static float theta_or_default(float t) { return t > 0 ? t : 10000.0f; }

void cuda_train_rope(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, int seq_len, int num_heads, int head_dim, float rope_theta) {
    CTX_OR_RETURN(ctx); NEED(x_in, x_out);
    if (seq_len <= 0 || index_single(c, seq_len, seq_len)) return;
    int op = sb_prof_begin(c, "rope");
    sb_rope(c, x_in->data, x_out->data, c->pos_ids, seq_len, num_heads, head_dim, theta_or_default(rope_theta), seq_len, 0);
    sb_prof_end(c, op, 0, (size_t)seq_len * num_heads * head_dim * 8);
}
void cuda_train_rope_backward(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, int seq_len, int num_heads, int head_dim, float rope_theta) {
    CTX_OR_RETURN(ctx); NEED(x_in, x_out);
    if (seq_len <= 0 || index_single(c, seq_len, seq_len)) return;
    int op = sb_prof_begin(c, "rope_bwd");
    sb_rope(c, x_in->data, x_out->data, c->pos_ids, seq_len, num_heads, head_dim, theta_or_default(rope_theta), seq_len, 1);
    sb_prof_end(c, op, 0, (size_t)seq_len * num_heads * head_dim * 8);
}
void cuda_train_rope_packed(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, cuda_buffer_t* seq_starts,
                            int total_tokens, int batch_size, int num_heads, int head_dim, float rope_theta) {
    CTX_OR_RETURN(ctx); NEED(x_in, x_out, seq_starts);
    if (total_tokens <= 0 || index_from_device_starts(c, (const uint32_t*)seq_starts->data, batch_size, total_tokens)) return;
    int op = sb_prof_begin(c, "rope_packed");
    sb_rope(c, x_in->data, x_out->data, c->pos_ids, total_tokens, num_heads, head_dim, theta_or_default(rope_theta), total_tokens, 0);
    sb_prof_end(c, op, 0, (size_t)total_tokens * num_heads * head_dim * 8);
}
void cuda_train_rope_backward_packed(cuda_train_context_t* ctx, cuda_buffer_t* x_in, cuda_buffer_t* x_out, cuda_buffer_t* seq_starts,
                                     int total_tokens, int batch_size, int num_heads, int head_dim, float rope_theta) {
    CTX_OR_RETURN(ctx); NEED(x_in, x_out, seq_starts);
    if (total_tokens <= 0 || index_from_device_starts(c, (const uint32_t*)seq_starts->data, batch_size, total_tokens)) return;
    int op = sb_prof_begin(c, "rope_bwd_packed");
    sb_rope(c, x_in->data, x_out->data, c->pos_ids, total_tokens, num_heads, head_dim, theta_or_default(rope_theta), total_tokens, 1);
    sb_prof_end(c, op, 0, (size_t)total_tokens * num_heads * head_dim * 8);
}

// lse_out may be NULL (the reference only fills it in its flash mode); here it is filled whenever given
void cuda_train_batch_attention(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V, cuda_buffer_t* out,
                                cuda_buffer_t* lse_out, int seq_len, int num_heads, int kv_heads, int head_dim) {
    CTX_OR_RETURN(ctx); NEED(Q, K, V, out);
    if (seq_len <= 0 || index_single(c, seq_len, seq_len)) return;
    int op = sb_prof_begin(c, "attention");
    sb_attention(c, Q->data, K->data, V->data, out->data, lse_out ? lse_out->data : NULL, c->seq_starts, c->seq_ids,
                 seq_len, num_heads, kv_heads, head_dim);
    sb_prof_end(c, op, (size_t)2 * seq_len * seq_len * num_heads * head_dim, 0);
}
void cuda_train_batch_attention_packed(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V, cuda_buffer_t* out,
                                       cuda_buffer_t* lse_out, cuda_buffer_t* seq_starts, int total_tokens, int batch_size,
                                       int num_heads, int kv_heads, int head_dim, int max_seq_in_batch) {
    CTX_OR_RETURN(ctx); NEED(Q, K, V, out, seq_starts);
    if (total_tokens <= 0 || index_from_device_starts(c, (const uint32_t*)seq_starts->data, batch_size, total_tokens)) return;
    int op = sb_prof_begin(c, "attention_packed");
    sb_attention(c, Q->data, K->data, V->data, out->data, lse_out ? lse_out->data : NULL, (const uint32_t*)seq_starts->data, c->seq_ids,
                 total_tokens, num_heads, kv_heads, head_dim);
    sb_prof_end(c, op, (size_t)2 * total_tokens * max_seq_in_batch * num_heads * head_dim, 0);
}

// ---------------------------------------------------------------------------
// Loss + backward ops (src/cuda_train_context.cu:2940-3200)
// ---------------------------------------------------------------------------
void cuda_train_cross_entropy_grad(cuda_train_context_t* ctx, cuda_buffer_t* logits, cuda_buffer_t* targets_u32, cuda_buffer_t* grad_logits,
                                   cuda_buffer_t* loss_rows, int rows, int cols) {
    CTX_OR_RETURN(ctx); NEED(logits, targets_u32, grad_logits, loss_rows);
    if (rows <= 0 || index_single(c, rows, rows + 1)) return;      // every row predicts
    int op = sb_prof_begin(c, "cross_entropy_grad");
    sb_cross_entropy(c, logits->data, (const uint32_t*)targets_u32->data, grad_logits->data, loss_rows->data,
                     c->pos_ids, c->seq_ids, c->seq_starts, rows, cols, rows);
    sb_prof_end(c, op, 0, (size_t)rows * cols * 12);
}
void cuda_train_cross_entropy_grad_packed(cuda_train_context_t* ctx, cuda_buffer_t* logits, cuda_buffer_t* targets_u32,
                                          cuda_buffer_t* grad_logits, cuda_buffer_t* loss_rows, cuda_buffer_t* seq_starts,
                                          int total_tokens, int batch_size, int vocab_size, int num_valid_predictions) {
    CTX_OR_RETURN(ctx); NEED(logits, targets_u32, grad_logits, loss_rows, seq_starts);
    if (total_tokens <= 0 || index_from_device_starts(c, (const uint32_t*)seq_starts->data, batch_size, total_tokens)) return;
    int op = sb_prof_begin(c, "cross_entropy_grad_packed");
    sb_cross_entropy(c, logits->data, (const uint32_t*)targets_u32->data, grad_logits->data, loss_rows->data,
                     c->pos_ids, c->seq_ids, (const uint32_t*)seq_starts->data, total_tokens, vocab_size, num_valid_predictions);
    sb_prof_end(c, op, 0, (size_t)total_tokens * vocab_size * 12);
}
// out[0] = sum(in[0..count)); deterministic (the reference adds block sums atomically)
void cuda_train_reduce_sum(cuda_train_context_t* ctx, cuda_buffer_t* in_buf, cuda_buffer_t* out_buf, size_t count) {
    CTX_OR_RETURN(ctx); NEED(in_buf, out_buf);
    int op = sb_prof_begin(c, "reduce_sum"); sb_reduce_sum(c, in_buf->data, out_buf->data, count); sb_prof_end(c, op, 0, count * 4);
}
void cuda_train_silu_backward(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* grad_output, cuda_buffer_t* grad_input, size_t count) {
    CTX_OR_RETURN(ctx); NEED(input, grad_output, grad_input);
    int op = sb_prof_begin(c, "silu_bwd"); sb_silu_backward(c, input->data, grad_output->data, grad_input->data, count);
    sb_prof_end(c, op, 0, count * 12);
}
void cuda_train_elementwise_mul_backward(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* grad_C,
                                         cuda_buffer_t* grad_A, cuda_buffer_t* grad_B, size_t count) {
    CTX_OR_RETURN(ctx); NEED(A, B, grad_C, grad_A, grad_B);
    int op = sb_prof_begin(c, "mul_bwd"); sb_mul_backward(c, A->data, B->data, grad_C->data, grad_A->data, grad_B->data, count);
    sb_prof_end(c, op, 0, count * 20);
}
// grad_scale is accumulated into, as in the reference (its kernel uses atomicAdd on it)
void cuda_train_rmsnorm_backward_batch(cuda_train_context_t* ctx, cuda_buffer_t* input, cuda_buffer_t* scale, cuda_buffer_t* grad_output,
                                       cuda_buffer_t* grad_input, cuda_buffer_t* grad_scale, int rows, int cols, float eps) {
    CTX_OR_RETURN(ctx); NEED(input, scale, grad_output, grad_input, grad_scale);
    int op = sb_prof_begin(c, "rmsnorm_bwd");
    sb_rmsnorm_backward(c, input->data, scale->data, grad_output->data, NULL, grad_input->data, grad_scale->data, rows, cols, eps);
    sb_prof_end(c, op, 0, (size_t)rows * cols * 12);
}
// Q or K normalised over the whole token row, in place (include/vulkan_backend.h:600, shaders/qk_norm.comp); rms_out may be NULL
void seraph_b200_qk_norm(cuda_train_context_t* ctx, cuda_buffer_t* qk, cuda_buffer_t* rms_out, int seq_len, int num_heads, int head_dim,
                         int use_qk_norm, float eps) {
    CTX_OR_RETURN(ctx); NEED(qk);
    if (!use_qk_norm || seq_len <= 0 || num_heads <= 0 || head_dim <= 0) return;
    int op = sb_prof_begin(c, "qk_norm");
    sb_qk_norm(c, qk->data, rms_out ? rms_out->data : NULL, seq_len, num_heads * head_dim, eps);
    sb_prof_end(c, op, 0, (size_t)seq_len * num_heads * head_dim * 8);
}
// its backward (the reference has none): qk_out and rms are what the forward call left; grad_in may alias grad_out
void seraph_b200_qk_norm_backward(cuda_train_context_t* ctx, cuda_buffer_t* qk_out, cuda_buffer_t* rms, cuda_buffer_t* grad_out,
                                  cuda_buffer_t* grad_in, int seq_len, int num_heads, int head_dim, int use_qk_norm, float eps) {
    CTX_OR_RETURN(ctx); NEED(qk_out, rms, grad_out, grad_in);
    if (seq_len <= 0 || num_heads <= 0 || head_dim <= 0) return;
    if (!use_qk_norm) {
        if (grad_in->data != grad_out->data) sb_copy(c, grad_in->data, grad_out->data, (size_t)seq_len * num_heads * head_dim * sizeof(float));
        return;
    }
    int op = sb_prof_begin(c, "qk_norm_bwd");
    sb_qk_norm_backward(c, qk_out->data, rms->data, grad_out->data, grad_in->data, seq_len, num_heads * head_dim, eps);
    sb_prof_end(c, op, 0, (size_t)seq_len * num_heads * head_dim * 12);
}
// grad_K and grad_V are accumulated into (callers zero them first, src/train_cuda.c:2234-2237); grad_Q is written.
// attn_out and lse must come from the forward call: this implementation always uses the log-sum-exp form.
void cuda_train_batch_attention_backward(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V,
                                         cuda_buffer_t* attn_out, cuda_buffer_t* lse, cuda_buffer_t* grad_out,
                                         cuda_buffer_t* grad_Q, cuda_buffer_t* grad_K, cuda_buffer_t* grad_V,
                                         int seq_len, int num_heads, int kv_heads, int head_dim) {
    CTX_OR_RETURN(ctx); NEED(Q, K, V, attn_out, lse, grad_out, grad_Q, grad_K, grad_V);
    if (seq_len <= 0 || index_single(c, seq_len, seq_len)) return;
    int op = sb_prof_begin(c, "attention_bwd");
    sb_attention_backward(c, Q->data, K->data, V->data, attn_out->data, lse->data, grad_out->data, grad_Q->data, grad_K->data,
                          grad_V->data, 1, c->seq_starts, c->seq_ids, 1, seq_len, num_heads, kv_heads, head_dim);
    sb_prof_end(c, op, (size_t)5 * seq_len * seq_len * num_heads * head_dim, 0);
}
void cuda_train_batch_attention_backward_packed(cuda_train_context_t* ctx, cuda_buffer_t* Q, cuda_buffer_t* K, cuda_buffer_t* V,
                                                cuda_buffer_t* attn_out, cuda_buffer_t* lse, cuda_buffer_t* grad_out,
                                                cuda_buffer_t* grad_Q, cuda_buffer_t* grad_K, cuda_buffer_t* grad_V,
                                                cuda_buffer_t* seq_starts, int total_tokens, int batch_size,
                                                int num_heads, int kv_heads, int head_dim, int max_seq_in_batch) {
    CTX_OR_RETURN(ctx); NEED(Q, K, V, attn_out, lse, grad_out, grad_Q, grad_K, grad_V, seq_starts);
    if (total_tokens <= 0 || index_from_device_starts(c, (const uint32_t*)seq_starts->data, batch_size, total_tokens)) return;
    int op = sb_prof_begin(c, "attention_bwd_packed");
    sb_attention_backward(c, Q->data, K->data, V->data, attn_out->data, lse->data, grad_out->data, grad_Q->data, grad_K->data,
                          grad_V->data, 1, (const uint32_t*)seq_starts->data, c->seq_ids, batch_size, total_tokens, num_heads, kv_heads, head_dim);
    sb_prof_end(c, op, (size_t)5 * total_tokens * max_seq_in_batch * num_heads * head_dim, 0);
}
void cuda_train_embedding_backward(cuda_train_context_t* ctx, cuda_buffer_t* tokens_u32, cuda_buffer_t* grad_hidden, cuda_buffer_t* grad_embed,
                                   int seq_len, int hidden_size, int vocab_size) {
    CTX_OR_RETURN(ctx); NEED(tokens_u32, grad_hidden, grad_embed);
    int op = sb_prof_begin(c, "embedding_bwd");
    sb_embedding_backward(c, (const uint32_t*)tokens_u32->data, grad_hidden->data, grad_embed->data, seq_len, hidden_size, vocab_size);
    sb_prof_end(c, op, 0, (size_t)seq_len * hidden_size * 12);
}

// reference: cuda_train_adamw_update, src/cuda_train_context.cu:3203 (no clipping there, none here)
void cuda_train_adamw_update(cuda_train_context_t* ctx, cuda_buffer_t* weight, cuda_buffer_t* grad, cuda_buffer_t* m, cuda_buffer_t* v,
                             float lr, float beta1, float beta2, float weight_decay, float eps, int step, size_t size,
                             const char* tensor_name, int rows, int cols) {
    (void)tensor_name; (void)rows; (void)cols;
    CTX_OR_RETURN(ctx); NEED(weight, grad, m, v);
    int op = sb_prof_begin(c, "adamw");
    sb_adamw(c, weight->data, grad->data, m->data, v->data, size, lr, beta1, beta2, weight_decay, eps, step, 1.0f, NULL, 0.f);
    sb_prof_end(c, op, 0, size * 28);
}

void cuda_train_nan_check(cuda_train_context_t* ctx, cuda_buffer_t* input, size_t count_floats, cuda_buffer_t* flags_u32, uint32_t flag_index) {
    CTX_OR_RETURN(ctx); NEED(input, flags_u32);
    sb_nan_check(c, input->data, count_floats, (uint32_t*)flags_u32->data, flag_index);
}

void cuda_train_set_profiler(cuda_train_context_t* ctx, cuda_profiler_t* prof) {
    sb_ctx_t* c = sb_priv(ctx);
    if (c) { c->profiler = prof; c->prof_depth = 0; c->tick_prof = 0; }
}

// Extension (test surface): C = op(A) op(B) as cuda_train_matmul_transpose does without accumulation, and the largest |C| the
// tensor-core kernel's epilogue (and its split-K fix-up) left behind for the next operand split.  Returns 1 with *amax_out set
// when the launch produced it, 0 when this shape does not run on that kernel (C is computed all the same), -1 on bad arguments.
int seraph_b200_matmul_amax(cuda_train_context_t* ctx, cuda_buffer_t* A, cuda_buffer_t* B, cuda_buffer_t* C, int M, int N, int K,
                            int transpose_A, int transpose_B, float* amax_out) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !A || !B || !C || !amax_out || M <= 0 || N <= 0 || K <= 0) return -1;
    sb_parts_open(c);
    sb_amax_announce(c, C->data, (size_t)M * N);
    sb_gemm(c, A->data, B->data, C->data, M, N, K, transpose_A, transpose_B, 0);
    float* w = sb_amax_lookup(c, C->data, (size_t)M * N);
    int got = 0;
    if (w && cudaMemcpyAsync(amax_out, w, sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)c->pub.stream) == cudaSuccess &&
        cudaStreamSynchronize((cudaStream_t)c->pub.stream) == cudaSuccess) got = 1;
    sb_parts_close(c);
    return got;
}

// ---------------------------------------------------------------------------
// LoRA (src/cuda_train_context.cu:3240-3290)
//   h = X A^T ; gB += dY^T (s h) ; gh = s (dY B) ; gA += gh^T X
// After the call `tmp` holds gh [T, r] (used by the exact-dX option of the step).
// ---------------------------------------------------------------------------
void sb_lora_backward(sb_ctx_t* c, const float* dY, const float* X, const float* A, const float* B, float* gA, float* gB,
                      float* tmp, int T, int in, int out, int r, float s) {
    sb_gemm_keep_forget(c, tmp);                       /* tmp is written twice below: parts a caller's keep region holds for it go stale */
    sb_gemm(c, X, A, tmp, T, r, in, 0, 1, 0);
    sb_scale(c, tmp, (size_t)T * r, s);
    sb_gemm(c, dY, tmp, gB, out, r, T, 1, 0, 1);
    sb_gemm_keep_forget(c, tmp);
    sb_gemm(c, dY, B, tmp, T, r, out, 0, 0, 0);
    sb_scale(c, tmp, (size_t)T * r, s);
    sb_gemm(c, tmp, X, gA, r, in, T, 1, 0, 1);
}

void cuda_train_lora_backward(cuda_train_context_t* ctx, cuda_buffer_t* grad_output, cuda_buffer_t* input, cuda_buffer_t* A, cuda_buffer_t* B,
                              cuda_buffer_t* gA, cuda_buffer_t* gB, cuda_buffer_t* hidden_tmp,
                              int seq_len, int in_dim, int out_dim, int rank, float scale) {
    CTX_OR_RETURN(ctx); NEED(grad_output, input, A, B, gA, gB, hidden_tmp);
    int op = sb_prof_begin(c, "lora_backward");
    sb_lora_backward(c, grad_output->data, input->data, A->data, B->data, gA->data, gB->data, hidden_tmp->data,
                     seq_len, in_dim, out_dim, rank, scale);
    sb_prof_end(c, op, (size_t)2 * seq_len * rank * (in_dim + out_dim) * 2, 0);
}

// ---------------------------------------------------------------------------
// Extension: the integer tables of the last embedding backward (test surface
// for "row indices and token counts are bit-exact")
// ---------------------------------------------------------------------------
int seraph_b200_embedding_segments(cuda_train_context_t* ctx, int T, int V, int* rows_out, int* counts_out, int* sorted_pos_out) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !rows_out || !counts_out || !sorted_pos_out) return -1;
    return sb_embedding_segments(c, T, V, rows_out, counts_out, sorted_pos_out);
}

// fused SwiGLU ops (no counterpart in the reference API; its step uses silu, mul, mul_backward, silu_backward)
void seraph_b200_swiglu(cuda_train_context_t* ctx, cuda_buffer_t* gate, cuda_buffer_t* up, cuda_buffer_t* out, size_t count) {
    CTX_OR_RETURN(ctx); NEED(gate, up, out);
    sb_swiglu(c, gate->data, up->data, out->data, count);
}
void seraph_b200_swiglu_backward(cuda_train_context_t* ctx, cuda_buffer_t* gate, cuda_buffer_t* up, cuda_buffer_t* grad_out,
                                 cuda_buffer_t* grad_gate, cuda_buffer_t* grad_up, size_t count) {
    CTX_OR_RETURN(ctx); NEED(gate, up, grad_out, grad_gate, grad_up);
    int op = sb_prof_begin(c, "swiglu_bwd");
    sb_swiglu_backward(c, gate->data, up->data, grad_out->data, grad_gate->data, grad_up->data, count);
    sb_prof_end(c, op, 0, count * 20);
}

// device timer on the context's stream (CUDA events), for callers that measure through the C ABI
static cudaEvent_t g_ev[2];
static int g_ev_init = 0;
void seraph_b200_timer_start(cuda_train_context_t* ctx) {
    if (!ctx) return;
    if (!g_ev_init) { cudaEventCreate(&g_ev[0]); cudaEventCreate(&g_ev[1]); g_ev_init = 1; }
    cudaEventRecord(g_ev[0], (cudaStream_t)ctx->stream);
}
float seraph_b200_timer_stop(cuda_train_context_t* ctx) {
    if (!ctx || !g_ev_init) return -1.0f;
    cudaEventRecord(g_ev[1], (cudaStream_t)ctx->stream);
    cudaEventSynchronize(g_ev[1]);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, g_ev[0], g_ev[1]);
    return ms;
}

}  // extern "C"
