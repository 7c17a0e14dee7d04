/*
 * ref_shim.c - flat C entry points around the UNMODIFIED reference sources.
 *
 * TEST INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile together with the
 * reference's own files, read in place from the reference checkout; nothing
 * of the reference is copied here.  Outputs go to oracle/_ref/.
 *
 *   -DREF_SHIM_CPU : wraps the reference's CPU training path
 *                    (train_forward_fp32 / train_step / lora_backward and the
 *                    static adamw_update_tensor, reached by including train.c
 *                    into this translation unit).
 *   -DREF_SHIM_CUDA: wraps the reference's CUDA backend
 *                    (cuda_train_step_gpu_full_batch and the per-op calls).
 *
 * The train_state_t is built by hand from flat arrays so that no model files
 * or tokenizer are needed.  Flat parameter order: see oracle/ref_step.c.
 */
#include <stdlib.h>
#include <string.h>
#include <stdio.h>

#ifdef REF_SHIM_CPU
#include "train.c"          /* found through -I<reference>/src */
#else
#include "train.h"
#include "train_cuda.h"
#endif

typedef struct {
    train_state_t st;
    model_config_t cfg;
    train_config_t tc;
    trainable_weights_t w;
    void* cuda;
} shim_t;

static void wt_alloc(weight_tensor_t* t, size_t n) {
    t->weight = calloc(n, 4); t->grad = calloc(n, 4); t->m = calloc(n, 4); t->v = calloc(n, 4); t->size = n;
}
static void wt_free(weight_tensor_t* t) { free(t->weight); free(t->grad); free(t->m); free(t->v); }

/* visit every tensor in the flat order */
typedef void (*visit_fn)(weight_tensor_t*, void*);
static void visit(shim_t* s, visit_fn f, void* arg) {
    f(&s->w.embed_tokens, arg); f(&s->w.final_norm, arg);
    for (int l = 0; l < s->w.num_layers; l++) {
        layer_weights_t* y = &s->w.layers[l];
        f(&y->q_proj, arg); f(&y->k_proj, arg); f(&y->v_proj, arg); f(&y->o_proj, arg);
        f(&y->gate_proj, arg); f(&y->up_proj, arg); f(&y->down_proj, arg);
        f(&y->input_norm, arg); f(&y->post_norm, arg);
    }
}

void* refshim_create(int V, int d, int L, int Hq, int Hkv, int hd, int F, float theta,
                     int max_seq, float lr, int accum) {
    shim_t* s = calloc(1, sizeof(shim_t));
    model_config_t* c = &s->cfg;
    c->vocab_size = V; c->hidden_size = d; c->num_hidden_layers = L; c->intermediate_size = F;
    c->num_attention_heads = Hq; c->num_key_value_heads = Hkv; c->head_dim = hd; c->kv_dim = Hkv * hd;
    c->rms_norm_eps = 1e-5f; c->rope_theta = theta; c->max_position_embeddings = max_seq;
    c->tie_word_embeddings = 1;
    size_t qd = (size_t)Hq * hd, kvd = (size_t)Hkv * hd;
    s->w.num_layers = L; s->w.hidden_size = d; s->w.intermediate_size = F; s->w.vocab_size = V;
    s->w.layers = calloc(L, sizeof(layer_weights_t));
    wt_alloc(&s->w.embed_tokens, (size_t)V * d); wt_alloc(&s->w.final_norm, d);
    for (int l = 0; l < L; l++) {
        layer_weights_t* y = &s->w.layers[l];
        wt_alloc(&y->q_proj, qd * d); wt_alloc(&y->k_proj, kvd * d); wt_alloc(&y->v_proj, kvd * d);
        wt_alloc(&y->o_proj, (size_t)d * qd); wt_alloc(&y->gate_proj, (size_t)F * d);
        wt_alloc(&y->up_proj, (size_t)F * d); wt_alloc(&y->down_proj, (size_t)d * F);
        wt_alloc(&y->input_norm, d); wt_alloc(&y->post_norm, d);
    }
    s->st.config = c; s->st.train_cfg = &s->tc; s->st.use_full_training = 1; s->st.full_weights = &s->w;
    s->st.learning_rate = lr; s->st.gradient_accumulation_steps = accum;
#ifdef REF_SHIM_CPU
    s->st.act_cache = activation_cache_alloc(L, d, F, (int)qd, (int)kvd, max_seq);
#endif
    return s;
}

static void f_free(weight_tensor_t* t, void* a) { (void)a; wt_free(t); }
void refshim_destroy(void* p) {
    shim_t* s = p;
#ifdef REF_SHIM_CUDA
    if (s->cuda) cuda_train_free(s->cuda);
#endif
    visit(s, f_free, NULL); free(s->w.layers); free(s);
}

typedef struct { float* flat; int which; int set; } io_t;
static void f_io(weight_tensor_t* t, void* a) {
    io_t* io = a;
    float* p = io->which == 0 ? t->weight : io->which == 1 ? t->grad : io->which == 2 ? t->m : t->v;
    if (io->set) memcpy(p, io->flat, t->size * 4); else memcpy(io->flat, p, t->size * 4);
    io->flat += t->size;
}
/* which: 0 weight, 1 grad, 2 m, 3 v */
void refshim_set(void* p, int which, const float* flat) { io_t io = {(float*)flat, which, 1}; visit(p, f_io, &io); }
void refshim_get(void* p, int which, float* flat) { io_t io = {flat, which, 0}; visit(p, f_io, &io); }
void refshim_set_counters(void* p, int optimizer_step, int accumulation_counter) {
    shim_t* s = p; s->st.optimizer_step = optimizer_step; s->st.accumulation_counter = accumulation_counter;
}

#ifdef REF_SHIM_CPU
/* forward only: logits [n,V] of the reference's exact CPU forward (src/train.c:3219) */
int refshim_forward(void* p, const int* tokens, int n, float* logits_out) {
    shim_t* s = p;
    float* lg = train_forward_fp32(&s->st, (int*)tokens, n, NULL);
    if (!lg) return -1;
    memcpy(logits_out, lg, (size_t)n * s->cfg.vocab_size * 4);
    free(lg);
    return 0;
}
/* the reference's whole CPU step (src/train.c:6808): forward, loss, truncated backward, AdamW */
float refshim_train_step(void* p, const int* tokens, int n) {
    shim_t* s = p; return train_step(&s->st, (int*)tokens, n);
}
/* static adamw_update_tensor (src/train.c:1710) on caller arrays */
void refshim_adamw(float* w, float* g, float* m, float* v, size_t n,
                   float lr, float b1, float b2, float wd, float eps, int step) {
    weight_tensor_t t = {w, g, m, v, n};
    adamw_update_tensor(&t, lr, b1, b2, wd, eps, step);
}
/* lora_backward (src/lora.c:150) on caller arrays; gA/gB accumulate */
void refshim_lora_backward(const float* A, const float* B, float* gA, float* gB, const float* x, const float* dy,
                           float* dx, int T, int in, int out, int rank, float alpha) {
    lora_adapter_t a; memset(&a, 0, sizeof a);
    a.in_dim = in; a.out_dim = out; a.rank = rank; a.alpha = alpha;
    a.A = (float*)A; a.B = (float*)B; a.grad_A = gA; a.grad_B = gB;
    lora_backward(&a, x, dy, dx, T);
}
void refshim_loss_gradient(float* g, float* logits, int target, int V) { compute_loss_gradient(g, logits, target, V); }
#endif

#ifdef REF_SHIM_CUDA
int refshim_cuda_init(void* p, int device, int flash) {
    shim_t* s = p;
    s->cuda = cuda_train_init(device);
    if (!s->cuda) return -1;
    ((cuda_train_context_t*)s->cuda)->use_flash_attn = flash;
    /* the reference CLI sizes this before the first step (tools/seraph_train_cuda.c:215-216) */
    ((cuda_train_context_t*)s->cuda)->max_fwd_buffer_size =
        (size_t)s->cfg.max_position_embeddings * (size_t)s->cfg.intermediate_size * sizeof(float);
    s->st.cuda_ctx = s->cuda;
    return 0;
}
/* one packed full-weight step on the reference CUDA backend (src/train_cuda.c:1966);
 * afterwards refshim_cuda_download makes grads/weights readable through refshim_get */
float refshim_cuda_step(void* p, const int* tokens, int T, const int* seq_starts, int B) {
    shim_t* s = p;
    return cuda_train_step_gpu_full_batch(&s->st, (int*)tokens, T, (int*)seq_starts, B, s->cuda);
}
void refshim_cuda_download(void* p) {
    shim_t* s = p;
    cuda_download_gpu_gradients(s->cuda, &s->st);
    cuda_download_full_weights(s->cuda, &s->st);
}
void* refshim_cuda_ctx(void* p) { return ((shim_t*)p)->cuda; }

/* The reference's packed causal attention on caller arrays: forward with the flash kernel (so that it writes the
 * log-sum-exp, src/cuda_train_context.cu:1289) and backward with flash_attention_bwd_packed_kernel (:2012) through the
 * reference's own wrappers (:3107).  Q, dO, O, dQ are [T, Hq*hd]; K, V, dK, dV [T, Hkv*hd]; lse [T, Hq].  dK and dV are
 * zeroed first (the kernel adds into them with atomics, as src/train_cuda.c:2234-2237 does before calling it).
 * ms[0], ms[1]: device time of the forward and of the backward call, the mean over `reps` repetitions after one
 * untimed run.  Returns 0, or -1 when the context or a buffer could not be made. */
#include <cuda_runtime_api.h>
int refshim_cuda_attention(int device, const float* Q, const float* K, const float* V, const float* dO, const int* seq_starts,
                           int B, int T, int Hq, int Hkv, int hd, int max_seq, int reps,
                           float* O, float* lse, float* dQ, float* dK, float* dV, float* ms) {
    cuda_train_context_t* c = cuda_train_init(device);
    if (!c) return -1;
    c->use_flash_attn = 1;
    size_t nq = (size_t)T * Hq * hd, nkv = (size_t)T * Hkv * hd, nl = (size_t)T * Hq;
    cuda_buffer_t* b[12]; size_t sz[12] = {nq, nkv, nkv, nq, nq, nl, nq, nkv, nkv, (size_t)B + 1, 0, 0};
    int rc = 0;
    for (int i = 0; i < 10; i++) { b[i] = cuda_train_buffer_create(c, sz[i] * 4); if (!b[i]) rc = -1; }
    if (rc == 0) {
        cuda_train_buffer_upload(c, b[0], Q, nq); cuda_train_buffer_upload(c, b[1], K, nkv); cuda_train_buffer_upload(c, b[2], V, nkv);
        cuda_train_buffer_upload(c, b[3], dO, nq); cuda_train_buffer_upload_u32(c, b[9], (const uint32_t*)seq_starts, (size_t)B + 1);
        cudaEvent_t e0, e1, e2; cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
        float tf = 0.f, tb = 0.f;
        for (int r = 0; r <= reps; r++) {
            cuda_train_fill_buffer(c, b[7], 0, nkv * 4); cuda_train_fill_buffer(c, b[8], 0, nkv * 4);
            cudaEventRecord(e0, (cudaStream_t)c->stream);
            cuda_train_batch_attention_packed(c, b[0], b[1], b[2], b[4], b[5], b[9], T, B, Hq, Hkv, hd, max_seq);
            cudaEventRecord(e1, (cudaStream_t)c->stream);
            cuda_train_batch_attention_backward_packed(c, b[0], b[1], b[2], b[4], b[5], b[3], b[6], b[7], b[8], b[9], T, B, Hq, Hkv, hd, max_seq);
            cudaEventRecord(e2, (cudaStream_t)c->stream);
            cuda_train_sync(c);
            if (cudaGetLastError() != cudaSuccess) { rc = -2; break; }
            if (r > 0) { float a = 0.f, d = 0.f; cudaEventElapsedTime(&a, e0, e1); cudaEventElapsedTime(&d, e1, e2); tf += a; tb += d; }
        }
        if (ms && reps > 0) { ms[0] = tf / reps; ms[1] = tb / reps; }
        if (rc == 0) {
            cuda_train_buffer_download(c, b[4], O, nq); cuda_train_buffer_download(c, b[5], lse, nl);
            cuda_train_buffer_download(c, b[6], dQ, nq); cuda_train_buffer_download(c, b[7], dK, nkv); cuda_train_buffer_download(c, b[8], dV, nkv);
        }
        cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    }
    for (int i = 0; i < 10; i++) if (b[i]) cuda_train_buffer_free(c, b[i]);
    cuda_train_free(c);
    return rc;
}
#endif
