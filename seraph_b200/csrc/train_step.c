/*
 * train_step.c - host orchestration of the training step, in C.
 *
 * Implements the step-level C ABI of the reference (include/train_cuda.h:12-64,
 * src/train_cuda.c): cuda_train_step_gpu_full[_batch], cuda_train_step_gpu_lora[_batch],
 * cuda_download_full_weights, cuda_download_gpu_gradients, cuda_download_lora_weights,
 * cuda_eval_forward, cuda_evaluate, cuda_train_zero_lora_grads, cuda_train_free.
 *
 * What is different from the reference's op list (src/train_cuda.c:2081-2287),
 * with identical results:
 *   - weights, gradients and both Adam moments live in four contiguous arenas
 *     (one memset zeroes all gradients, one kernel launch is the whole AdamW
 *     step, gradient buckets for data parallel are plain ranges);
 *   - activations are written straight into their per-layer cache slots (the
 *     reference copies every one of them, 12 device copies per layer);
 *   - residual adds ride on the GEMM's `C +=` epilogue; the residual-gradient
 *     add is fused into the RMSNorm backward; SwiGLU forward/backward are one
 *     kernel each; dK/dV need no zero fill (attention backward owns them).
 * The LoRA steps follow the complete chain rule of the reference's Vulkan
 * LoRA step (src/train.c:6095-6186 forward adds, :6287-6615 backward), not the
 * reference CUDA LoRA step, which feeds the LM-head gradient to every adapter
 * (src/train_cuda.c:1847-1906).
 */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

int sb_ensure_tokens(sb_ctx_t* c, int T, int B);
int sb_dp_bucket_ready(sb_ctx_t* c, float* p, size_t n);      /* dp.c: no-ops when not data parallel */
int sb_dp_bucket_ready_last(sb_ctx_t* c, float* p, size_t n);
int sb_dp_join(sb_ctx_t* c);
int sb_dp_mark_partial(sb_ctx_t* c);
int sb_dp_wait_partial(sb_ctx_t* c);

#define RMS_EPS 1e-5f   /* hard-coded in every training path of the reference (src/train_cuda.c:1984) */

/* ------------------------------------------------------------------------ */
/* geometry                                                                  */
/* ------------------------------------------------------------------------ */
static size_t layout_offsets(int V, int d, int L, int qd, int kvd, int F, sb_layer_off_t* off) {
    size_t n = (size_t)V * d + (size_t)d;      /* embed, final_norm */
    for (int l = 0; l < L; l++) {
        sb_layer_off_t o;
        o.q = n; n += (size_t)qd * d;
        o.k = n; n += (size_t)kvd * d;
        o.v = n; n += (size_t)kvd * d;
        o.o = n; n += (size_t)d * qd;
        o.gate = n; n += (size_t)F * d;
        o.up = n; n += (size_t)F * d;
        o.down = n; n += (size_t)d * F;
        o.in_norm = n; n += (size_t)d;
        o.post_norm = n; n += (size_t)d;
        if (off) off[l] = o;
    }
    return n;
}

static void lora_dims(const sb_ctx_t* c, int a, int* in, int* out) {
    switch (a) {
        case 0: *in = c->d; *out = c->qd; break;
        case 1: case 2: *in = c->d; *out = c->kvd; break;
        case 3: *in = c->qd; *out = c->d; break;
        case 4: case 5: *in = c->d; *out = c->F; break;
        default: *in = c->F; *out = c->d; break;
    }
}
static size_t lora_layer_params(const sb_ctx_t* c) {
    size_t n = 0;
    for (int a = 0; a < 7; a++) if (c->lora_mask & (1 << a)) { int in, out; lora_dims(c, a, &in, &out); n += (size_t)c->lora_rank * in + (size_t)out * c->lora_rank; }
    return n;
}
/* offset of A of adapter a in layer l; B follows at + rank*in */
static size_t lora_off(const sb_ctx_t* c, int l, int a) {
    size_t n = lora_layer_params(c) * (size_t)l;
    for (int b = 0; b < a; b++) if (c->lora_mask & (1 << b)) { int in, out; lora_dims(c, b, &in, &out); n += (size_t)c->lora_rank * in + (size_t)out * c->lora_rank; }
    return n;
}

/* the same for the rank-padded working copies */
static size_t lora_layer_params_pad(const sb_ctx_t* c) {
    size_t n = 0;
    for (int a = 0; a < 7; a++) if (c->lora_mask & (1 << a)) { int in, out; lora_dims(c, a, &in, &out); n += (size_t)c->lora_R * in + (size_t)out * c->lora_R; }
    return n;
}
static size_t lora_off_pad(const sb_ctx_t* c, int l, int a) {
    size_t n = lora_layer_params_pad(c) * (size_t)l;
    for (int b = 0; b < a; b++) if (c->lora_mask & (1 << b)) { int in, out; lora_dims(c, b, &in, &out); n += (size_t)c->lora_R * in + (size_t)out * c->lora_R; }
    return n;
}

static cudaStream_t S(sb_ctx_t* c) { return (cudaStream_t)c->pub.stream; }

static cuda_buffer_t* view(float* p, size_t floats) {
    cuda_buffer_t* b = (cuda_buffer_t*)malloc(sizeof(cuda_buffer_t));
    if (b) { b->data = p; b->size = floats * sizeof(float); }
    return b;
}
static cuda_buffer_t** view_array(int n) { return (cuda_buffer_t**)calloc((size_t)n, sizeof(cuda_buffer_t*)); }
static void free_view_array(cuda_buffer_t** a, int n) { if (!a) return; for (int i = 0; i < n; i++) free(a[i]); free(a); }

/* ------------------------------------------------------------------------ */
/* resident model                                                            */
/* ------------------------------------------------------------------------ */
static void free_model(sb_ctx_t* c) {
    cuda_train_context_t* p = &c->pub;
    int L = c->L;
    sb_parts_unregister(c, 0);
    if (c->W) cudaFree(c->W);
    if (c->G) cudaFree(c->G);
    if (c->M) cudaFree(c->M);
    if (c->Vv) cudaFree(c->Vv);
    c->W = c->G = c->M = c->Vv = NULL;
    if (c->XW) cudaFree(c->XW);
    if (c->XG) cudaFree(c->XG);
    if (c->XM) cudaFree(c->XM);
    if (c->XV) cudaFree(c->XV);
    c->XW = c->XG = c->XM = c->XV = NULL; c->n_extras = 0;
    free(c->off); c->off = NULL;
#define FREE1(f) do { free(p->f); p->f = NULL; } while (0)
#define FREEL(f) do { free_view_array(p->f, L); p->f = NULL; } while (0)
    FREE1(gpu_w_embed); FREE1(gpu_g_embed); FREE1(gpu_m_embed); FREE1(gpu_v_embed);
    FREE1(gpu_w_final_norm); FREE1(gpu_g_final_norm); FREE1(gpu_m_final_norm); FREE1(gpu_v_final_norm);
    FREEL(gpu_w_q); FREEL(gpu_g_q); FREEL(gpu_m_q); FREEL(gpu_v_q);
    FREEL(gpu_w_k); FREEL(gpu_g_k); FREEL(gpu_m_k); FREEL(gpu_v_k);
    FREEL(gpu_w_v); FREEL(gpu_g_v); FREEL(gpu_m_v); FREEL(gpu_v_v);
    FREEL(gpu_w_o); FREEL(gpu_g_o); FREEL(gpu_m_o); FREEL(gpu_v_o);
    FREEL(gpu_w_gate); FREEL(gpu_g_gate); FREEL(gpu_m_gate); FREEL(gpu_v_gate);
    FREEL(gpu_w_up); FREEL(gpu_g_up); FREEL(gpu_m_up); FREEL(gpu_v_up);
    FREEL(gpu_w_down); FREEL(gpu_g_down); FREEL(gpu_m_down); FREEL(gpu_v_down);
    FREEL(gpu_w_in_norm); FREEL(gpu_g_in_norm); FREEL(gpu_m_in_norm); FREEL(gpu_v_in_norm);
    FREEL(gpu_w_post_norm); FREEL(gpu_g_post_norm); FREEL(gpu_m_post_norm); FREEL(gpu_v_post_norm);
#undef FREE1
#undef FREEL
    c->n_params = 0; c->L = 0;
}

/* expose the arenas through the reference's per-tensor buffer fields (views, not owners) */
static void publish_views(sb_ctx_t* c) {
    cuda_train_context_t* p = &c->pub;
    int L = c->L, d = c->d, qd = c->qd, kvd = c->kvd, F = c->F;
    size_t nE = (size_t)c->V * d;
    float* A[4] = {c->W, c->G, c->M, c->Vv};
    cuda_buffer_t** e[4] = {&p->gpu_w_embed, &p->gpu_g_embed, &p->gpu_m_embed, &p->gpu_v_embed};
    cuda_buffer_t** f[4] = {&p->gpu_w_final_norm, &p->gpu_g_final_norm, &p->gpu_m_final_norm, &p->gpu_v_final_norm};
    cuda_buffer_t*** lq[4] = {&p->gpu_w_q, &p->gpu_g_q, &p->gpu_m_q, &p->gpu_v_q};
    cuda_buffer_t*** lk[4] = {&p->gpu_w_k, &p->gpu_g_k, &p->gpu_m_k, &p->gpu_v_k};
    cuda_buffer_t*** lv[4] = {&p->gpu_w_v, &p->gpu_g_v, &p->gpu_m_v, &p->gpu_v_v};
    cuda_buffer_t*** lo[4] = {&p->gpu_w_o, &p->gpu_g_o, &p->gpu_m_o, &p->gpu_v_o};
    cuda_buffer_t*** lg[4] = {&p->gpu_w_gate, &p->gpu_g_gate, &p->gpu_m_gate, &p->gpu_v_gate};
    cuda_buffer_t*** lu[4] = {&p->gpu_w_up, &p->gpu_g_up, &p->gpu_m_up, &p->gpu_v_up};
    cuda_buffer_t*** ld[4] = {&p->gpu_w_down, &p->gpu_g_down, &p->gpu_m_down, &p->gpu_v_down};
    cuda_buffer_t*** li[4] = {&p->gpu_w_in_norm, &p->gpu_g_in_norm, &p->gpu_m_in_norm, &p->gpu_v_in_norm};
    cuda_buffer_t*** lp[4] = {&p->gpu_w_post_norm, &p->gpu_g_post_norm, &p->gpu_m_post_norm, &p->gpu_v_post_norm};
    for (int k = 0; k < 4; k++) {
        if (!A[k]) continue;
        *e[k] = view(A[k], nE);
        *f[k] = view(A[k] + nE, (size_t)d);
        *lq[k] = view_array(L); *lk[k] = view_array(L); *lv[k] = view_array(L); *lo[k] = view_array(L);
        *lg[k] = view_array(L); *lu[k] = view_array(L); *ld[k] = view_array(L); *li[k] = view_array(L); *lp[k] = view_array(L);
        for (int l = 0; l < L; l++) {
            const sb_layer_off_t* o = &c->off[l];
            (*lq[k])[l] = view(A[k] + o->q, (size_t)qd * d);
            (*lk[k])[l] = view(A[k] + o->k, (size_t)kvd * d);
            (*lv[k])[l] = view(A[k] + o->v, (size_t)kvd * d);
            (*lo[k])[l] = view(A[k] + o->o, (size_t)d * qd);
            (*lg[k])[l] = view(A[k] + o->gate, (size_t)F * d);
            (*lu[k])[l] = view(A[k] + o->up, (size_t)F * d);
            (*ld[k])[l] = view(A[k] + o->down, (size_t)d * F);
            (*li[k])[l] = view(A[k] + o->in_norm, (size_t)d);
            (*lp[k])[l] = view(A[k] + o->post_norm, (size_t)d);
        }
    }
    p->gpu_weights_num_layers = L; p->gpu_weights_hidden_size = d; p->gpu_weights_intermediate_size = F;
    p->gpu_weights_q_dim = qd; p->gpu_weights_kv_dim = kvd; p->gpu_weights_vocab_size = c->V;
}

typedef void (*tensor_fn)(sb_ctx_t* c, weight_tensor_t* t, size_t off, void* arg);
static void for_each_tensor(sb_ctx_t* c, trainable_weights_t* w, tensor_fn fn, void* arg) {
    fn(c, &w->embed_tokens, 0, arg);
    fn(c, &w->final_norm, (size_t)c->V * c->d, arg);
    for (int l = 0; l < c->L; l++) {
        layer_weights_t* y = &w->layers[l]; const sb_layer_off_t* o = &c->off[l];
        fn(c, &y->q_proj, o->q, arg); fn(c, &y->k_proj, o->k, arg); fn(c, &y->v_proj, o->v, arg); fn(c, &y->o_proj, o->o, arg);
        fn(c, &y->gate_proj, o->gate, arg); fn(c, &y->up_proj, o->up, arg); fn(c, &y->down_proj, o->down, arg);
        fn(c, &y->input_norm, o->in_norm, arg); fn(c, &y->post_norm, o->post_norm, arg);
    }
}
static size_t tensor_len(sb_ctx_t* c, size_t off) {
    /* length of the tensor that starts at `off`, from the layout */
    size_t nE = (size_t)c->V * c->d;
    if (off == 0) return nE;
    if (off == nE) return (size_t)c->d;
    for (int l = 0; l < c->L; l++) {
        const sb_layer_off_t* o = &c->off[l];
        if (off == o->q) return (size_t)c->qd * c->d;
        if (off == o->k || off == o->v) return (size_t)c->kvd * c->d;
        if (off == o->o) return (size_t)c->d * c->qd;
        if (off == o->gate || off == o->up || off == o->down) return (size_t)c->F * c->d;
        if (off == o->in_norm || off == o->post_norm) return (size_t)c->d;
    }
    return 0;
}
static void up_tensor(sb_ctx_t* c, weight_tensor_t* t, size_t off, void* arg) {
    (void)arg;
    size_t n = tensor_len(c, off);
    if (t->weight) cudaMemcpyAsync(c->W + off, t->weight, n * 4, cudaMemcpyHostToDevice, S(c));
    if (!c->frozen_base) {
        if (t->m) cudaMemcpyAsync(c->M + off, t->m, n * 4, cudaMemcpyHostToDevice, S(c));
        if (t->v) cudaMemcpyAsync(c->Vv + off, t->v, n * 4, cudaMemcpyHostToDevice, S(c));
    }
}
static void down_tensor(sb_ctx_t* c, weight_tensor_t* t, size_t off, void* arg) {
    int what = *(int*)arg;     /* 0: weights + moments, 1: gradients */
    size_t n = tensor_len(c, off);
    if (what == 0) {
        if (t->weight) cudaMemcpyAsync(t->weight, c->W + off, n * 4, cudaMemcpyDeviceToHost, S(c));
        if (t->m && c->M) cudaMemcpyAsync(t->m, c->M + off, n * 4, cudaMemcpyDeviceToHost, S(c));
        if (t->v && c->Vv) cudaMemcpyAsync(t->v, c->Vv + off, n * 4, cudaMemcpyDeviceToHost, S(c));
    } else if (t->grad && c->G) {
        cudaMemcpyAsync(t->grad, c->G + off, n * 4, cudaMemcpyDeviceToHost, S(c));
    }
}

/* The frozen base of a LoRA state the reference's train_init built: no FP32 host copies (full_weights is NULL in LoRA mode,
 * src/train.c:7900-7909), the weights are the BF16 tensors of the memory-mapped model, found by name as
 * ensure_cuda_lora_base_weights does (src/train_cuda.c:1376-1460) and read as raw BF16 whatever the file's dtype says. */
int sb_upload_bf16(sb_ctx_t* c, const uint16_t* src, float* dst, size_t n);
static const uint16_t* model_tensor(const seraph_model_t* m, const char* name, size_t want) {
    for (int i = 0; i < m->num_tensors; i++) {
        if (strcmp(m->tensor_map[i].name, name)) continue;
        const int fi = m->tensor_map[i].file_idx;
        if (fi < 0 || fi >= 8 || !m->st[fi]) return NULL;
        const safetensors_t* f = m->st[fi];
        for (int t = 0; t < f->num_tensors; t++)
            if (f->tensors[t].name && !strcmp(f->tensors[t].name, m->tensor_map[i].orig_name)) {
                if (f->tensors[t].num_elements != want) return NULL;
                /* the offsets come from the file's header: stay inside the mapping whatever it claims */
                if (f->tensors[t].offset_start < 0 || f->data_offset + (size_t)f->tensors[t].offset_start + want * 2 > f->file_size) return NULL;
                return (const uint16_t*)(f->data + f->data_offset + f->tensors[t].offset_start);
            }
        return NULL;
    }
    return NULL;
}
static int upload_base_from_model(sb_ctx_t* c, const seraph_model_t* m) {
    static const char* per_layer[9] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
                                       "mlp.up_proj", "mlp.down_proj", "input_layernorm", "post_attention_layernorm"};
    char name[320];
    const size_t nE = (size_t)c->V * c->d;
    const uint16_t* p = model_tensor(m, "model.embed_tokens.weight", nE);
    if (!p || sb_upload_bf16(c, p, c->W, nE)) { fprintf(stderr, "seraph_b200: model.embed_tokens.weight missing from the model or of another size\n"); return 1; }
    p = model_tensor(m, "model.norm.weight", (size_t)c->d);
    if (!p || sb_upload_bf16(c, p, c->W + nE, (size_t)c->d)) { fprintf(stderr, "seraph_b200: model.norm.weight missing from the model or of another size\n"); return 1; }
    for (int l = 0; l < c->L; l++) {
        const sb_layer_off_t* o = &c->off[l];
        const size_t offs[9] = {o->q, o->k, o->v, o->o, o->gate, o->up, o->down, o->in_norm, o->post_norm};
        for (int t = 0; t < 9; t++) {
            snprintf(name, sizeof name, "model.layers.%d.%s.weight", l, per_layer[t]);
            const size_t n = tensor_len(c, offs[t]);
            p = model_tensor(m, name, n);
            if (!p || sb_upload_bf16(c, p, c->W + offs[t], n)) { fprintf(stderr, "seraph_b200: %s missing from the model or of another size\n", name); return 1; }
        }
    }
    return 0;
}

/* Allocate the arenas for this geometry and upload the host master copy once
 * (the reference uploads once and afterwards only downloads, src/train_cuda.c:286-291). */
static void free_lora(sb_ctx_t* c);
static void free_activations(sb_ctx_t* c);
static int ensure_model(sb_ctx_t* c, const train_state_t* st, int frozen_base) {
    const model_config_t* cfg = st->config;
    int V = cfg->vocab_size, d = cfg->hidden_size, L = cfg->num_hidden_layers, F = cfg->intermediate_size;
    int Hq = cfg->num_attention_heads, Hkv = cfg->num_key_value_heads, hd = cfg->head_dim;
    if (V <= 0 || d <= 0 || L <= 0 || F <= 0 || Hq <= 0 || Hkv <= 0 || hd <= 0 || Hq % Hkv) { sb_set_status(c, SB_ERR_ARG); return 1; }
    if (c->W && c->V == V && c->d == d && c->L == L && c->F == F && c->Hq == Hq && c->Hkv == Hkv && c->hd == hd &&
        c->frozen_base == frozen_base) return 0;
    if (!st->full_weights && !(frozen_base && st->model)) { sb_set_status(c, SB_ERR_ARG); return 1; }
    cudaStreamSynchronize(S(c));
    /* the activation slots, the registered operand parts and the adapter arenas were carved for the old geometry
       (the reference reallocates on a geometry change too, src/train.c:2705) */
    if (c->V != V || c->d != d || c->L != L || c->F != F || c->Hq != Hq || c->Hkv != Hkv || c->hd != hd) { free_activations(c); free_lora(c); }
    free_model(c);
    c->V = V; c->d = d; c->L = L; c->F = F; c->Hq = Hq; c->Hkv = Hkv; c->hd = hd; c->qd = Hq * hd; c->kvd = Hkv * hd;
    c->frozen_base = frozen_base;
    c->off = (sb_layer_off_t*)calloc((size_t)L, sizeof(sb_layer_off_t));
    if (!c->off) return 1;
    c->n_params = layout_offsets(V, d, L, c->qd, c->kvd, F, c->off);
    size_t bytes = c->n_params * sizeof(float);
    if (sb_check(c, cudaMalloc((void**)&c->W, bytes), "weight arena")) { c->status = SB_ERR_OOM; return 1; }
    if (!frozen_base) {
        if (sb_check(c, cudaMalloc((void**)&c->G, bytes), "gradient arena") ||
            sb_check(c, cudaMalloc((void**)&c->M, bytes), "Adam m arena") ||
            sb_check(c, cudaMalloc((void**)&c->Vv, bytes), "Adam v arena")) { c->status = SB_ERR_OOM; return 1; }
        cudaMemsetAsync(c->G, 0, bytes, S(c));
        cudaMemsetAsync(c->M, 0, bytes, S(c));
        cudaMemsetAsync(c->Vv, 0, bytes, S(c));
    }
    sb_parts_register(c, 0, c->W, (size_t)V * d);
    for (int l = 0; l < L; l++) {
        const sb_layer_off_t* o = &c->off[l];
        sb_parts_register(c, 0, c->W + o->q, (size_t)c->qd * d); sb_parts_register(c, 0, c->W + o->k, (size_t)c->kvd * d);
        sb_parts_register(c, 0, c->W + o->v, (size_t)c->kvd * d); sb_parts_register(c, 0, c->W + o->o, (size_t)c->qd * d);
        sb_parts_register(c, 0, c->W + o->gate, (size_t)F * d); sb_parts_register(c, 0, c->W + o->up, (size_t)F * d);
        sb_parts_register(c, 0, c->W + o->down, (size_t)F * d);
    }
    if (st->full_weights) for_each_tensor(c, st->full_weights, up_tensor, NULL);
    else if (upload_base_from_model(c, (const seraph_model_t*)st->model)) { sb_set_status(c, SB_ERR_ARG); return 1; }
    publish_views(c);
    return sb_check(c, cudaStreamSynchronize(S(c)), "weight upload");
}

/* Parameters of the model options (per-head q/k norm scales, separate lm_head): resident beside the arenas, uploaded from the
 * host copy seraph_b200_set_model_extras left; gradients and Adam moments only in full-weight mode. */
static size_t extras_lm_off(const sb_ctx_t* c) { return c->head_norm ? (size_t)c->L * 2 * c->hd : 0; }
static int ensure_extras(sb_ctx_t* c, int full) {
    const size_t n = extras_lm_off(c) + (c->untied ? (size_t)c->V * c->d : 0);
    if (n == 0) return 0;
    if (!c->XW) {
        if (!c->h_extras || c->n_extras_host != n) {
            fprintf(stderr, "seraph_b200: the model options need %zu extra parameters, seraph_b200_set_model_extras gave %zu\n", n, c->n_extras_host);
            sb_set_status(c, SB_ERR_ARG); return 1;
        }
        if (sb_check(c, cudaMalloc((void**)&c->XW, n * 4), "extra parameters")) { c->status = SB_ERR_OOM; return 1; }
        c->n_extras = n;
        cudaMemcpyAsync(c->XW, c->h_extras, n * 4, cudaMemcpyHostToDevice, S(c));
        if (c->untied) sb_parts_register(c, 0, c->XW + extras_lm_off(c), (size_t)c->V * c->d);
        if (sb_check(c, cudaStreamSynchronize(S(c)), "extra parameter upload")) return 1;
    }
    if (full && !c->XG) {
        if (sb_check(c, cudaMalloc((void**)&c->XG, n * 4), "extra gradients") || sb_check(c, cudaMalloc((void**)&c->XM, n * 4), "extra Adam m") ||
            sb_check(c, cudaMalloc((void**)&c->XV, n * 4), "extra Adam v")) { c->status = SB_ERR_OOM; return 1; }
        cudaMemsetAsync(c->XG, 0, n * 4, S(c)); cudaMemsetAsync(c->XM, 0, n * 4, S(c)); cudaMemsetAsync(c->XV, 0, n * 4, S(c));
    }
    return 0;
}

/* Model options beyond the reference's training step (its trainable_weights_t has no tensors for them, include/train.h:75-90):
 * per_head_qk_norm: q and k pass through a learned RMSNorm over each head before RoPE (scales q_norm [hd], k_norm [hd] per layer);
 * untied_lm_head: logits come from a separate lm_head [V,d] instead of the embedding matrix.  `flat` holds the parameters
 * (per layer q_norm then k_norm; then lm_head), n their count; both options off takes flat = NULL.  Takes effect at the next
 * step, which uploads them; in full-weight mode they are trained by the same AdamW, in LoRA mode they are frozen. */
int seraph_b200_set_model_extras(cuda_train_context_t* ctx, int per_head_qk_norm, int untied_lm_head, const float* flat, size_t n) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || ((per_head_qk_norm || untied_lm_head) && (!flat || !n))) return SB_ERR_ARG;
    cudaStreamSynchronize(S(c));
    if (c->XW) { sb_parts_unregister(c, 0); }          /* weight parts are registered again with the model */
    free_activations(c); free_lora(c); free_model(c);
    free(c->h_extras); c->h_extras = NULL; c->n_extras_host = 0;
    c->head_norm = per_head_qk_norm ? 1 : 0; c->untied = untied_lm_head ? 1 : 0;
    if (c->head_norm || c->untied) {
        c->h_extras = (float*)malloc(n * 4);
        if (!c->h_extras) { c->head_norm = c->untied = 0; return SB_ERR_OOM; }
        memcpy(c->h_extras, flat, n * 4); c->n_extras_host = n;
    }
    return SB_OK;
}
/* which: 0 parameters, 1 gradients, 2 Adam m, 3 Adam v of the extra parameters, copied to out[n]; reading the parameters also
 * refreshes the host copy, so that a later seraph_b200_reset_model continues from the trained values. */
int seraph_b200_get_model_extras(cuda_train_context_t* ctx, int which, float* out, size_t n) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !out || which < 0 || which > 3) return SB_ERR_ARG;
    const float* src = which == 0 ? c->XW : which == 1 ? c->XG : which == 2 ? c->XM : c->XV;
    if (!src || n != c->n_extras) return SB_ERR_ARG;
    cudaMemcpyAsync(out, src, n * 4, cudaMemcpyDeviceToHost, S(c));
    if (sb_check(c, cudaStreamSynchronize(S(c)), "extra parameter download")) return SB_ERR_CUDA;
    if (which == 0 && c->h_extras && c->n_extras_host == n) memcpy(c->h_extras, out, n * 4);
    return SB_OK;
}

/* ------------------------------------------------------------------------ */
/* LoRA adapters                                                             */
/* ------------------------------------------------------------------------ */
static lora_adapter_t** lora_list(const lora_model_t* m, int a) {
    switch (a) { case 0: return m->q_adapters; case 1: return m->k_adapters; case 2: return m->v_adapters; case 3: return m->o_adapters;
                 case 4: return m->gate_adapters; case 5: return m->up_adapters; default: return m->down_adapters; }
}
static cuda_lora_gpu_adapter_t* lora_pub(cuda_lora_gpu_state_t* s, int a) {
    switch (a) { case 0: return &s->q; case 1: return &s->k; case 2: return &s->v; case 3: return &s->o;
                 case 4: return &s->gate; case 5: return &s->up; default: return &s->down; }
}
static void free_lora(sb_ctx_t* c) {
    if (c->LW) cudaFree(c->LW);
    if (c->LG) cudaFree(c->LG);
    if (c->LM) cudaFree(c->LM);
    if (c->LV) cudaFree(c->LV);
    if (c->lora_tmp) cudaFree(c->lora_tmp);
    if (c->LWp) cudaFree(c->LWp);
    if (c->LGp) cudaFree(c->LGp);
    c->LW = c->LG = c->LM = c->LV = c->lora_tmp = c->LWp = c->LGp = NULL; c->lora_tmp_cap = 0; c->n_lora_pad = 0; c->lora_R = 0;
    cuda_lora_gpu_state_t* s = (cuda_lora_gpu_state_t*)c->pub.lora_gpu;
    if (s) {
        for (int a = 0; a < 7; a++) {
            cuda_lora_gpu_adapter_t* g = lora_pub(s, a);
            free_view_array(g->A, s->num_layers); free_view_array(g->B, s->num_layers);
            free_view_array(g->gA, s->num_layers); free_view_array(g->gB, s->num_layers);
            free_view_array(g->mA, s->num_layers); free_view_array(g->vA, s->num_layers);
            free_view_array(g->mB, s->num_layers); free_view_array(g->vB, s->num_layers);
        }
        free(s);
        c->pub.lora_gpu = NULL;
    }
    c->n_lora = 0; c->lora_rank = 0; c->lora_mask = 0;
}

/* the host adapters changed (a file was loaded into them): the next LoRA step uploads them again */
void sb_lora_mark_stale(sb_ctx_t* c) {
    if (!c || !c->LW) return;
    cudaStreamSynchronize(S(c));
    free_lora(c);
}

static int ensure_lora(sb_ctx_t* c, const lora_model_t* m) {
    int mask = 0;
    for (int a = 0; a < 7; a++) { lora_adapter_t** ls = lora_list(m, a); if (ls && ls[0]) mask |= 1 << a; }
    if (c->LW && c->lora_rank == m->rank && c->lora_mask == mask) return 0;
    if (m->rank <= 0 || mask == 0) { sb_set_status(c, SB_ERR_ARG); return 1; }
    cudaStreamSynchronize(S(c));
    free_lora(c);
    c->lora_rank = m->rank; c->lora_mask = mask; c->lora_alpha = m->alpha;
    c->lora_R = (m->rank + 127) / 128 * 128;
    c->n_lora = lora_layer_params(c) * (size_t)c->L;
    c->n_lora_pad = lora_layer_params_pad(c) * (size_t)c->L;
    if (sb_check(c, cudaMalloc((void**)&c->LWp, c->n_lora_pad * sizeof(float)), "lora padded weights") ||
        sb_check(c, cudaMalloc((void**)&c->LGp, c->n_lora_pad * sizeof(float)), "lora padded grads")) { c->status = SB_ERR_OOM; return 1; }
    cudaMemsetAsync(c->LWp, 0, c->n_lora_pad * sizeof(float), S(c)); cudaMemsetAsync(c->LGp, 0, c->n_lora_pad * sizeof(float), S(c));
    c->lora_pad_stale = 1;
    size_t bytes = c->n_lora * sizeof(float);
    if (sb_check(c, cudaMalloc((void**)&c->LW, bytes), "lora weights") || sb_check(c, cudaMalloc((void**)&c->LG, bytes), "lora grads") ||
        sb_check(c, cudaMalloc((void**)&c->LM, bytes), "lora m") || sb_check(c, cudaMalloc((void**)&c->LV, bytes), "lora v")) {
        c->status = SB_ERR_OOM; return 1;
    }
    cudaMemsetAsync(c->LG, 0, bytes, S(c)); cudaMemsetAsync(c->LM, 0, bytes, S(c)); cudaMemsetAsync(c->LV, 0, bytes, S(c));
    cuda_lora_gpu_state_t* s = (cuda_lora_gpu_state_t*)calloc(1, sizeof(cuda_lora_gpu_state_t));
    if (!s) return 1;
    s->num_layers = c->L; s->rank = m->rank; s->alpha = m->alpha; s->scale = m->alpha / (float)m->rank;
    for (int a = 0; a < 7; a++) {
        if (!(mask & (1 << a))) continue;
        int in, out; lora_dims(c, a, &in, &out);
        size_t nA = (size_t)m->rank * in, nB = (size_t)out * m->rank;
        cuda_lora_gpu_adapter_t* g = lora_pub(s, a);
        g->active = 1;
        g->A = view_array(c->L); g->B = view_array(c->L); g->gA = view_array(c->L); g->gB = view_array(c->L);
        g->mA = view_array(c->L); g->vA = view_array(c->L); g->mB = view_array(c->L); g->vB = view_array(c->L);
        lora_adapter_t** ls = lora_list(m, a);
        for (int l = 0; l < c->L; l++) {
            size_t o = lora_off(c, l, a);
            g->A[l] = view(c->LW + o, nA); g->B[l] = view(c->LW + o + nA, nB);
            g->gA[l] = view(c->LG + o, nA); g->gB[l] = view(c->LG + o + nA, nB);
            g->mA[l] = view(c->LM + o, nA); g->mB[l] = view(c->LM + o + nA, nB);
            g->vA[l] = view(c->LV + o, nA); g->vB[l] = view(c->LV + o + nA, nB);
            const lora_adapter_t* ad = ls[l];
            if (!ad || ad->in_dim != in || ad->out_dim != out || ad->rank != m->rank) { sb_set_status(c, SB_ERR_ARG); free(s); return 1; }
            cudaMemcpyAsync(c->LW + o, ad->A, nA * 4, cudaMemcpyHostToDevice, S(c));
            cudaMemcpyAsync(c->LW + o + nA, ad->B, nB * 4, cudaMemcpyHostToDevice, S(c));
            if (ad->m_A) cudaMemcpyAsync(c->LM + o, ad->m_A, nA * 4, cudaMemcpyHostToDevice, S(c));
            if (ad->m_B) cudaMemcpyAsync(c->LM + o + nA, ad->m_B, nB * 4, cudaMemcpyHostToDevice, S(c));
            if (ad->v_A) cudaMemcpyAsync(c->LV + o, ad->v_A, nA * 4, cudaMemcpyHostToDevice, S(c));
            if (ad->v_B) cudaMemcpyAsync(c->LV + o + nA, ad->v_B, nB * 4, cudaMemcpyHostToDevice, S(c));
        }
    }
    c->pub.lora_gpu = s;
    return sb_check(c, cudaStreamSynchronize(S(c)), "lora upload");
}

/* ------------------------------------------------------------------------ */
/* activations                                                               */
/* ------------------------------------------------------------------------ */
static void free_activations(sb_ctx_t* c) {
    sb_parts_unregister(c, 1);
    if (c->act_arena) cudaFree(c->act_arena);
    c->act_arena = NULL; c->act_arena_bytes = 0; c->T_cap = 0;
    free(c->act); c->act = NULL;
}

static size_t r4(size_t n) { return (n + 63) & ~(size_t)63; }     /* keep every slot 256-byte aligned */

static int ensure_activations(sb_ctx_t* c, int T, int need_logits_grad) {
    if (c->act_arena && c->T_cap >= T) return 0;
    cudaStreamSynchronize(S(c));
    free_activations(c);
    size_t Td = r4((size_t)T * c->d), TF = r4((size_t)T * c->F), Tq = r4((size_t)T * c->qd), Tkv = r4((size_t)T * c->kvd);
    size_t TH = r4((size_t)T * c->Hq), TV = r4((size_t)T * c->V);
    size_t per_layer = 4 * Td + 2 * Tq + 2 * Tkv + TH + 3 * TF + 2 * r4((size_t)T);    /* layer_in x_norm_attn post_attn_in x_norm_ffn | q attn_out | k v | lse | gate up ffn_hidden */
    if (c->head_norm) per_layer += Tq + Tkv;                                          /* q_pre k_pre */
    size_t shared = 3 * Td /* hidden_norm final_in (+1 spare) */ + 2 * TV + r4((size_t)T)
                  + 3 * Td /* g_hidden g_tmp g_xnorm */ + 2 * Tq + 2 * Tkv + 3 * TF + (c->head_norm ? Tq + Tkv : 0);
    (void)need_logits_grad;
    size_t total = per_layer * (size_t)c->L + shared;
    if (sb_check(c, cudaMalloc((void**)&c->act_arena, total * sizeof(float)), "activation arena")) { c->status = SB_ERR_OOM; return 1; }
    c->act_arena_bytes = total * sizeof(float); c->T_cap = T;
    c->act = (sb_layer_act_t*)calloc((size_t)c->L, sizeof(sb_layer_act_t));
    if (!c->act) return 1;
    float* p = c->act_arena;
#define TAKE(dst, n) do { dst = p; p += (n); } while (0)
    for (int l = 0; l < c->L; l++) {
        sb_layer_act_t* a = &c->act[l];
        TAKE(a->layer_in, Td); TAKE(a->x_norm_attn, Td); TAKE(a->post_attn_in, Td); TAKE(a->x_norm_ffn, Td);
        TAKE(a->q, Tq); TAKE(a->attn_out, Tq); TAKE(a->k, Tkv); TAKE(a->v, Tkv); TAKE(a->lse, TH); TAKE(a->q_rms, r4((size_t)T)); TAKE(a->k_rms, r4((size_t)T));
        TAKE(a->gate, TF); TAKE(a->up, TF); TAKE(a->ffn_hidden, TF);
        if (c->head_norm) { TAKE(a->q_pre, Tq); TAKE(a->k_pre, Tkv); }
    }
    TAKE(c->hidden_norm, Td); TAKE(c->final_in, Td); TAKE(c->hidden, Td);
    TAKE(c->logits, TV); TAKE(c->dlogits, TV); TAKE(c->loss_rows, r4((size_t)T));
    TAKE(c->g_hidden, Td); TAKE(c->g_tmp, Td); TAKE(c->g_xnorm, Td);
    TAKE(c->g_q, Tq); TAKE(c->g_attn, Tq); TAKE(c->g_k, Tkv); TAKE(c->g_v, Tkv);
    TAKE(c->g_ffn, TF); TAKE(c->g_gate, TF); TAKE(c->g_up, TF);
    if (c->head_norm) { TAKE(c->g_q2, Tq); TAKE(c->g_k2, Tkv); }
#undef TAKE
    /* operands of more than one product per step, written once by the forward pass */
    for (int l = 0; l < c->L; l++) {
        const sb_layer_act_t* a = &c->act[l];
        sb_parts_register(c, 1, a->x_norm_attn, (size_t)T * c->d); sb_parts_register(c, 1, a->x_norm_ffn, (size_t)T * c->d);
        sb_parts_register(c, 1, a->attn_out, (size_t)T * c->qd); sb_parts_register(c, 1, a->ffn_hidden, (size_t)T * c->F);
        sb_parts_register(c, 1, a->q, (size_t)T * c->qd); sb_parts_register(c, 1, a->k, (size_t)T * c->kvd);
        sb_parts_register(c, 1, a->v, (size_t)T * c->kvd);
    }
    sb_parts_register(c, 1, c->hidden_norm, (size_t)T * c->d);
    sb_parts_register(c, 1, c->dlogits, (size_t)T * c->V);
    sb_parts_register(c, 1, c->g_gate, (size_t)T * c->F); sb_parts_register(c, 1, c->g_up, (size_t)T * c->F);      /* written as parts by the SwiGLU backward */
    return 0;
}

static int ensure_pinned(sb_ctx_t* c, size_t bytes) {
    if (c->h_pinned && c->h_pinned_bytes >= bytes) return 0;
    cudaStreamSynchronize(S(c));
    if (c->h_pinned) cudaFreeHost(c->h_pinned);
    c->h_pinned = NULL; c->h_pinned_bytes = 0;
    size_t want = bytes < 65536 ? 65536 : bytes;
    if (sb_check(c, cudaMallocHost(&c->h_pinned, want), "pinned staging")) return 1;
    c->h_pinned_bytes = want;
    return 0;
}

/* ------------------------------------------------------------------------ */
/* the step                                                                  */
/* ------------------------------------------------------------------------ */
typedef struct { const float *A, *B; float *gA, *gB; int in, out; } lora_ref_t;
/* the rank-padded working copies of adapter a of layer l */
static int lora_get(sb_ctx_t* c, int l, int a, lora_ref_t* r) {
    if (!c->LW || !(c->lora_mask & (1 << a))) return 0;
    lora_dims(c, a, &r->in, &r->out);
    size_t o = lora_off_pad(c, l, a), nA = (size_t)c->lora_R * r->in;
    r->A = c->LWp + o; r->B = c->LWp + o + nA; r->gA = c->LGp + o; r->gB = c->LGp + o + nA;
    return 1;
}
/* LWp <- LW (all layers) when the adapters changed: A's r rows are the head of the padded block, B's r columns a strided copy */
static void lora_refresh_padded(sb_ctx_t* c) {
    if (!c->lora_pad_stale || !c->LWp) return;
    const int r = c->lora_rank, R = c->lora_R;
    for (int l = 0; l < c->L; l++)
        for (int a = 0; a < 7; a++) {
            if (!(c->lora_mask & (1 << a))) continue;
            int in, out; lora_dims(c, a, &in, &out);
            const size_t o = lora_off(c, l, a), op = lora_off_pad(c, l, a);
            cudaMemcpyAsync(c->LWp + op, c->LW + o, (size_t)r * in * 4, cudaMemcpyDeviceToDevice, S(c));
            cudaMemcpy2DAsync(c->LWp + op + (size_t)R * in, (size_t)R * 4, c->LW + o + (size_t)r * in, (size_t)r * 4, (size_t)r * 4, (size_t)out,
                              cudaMemcpyDeviceToDevice, S(c));
        }
    c->lora_pad_stale = 0;
}
/* LG <- live part of LGp for layer l (the running total of this accumulation cycle) */
static void lora_compact_grads(sb_ctx_t* c, int l) {
    const int r = c->lora_rank, R = c->lora_R;
    for (int a = 0; a < 7; a++) {
        if (!(c->lora_mask & (1 << a))) continue;
        int in, out; lora_dims(c, a, &in, &out);
        const size_t o = lora_off(c, l, a), op = lora_off_pad(c, l, a);
        cudaMemcpyAsync(c->LG + o, c->LGp + op, (size_t)r * in * 4, cudaMemcpyDeviceToDevice, S(c));
        cudaMemcpy2DAsync(c->LG + o + (size_t)r * in, (size_t)r * 4, c->LGp + op + (size_t)R * in, (size_t)R * 4, (size_t)r * 4, (size_t)out,
                          cudaMemcpyDeviceToDevice, S(c));
    }
}

/* Y[T,out] (+)= X[T,in] W[out,in]^T, plus the adapter's (s X A^T) B^T when one is active */
static void linear_fwd(sb_ctx_t* c, int use_lora, int l, int a, const float* X, const float* W, float* Y, int T, int in, int out, int acc) {
    sb_gemm(c, X, W, Y, T, out, in, 0, 1, acc);
    lora_ref_t r;
    if (use_lora && lora_get(c, l, a, &r)) {
        float s = c->lora_alpha / (float)c->lora_rank;
        sb_gemm_keep_forget(c, c->lora_tmp);
        sb_gemm(c, X, r.A, c->lora_tmp, T, c->lora_R, in, 0, 1, 0);
        sb_scale(c, c->lora_tmp, (size_t)T * c->lora_R, s);
        sb_gemm(c, c->lora_tmp, r.B, Y, T, out, c->lora_R, 0, 1, 1);
    }
}
/* adapter gradients for one projection; in exact mode also dX += (s dY B) A */
static void lora_bwd(sb_ctx_t* c, int l, int a, const float* dY, const float* X, float* dX, int T) {
    lora_ref_t r;
    if (!lora_get(c, l, a, &r)) return;
    float s = c->lora_alpha / (float)c->lora_rank;
    sb_lora_backward(c, dY, X, r.A, r.B, r.gA, r.gB, c->lora_tmp, T, r.in, r.out, c->lora_R, s);
    if (c->lora_exact && dX) sb_gemm(c, c->lora_tmp, r.A, dX, T, r.in, c->lora_R, 0, 0, 1);
}

/* NaN/Inf flags of a training step with state->debug_nan_check set, indexed as the reference indexes them
 * (src/train_cuda.c:626-645): [0..9] fixed buffers, [10 + l] hidden after layer l, [10 + L + 5 l + 0..3] grad_attn,
 * grad_q, grad_k, grad_v of layer l, [10 + 6 L + l] grad_hidden after layer l's backward, [10 + 7 L] embedding weights. */
static uint32_t nan_fwd_base(const sb_ctx_t* c) { (void)c; return 10u; }
static uint32_t nan_bwd_base(const sb_ctx_t* c) { return 10u + (uint32_t)c->L; }
static uint32_t nan_ghid_base(const sb_ctx_t* c) { return 10u + 6u * (uint32_t)c->L; }
static uint32_t nan_weight_idx(const sb_ctx_t* c) { return 10u + 7u * (uint32_t)c->L; }
static void nan_mark(sb_ctx_t* c, const float* p, size_t n, uint32_t idx) {
    if (!c->nan_on || !c->pub.debug_nan_flags || idx >= c->nan_count) return;
    sb_nan_check(c, p, n, (uint32_t*)c->pub.debug_nan_flags->data, idx);
}
static int nan_begin(sb_ctx_t* c, int on) {
    c->nan_on = 0;
    if (!on) return 0;
    uint32_t count = nan_weight_idx(c) + 5u;
    if (!c->pub.debug_nan_flags || c->pub.debug_nan_flags->size < (size_t)count * 4) {
        cudaStreamSynchronize(S(c));
        if (c->pub.debug_nan_flags) cuda_train_buffer_free(&c->pub, c->pub.debug_nan_flags);
        c->pub.debug_nan_flags = cuda_train_buffer_create(&c->pub, (size_t)count * 4);
        if (!c->pub.debug_nan_flags) return 1;
    }
    c->nan_count = count; c->nan_on = 1;
    sb_memset(c, c->pub.debug_nan_flags->data, 0, (size_t)count * 4);
    return 0;
}
/* Reads the flags back (synchronises).  Returns 1 and reports the buffers when any is set. */
static int nan_tripped(sb_ctx_t* c, const train_state_t* st, int T) {
    if (!c->nan_on) return 0;
    uint32_t* h = (uint32_t*)calloc(c->nan_count, sizeof(uint32_t));
    if (!h) return 0;
    int any = 0;
    if (cudaMemcpyAsync(h, c->pub.debug_nan_flags->data, (size_t)c->nan_count * 4, cudaMemcpyDeviceToHost, S(c)) == cudaSuccess &&
        cudaStreamSynchronize(S(c)) == cudaSuccess)
        for (uint32_t i = 0; i < c->nan_count; i++) if (h[i]) { any = 1; break; }
    if (any) {
        static const char* fixed[10] = {"grad_hidden (post final-norm backward)", "logits (LM head output)", "hidden_norm (LM head input)",
            "grad_logits (cross-entropy grad)", "grad_hidden (after LM head backward)", "grad_tmp_hidden (final rmsnorm backward output)",
            "final_input (pre final rmsnorm)", "hidden (post embedding)", "grad_hidden (pre embedding_backward)", "g_embed (post embedding_backward)"};
        fprintf(stderr, "[NAN] detected at step=%d seq=%d (optimizer skipped)\n", st->current_step + 1, T);
        fprintf(stderr, "  - lr(base)=%g opt_step=%d accum=%d/%d\n", (double)st->learning_rate, st->optimizer_step, st->accumulation_counter,
                st->gradient_accumulation_steps);
        for (int i = 0; i < 10; i++) if (h[i]) fprintf(stderr, "  - buffer: %s\n", fixed[i]);
        if (h[nan_weight_idx(c)]) fprintf(stderr, "  - buffer: w_embed (weights already NaN/Inf at step start)\n");
        for (int l = 0; l < c->L; l++) if (h[nan_fwd_base(c) + l]) { fprintf(stderr, "  - buffer: hidden (post layer) layer=%d\n", l); break; }
        for (int l = 0; l < c->L; l++) {
            const uint32_t* b = h + nan_bwd_base(c) + 5u * (uint32_t)l;
            static const char* nm[4] = {"grad_attn (input to attn backward)", "grad_q (post rope_backward)", "grad_k (post attn backward)", "grad_v (post attn backward)"};
            int hit = -1;
            for (int k = 0; k < 4; k++) if (b[k]) { hit = k; break; }
            if (hit >= 0) { fprintf(stderr, "  - buffer: %s layer=%d\n", nm[hit], l); break; }
        }
        for (int l = 0; l < c->L; l++) if (h[nan_ghid_base(c) + l]) { fprintf(stderr, "  - buffer: grad_hidden (after layer backward) layer=%d\n", l); break; }
    }
    free(h);
    return any;
}

static void forward_pass(sb_ctx_t* c, int T, int max_seq, float theta, int use_lora) {
    const int d = c->d, F = c->F, qd = c->qd, kvd = c->kvd, L = c->L;
    const size_t Td = (size_t)T * d;
    /* producers that may write an operand only as FP16 parts: every product that reads it must take parts */
    const int ffn_lora = use_lora && (c->lora_mask & 0x70);
    const int ffn_parts = !c->nan_on && !ffn_lora && sb_gemm_reads_f16_parts(c, T, d, F, 0, 1) && sb_gemm_reads_f16_parts(c, d, F, T, 1, 0);
    /* the normalised rows are read by the projections and by their weight gradients only (adapters read them too: FP32 stays then) */
    const int xa_parts = !c->nan_on && !(use_lora && (c->lora_mask & 0x07)) &&
                         sb_gemm_reads_f16_parts(c, T, qd, d, 0, 1) && sb_gemm_reads_f16_parts(c, T, kvd, d, 0, 1) &&
                         sb_gemm_reads_f16_parts(c, qd, d, T, 1, 0) && sb_gemm_reads_f16_parts(c, kvd, d, T, 1, 0);
    const int xf_parts = !c->nan_on && !(use_lora && (c->lora_mask & 0x30)) &&
                         sb_gemm_reads_f16_parts(c, T, F, d, 0, 1) && sb_gemm_reads_f16_parts(c, F, d, T, 1, 0);
    const int hn_parts = !c->nan_on && sb_gemm_reads_f16_parts(c, T, c->V, d, 0, 1) && sb_gemm_reads_f16_parts(c, c->V, d, T, 1, 0);
    nan_mark(c, c->W, (size_t)c->V * d, nan_weight_idx(c));
    sb_embed_lookup(c, c->tokens, c->W, c->act[0].layer_in, T, d, c->V);
    nan_mark(c, c->act[0].layer_in, Td, 7);
    for (int l = 0; l < L; l++) {
        const sb_layer_off_t* o = &c->off[l];
        sb_layer_act_t* a = &c->act[l];
        float* next_in = (l + 1 < L) ? c->act[l + 1].layer_in : c->final_in;
        if (!(xa_parts && sb_rmsnorm_parts(c, a->layer_in, c->W + o->in_norm, a->x_norm_attn, T, d, RMS_EPS))) {
            sb_amax_announce(c, a->x_norm_attn, Td);       /* producers of GEMM operands leave max |x| behind for the operand split */
            sb_rmsnorm(c, a->layer_in, c->W + o->in_norm, a->x_norm_attn, T, d, RMS_EPS);
        }
        /* runs of products that share an operand keep its prepared parts (the adapters' scratch, rewritten in between, is dropped from the kept set at every write) */
        sb_gemm_keep_begin(c);
        linear_fwd(c, use_lora, l, 0, a->x_norm_attn, c->W + o->q, c->head_norm ? a->q_pre : a->q, T, d, qd, 0);
        linear_fwd(c, use_lora, l, 1, a->x_norm_attn, c->W + o->k, c->head_norm ? a->k_pre : a->k, T, d, kvd, 0);
        linear_fwd(c, use_lora, l, 2, a->x_norm_attn, c->W + o->v, a->v, T, d, kvd, 0);
        sb_gemm_keep_end(c);
        if (c->head_norm) {       /* learned RMSNorm over each head (rows of head_dim), before RoPE */
            const float* wn = c->XW + (size_t)l * 2 * c->hd;
            sb_rmsnorm(c, a->q_pre, wn, a->q, T * c->Hq, c->hd, RMS_EPS);
            sb_rmsnorm(c, a->k_pre, wn + c->hd, a->k, T * c->Hkv, c->hd, RMS_EPS);
        }
        if (!c->qk_norm) { sb_amax_announce(c, a->q, (size_t)T * qd); sb_amax_announce(c, a->k, (size_t)T * kvd); }
        sb_rope2(c, a->q, a->k, c->pos_ids, T, c->Hq, c->Hkv, c->hd, theta, max_seq, 0);
        if (c->qk_norm) {
            /* whole-row normalisation of q and k after RoPE (shaders/qk_norm.comp, src/train.c:4688-4689); the row statistic is kept for the backward pass */
            sb_qk_norm(c, a->q, a->q_rms, T, qd, RMS_EPS);
            sb_qk_norm(c, a->k, a->k_rms, T, kvd, RMS_EPS);
        }
        sb_amax_announce(c, a->attn_out, (size_t)T * qd);
        sb_attention(c, a->q, a->k, a->v, a->attn_out, a->lse, c->seq_starts, c->seq_ids, T, c->Hq, c->Hkv, c->hd);
        sb_copy(c, a->post_attn_in, a->layer_in, Td * sizeof(float));
        linear_fwd(c, use_lora, l, 3, a->attn_out, c->W + o->o, a->post_attn_in, T, qd, d, 1);
        if (!(xf_parts && sb_rmsnorm_parts(c, a->post_attn_in, c->W + o->post_norm, a->x_norm_ffn, T, d, RMS_EPS))) {
            sb_amax_announce(c, a->x_norm_ffn, Td);
            sb_rmsnorm(c, a->post_attn_in, c->W + o->post_norm, a->x_norm_ffn, T, d, RMS_EPS);
        }
        sb_gemm_keep_begin(c);
        sb_amax_announce(c, a->gate, (size_t)T * F);        /* the products' epilogues leave max |gate|, max |up| for the bound below */
        linear_fwd(c, use_lora, l, 4, a->x_norm_ffn, c->W + o->gate, a->gate, T, d, F, 0);
        sb_amax_announce(c, a->up, (size_t)T * F);
        linear_fwd(c, use_lora, l, 5, a->x_norm_ffn, c->W + o->up, a->up, T, d, F, 0);
        sb_gemm_keep_end(c);
        /* silu(gate) * up is read only as an operand (down projection, its weight gradient): when those products take FP16 parts
           the kernel writes the parts and no FP32 copy */
        if (!(ffn_parts && sb_swiglu_parts(c, a->gate, a->up, a->ffn_hidden, (size_t)T * F))) {
            sb_amax_announce(c, a->ffn_hidden, (size_t)T * F);
            sb_swiglu(c, a->gate, a->up, a->ffn_hidden, (size_t)T * F);
        }
        sb_copy(c, next_in, a->post_attn_in, Td * sizeof(float));
        linear_fwd(c, use_lora, l, 6, a->ffn_hidden, c->W + o->down, next_in, T, F, d, 1);
        nan_mark(c, next_in, Td, nan_fwd_base(c) + (uint32_t)l);
    }
    if (!(hn_parts && sb_rmsnorm_parts(c, c->final_in, c->W + (size_t)c->V * d, c->hidden_norm, T, d, RMS_EPS))) {
        sb_amax_announce(c, c->hidden_norm, Td);
        sb_rmsnorm(c, c->final_in, c->W + (size_t)c->V * d, c->hidden_norm, T, d, RMS_EPS);
    }
    nan_mark(c, c->hidden_norm, Td, 2); nan_mark(c, c->final_in, Td, 6);
    sb_gemm(c, c->hidden_norm, c->untied ? c->XW + extras_lm_off(c) : c->W, c->logits, T, c->V, d, 0, 1, 0);       /* tied LM head, or the separate one */
    nan_mark(c, c->logits, (size_t)T * c->V, 1);
}

/* AdamW of the layer ranges, run from inside the backward pass of a data-parallel step (see there) */
typedef struct { int on, done, step; float lr, gscale; } early_adamw_t;

/* `reduce`: hand every finished gradient range to the data-parallel all-reduce as soon as it is complete */
static void backward_pass(sb_ctx_t* c, int T, int B, int max_seq, float theta, int full, int reduce, early_adamw_t* early) {
    const int d = c->d, F = c->F, qd = c->qd, kvd = c->kvd, L = c->L, V = c->V;
    float* gh = c->g_hidden; float* gx = c->g_xnorm;
    float* Gd = full ? c->G : NULL;
    float* norm_sink = c->g_tmp;                 /* LoRA mode: norm-scale gradients are discarded */
    if (!full) sb_memset(c, norm_sink, 0, (size_t)d * sizeof(float));
    sb_gemm_keep_begin(c);
    sb_gemm(c, c->dlogits, c->untied ? c->XW + extras_lm_off(c) : c->W, gx, T, d, V, 0, 0, 0);
    if (full) sb_gemm(c, c->dlogits, c->hidden_norm, c->untied ? c->XG + extras_lm_off(c) : Gd, V, d, T, 1, 0, 1);
    sb_gemm_keep_end(c);
    nan_mark(c, c->dlogits, (size_t)T * V, 3); nan_mark(c, gx, (size_t)T * d, 4);
    sb_amax_announce(c, gh, (size_t)T * d);
    sb_rmsnorm_backward(c, c->final_in, c->W + (size_t)V * d, gx, NULL, gh, full ? Gd + (size_t)V * d : norm_sink, T, d, RMS_EPS);
    nan_mark(c, gh, (size_t)T * d, 5); nan_mark(c, gh, (size_t)T * d, 0);
    const int ffn_lora = !full && (c->lora_mask & 0x70);
    const int ffn_parts_bwd = !c->nan_on && !ffn_lora && sb_gemm_reads_f16_parts(c, T, d, F, 0, 0) && (!full || sb_gemm_reads_f16_parts(c, F, d, T, 1, 0));
    for (int l = L - 1; l >= 0; l--) {
        const sb_layer_off_t* o = &c->off[l];
        sb_layer_act_t* a = &c->act[l];
        /* FFN */
        sb_gemm_keep_begin(c);                       /* gh (and, with adapters, what they read) is split once for the whole group */
        if (full) sb_gemm(c, gh, a->ffn_hidden, Gd + o->down, d, F, T, 1, 0, 1);
        sb_amax_announce(c, c->g_ffn, (size_t)T * F);
        sb_gemm(c, gh, c->W + o->down, c->g_ffn, T, F, d, 0, 0, 0);
        if (!full) lora_bwd(c, l, 6, gh, a->ffn_hidden, c->g_ffn, T);
        sb_gemm_keep_end(c);
        if (!(ffn_parts_bwd && sb_swiglu_backward_parts(c, a->gate, a->up, c->g_ffn, c->g_gate, c->g_up, (size_t)T * F))) {
            sb_amax_announce(c, c->g_gate, (size_t)T * F); sb_amax_announce(c, c->g_up, (size_t)T * F);
            sb_swiglu_backward(c, a->gate, a->up, c->g_ffn, c->g_gate, c->g_up, (size_t)T * F);
        }
        sb_gemm_keep_begin(c);
        if (full) {
            sb_gemm(c, c->g_gate, a->x_norm_ffn, Gd + o->gate, F, d, T, 1, 0, 1);
            sb_gemm(c, c->g_up, a->x_norm_ffn, Gd + o->up, F, d, T, 1, 0, 1);
        }
        sb_gemm(c, c->g_gate, c->W + o->gate, gx, T, d, F, 0, 0, 0);
        sb_gemm(c, c->g_up, c->W + o->up, gx, T, d, F, 0, 0, 1);
        if (!full) { lora_bwd(c, l, 4, c->g_gate, a->x_norm_ffn, gx, T); lora_bwd(c, l, 5, c->g_up, a->x_norm_ffn, gx, T); }
        sb_gemm_keep_end(c);
        sb_amax_announce(c, gh, (size_t)T * d);
        sb_rmsnorm_backward(c, a->post_attn_in, c->W + o->post_norm, gx, gh, gh, full ? Gd + o->post_norm : norm_sink, T, d, RMS_EPS);
        /* attention */
        sb_gemm_keep_begin(c);
        if (full) sb_gemm(c, gh, a->attn_out, Gd + o->o, d, qd, T, 1, 0, 1);
        sb_gemm(c, gh, c->W + o->o, c->g_attn, T, qd, d, 0, 0, 0);
        if (!full) lora_bwd(c, l, 3, gh, a->attn_out, c->g_attn, T);
        sb_gemm_keep_end(c);
        nan_mark(c, c->g_attn, (size_t)T * qd, nan_bwd_base(c) + 5u * (uint32_t)l);
        sb_attention_backward(c, a->q, a->k, a->v, a->attn_out, a->lse, c->g_attn, c->g_q, c->g_k, c->g_v, 0,
                              c->seq_starts, c->seq_ids, B, T, c->Hq, c->Hkv, c->hd);
        if (c->qk_norm) {
            /* the reference has no backward for qk_norm; this is the derivative of its forward */
            sb_qk_norm_backward(c, a->q, a->q_rms, c->g_q, c->g_q, T, qd, RMS_EPS);
            sb_qk_norm_backward(c, a->k, a->k_rms, c->g_k, c->g_k, T, kvd, RMS_EPS);
        }
        sb_amax_announce(c, c->g_q, (size_t)T * qd); sb_amax_announce(c, c->g_k, (size_t)T * kvd);
        sb_rope2(c, c->g_q, c->g_k, c->pos_ids, T, c->Hq, c->Hkv, c->hd, theta, max_seq, 1);
        if (c->nan_on) {
            const uint32_t nb = nan_bwd_base(c) + 5u * (uint32_t)l;
            nan_mark(c, c->g_q, (size_t)T * qd, nb + 1); nan_mark(c, c->g_k, (size_t)T * kvd, nb + 2); nan_mark(c, c->g_v, (size_t)T * kvd, nb + 3);
        }
        float* gq = c->g_q; float* gk = c->g_k;
        if (c->head_norm) {
            const size_t xo = (size_t)l * 2 * c->hd;
            sb_amax_announce(c, c->g_q2, (size_t)T * qd); sb_amax_announce(c, c->g_k2, (size_t)T * kvd);
            sb_rmsnorm_backward(c, a->q_pre, c->XW + xo, c->g_q, NULL, c->g_q2, full ? c->XG + xo : norm_sink, T * c->Hq, c->hd, RMS_EPS);
            sb_rmsnorm_backward(c, a->k_pre, c->XW + xo + c->hd, c->g_k, NULL, c->g_k2, full ? c->XG + xo + c->hd : norm_sink, T * c->Hkv, c->hd, RMS_EPS);
            gq = c->g_q2; gk = c->g_k2;
        }
        sb_gemm_keep_begin(c);
        if (full) {
            sb_gemm(c, gq, a->x_norm_attn, Gd + o->q, qd, d, T, 1, 0, 1);
            sb_gemm(c, gk, a->x_norm_attn, Gd + o->k, kvd, d, T, 1, 0, 1);
            sb_gemm(c, c->g_v, a->x_norm_attn, Gd + o->v, kvd, d, T, 1, 0, 1);
        }
        sb_gemm(c, gq, c->W + o->q, gx, T, d, qd, 0, 0, 0);
        sb_gemm(c, gk, c->W + o->k, gx, T, d, kvd, 0, 0, 1);
        sb_gemm(c, c->g_v, c->W + o->v, gx, T, d, kvd, 0, 0, 1);
        if (!full) { lora_bwd(c, l, 0, gq, a->x_norm_attn, gx, T); lora_bwd(c, l, 1, gk, a->x_norm_attn, gx, T); lora_bwd(c, l, 2, c->g_v, a->x_norm_attn, gx, T); }
        sb_gemm_keep_end(c);
        sb_amax_announce(c, gh, (size_t)T * d);
        sb_rmsnorm_backward(c, a->layer_in, c->W + o->in_norm, gx, gh, gh, full ? Gd + o->in_norm : norm_sink, T, d, RMS_EPS);
        nan_mark(c, gh, (size_t)T * d, nan_ghid_base(c) + (uint32_t)l);
        if (!full && c->LW) lora_compact_grads(c, l);
        if (reduce) {
            if (full) sb_dp_bucket_ready(c, Gd + o->q, o->post_norm + (size_t)d - o->q);
            else { size_t per = lora_layer_params(c); sb_dp_bucket_ready(c, c->LG + per * (size_t)l, per); }
        }
    }
    if (full) {
        nan_mark(c, gh, (size_t)T * d, 8);
        sb_embedding_backward(c, c->tokens, gh, Gd, T, d, V);
        nan_mark(c, Gd, (size_t)V * d, 9);
    }
    /* Every layer's gradients are with the all-reduce.  The last bucket (embedding with the LM head's share, and the final norm:
       1.2 GB at the benchmark size) is handed over now; AdamW of the layer ranges starts as soon as the layers' buckets are back
       and runs beside its reduction.  The update is elementwise, so doing it in two launches changes no value. */
    const int early_on = full && reduce && early && early->on && sb_dp_mark_partial(c) == 0;
    if (full && reduce) {
        sb_dp_bucket_ready_last(c, Gd, c->off[0].q);
        if (c->XG) sb_dp_bucket_ready_last(c, c->XG, c->n_extras);
    }
    if (early_on && sb_dp_wait_partial(c) == 0) {
        const size_t o0 = c->off[0].q;
        sb_adamw(c, c->W + o0, c->G + o0, c->M + o0, c->Vv + o0, c->n_params - o0, early->lr, 0.9f, 0.999f, 0.01f, 1e-8f, early->step,
                 early->gscale, NULL, 0.f);
        early->done = 1;
    }
}

/* tokens, targets and sequence starts: clamp negative ids to 0, last token of a
 * sequence has target 0 (src/train_cuda.c:2030-2043); staged in pinned memory */
static int upload_batch(sb_ctx_t* c, const int* tokens, int T, const int* seq_starts, int B, int* max_seq_out) {
    if (sb_ensure_tokens(c, T, B)) return 1;
    size_t words = (size_t)2 * T + (size_t)B + 1 + 4;
    if (ensure_pinned(c, words * sizeof(uint32_t) + 64)) return 1;
    uint32_t* h_tok = (uint32_t*)c->h_pinned; uint32_t* h_tgt = h_tok + T; uint32_t* h_ss = h_tgt + T;
    int max_seq = 0;
    for (int b = 0; b < B; b++) {
        int s = seq_starts[b], e = seq_starts[b + 1];
        if (s < 0 || e < s || e > T) { sb_set_status(c, SB_ERR_ARG); return 1; }
        if (e - s > max_seq) max_seq = e - s;
        for (int t = s; t < e; t++) {
            int tk = tokens[t];
            h_tok[t] = tk < 0 ? 0u : (uint32_t)tk;
            if (t < e - 1) { int nx = tokens[t + 1]; h_tgt[t] = nx < 0 ? 0u : (uint32_t)nx; } else h_tgt[t] = 0u;
        }
    }
    if (seq_starts[0] != 0 || seq_starts[B] != T) { sb_set_status(c, SB_ERR_ARG); return 1; }
    for (int b = 0; b <= B; b++) h_ss[b] = (uint32_t)seq_starts[b];
    cudaMemcpyAsync(c->tokens, h_tok, (size_t)T * 4, cudaMemcpyHostToDevice, S(c));
    cudaMemcpyAsync(c->targets, h_tgt, (size_t)T * 4, cudaMemcpyHostToDevice, S(c));
    cudaMemcpyAsync(c->seq_starts, h_ss, (size_t)(B + 1) * 4, cudaMemcpyHostToDevice, S(c));
    sb_seq_index(c, c->seq_starts, B, T, c->pos_ids, c->seq_ids);
    sb_set_host_seq(c, seq_starts, B);
    *max_seq_out = max_seq;
    return 0;
}

static float lr_for_step(const train_state_t* st, int accum) {
    /* 100-step linear warm-up, then divided by the accumulation count (src/train_cuda.c:2298-2303) */
    float lr = st->learning_rate;
    if (st->optimizer_step < 100.0f) lr = st->learning_rate * (st->optimizer_step / 100.0f);
    return lr / accum;
}

static float step_body(train_state_t* st, int* tokens, int T, int* seq_starts, int B, cuda_train_context_t* ctx, int full, int train, int resident) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!st || !st->config || !c || T <= 0 || B <= 0) return -1.0f;
    if (!resident && (!tokens || !seq_starts)) return -1.0f;
    if (full && !st->full_weights) return -1.0f;
    if (!full && train && !st->lora) return -1.0f;
    int num_valid = T - B;
    if (num_valid <= 0) return 0.0f;
    int use_lora = (!full && st->lora != NULL);
    c->qk_norm = st->config->use_qk_norm ? 1 : 0;
    if (ensure_model(c, st, full ? 0 : (use_lora ? 1 : c->frozen_base))) return -1.0f;
    if (use_lora && ensure_lora(c, st->lora)) return -1.0f;
    if (ensure_extras(c, full && train)) return -1.0f;
    if (ensure_activations(c, T, train)) return -1.0f;
    if (use_lora && c->lora_tmp_cap < (size_t)T * c->lora_R) {
        cudaStreamSynchronize(S(c));
        if (c->lora_tmp) cudaFree(c->lora_tmp);
        c->lora_tmp = NULL;
        if (sb_check(c, cudaMalloc((void**)&c->lora_tmp, (size_t)T * c->lora_R * sizeof(float)), "lora tmp")) return -1.0f;
        c->lora_tmp_cap = (size_t)T * c->lora_R;
    }
    if (use_lora) lora_refresh_padded(c);
    float theta = st->config->rope_theta > 0 ? st->config->rope_theta : 10000.0f;
    int max_seq = 0;
    if (resident) {
        /* batch of the previous call is still on the device: no host-to-device copy, no loss read-back */
        if (c->res_T != T || c->res_B != B) { sb_set_status(c, SB_ERR_ARG); return -1.0f; }
        max_seq = c->res_max_seq;
    } else {
        if (upload_batch(c, tokens, T, seq_starts, B, &max_seq)) return -1.0f;
        c->res_T = T; c->res_B = B; c->res_max_seq = max_seq;
    }
    c->pub.batch_size = B;

    if (nan_begin(c, train && st->debug_nan_check)) return -1.0f;
    if (train && st->accumulation_counter == 0) {
        if (full) sb_memset(c, c->G, 0, c->n_params * sizeof(float));
        else { sb_memset(c, c->LG, 0, c->n_lora * sizeof(float)); sb_memset(c, c->LGp, 0, c->n_lora_pad * sizeof(float)); }
        if (full && c->XG) sb_memset(c, c->XG, 0, c->n_extras * sizeof(float));
    }
    forward_pass(c, T, max_seq, theta, use_lora);
    /* training: the gradient of the logits leaves the loss kernel as the FP16 parts the two LM-head backward products read (its
       FP32 form is never written); evaluation, the NaN guard (which inspects the FP32 array) and contexts without the parts arena
       take the plain kernel */
    const int ce_parts = train && !c->nan_on && sb_gemm_reads_f16_parts(c, T, c->d, c->V, 0, 0) && (!full || sb_gemm_reads_f16_parts(c, c->V, c->d, T, 1, 0));
    if (!(ce_parts && sb_cross_entropy_parts(c, c->logits, c->targets, c->dlogits, c->loss_rows, c->pos_ids, c->seq_ids, c->seq_starts,
                                                          T, c->V, num_valid))) {
        if (train) sb_amax_announce(c, c->dlogits, (size_t)T * c->V);
        sb_cross_entropy(c, c->logits, c->targets, c->dlogits, c->loss_rows, c->pos_ids, c->seq_ids, c->seq_starts, T, c->V, num_valid);
    }
    sb_reduce_sum(c, c->loss_rows, c->d_loss, (size_t)T);

    if (train) {
        int accum = st->gradient_accumulation_steps < 1 ? 1 : st->gradient_accumulation_steps;
        int last_micro = (st->accumulation_counter + 1 >= accum);
        /* data parallel, last micro-batch, no clipping (its norm needs every gradient first): the optimizer's parameters are known
           now, so the layer ranges can be updated while the last bucket is still being reduced */
        early_adamw_t early = {0, 0, 0, 0.f, 0.f};
        if (full && last_micro && c->dp_world > 1 && c->grad_clip <= 0.f && !c->nan_on) {
            early.on = 1; early.step = st->optimizer_step + 1; early.gscale = 1.0f / (float)c->dp_world;
            train_state_t tmp = *st; tmp.optimizer_step = early.step;
            early.lr = lr_for_step(&tmp, accum);
        }
        backward_pass(c, T, B, max_seq, theta, full, last_micro && c->dp_world > 1, &early);
        if (c->nan_on) {
            /* the reference reads its flags back before the optimizer and skips it when one is set, leaving the counters alone
               (src/train_cuda.c:1086-1187).  Data parallel: the buckets are already in flight, so every rank first waits for them and
               then looks at the whole reduced gradient, which is the same on all ranks, so that all of them skip or none does. */
            if (last_micro && c->dp_world > 1) {
                if (sb_dp_join(c)) return -1.0f;
                nan_mark(c, full ? c->G : c->LG, full ? c->n_params : c->n_lora, 9);
            }
            if (nan_tripped(c, st, T)) { c->nan_on = 0; st->nan_detected = 1; return NAN; }
            c->nan_on = 0;
        }
        st->accumulation_counter++;
        if (st->accumulation_counter >= accum) {
            st->optimizer_step++;
            float lr = lr_for_step(st, accum);
            float* w = full ? c->W : c->LW; float* g = full ? c->G : c->LG;
            float* m = full ? c->M : c->LM; float* v = full ? c->Vv : c->LV;
            size_t n = full ? c->n_params : c->n_lora;
            float gscale = 1.0f;
            if (c->dp_world > 1) {
                if (sb_dp_join(c)) return -1.0f;
                gscale = 1.0f / (float)c->dp_world;
            }
            const float* sumsq = NULL;
            const int extras = full && c->XG != NULL;
            if (c->grad_clip > 0.f) {
                sb_sumsq(c, g, n, c->d_gnorm); sumsq = c->d_gnorm;
                if (extras) { sb_sumsq(c, c->XG, c->n_extras, c->d_gnorm + 1); sb_add(c, c->d_gnorm, c->d_gnorm + 1, c->d_gnorm, 1); }   /* one norm over all trained parameters */
            }
            if (early.done) n = c->off[0].q;           /* the layer ranges were updated inside the backward pass: embedding and final norm remain */
            sb_adamw(c, w, g, m, v, n, lr, 0.9f, 0.999f, 0.01f, 1e-8f, st->optimizer_step, gscale, sumsq, c->grad_clip);
            if (extras) sb_adamw(c, c->XW, c->XG, c->XM, c->XV, c->n_extras, lr, 0.9f, 0.999f, 0.01f, 1e-8f, st->optimizer_step, gscale, sumsq, c->grad_clip);
            if (!full) c->lora_pad_stale = 1;          /* the adapters moved: the padded copies follow before the next step */
            st->accumulation_counter = 0;
        }
    }
    if (resident) return sb_check(c, cudaGetLastError(), "training step (resident batch)") ? -1.0f : 0.0f;
    /* data parallel: a peer that died leaves this rank's collectives unfinished for ever; wait for them with a limit on the host
       (the communicator is aborted when it runs out) instead of inside the unbounded stream synchronisation below */
    if (train && c->dp_world > 1 && seraph_dp_wait(ctx, c->dp_timeout_ms) != SB_OK) return -1.0f;
    float* h_loss = (float*)((char*)c->h_pinned + c->h_pinned_bytes - 64);
    cudaMemcpyAsync(h_loss, c->d_loss, sizeof(float), cudaMemcpyDeviceToHost, S(c));
    if (sb_check(c, cudaStreamSynchronize(S(c)), "training step")) return -1.0f;
    float loss = *h_loss / (float)num_valid;
    if (train && st->debug_nan_check && (isnan(loss) || isinf(loss))) { st->nan_detected = 1; return NAN; }
    return loss;
}

/* prepared operand parts of weights and saved activations are shared by the products of one call and dropped when it returns */
static float step_common(train_state_t* st, int* tokens, int T, int* seq_starts, int B, cuda_train_context_t* ctx, int full, int train, int resident) {
    sb_ctx_t* c = sb_priv(ctx);
    if (c) sb_parts_open(c);
    float r = step_body(st, tokens, T, seq_starts, B, ctx, full, train, resident);
    if (c) sb_parts_close(c);
    return r;
}

float cuda_train_step_gpu_full_batch(train_state_t* state, int* tokens_packed, int total_tokens, int* seq_starts, int batch_size,
                                     cuda_train_context_t* ctx) {
    return step_common(state, tokens_packed, total_tokens, seq_starts, batch_size, ctx, 1, 1, 0);
}
float cuda_train_step_gpu_full(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx) {
    int ss[2] = {0, num_tokens};
    return step_common(state, tokens, num_tokens, ss, 1, ctx, 1, 1, 0);
}
float cuda_train_step_gpu_lora_batch(train_state_t* state, int* tokens_packed, int total_tokens, int* seq_starts, int batch_size,
                                     cuda_train_context_t* ctx) {
    return step_common(state, tokens_packed, total_tokens, seq_starts, batch_size, ctx, 0, 1, 0);
}
float cuda_train_step_gpu_lora(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx) {
    int ss[2] = {0, num_tokens};
    return step_common(state, tokens, num_tokens, ss, 1, ctx, 0, 1, 0);
}

/* forward + loss only (src/train_cuda.c:2677); uses the adapters when the state trains LoRA */
float cuda_eval_forward(train_state_t* state, int* tokens, int num_tokens, cuda_train_context_t* ctx) {
    if (!state || !state->config || !ctx || num_tokens < 2) return -1.0f;
    int ss[2] = {0, num_tokens};
    int full = state->lora == NULL;
    return step_common(state, tokens, num_tokens, ss, 1, ctx, full, 0, 0);
}

/* One packed forward pass over the samples gathered in pk[0..T) / ss[0..B]: every sample's mean loss is added to *total
 * (and counted in *valid) from the per-token losses of the pass, summed per sample on the host in token order. */
static void eval_flush(train_state_t* state, cuda_train_context_t* ctx, int* pk, int* ss, int B, int full, float* rows,
                       double* total, int* valid) {
    sb_ctx_t* c = sb_priv(ctx);
    int T = ss[B];
    if (B <= 0 || T <= 0) return;
    float loss = step_common(state, pk, T, ss, B, ctx, full, 0, 0);
    if (loss < 0.0f || isnan(loss)) return;
    if (cudaMemcpy(rows, c->loss_rows, (size_t)T * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    for (int b = 0; b < B; b++) {
        double sum = 0.0;
        int n = ss[b + 1] - ss[b];
        for (int t = ss[b]; t < ss[b + 1] - 1; t++) sum += rows[t];       /* the last token of a sample predicts nothing */
        float l = (float)(sum / (double)(n - 1));
        if (l >= 0.0f && !isnan(l)) { *total += l; (*valid)++; }
    }
}

/* src/train_cuda.c:2812-2846: evenly spaced samples, mean of the samples' mean losses, perplexity = exp(mean).  The reference
 * runs one forward pass per sample; here the samples are packed, as many as fit eval_batch_tokens tokens (and at most 256),
 * into one pass each (seraph_b200_set_eval_batch_tokens(ctx, 0) restores one pass per sample). */
#define EVAL_MAX_SEQS 256
float cuda_evaluate(train_state_t* state, int* val_tokens, int num_val_tokens, int* offsets, int num_samples, int max_seq_len,
                    int max_eval_samples, cuda_train_context_t* ctx, float* out_perplexity) {
    if (!state || !val_tokens || !offsets || num_samples <= 0 || !ctx) { if (out_perplexity) *out_perplexity = 0.0f; return -1.0f; }
    sb_ctx_t* c = sb_priv(ctx);
    int max_eval = max_eval_samples > 0 ? max_eval_samples : num_samples;
    int stride = num_samples > max_eval ? num_samples / max_eval : 1;
    int budget = c ? c->eval_batch_tokens : 0;
    double total = 0.0; int valid = 0;
    int* pk = NULL; int* ss = NULL; float* rows = NULL;
    if (budget > 0) {
        if (budget < max_seq_len) budget = max_seq_len;
        pk = (int*)malloc((size_t)budget * sizeof(int));
        ss = (int*)malloc((EVAL_MAX_SEQS + 1) * sizeof(int));
        rows = (float*)malloc((size_t)budget * sizeof(float));
        if (!pk || !ss || !rows) { free(pk); free(ss); free(rows); pk = NULL; budget = 0; }
    }
    int full = state->lora == NULL;
    int B = 0;
    if (budget > 0) ss[0] = 0;
    for (int s = 0; s < num_samples; s += stride) {
        int start = offsets[s], end = (s + 1 < num_samples) ? offsets[s + 1] : num_val_tokens;
        int n = end - start;
        if (n > max_seq_len) n = max_seq_len;
        if (n < 2) continue;
        if (budget <= 0) {
            float loss = cuda_eval_forward(state, &val_tokens[start], n, ctx);
            if (loss >= 0.0f && !isnan(loss)) { total += loss; valid++; }
            continue;
        }
        if (B == EVAL_MAX_SEQS || ss[B] + n > budget) { eval_flush(state, ctx, pk, ss, B, full, rows, &total, &valid); B = 0; }
        memcpy(pk + ss[B], &val_tokens[start], (size_t)n * sizeof(int));
        ss[B + 1] = ss[B] + n;
        B++;
    }
    if (budget > 0) {
        eval_flush(state, ctx, pk, ss, B, full, rows, &total, &valid);
        free(pk); free(ss); free(rows);
    }
    float avg = valid > 0 ? (float)(total / valid) : -1.0f;
    if (out_perplexity) *out_perplexity = avg > 0.0f ? expf(avg) : 0.0f;
    return avg;
}

/* src/train_cuda.c:1244 / :1317 */
void cuda_download_full_weights(cuda_train_context_t* ctx, train_state_t* state) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || !state->full_weights || !c->W) return;
    int what = 0;
    for_each_tensor(c, state->full_weights, down_tensor, &what);
    sb_check(c, cudaStreamSynchronize(S(c)), "weight download");
}
void cuda_download_gpu_gradients(cuda_train_context_t* ctx, train_state_t* state) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || !state->full_weights || !c->G) return;
    int what = 1;
    for_each_tensor(c, state->full_weights, down_tensor, &what);
    sb_check(c, cudaStreamSynchronize(S(c)), "gradient download");
}
/* src/cuda_train_context.cu:3330: adapters A, B and their Adam moments back to the host model.
 * Gradients are copied too when the host adapter has room for them. */
void cuda_download_lora_weights(cuda_train_context_t* ctx, void* lora_ptr) {
    sb_ctx_t* c = sb_priv(ctx);
    lora_model_t* m = (lora_model_t*)lora_ptr;
    if (!c || !m || !c->LW) return;
    for (int a = 0; a < 7; a++) {
        if (!(c->lora_mask & (1 << a))) continue;
        lora_adapter_t** ls = lora_list(m, a);
        if (!ls) continue;
        int in, out; lora_dims(c, a, &in, &out);
        size_t nA = (size_t)c->lora_rank * in, nB = (size_t)out * c->lora_rank;
        for (int l = 0; l < c->L; l++) {
            lora_adapter_t* ad = ls[l];
            if (!ad) continue;
            size_t o = lora_off(c, l, a);
            cudaMemcpyAsync(ad->A, c->LW + o, nA * 4, cudaMemcpyDeviceToHost, S(c));
            cudaMemcpyAsync(ad->B, c->LW + o + nA, nB * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->m_A) cudaMemcpyAsync(ad->m_A, c->LM + o, nA * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->m_B) cudaMemcpyAsync(ad->m_B, c->LM + o + nA, nB * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->v_A) cudaMemcpyAsync(ad->v_A, c->LV + o, nA * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->v_B) cudaMemcpyAsync(ad->v_B, c->LV + o + nA, nB * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->grad_A) cudaMemcpyAsync(ad->grad_A, c->LG + o, nA * 4, cudaMemcpyDeviceToHost, S(c));
            if (ad->grad_B) cudaMemcpyAsync(ad->grad_B, c->LG + o + nA, nB * 4, cudaMemcpyDeviceToHost, S(c));
        }
    }
    sb_check(c, cudaStreamSynchronize(S(c)), "lora download");
}
void cuda_train_zero_lora_grads(cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !c->LG) return;
    sb_memset(c, c->LG, 0, c->n_lora * sizeof(float));
    if (c->LGp) sb_memset(c, c->LGp, 0, c->n_lora_pad * sizeof(float));
}

/* Extension: repeat the full-weight step on the batch the previous step call left on the device.
 * Nothing crosses the host-device boundary and the call does not wait for the GPU; the loss stays
 * on the device (seraph_b200_last_loss).  Returns 0 or a status code. */
int seraph_b200_step_full_resident(train_state_t* state, cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || c->res_T <= 0) return SB_ERR_ARG;
    float r = step_common(state, NULL, c->res_T, NULL, c->res_B, ctx, 1, 1, 1);
    return r < 0.f ? (c->status ? c->status : SB_ERR_ARG) : SB_OK;
}
/* the same for either kind of step: full != 0 the full-weight step, 0 the LoRA step of a state with adapters attached */
int seraph_b200_step_resident(train_state_t* state, cuda_train_context_t* ctx, int full) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || c->res_T <= 0) return SB_ERR_ARG;
    float r = step_common(state, NULL, c->res_T, NULL, c->res_B, ctx, full ? 1 : 0, 1, 1);
    return r < 0.f ? (c->status ? c->status : SB_ERR_ARG) : SB_OK;
}
/* mean loss of the last step, read from the device (synchronises) */
float seraph_b200_last_loss(cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || c->res_T <= c->res_B) return -1.0f;
    float v = 0.f;
    cudaStreamSynchronize(S(c));
    if (cudaMemcpy(&v, c->d_loss, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return -1.0f;
    return v / (float)(c->res_T - c->res_B);
}

/* Extension: logits [T,V] of the last step/eval, copied to the host */
int seraph_b200_download_logits(cuda_train_context_t* ctx, float* out, int T) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !out || !c->logits || T > c->T_cap) return SB_ERR_ARG;
    cudaMemcpyAsync(out, c->logits, (size_t)T * c->V * 4, cudaMemcpyDeviceToHost, S(c));
    return sb_check(c, cudaStreamSynchronize(S(c)), "logits download") ? SB_ERR_CUDA : SB_OK;
}

/* Extension: forget the resident weights, adapters and optimizer state, so that the next step uploads
 * them again from the host state (the reference uploads once per context, src/train_cuda.c:286-291). */
/* the full-weight model of `st` resident on the device (uploaded from the host copies if it is not yet); 0 on success */
int sb_ensure_full_model(sb_ctx_t* c, const train_state_t* st) {
    if (!c || !st || !st->config || !st->full_weights) return 1;
    return ensure_model(c, st, 0);
}

int seraph_b200_reset_model(cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    cudaStreamSynchronize(S(c));
    free_lora(c);
    free_activations(c);
    free_model(c);
    return SB_OK;
}

/* src/cuda_train_context.cu:2404 */
void sb_dp_finalize(sb_ctx_t* c);
void cuda_train_free(cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return;
    cudaStreamSynchronize(S(c));
    sb_dp_finalize(c);
    free_lora(c);
    free_activations(c);
    free_model(c);
    if (c->tokens) cudaFree(c->tokens);
    if (c->seq_starts) cudaFree(c->seq_starts);
    if (c->scratch) cudaFree(c->scratch);
    for (int i = 0; i < 5; i++) if (c->gemm_stage[i]) cudaFree(c->gemm_stage[i]);
    if (c->side_ready) {
        for (int i = 0; i < 4; i++) cudaStreamDestroy((cudaStream_t)c->side_stream[i]);
        for (int i = 0; i < 5; i++) cudaEventDestroy((cudaEvent_t)c->side_ev[i]);
    }
    if (c->rope_tab) cudaFree(c->rope_tab);
    sb_parts_free(c);
    if (c->d_amax) cudaFree(c->d_amax);
    for (int i = 0; i < SB_F16_SLOTS; i++) if (c->f16_slot[i].h) cudaFree(c->f16_slot[i].h);
    if (c->d_status) cudaFree(c->d_status);
    if (c->d_loss) cudaFree(c->d_loss);
    if (c->h_pinned) cudaFreeHost(c->h_pinned);
    free(c->h_seq);
    free(c->h_extras);
    if (c->pub.debug_nan_flags) cuda_train_buffer_free(ctx, c->pub.debug_nan_flags);
    cudaStreamDestroy(S(c));
    c->magic = 0;
    free(c);
}
