/*
 * ref_step.c - CPU restatement of one Seraph training step (forward, loss,
 * backward) as the fixed op sequence the reference issues on the GPU.
 *
 * TEST INFRASTRUCTURE ONLY (see ref_ops.c).
 *
 * Full-weight step: src/train_cuda.c:1966-2326 (cuda_train_step_gpu_full_batch;
 * the single-sequence twin :597 is the same sequence with batch_size 1).
 * LoRA step: forward adds src/train.c:6095-6186 and backward src/train.c:6287-6615
 * (train_step_gpu_lora, the only complete LoRA chain rule in the reference),
 * carried over to packed batches.
 *
 * Flat parameter order used here and by the tests:
 *   embed [V,d], final_norm [d], then per layer
 *   q [qd,d], k [kvd,d], v [kvd,d], o [d,qd], gate [F,d], up [F,d], down [d,F],
 *   in_norm [d], post_norm [d].
 * Flat LoRA order: per layer, for each of q,k,v,o,gate,up,down: A [r,in] then
 * B [out,r]; adapters switched off by the mask are skipped.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

void ref_embed_lookup(const uint32_t*, const float*, float*, int, int);
void ref_rmsnorm(const float*, const float*, float*, int, int, float);
void ref_matmul(const float*, const float*, float*, int, int, int, int, int, int);
void ref_rope(const float*, float*, const uint32_t*, int, int, int, int, float, int);
void ref_qk_norm(float*, float*, int, int, int, int, float);
void ref_qk_norm_backward(const float*, const float*, const float*, float*, int, int, int, int, float);
void ref_attention(const float*, const float*, const float*, float*, float*, const uint32_t*, int, int, int, int, int);
void ref_attention_backward(const float*, const float*, const float*, const float*, float*, float*, float*,
                            const uint32_t*, int, int, int, int, int);
void ref_add(const float*, const float*, float*, size_t);
void ref_mul(const float*, const float*, float*, size_t);
void ref_silu(const float*, float*, size_t);
void ref_cross_entropy_grad(const float*, const uint32_t*, float*, float*, const uint32_t*, int, int, int, int);
float ref_reduce_sum(const float*, size_t);
void ref_silu_backward(const float*, const float*, float*, size_t);
void ref_mul_backward(const float*, const float*, const float*, float*, float*, size_t);
void ref_rmsnorm_backward(const float*, const float*, const float*, float*, float*, int, int, float);
void ref_embedding_backward(const uint32_t*, const float*, float*, int, int);
void ref_lora_backward(const float*, const float*, const float*, const float*, float*, float*, float*, int, int, int, int, float);
void ref_lora_forward_add(const float*, float*, const float*, const float*, float*, int, int, int, int, float);

/* head_norm: learned RMSNorm over each head of q and k before RoPE (weights q_norm [hd], k_norm [hd] per layer);
 * untied: a separate lm_head [V,d] instead of the embedding matrix.  Neither exists in the reference's training step
 * (trainable_weights_t has no such tensors, include/train.h:75-90): they are options of the new library, and their
 * parameters travel in a second flat array ("extras": per layer q_norm, k_norm; then lm_head). */
typedef struct { int V, d, L, Hq, Hkv, hd, F; float eps, theta; int qk_norm, head_norm, untied; } ref_cfg_t;

size_t ref_extras_count(const ref_cfg_t* c) {
    return (c->head_norm ? (size_t)c->L * 2 * c->hd : 0) + (c->untied ? (size_t)c->V * c->d : 0);
}

typedef struct { size_t q, k, v, o, gate, up, down, in_norm, post_norm; } layer_off_t;

static size_t layer_offsets(const ref_cfg_t* c, size_t base, layer_off_t* o) {
    size_t qd = (size_t)c->Hq * c->hd, kvd = (size_t)c->Hkv * c->hd, d = c->d, F = c->F;
    o->q = base; base += qd * d;
    o->k = base; base += kvd * d;
    o->v = base; base += kvd * d;
    o->o = base; base += d * qd;
    o->gate = base; base += F * d;
    o->up = base; base += F * d;
    o->down = base; base += d * F;
    o->in_norm = base; base += d;
    o->post_norm = base; base += d;
    return base;
}

size_t ref_param_count(const ref_cfg_t* c) {
    size_t n = (size_t)c->V * c->d + c->d;
    layer_off_t o;
    for (int l = 0; l < c->L; l++) n = layer_offsets(c, n, &o);
    return n;
}

/* adapter index: 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down */
static void lora_dims(const ref_cfg_t* c, int a, int* in, int* out) {
    int qd = c->Hq * c->hd, kvd = c->Hkv * c->hd;
    switch (a) {
        case 0: *in = c->d; *out = qd; break;
        case 1: case 2: *in = c->d; *out = kvd; break;
        case 3: *in = qd; *out = c->d; break;
        case 4: case 5: *in = c->d; *out = c->F; break;
        default: *in = c->F; *out = c->d; break;
    }
}

size_t ref_lora_param_count(const ref_cfg_t* c, int rank, int mask) {
    size_t n = 0;
    for (int a = 0; a < 7; a++) if (mask & (1 << a)) { int in, out; lora_dims(c, a, &in, &out); n += (size_t)rank * in + (size_t)out * rank; }
    return n * c->L;
}

/* offset of adapter a of layer l (A first, then B); (size_t)-1 if masked off */
static size_t lora_off(const ref_cfg_t* c, int rank, int mask, int l, int a) {
    if (!(mask & (1 << a))) return (size_t)-1;
    size_t per_layer = ref_lora_param_count(c, rank, mask) / c->L, n = per_layer * l;
    for (int b = 0; b < a; b++) if (mask & (1 << b)) { int in, out; lora_dims(c, b, &in, &out); n += (size_t)rank * in + (size_t)out * rank; }
    return n;
}

static float* fbuf(size_t n) { return (float*)calloc(n ? n : 1, sizeof(float)); }

/*
 * One forward + loss + backward.  grads (full-weight mode) or lora_grads (LoRA
 * mode) are accumulated into, as the reference's `accumulate=1` GEMMs and
 * atomics do; the caller zeroes them at the start of an accumulation cycle
 * (src/train_cuda.c:2011-2013).
 *
 * lora == NULL: full-weight step.  Otherwise base weights are frozen and only
 * adapter gradients are produced.  lora_exact = 0 reproduces the reference,
 * which leaves the adapters' own contribution out of dX (grad_input=NULL at
 * every call, e.g. src/train.c:6427); lora_exact = 1 adds s*(dY B) A.
 *
 * Returns the mean loss over the valid predictions, or 0 when there is none
 * (src/train_cuda.c:1990-1991).  logits_out (optional) receives [T,V].
 */
float ref_train_step(const ref_cfg_t* c, const float* P, float* G,
                     const float* lora, float* lora_grads, int rank, float alpha, int mask, int lora_exact,
                     const int* tokens, int T, const int* seq_starts, int B,
                     float* logits_out, float* dhidden0_out, const float* X, float* GX) {
    const int d = c->d, F = c->F, V = c->V, L = c->L, Hq = c->Hq, Hkv = c->Hkv, hd = c->hd;
    const int qd = Hq * hd, kvd = Hkv * hd;
    const float eps = c->eps, theta = c->theta > 0 ? c->theta : 10000.0f;
    const float ls = rank > 0 ? alpha / rank : 0.f;
    int num_valid = T - B;
    if (num_valid <= 0) return 0.0f;

    uint32_t* tok = (uint32_t*)malloc((size_t)T * 4);
    uint32_t* tgt = (uint32_t*)malloc((size_t)T * 4);
    uint32_t* ss = (uint32_t*)malloc((size_t)(B + 1) * 4);
    for (int b = 0; b <= B; b++) ss[b] = (uint32_t)seq_starts[b];
    /* negative ids clamp to 0; last token of each sequence has target 0
     * (src/train_cuda.c:2030-2043) */
    for (int b = 0; b < B; b++)
        for (int t = seq_starts[b]; t < seq_starts[b + 1]; t++) {
            tok[t] = tokens[t] < 0 ? 0u : (uint32_t)tokens[t];
            tgt[t] = (t < seq_starts[b + 1] - 1) ? (tokens[t + 1] < 0 ? 0u : (uint32_t)tokens[t + 1]) : 0u;
        }

    const float* E = P;
    const float* wfin = P + (size_t)V * d;
    layer_off_t* off = (layer_off_t*)malloc(sizeof(layer_off_t) * L);
    { size_t n = (size_t)V * d + d; for (int l = 0; l < L; l++) n = layer_offsets(c, n, &off[l]); }

    size_t Td = (size_t)T * d, TF = (size_t)T * F, Tq = (size_t)T * qd, Tkv = (size_t)T * kvd;
    /* per-layer caches, as the reference keeps them (src/train_cuda.c:2064-2075) */
    float **c_in = malloc(sizeof(float*) * L), **c_xa = malloc(sizeof(float*) * L), **c_q = malloc(sizeof(float*) * L),
          **c_k = malloc(sizeof(float*) * L), **c_v = malloc(sizeof(float*) * L), **c_att = malloc(sizeof(float*) * L),
          **c_pa = malloc(sizeof(float*) * L), **c_xf = malloc(sizeof(float*) * L), **c_g = malloc(sizeof(float*) * L),
          **c_u = malloc(sizeof(float*) * L), **c_s = malloc(sizeof(float*) * L), **c_fh = malloc(sizeof(float*) * L);
    float **c_qr = calloc((size_t)L, sizeof(float*)), **c_kr = calloc((size_t)L, sizeof(float*));      /* row statistics of qk_norm */
    float **c_qp = calloc((size_t)L, sizeof(float*)), **c_kp = calloc((size_t)L, sizeof(float*));      /* q, k before the per-head norm */
    const float* Wlm = (c->untied && X) ? X + (c->head_norm ? (size_t)L * 2 * hd : 0) : NULL;
    float* GWlm = (c->untied && GX) ? GX + (c->head_norm ? (size_t)L * 2 * hd : 0) : NULL;
    float* hidden = fbuf(Td); float* tmp = fbuf(Td); float* ltmp = fbuf((size_t)T * (rank > 0 ? rank : 1));

#define LA(l, a) (lora + lora_off(c, rank, mask, l, a))
#define LB(l, a, in) (lora + lora_off(c, rank, mask, l, a) + (size_t)rank * (in))
#define LGA(l, a) (lora_grads + lora_off(c, rank, mask, l, a))
#define LGB(l, a, in) (lora_grads + lora_off(c, rank, mask, l, a) + (size_t)rank * (in))
#define HAS(a) (lora && (mask & (1 << (a))))

    ref_embed_lookup(tok, E, hidden, T, d);
    for (int l = 0; l < L; l++) {
        const layer_off_t* o = &off[l];
        c_in[l] = fbuf(Td); memcpy(c_in[l], hidden, Td * 4);
        c_xa[l] = fbuf(Td); ref_rmsnorm(hidden, P + o->in_norm, c_xa[l], T, d, eps);
        c_q[l] = fbuf(Tq); c_k[l] = fbuf(Tkv); c_v[l] = fbuf(Tkv);
        ref_matmul(c_xa[l], P + o->q, c_q[l], T, qd, d, 0, 1, 0);
        if (HAS(0)) ref_lora_forward_add(c_xa[l], c_q[l], LA(l, 0), LB(l, 0, d), ltmp, T, d, qd, rank, ls);
        ref_matmul(c_xa[l], P + o->k, c_k[l], T, kvd, d, 0, 1, 0);
        if (HAS(1)) ref_lora_forward_add(c_xa[l], c_k[l], LA(l, 1), LB(l, 1, d), ltmp, T, d, kvd, rank, ls);
        ref_matmul(c_xa[l], P + o->v, c_v[l], T, kvd, d, 0, 1, 0);
        if (HAS(2)) ref_lora_forward_add(c_xa[l], c_v[l], LA(l, 2), LB(l, 2, d), ltmp, T, d, kvd, rank, ls);
        if (c->head_norm && X) {    /* every head of q and k normalised with a learned scale, before RoPE */
            c_qp[l] = fbuf(Tq); memcpy(c_qp[l], c_q[l], Tq * 4);
            c_kp[l] = fbuf(Tkv); memcpy(c_kp[l], c_k[l], Tkv * 4);
            ref_rmsnorm(c_qp[l], X + (size_t)l * 2 * hd, c_q[l], T * Hq, hd, eps);
            ref_rmsnorm(c_kp[l], X + (size_t)l * 2 * hd + hd, c_k[l], T * Hkv, hd, eps);
        }
        ref_rope(c_q[l], c_q[l], ss, T, B, Hq, hd, theta, 0);
        ref_rope(c_k[l], c_k[l], ss, T, B, Hkv, hd, theta, 0);
        if (c->qk_norm) {       /* shaders/qk_norm.comp after RoPE (src/train.c:4688-4689) */
            c_qr[l] = fbuf((size_t)T); c_kr[l] = fbuf((size_t)T);
            ref_qk_norm(c_q[l], c_qr[l], T, Hq, hd, 1, eps);
            ref_qk_norm(c_k[l], c_kr[l], T, Hkv, hd, 1, eps);
        }
        c_att[l] = fbuf(Tq);
        ref_attention(c_q[l], c_k[l], c_v[l], c_att[l], NULL, ss, T, B, Hq, Hkv, hd);
        ref_matmul(c_att[l], P + o->o, tmp, T, d, qd, 0, 1, 0);
        if (HAS(3)) ref_lora_forward_add(c_att[l], tmp, LA(l, 3), LB(l, 3, qd), ltmp, T, qd, d, rank, ls);
        ref_add(hidden, tmp, hidden, Td);
        c_pa[l] = fbuf(Td); memcpy(c_pa[l], hidden, Td * 4);
        c_xf[l] = fbuf(Td); ref_rmsnorm(hidden, P + o->post_norm, c_xf[l], T, d, eps);
        c_g[l] = fbuf(TF); c_u[l] = fbuf(TF); c_s[l] = fbuf(TF); c_fh[l] = fbuf(TF);
        ref_matmul(c_xf[l], P + o->gate, c_g[l], T, F, d, 0, 1, 0);
        if (HAS(4)) ref_lora_forward_add(c_xf[l], c_g[l], LA(l, 4), LB(l, 4, d), ltmp, T, d, F, rank, ls);
        ref_matmul(c_xf[l], P + o->up, c_u[l], T, F, d, 0, 1, 0);
        if (HAS(5)) ref_lora_forward_add(c_xf[l], c_u[l], LA(l, 5), LB(l, 5, d), ltmp, T, d, F, rank, ls);
        ref_silu(c_g[l], c_s[l], TF);
        ref_mul(c_s[l], c_u[l], c_fh[l], TF);
        ref_matmul(c_fh[l], P + o->down, tmp, T, d, F, 0, 1, 0);
        if (HAS(6)) ref_lora_forward_add(c_fh[l], tmp, LA(l, 6), LB(l, 6, F), ltmp, T, F, d, rank, ls);
        ref_add(hidden, tmp, hidden, Td);
    }
    float* final_in = fbuf(Td); memcpy(final_in, hidden, Td * 4);
    float* hn = fbuf(Td); ref_rmsnorm(hidden, wfin, hn, T, d, eps);
    float* logits = fbuf((size_t)T * V);
    ref_matmul(hn, Wlm ? Wlm : E, logits, T, V, d, 0, 1, 0);   /* tied LM head, src/train_cuda.c:2156 (or the separate lm_head) */
    if (logits_out) memcpy(logits_out, logits, (size_t)T * V * 4);

    float* dlog = fbuf((size_t)T * V); float* loss_rows = fbuf(T);
    ref_cross_entropy_grad(logits, tgt, dlog, loss_rows, ss, T, B, V, num_valid);
    float loss = ref_reduce_sum(loss_rows, T) / (float)num_valid;

    float* gh = fbuf(Td); float* gt = fbuf(Td); float* gx = fbuf(Td);
    float* gq = fbuf(Tq); float* gk = fbuf(Tkv); float* gv = fbuf(Tkv); float* ga = fbuf(Tq);
    float* gf = fbuf(TF); float* gg = fbuf(TF); float* gu = fbuf(TF);
    float* scratch_norm = fbuf(d);
    int full = (lora == NULL);

    ref_matmul(dlog, Wlm ? Wlm : E, gh, T, d, V, 0, 0, 0);
    if (full) ref_matmul(dlog, hn, (Wlm && GWlm) ? GWlm : G, V, d, T, 1, 0, 1);
    ref_rmsnorm_backward(final_in, wfin, gh, gt, full ? G + (size_t)V * d : scratch_norm, T, d, eps);
    memcpy(gh, gt, Td * 4);

/* LoRA gradient for one adapter, plus (exact mode) its share of dX */
#define LORA_BWD(a, dY, X, in, out, dXacc) \
    if (HAS(a)) { \
        ref_lora_backward(dY, X, LA(l, a), LB(l, a, in), LGA(l, a), LGB(l, a, in), ltmp, T, in, out, rank, ls); \
        if (lora_exact && (dXacc)) ref_matmul(ltmp, LA(l, a), dXacc, T, in, rank, 0, 0, 1); \
    }

    for (int l = L - 1; l >= 0; l--) {
        const layer_off_t* o = &off[l];
        if (full) ref_matmul(gh, c_fh[l], G + o->down, d, F, T, 1, 0, 1);
        ref_matmul(gh, P + o->down, gf, T, F, d, 0, 0, 0);
        LORA_BWD(6, gh, c_fh[l], F, d, gf)
        ref_mul_backward(c_s[l], c_u[l], gf, gg, gu, TF);
        ref_silu_backward(c_g[l], gg, gg, TF);
        if (full) {
            ref_matmul(gg, c_xf[l], G + o->gate, F, d, T, 1, 0, 1);
            ref_matmul(gu, c_xf[l], G + o->up, F, d, T, 1, 0, 1);
        }
        ref_matmul(gg, P + o->gate, gx, T, d, F, 0, 0, 0);
        ref_matmul(gu, P + o->up, gt, T, d, F, 0, 0, 0);
        ref_add(gx, gt, gx, Td);
        LORA_BWD(4, gg, c_xf[l], d, F, gx)
        LORA_BWD(5, gu, c_xf[l], d, F, gx)
        ref_rmsnorm_backward(c_pa[l], P + o->post_norm, gx, gt, full ? G + o->post_norm : scratch_norm, T, d, eps);
        ref_add(gt, gh, gh, Td);

        if (full) ref_matmul(gh, c_att[l], G + o->o, d, qd, T, 1, 0, 1);
        ref_matmul(gh, P + o->o, ga, T, qd, d, 0, 0, 0);
        LORA_BWD(3, gh, c_att[l], qd, d, ga)
        memset(gk, 0, Tkv * 4); memset(gv, 0, Tkv * 4);
        ref_attention_backward(c_q[l], c_k[l], c_v[l], ga, gq, gk, gv, ss, T, B, Hq, Hkv, hd);
        if (c->qk_norm) {
            ref_qk_norm_backward(c_q[l], c_qr[l], gq, gq, T, Hq, hd, 1, eps);
            ref_qk_norm_backward(c_k[l], c_kr[l], gk, gk, T, Hkv, hd, 1, eps);
        }
        ref_rope(gq, gq, ss, T, B, Hq, hd, theta, 1);
        ref_rope(gk, gk, ss, T, B, Hkv, hd, theta, 1);
        if (c->head_norm && X) {
            float* t1 = fbuf(Tq); float* t2 = fbuf(Tkv); float* sink = fbuf((size_t)hd);
            ref_rmsnorm_backward(c_qp[l], X + (size_t)l * 2 * hd, gq, t1, (full && GX) ? GX + (size_t)l * 2 * hd : sink, T * Hq, hd, eps);
            ref_rmsnorm_backward(c_kp[l], X + (size_t)l * 2 * hd + hd, gk, t2, (full && GX) ? GX + (size_t)l * 2 * hd + hd : sink, T * Hkv, hd, eps);
            memcpy(gq, t1, Tq * 4); memcpy(gk, t2, Tkv * 4);
            free(t1); free(t2); free(sink);
        }
        if (full) {
            ref_matmul(gq, c_xa[l], G + o->q, qd, d, T, 1, 0, 1);
            ref_matmul(gk, c_xa[l], G + o->k, kvd, d, T, 1, 0, 1);
            ref_matmul(gv, c_xa[l], G + o->v, kvd, d, T, 1, 0, 1);
        }
        ref_matmul(gq, P + o->q, gx, T, d, qd, 0, 0, 0);
        ref_matmul(gk, P + o->k, gt, T, d, kvd, 0, 0, 0);
        ref_add(gx, gt, gx, Td);
        ref_matmul(gv, P + o->v, gt, T, d, kvd, 0, 0, 0);
        ref_add(gx, gt, gx, Td);
        LORA_BWD(0, gq, c_xa[l], d, qd, gx)
        LORA_BWD(1, gk, c_xa[l], d, kvd, gx)
        LORA_BWD(2, gv, c_xa[l], d, kvd, gx)
        ref_rmsnorm_backward(c_in[l], P + o->in_norm, gx, gt, full ? G + o->in_norm : scratch_norm, T, d, eps);
        ref_add(gt, gh, gh, Td);
    }
    if (full) ref_embedding_backward(tok, gh, G, T, d);
    if (dhidden0_out) memcpy(dhidden0_out, gh, Td * 4);

    for (int l = 0; l < L; l++) {
        free(c_in[l]); free(c_xa[l]); free(c_q[l]); free(c_k[l]); free(c_v[l]); free(c_att[l]);
        free(c_pa[l]); free(c_xf[l]); free(c_g[l]); free(c_u[l]); free(c_s[l]); free(c_fh[l]);
        free(c_qr[l]); free(c_kr[l]); free(c_qp[l]); free(c_kp[l]);
    }
    free(c_qr); free(c_kr); free(c_qp); free(c_kp);
    free(c_in); free(c_xa); free(c_q); free(c_k); free(c_v); free(c_att); free(c_pa); free(c_xf);
    free(c_g); free(c_u); free(c_s); free(c_fh);
    free(hidden); free(tmp); free(ltmp); free(final_in); free(hn); free(logits); free(dlog); free(loss_rows);
    free(gh); free(gt); free(gx); free(gq); free(gk); free(gv); free(ga); free(gf); free(gg); free(gu);
    free(scratch_norm); free(off); free(tok); free(tgt); free(ss);
    return loss;
}

/* learning rate the reference applies at a given optimizer step:
 * 100-step linear warm-up, then divided by the accumulation count
 * (src/train_cuda.c:2298-2303) */
float ref_effective_lr(float base_lr, int optimizer_step, int accum_steps) {
    float lr = base_lr;
    if (optimizer_step < 100.0f) lr = base_lr * (optimizer_step / 100.0f);
    if (accum_steps < 1) accum_steps = 1;
    return lr / accum_steps;
}
