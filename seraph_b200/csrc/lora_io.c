/*
 * lora_io.c - LoRA adapter files.
 *
 * Version 2 is the reference's format, byte for byte (lora_save / lora_load, src/lora.c:441-560): a 36-byte header
 * (magic "LORA", version 2, num_layers, rank, alpha, hidden size, q out dim, kv out dim, apply mask with Q=1 K=2 V=4 O=8
 * FFN=16) followed per layer by A [rank,in] and B [out,rank] of the Q adapter and then of the V adapter.  Adapters on
 * k, o, gate, up, down are not part of that format: the reference trains them (src/train.c:6421-6557) and drops them on
 * save (src/lora.c:478-489).
 *
 * Version 3 is this library's extension for those adapters and for resuming: a 64-byte header (the version-2 fields, then
 * o in dim, ffn dim, a 7-bit adapter mask q k v o gate up down, a flag for Adam moments, the optimizer step) and per layer,
 * per adapter in mask order: A, B and, when the flag is set, m_A, m_B, v_A, v_B.
 *
 * Both directions work on the host lora_model_t the training state owns.  Saving first brings the resident adapters and
 * moments back from the GPU (cuda_download_lora_weights); loading marks the resident copy stale so that the next LoRA step
 * uploads what was read.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

#define LORA_MAGIC 0x4C4F5241u

static lora_adapter_t** list_of(const lora_model_t* m, int a) {
    switch (a) { case 0: return m->q_adapters; case 1: return m->k_adapters; case 2: return m->v_adapters; case 3: return m->o_adapters;
                 case 4: return m->gate_adapters; case 5: return m->up_adapters; default: return m->down_adapters; }
}
static int present_mask(const lora_model_t* m) {
    int mask = 0;
    for (int a = 0; a < 7; a++) { lora_adapter_t** ls = list_of(m, a); if (ls && ls[0]) mask |= 1 << a; }
    return mask;
}
static int put(FILE* f, const void* p, size_t n) { return fwrite(p, 1, n, f) == n ? 0 : 1; }
static int get(FILE* f, void* p, size_t n) { return fread(p, 1, n, f) == n ? 0 : 1; }
static int put_f(FILE* f, const float* p, size_t n) {
    if (p) return put(f, p, n * 4);
    static const float zeros[256];                       /* a moment array the host model does not hold is written as zeros */
    while (n) { size_t k = n < 256 ? n : 256; if (put(f, zeros, k * 4)) return 1; n -= k; }
    return 0;
}
static int get_f(FILE* f, float* p, size_t n) {
    if (p) return get(f, p, n * 4);
    return fseek(f, (long)(n * 4), SEEK_CUR) != 0;
}

void sb_lora_mark_stale(sb_ctx_t* c);        /* train_step.c */

int seraph_b200_lora_save(cuda_train_context_t* ctx, train_state_t* state, const char* path, int version, int with_moments) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!state || !state->lora || !path || (version != 2 && version != 3)) return SB_ERR_ARG;
    lora_model_t* m = state->lora;
    if (c && c->LW) cuda_download_lora_weights(ctx, m);
    FILE* f = fopen(path, "wb");
    if (!f) return SB_ERR_ARG;
    int bad = 0;
    uint32_t magic = LORA_MAGIC, ver = (uint32_t)version;
    int hidden = 0, q_out = 0, kv_out = 0;
    if (m->q_adapters && m->q_adapters[0]) { hidden = m->q_adapters[0]->in_dim; q_out = m->q_adapters[0]->out_dim; }
    if (m->v_adapters && m->v_adapters[0]) kv_out = m->v_adapters[0]->out_dim;
    if (version == 3) {                                               /* the reference takes these from the Q and V adapters only */
        static const int in_is_hidden[7] = {1, 1, 1, 0, 1, 1, 0};
        for (int a = 0; a < 7 && !hidden; a++) { lora_adapter_t** ls = list_of(m, a); if (ls && ls[0]) hidden = in_is_hidden[a] ? ls[0]->in_dim : ls[0]->out_dim; }
        if (!kv_out && m->k_adapters && m->k_adapters[0]) kv_out = m->k_adapters[0]->out_dim;
    }
    uint32_t apply = (m->apply_to_q ? 1u : 0u) | (m->apply_to_k ? 2u : 0u) | (m->apply_to_v ? 4u : 0u) | (m->apply_to_o ? 8u : 0u) |
                     (m->apply_to_ffn ? 16u : 0u);
    bad |= put(f, &magic, 4) | put(f, &ver, 4) | put(f, &m->num_layers, 4) | put(f, &m->rank, 4) | put(f, &m->alpha, 4);
    bad |= put(f, &hidden, 4) | put(f, &q_out, 4) | put(f, &kv_out, 4) | put(f, &apply, 4);
    if (version == 2) {
        for (int l = 0; l < m->num_layers && !bad; l++)
            for (int a = 0; a <= 2; a += 2) {                         /* q, then v: all the format holds */
                lora_adapter_t** ls = list_of(m, a);
                if (!ls || !ls[l]) continue;
                const lora_adapter_t* ad = ls[l];
                bad |= put_f(f, ad->A, (size_t)ad->rank * ad->in_dim) | put_f(f, ad->B, (size_t)ad->out_dim * ad->rank);
            }
    } else {
        const int mask = present_mask(m);
        int o_in = 0, ffn = 0;
        if (m->o_adapters && m->o_adapters[0]) o_in = m->o_adapters[0]->in_dim;
        if (m->gate_adapters && m->gate_adapters[0]) ffn = m->gate_adapters[0]->out_dim;
        else if (m->up_adapters && m->up_adapters[0]) ffn = m->up_adapters[0]->out_dim;
        else if (m->down_adapters && m->down_adapters[0]) ffn = m->down_adapters[0]->in_dim;
        int32_t ext[7] = {o_in, ffn, mask, with_moments ? 1 : 0, state->optimizer_step, 0, 0};
        bad |= put(f, ext, sizeof ext);
        for (int l = 0; l < m->num_layers && !bad; l++)
            for (int a = 0; a < 7; a++) {
                if (!(mask & (1 << a))) continue;
                const lora_adapter_t* ad = list_of(m, a)[l];
                if (!ad) { bad = 1; break; }
                const size_t nA = (size_t)ad->rank * ad->in_dim, nB = (size_t)ad->out_dim * ad->rank;
                bad |= put_f(f, ad->A, nA) | put_f(f, ad->B, nB);
                if (with_moments) bad |= put_f(f, ad->m_A, nA) | put_f(f, ad->m_B, nB) | put_f(f, ad->v_A, nA) | put_f(f, ad->v_B, nB);
            }
    }
    if (fclose(f)) bad = 1;
    return bad ? SB_ERR_ARG : SB_OK;
}

/* Reads a version-2 or version-3 file into the adapters the state already holds (created with the same rank and
 * shapes, as lora_model_create does for the CLI); adapters the file lacks keep their values.  Returns SB_OK, or
 * SB_ERR_ARG for a file that cannot be read, has another magic or version, or whose shapes differ from the model's. */
int seraph_b200_lora_load(cuda_train_context_t* ctx, train_state_t* state, const char* path) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!state || !state->lora || !path) return SB_ERR_ARG;
    lora_model_t* m = state->lora;
    FILE* f = fopen(path, "rb");
    if (!f) return SB_ERR_ARG;
    uint32_t magic = 0, ver = 0, apply = 0; int L = 0, rank = 0, hidden = 0, q_out = 0, kv_out = 0; float alpha = 0.f;
    int bad = get(f, &magic, 4) | get(f, &ver, 4) | get(f, &L, 4) | get(f, &rank, 4) | get(f, &alpha, 4) | get(f, &hidden, 4) |
              get(f, &q_out, 4) | get(f, &kv_out, 4) | get(f, &apply, 4);
    if (bad || magic != LORA_MAGIC || (ver != 2 && ver != 3) || L != m->num_layers || rank != m->rank) { fclose(f); return SB_ERR_ARG; }
    int mask = 0, moments = 0, o_in = 0, ffn = 0;
    if (ver == 2) mask = ((apply & 1) ? 1 : 0) | ((apply & 4) ? 4 : 0);
    else {
        int32_t ext[7];
        if (get(f, ext, sizeof ext)) { fclose(f); return SB_ERR_ARG; }
        o_in = ext[0]; ffn = ext[1]; mask = ext[2] & 0x7f; moments = ext[3];
        if (moments) state->optimizer_step = ext[4];
    }
    const int want_in[7] = {hidden, hidden, hidden, o_in, hidden, hidden, ffn}, want_out[7] = {q_out, kv_out, kv_out, hidden, ffn, ffn, hidden};
    for (int l = 0; l < L && !bad; l++)
        for (int a = 0; a < 7 && !bad; a++) {
            if (!(mask & (1 << a))) continue;
            lora_adapter_t** ls = list_of(m, a);
            lora_adapter_t* ad = ls ? ls[l] : NULL;
            if (!ad || ad->rank != rank) { bad = 1; break; }
            if ((want_in[a] && ad->in_dim != want_in[a]) || (want_out[a] && ad->out_dim != want_out[a])) { bad = 1; break; }
            const size_t nA = (size_t)rank * ad->in_dim, nB = (size_t)ad->out_dim * rank;
            bad |= get_f(f, ad->A, nA) | get_f(f, ad->B, nB);
            if (moments) bad |= get_f(f, ad->m_A, nA) | get_f(f, ad->m_B, nB) | get_f(f, ad->v_A, nA) | get_f(f, ad->v_B, nB);
        }
    fclose(f);
    if (bad) return SB_ERR_ARG;
    m->alpha = alpha;
    if (c) sb_lora_mark_stale(c);
    return SB_OK;
}
