/*
 * harness.c - build a train_state_t in memory, without model files or a
 * tokenizer, from flat float arrays.  The reference only builds one through
 * train_init() (src/train.c:7854), which needs a model directory; tests,
 * benchmarks and embedders that already hold the weights use this instead.
 *
 * Flat parameter order: embed [V,d], final_norm [d], then per layer
 * q [qd,d], k [kvd,d], v [kvd,d], o [d,qd], gate [F,d], up [F,d], down [d,F],
 * in_norm [d], post_norm [d].  Flat LoRA order: per layer, for each adapter
 * selected by the mask (bit 0 q, 1 k, 2 v, 3 o, 4 gate, 5 up, 6 down): A [r,in]
 * then B [out,r].
 */
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include "sb_internal.h"

typedef struct {
    train_state_t st;          /* must stay first: the handle is a train_state_t* */
    model_config_t cfg;
    trainable_weights_t w;
    lora_model_t lora;
    int lora_mask;
    seraph_model_t model;      /* a memory-mapped safetensors file as the frozen LoRA base (seraph_b200_state_attach_model_file) */
    safetensors_t file;
} harness_t;

static int g_lean = 0;     /* weights only: no host copies of gradients and Adam moments */
static int wt_alloc(weight_tensor_t* t, size_t n) {
    t->weight = (float*)calloc(n, 4);
    t->size = n;
    if (g_lean) { t->grad = t->m = t->v = NULL; return !t->weight; }
    t->grad = (float*)calloc(n, 4); t->m = (float*)calloc(n, 4); t->v = (float*)calloc(n, 4);
    return !(t->weight && t->grad && t->m && t->v);
}
static void wt_free(weight_tensor_t* t) { free(t->weight); free(t->grad); free(t->m); free(t->v); }

typedef void (*visit_fn)(weight_tensor_t*, void*);
static void visit(harness_t* h, visit_fn f, void* arg) {
    f(&h->w.embed_tokens, arg); f(&h->w.final_norm, arg);
    for (int l = 0; l < h->w.num_layers; l++) {
        layer_weights_t* y = &h->w.layers[l];
        f(&y->q_proj, arg); f(&y->k_proj, arg); f(&y->v_proj, arg); f(&y->o_proj, arg);
        f(&y->gate_proj, arg); f(&y->up_proj, arg); f(&y->down_proj, arg); f(&y->input_norm, arg); f(&y->post_norm, arg);
    }
}

train_state_t* seraph_b200_state_create(int V, int d, int L, int Hq, int Hkv, int hd, int F, float theta, float lr, int accum) {
    if (V <= 0 || d <= 0 || L <= 0 || Hq <= 0 || Hkv <= 0 || hd <= 0 || F <= 0) return NULL;
    harness_t* h = (harness_t*)calloc(1, sizeof(harness_t));
    if (!h) return NULL;
    model_config_t* c = &h->cfg;
    c->vocab_size = V; c->hidden_size = d; c->num_hidden_layers = L; c->intermediate_size = F;
    c->num_attention_heads = Hq; c->num_key_value_heads = Hkv; c->head_dim = hd; c->kv_dim = Hkv * hd;
    c->rms_norm_eps = 1e-5f; c->rope_theta = theta; c->tie_word_embeddings = 1;
    size_t qd = (size_t)Hq * hd, kvd = (size_t)Hkv * hd;
    h->w.num_layers = L; h->w.hidden_size = d; h->w.intermediate_size = F; h->w.vocab_size = V;
    h->w.layers = (layer_weights_t*)calloc((size_t)L, sizeof(layer_weights_t));
    int bad = !h->w.layers;
    bad |= wt_alloc(&h->w.embed_tokens, (size_t)V * d); bad |= wt_alloc(&h->w.final_norm, (size_t)d);
    for (int l = 0; l < L && !bad; l++) {
        layer_weights_t* y = &h->w.layers[l];
        bad |= wt_alloc(&y->q_proj, qd * d); bad |= wt_alloc(&y->k_proj, kvd * d); bad |= wt_alloc(&y->v_proj, kvd * d);
        bad |= wt_alloc(&y->o_proj, (size_t)d * qd); bad |= wt_alloc(&y->gate_proj, (size_t)F * d);
        bad |= wt_alloc(&y->up_proj, (size_t)F * d); bad |= wt_alloc(&y->down_proj, (size_t)d * F);
        bad |= wt_alloc(&y->input_norm, (size_t)d); bad |= wt_alloc(&y->post_norm, (size_t)d);
    }
    h->st.config = c; h->st.use_full_training = 1; h->st.full_weights = &h->w;
    h->st.learning_rate = lr; h->st.gradient_accumulation_steps = accum;
    if (bad) return NULL;
    h->w.total_params = (size_t)V * d + (size_t)d + (size_t)L * (2 * qd * d + 2 * kvd * d + 3 * (size_t)F * d + 2 * (size_t)d);
    return &h->st;
}

/* same, but the host state holds the weights only (a quarter of the host memory): gradients and
 * Adam moments then live on the device alone and cannot be downloaded into this state */
train_state_t* seraph_b200_state_create_lean(int V, int d, int L, int Hq, int Hkv, int hd, int F, float theta, float lr, int accum) {
    g_lean = 1;
    train_state_t* st = seraph_b200_state_create(V, d, L, Hq, Hkv, hd, F, theta, lr, accum);
    g_lean = 0;
    return st;
}

static void f_free(weight_tensor_t* t, void* a) { (void)a; wt_free(t); }
static void lora_free_all(harness_t* h);
static void model_file_close(harness_t* h) {
    if (h->file.tensors) { for (int i = 0; i < h->file.num_tensors; i++) { free(h->file.tensors[i].name); free(h->file.tensors[i].shape); } free(h->file.tensors); }
    if (h->file.data) munmap(h->file.data, h->file.file_size);
    if (h->file.fd > 0) close(h->file.fd);
    free(h->model.tensor_map);
    memset(&h->file, 0, sizeof h->file); memset(&h->model, 0, sizeof h->model);
    h->st.model = NULL;
}

/* A state shaped like the one the reference's train_init builds for LoRA training (src/train.c:7900-7909): no FP32 host
 * copies of the base (full_weights = NULL), state->model = the safetensors file at `path`, memory-mapped, its tensors
 * found by their Hugging Face names.  The library then reads the frozen base as raw BF16 from that mapping.  The header
 * is scanned for every tensor's name, shape and data_offsets; returns 0, or 1 when the file cannot be mapped or parsed. */
static const char* skip_string(const char* p, const char* end) {      /* p at the opening quote; returns past the closing one */
    for (p++; p < end && *p != '"'; p++) if (*p == '\\' && p + 1 < end) p++;
    return p < end ? p + 1 : end;
}
static const char* find_key(const char* p, const char* end, const char* key) {   /* inside one object: value position of "key": */
    size_t n = strlen(key);
    while (p < end) {
        if (*p == '"') {
            const char* q = skip_string(p, end);
            if ((size_t)(q - p - 2) == n && !memcmp(p + 1, key, n)) { while (q < end && (*q == ':' || *q == ' ')) q++; return q; }
            p = q;
        } else p++;
    }
    return NULL;
}
int seraph_b200_state_attach_model_file(train_state_t* st, const char* path) {
    harness_t* h = (harness_t*)st;
    if (!h || !path) return 1;
    model_file_close(h);
    int fd = open(path, O_RDONLY);
    if (fd < 0) return 1;
    struct stat sb;
    if (fstat(fd, &sb) || sb.st_size < 16) { close(fd); return 1; }
    uint8_t* data = (uint8_t*)mmap(NULL, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (data == MAP_FAILED) { close(fd); return 1; }
    uint64_t hlen; memcpy(&hlen, data, 8);
    if (hlen + 8 > (uint64_t)sb.st_size) { munmap(data, (size_t)sb.st_size); close(fd); return 1; }
    h->file.fd = fd; h->file.data = data; h->file.file_size = (size_t)sb.st_size; h->file.data_offset = 8 + (size_t)hlen;
    const char* p = (const char*)data + 8; const char* end = p + hlen;
    int cap = 64, n = 0;
    tensor_metadata_t* tm = (tensor_metadata_t*)calloc((size_t)cap, sizeof *tm);
    while (p < end && *p != '{') p++;
    p++;
    while (tm && p < end) {
        while (p < end && *p != '"' && *p != '}') p++;
        if (p >= end || *p == '}') break;
        const char* q = skip_string(p, end);
        size_t kl = (size_t)(q - p - 2);
        const char* key = p + 1;
        p = q;
        while (p < end && *p != '{') p++;                     /* the value object: find its end with brace matching */
        const char* ob = p; int depth = 0;
        for (; p < end; p++) { if (*p == '"') { p = skip_string(p, end) - 1; continue; } if (*p == '{') depth++; else if (*p == '}' && --depth == 0) { p++; break; } }
        const char* oe = p;
        if (kl == 12 && !memcmp(key, "__metadata__", 12)) continue;
        const char* v = find_key(ob, oe, "data_offsets");
        if (!v) continue;
        long long a = 0, b = 0;
        if (sscanf(v, "[%lld,%lld]", &a, &b) != 2 && sscanf(v, "[%lld, %lld]", &a, &b) != 2) continue;
        if (n == cap) { cap *= 2; tensor_metadata_t* t2 = (tensor_metadata_t*)realloc(tm, (size_t)cap * sizeof *tm); if (!t2) break; tm = t2; memset(tm + n, 0, (size_t)(cap - n) * sizeof *tm); }
        tensor_metadata_t* t = &tm[n++];
        t->name = (char*)malloc(kl + 1); memcpy(t->name, key, kl); t->name[kl] = 0;
        t->offset_start = a; t->offset_end = b;
        const char* d = find_key(ob, oe, "dtype");
        t->dtype = (d && !strncmp(d, "\"BF16\"", 6)) ? 3 : (d && !strncmp(d, "\"F16\"", 5)) ? 2 : (d && !strncmp(d, "\"F32\"", 5)) ? 1 : 0;
        t->num_elements = (size_t)(b - a) / (t->dtype == 1 ? 4 : 2);
        const char* sh = find_key(ob, oe, "shape");
        if (sh && *sh == '[') {
            int64_t dims[8]; int nd = 0; const char* r = sh + 1;
            while (r < oe && *r != ']' && nd < 8) { dims[nd++] = strtoll(r, (char**)&r, 10); while (r < oe && (*r == ',' || *r == ' ')) r++; }
            t->n_dims = nd; t->shape = (int64_t*)malloc(sizeof(int64_t) * (size_t)(nd ? nd : 1)); memcpy(t->shape, dims, sizeof(int64_t) * (size_t)nd);
        }
    }
    if (!tm || n == 0) { free(tm); model_file_close(h); return 1; }
    h->file.tensors = tm; h->file.num_tensors = n;
    h->model.st[0] = &h->file; h->model.num_files = 1; h->model.config = &h->cfg; h->model.num_tensors = n;
    h->model.tensor_map = (tensor_location_t*)calloc((size_t)n, sizeof(tensor_location_t));
    if (!h->model.tensor_map) { model_file_close(h); return 1; }
    for (int i = 0; i < n; i++) {
        strncpy(h->model.tensor_map[i].name, tm[i].name, 255); strncpy(h->model.tensor_map[i].orig_name, tm[i].name, 255);
        h->model.tensor_map[i].file_idx = 0;
    }
    h->st.model = &h->model;
    h->st.full_weights = NULL; h->st.use_full_training = 0;          /* the host FP32 copies stay allocated inside the harness, unused */
    return 0;
}

void seraph_b200_state_free(train_state_t* st) {
    harness_t* h = (harness_t*)st;
    if (!h) return;
    model_file_close(h);
    lora_free_all(h);
    visit(h, f_free, NULL);
    free(h->w.layers);
    free(h);
}

static void f_count(weight_tensor_t* t, void* a) { *(size_t*)a += t->size; }
size_t seraph_b200_state_param_count(train_state_t* st) { size_t n = 0; visit((harness_t*)st, f_count, &n); return n; }

typedef struct { float* flat; int which; int set; } io_t;
static void f_io(weight_tensor_t* t, void* a) {
    io_t* io = (io_t*)a;
    float* p = io->which == 0 ? t->weight : io->which == 1 ? t->grad : io->which == 2 ? t->m : t->v;
    if (!p) { if (!io->set) memset(io->flat, 0, t->size * 4); }
    else if (io->set) memcpy(p, io->flat, t->size * 4); else memcpy(io->flat, p, t->size * 4);
    io->flat += t->size;
}
/* which: 0 weights, 1 gradients, 2 Adam m, 3 Adam v */
void seraph_b200_state_set(train_state_t* st, int which, const float* flat) { io_t io = {(float*)flat, which, 1}; visit((harness_t*)st, f_io, &io); }
void seraph_b200_state_get(train_state_t* st, int which, float* flat) { io_t io = {flat, which, 0}; visit((harness_t*)st, f_io, &io); }

void seraph_b200_state_set_counters(train_state_t* st, int optimizer_step, int accumulation_counter) {
    st->optimizer_step = optimizer_step; st->accumulation_counter = accumulation_counter;
}
void seraph_b200_state_get_counters(train_state_t* st, int* optimizer_step, int* accumulation_counter) {
    if (optimizer_step) *optimizer_step = st->optimizer_step;
    if (accumulation_counter) *accumulation_counter = st->accumulation_counter;
}
void seraph_b200_state_set_lr(train_state_t* st, float lr, int accum) { st->learning_rate = lr; st->gradient_accumulation_steps = accum; }
void* seraph_b200_state_weights(train_state_t* st) { return st ? (void*)st->full_weights : NULL; }
void seraph_b200_state_set_qk_norm(train_state_t* st, int on) { if (st && st->config) st->config->use_qk_norm = on ? 1 : 0; }
/* train_state_t.debug_nan_check (the CLI's --debug-nan) and the flag the step sets when it trips */
void seraph_b200_state_set_debug_nan(train_state_t* st, int on) { if (st) { st->debug_nan_check = on ? 1 : 0; st->nan_detected = 0; } }
int seraph_b200_state_nan_detected(train_state_t* st) { return st ? st->nan_detected : 0; }

/* ---- LoRA ---- */
static void dims(const model_config_t* c, int a, int* in, int* out) {
    int qd = c->num_attention_heads * c->head_dim, kvd = c->num_key_value_heads * c->head_dim;
    switch (a) {
        case 0: *in = c->hidden_size; *out = qd; break;
        case 1: case 2: *in = c->hidden_size; *out = kvd; break;
        case 3: *in = qd; *out = c->hidden_size; break;
        case 4: case 5: *in = c->hidden_size; *out = c->intermediate_size; break;
        default: *in = c->intermediate_size; *out = c->hidden_size; break;
    }
}
static lora_adapter_t*** slot(lora_model_t* m, int a) {
    switch (a) { case 0: return &m->q_adapters; case 1: return &m->k_adapters; case 2: return &m->v_adapters; case 3: return &m->o_adapters;
                 case 4: return &m->gate_adapters; case 5: return &m->up_adapters; default: return &m->down_adapters; }
}
static void lora_free_all(harness_t* h) {
    for (int a = 0; a < 7; a++) {
        lora_adapter_t** ls = *slot(&h->lora, a);
        if (!ls) continue;
        for (int l = 0; l < h->lora.num_layers; l++) {
            lora_adapter_t* ad = ls[l];
            if (!ad) continue;
            free(ad->A); free(ad->B); free(ad->grad_A); free(ad->grad_B); free(ad->m_A); free(ad->v_A); free(ad->m_B); free(ad->v_B);
            free(ad);
        }
        free(ls);
        *slot(&h->lora, a) = NULL;
    }
    h->st.lora = NULL; h->lora_mask = 0;
}

size_t seraph_b200_state_lora_count(train_state_t* st, int rank, int mask) {
    harness_t* h = (harness_t*)st; size_t n = 0;
    for (int a = 0; a < 7; a++) if (mask & (1 << a)) { int in, out; dims(&h->cfg, a, &in, &out); n += (size_t)rank * in + (size_t)out * rank; }
    return n * (size_t)h->cfg.num_hidden_layers;
}

/* switch the state to LoRA training with adapters taken from `flat` (NULL: zeros) */
int seraph_b200_state_attach_lora(train_state_t* st, int rank, float alpha, int mask, const float* flat) {
    harness_t* h = (harness_t*)st;
    if (!h || rank <= 0 || !(mask & 0x7f)) return 1;
    lora_free_all(h);
    int L = h->cfg.num_hidden_layers;
    lora_model_t* m = &h->lora;
    m->num_layers = L; m->rank = rank; m->alpha = alpha; m->dropout = 0.f;
    m->apply_to_q = mask & 1; m->apply_to_k = (mask >> 1) & 1; m->apply_to_v = (mask >> 2) & 1; m->apply_to_o = (mask >> 3) & 1;
    m->apply_to_ffn = (mask >> 4) & 7 ? 1 : 0;
    for (int a = 0; a < 7; a++) if (mask & (1 << a)) *slot(m, a) = (lora_adapter_t**)calloc((size_t)L, sizeof(lora_adapter_t*));
    const float* p = flat;
    for (int l = 0; l < L; l++)
        for (int a = 0; a < 7; a++) {
            if (!(mask & (1 << a))) continue;
            int in, out; dims(&h->cfg, a, &in, &out);
            size_t nA = (size_t)rank * in, nB = (size_t)out * rank;
            lora_adapter_t* ad = (lora_adapter_t*)calloc(1, sizeof(lora_adapter_t));
            ad->in_dim = in; ad->out_dim = out; ad->rank = rank; ad->alpha = alpha;
            ad->A = (float*)calloc(nA, 4); ad->grad_A = (float*)calloc(nA, 4); ad->m_A = (float*)calloc(nA, 4); ad->v_A = (float*)calloc(nA, 4);
            ad->B = (float*)calloc(nB, 4); ad->grad_B = (float*)calloc(nB, 4); ad->m_B = (float*)calloc(nB, 4); ad->v_B = (float*)calloc(nB, 4);
            if (p) { memcpy(ad->A, p, nA * 4); p += nA; memcpy(ad->B, p, nB * 4); p += nB; }
            (*slot(m, a))[l] = ad;
        }
    h->lora_mask = mask;
    h->st.lora = m; h->st.use_full_training = 0;
    return 0;
}

/* which: 0 weights, 1 gradients, 2 Adam m, 3 Adam v (host copies; call cuda_download_lora_weights first) */
void seraph_b200_state_lora_get(train_state_t* st, int which, float* flat) {
    harness_t* h = (harness_t*)st;
    if (!h || !h->st.lora) return;
    float* p = flat;
    for (int l = 0; l < h->lora.num_layers; l++)
        for (int a = 0; a < 7; a++) {
            if (!(h->lora_mask & (1 << a))) continue;
            lora_adapter_t* ad = (*slot(&h->lora, a))[l];
            size_t nA = (size_t)ad->rank * ad->in_dim, nB = (size_t)ad->out_dim * ad->rank;
            const float* sa = which == 0 ? ad->A : which == 1 ? ad->grad_A : which == 2 ? ad->m_A : ad->v_A;
            const float* sb = which == 0 ? ad->B : which == 1 ? ad->grad_B : which == 2 ? ad->m_B : ad->v_B;
            memcpy(p, sa, nA * 4); p += nA; memcpy(p, sb, nB * 4); p += nB;
        }
}
