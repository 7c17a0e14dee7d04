// checkpoint.cu - the resident FP32 weights written as a BF16 safetensors file, byte for byte the file
// trainable_weights_save_to_safetensors (src/train.c:433-569) writes from the host copies after
// cuda_download_full_weights (src/train_cuda.c:1244): same JSON header (key order, metadata, the reference's header
// shapes, data offsets), same tensor order (embed_tokens, per layer q k v o gate up down input_norm post_norm,
// final norm), same FP32 -> BF16 conversion (the upper 16 bits of the word, src/train.c:263-267).
//
// The reference moves 4 bytes per parameter to the host in three synchronous copies per tensor, converts on one core and
// calls fwrite once per element.  Here the conversion runs on the GPU (4 B read, 2 B written per parameter), 2 bytes
// per parameter cross to the host in chunks through two pinned buffers, and the file is written chunk by chunk while
// the next chunk is converted and copied.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

#define CK_CHUNK_DEFAULT ((size_t)32 << 20) // parameters per chunk: 64 MB of BF16 per pinned buffer (SERAPH_B200_CKPT_CHUNK overrides)

__global__ void __launch_bounds__(256) pack_bf16_trunc_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, size_t n) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = (((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 7) == 0) ? n >> 2 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const uint4 v = ((const uint4*)src)[i];
        uint2 o;
        o.x = (v.x >> 16) | (v.y & 0xffff0000u);
        o.y = (v.z >> 16) | (v.w & 0xffff0000u);
        ((uint2*)dst)[i] = o;
    }
    for (size_t i = (n4 << 2) + tid; i < n; i += nth) dst[i] = (uint16_t)(__float_as_uint(src[i]) >> 16);
}

// growing string for the header
typedef struct { char* s; size_t n, cap; } ck_str_t;
static int ck_put(ck_str_t* b, const char* fmt, unsigned long long a, unsigned long long c2, unsigned long long d, unsigned long long e, const char* name) {
    char tmp[512];
    int k = name ? snprintf(tmp, sizeof tmp, fmt, name, a, c2, d, e) : snprintf(tmp, sizeof tmp, fmt, a, c2, d, e);
    if (k < 0 || (size_t)k >= sizeof tmp) return 1;
    if (b->n + (size_t)k + 1 > b->cap) {
        size_t cap = b->cap ? b->cap * 2 : 4096;
        while (cap < b->n + (size_t)k + 1) cap *= 2;
        char* p = (char*)realloc(b->s, cap);
        if (!p) return 1;
        b->s = p; b->cap = cap;
    }
    memcpy(b->s + b->n, tmp, (size_t)k + 1);
    b->n += (size_t)k;
    return 0;
}

extern "C" int seraph_b200_save_safetensors(cuda_train_context_t* ctx, train_state_t* state, const char* path) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || !state->full_weights || !path) return SB_ERR_ARG;
    if (!c->W || !c->off) { sb_set_status(c, SB_ERR_ARG); return SB_ERR_ARG; }
    const trainable_weights_t* w = state->full_weights;
    const int L = c->L, d = c->d, V = c->V, F = c->F;
    if (w->num_layers != L || w->hidden_size != d || w->vocab_size != V || w->intermediate_size != F) { sb_set_status(c, SB_ERR_ARG); return SB_ERR_ARG; }

    // ---- header: what cJSON_PrintUnformatted makes of the reference's object (numbers below 1e15 print as plain integers).
    // The reference's header gives q/k/v/o the shape [hidden, hidden] whatever the head geometry (src/train.c:472-473); the data
    // section has every tensor at its true size, so offsets here follow the header's sizes exactly as there.
    ck_str_t h = {NULL, 0, 0};
    unsigned long long off = 0;
    int bad = ck_put(&h, "{\"__metadata__\":{\"format\":\"pt\",\"framework\":\"tetyah\",\"trained\":\"full_weight_fp32_adamw\"}", 0, 0, 0, 0, NULL);
#define CK_T2(name, d0, d1) do { unsigned long long sz_ = (unsigned long long)(d0) * (unsigned long long)(d1) * 2ull; \
        bad |= ck_put(&h, ",\"%s\":{\"dtype\":\"BF16\",\"shape\":[%llu,%llu],\"data_offsets\":[%llu,%llu]}", (unsigned long long)(d0), (unsigned long long)(d1), off, off + sz_, name); off += sz_; } while (0)
#define CK_T1(name, d0) do { unsigned long long sz_ = (unsigned long long)(d0) * 2ull; \
        bad |= ck_put(&h, ",\"%s\":{\"dtype\":\"BF16\",\"shape\":[%llu],\"data_offsets\":[%llu,%llu]}", (unsigned long long)(d0), off, off + sz_, 0, name); off += sz_; } while (0)
    char nm[256];
    CK_T2("model.embed_tokens.weight", V, d);
    for (int l = 0; l < L && !bad; l++) {
        snprintf(nm, sizeof nm, "model.layers.%d.self_attn.q_proj.weight", l); CK_T2(nm, d, d);
        snprintf(nm, sizeof nm, "model.layers.%d.self_attn.k_proj.weight", l); CK_T2(nm, d, d);
        snprintf(nm, sizeof nm, "model.layers.%d.self_attn.v_proj.weight", l); CK_T2(nm, d, d);
        snprintf(nm, sizeof nm, "model.layers.%d.self_attn.o_proj.weight", l); CK_T2(nm, d, d);
        snprintf(nm, sizeof nm, "model.layers.%d.mlp.gate_proj.weight", l); CK_T2(nm, F, d);
        snprintf(nm, sizeof nm, "model.layers.%d.mlp.up_proj.weight", l); CK_T2(nm, F, d);
        snprintf(nm, sizeof nm, "model.layers.%d.mlp.down_proj.weight", l); CK_T2(nm, d, F);
        snprintf(nm, sizeof nm, "model.layers.%d.input_layernorm.weight", l); CK_T1(nm, d);
        snprintf(nm, sizeof nm, "model.layers.%d.post_attention_layernorm.weight", l); CK_T1(nm, d);
    }
    CK_T1("model.norm.weight", d);
    bad |= ck_put(&h, "}", 0, 0, 0, 0, NULL);
#undef CK_T2
#undef CK_T1
    if (bad) { free(h.s); sb_set_status(c, SB_ERR_OOM); return SB_ERR_OOM; }

    // ---- data: three contiguous ranges of the weight arena in file order
    const size_t nE = (size_t)V * d;
    const size_t layers_begin = c->off[0].q, layers_end = c->n_params;       // arena: embed, final norm, then the layers
    struct { size_t begin, n; } seg[3] = {{0, nE}, {layers_begin, layers_end - layers_begin}, {nE, (size_t)d}};

    size_t CK_CHUNK = CK_CHUNK_DEFAULT;
    { const char* e = getenv("SERAPH_B200_CKPT_CHUNK"); if (e && atol(e) >= 1024) CK_CHUNK = ((size_t)atol(e) + 3) & ~(size_t)3; }
    FILE* out = fopen(path, "wb");
    if (!out) { fprintf(stderr, "ERROR: Cannot create %s\n", path); free(h.s); return SB_ERR_ARG; }
    uint64_t hsize = (uint64_t)h.n;
    int rc = SB_OK;
    if (fwrite(&hsize, sizeof hsize, 1, out) != 1 || fwrite(h.s, 1, h.n, out) != h.n) rc = SB_ERR_ARG;
    free(h.s);

    uint16_t* dbuf[2] = {NULL, NULL}; uint16_t* hbuf[2] = {NULL, NULL};
    cudaEvent_t ev[2] = {NULL, NULL};
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    for (int i = 0; i < 2 && rc == SB_OK; i++)
        if (cudaMalloc((void**)&dbuf[i], CK_CHUNK * 2) != cudaSuccess || cudaMallocHost((void**)&hbuf[i], CK_CHUNK * 2) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); rc = SB_ERR_OOM; }
    // pipeline: chunk k is converted and copied into buffer k & 1 while chunk k - 1 is written to the file
    size_t pend_n = 0; int pend_buf = -1, k = 0;
    const int blocks = (c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148) * 8;
    for (int s = 0; s < 3 && rc == SB_OK; s++)
        for (size_t o = 0; o < seg[s].n && rc == SB_OK; o += CK_CHUNK, k++) {
            const size_t n = seg[s].n - o < CK_CHUNK ? seg[s].n - o : CK_CHUNK;
            const int b = k & 1;
            pack_bf16_trunc_kernel<<<blocks, 256, 0, st>>>(c->W + seg[s].begin + o, dbuf[b], n);
            c->launches++;
            cudaMemcpyAsync(hbuf[b], dbuf[b], n * 2, cudaMemcpyDeviceToHost, st);
            cudaEventRecord(ev[b], st);
            if (pend_buf >= 0) {
                if (cudaEventSynchronize(ev[pend_buf]) != cudaSuccess) { rc = SB_ERR_CUDA; break; }
                if (fwrite(hbuf[pend_buf], 2, pend_n, out) != pend_n) rc = SB_ERR_ARG;
            }
            pend_buf = b; pend_n = n;
        }
    if (rc == SB_OK && pend_buf >= 0) {
        if (cudaEventSynchronize(ev[pend_buf]) != cudaSuccess) rc = SB_ERR_CUDA;
        else if (fwrite(hbuf[pend_buf], 2, pend_n, out) != pend_n) rc = SB_ERR_ARG;
    }
    cudaStreamSynchronize(st);
    if (sb_check(c, cudaGetLastError(), "safetensors export")) rc = SB_ERR_CUDA;
    for (int i = 0; i < 2; i++) { if (dbuf[i]) cudaFree(dbuf[i]); if (hbuf[i]) cudaFreeHost(hbuf[i]); if (ev[i]) cudaEventDestroy(ev[i]); }
    if (fclose(out) != 0 && rc == SB_OK) rc = SB_ERR_ARG;
    if (rc != SB_OK) sb_set_status(c, rc);
    return rc;
}

// save_checkpoint (src/train.c:7760-7804) for a full-weight state whose weights live on the GPU: the safetensors file
// as above, then "<path>.state" with current_epoch, current_step, current_loss, optimizer_step (4 + 4 + 4 + 4 bytes).
// LoRA states are saved by the reference's own lora_save after cuda_download_lora_weights; this returns SB_ERR_ARG for them.
extern "C" int seraph_b200_save_checkpoint(cuda_train_context_t* ctx, train_state_t* state, const char* path) {
    if (!state || !path || state->lora) return SB_ERR_ARG;
    int rc = seraph_b200_save_safetensors(ctx, state, path);
    if (rc != SB_OK) return rc;
    char sp[600];
    if (snprintf(sp, sizeof sp, "%s.state", path) >= (int)sizeof sp) return SB_ERR_ARG;
    FILE* f = fopen(sp, "wb");
    if (!f) return SB_ERR_ARG;
    int ok = fwrite(&state->current_epoch, sizeof(int), 1, f) == 1 && fwrite(&state->current_step, sizeof(int), 1, f) == 1 &&
             fwrite(&state->current_loss, sizeof(float), 1, f) == 1 && fwrite(&state->optimizer_step, sizeof(int), 1, f) == 1;
    if (fclose(f) != 0) ok = 0;
    return ok ? SB_OK : SB_ERR_ARG;
}

// ---- the way back: trainable_weights_load_from_safetensors (src/train.c:571-629) skips the header and reads the tensors in
// the order they were saved, BF16 -> FP32 by a 16-bit shift.  Here the BF16 words go to the GPU in chunks (2 bytes per
// parameter) and are widened there, straight into the weight arena; the Adam moments and the host copies stay as they are
// (as in the reference, which loads weights only).
__global__ void __launch_bounds__(256) unpack_bf16_kernel(const uint16_t* __restrict__ src, float* __restrict__ dst, size_t n) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = (((uintptr_t)dst & 15) == 0 && ((uintptr_t)src & 7) == 0) ? n >> 2 : 0;
    for (size_t i = tid; i < n4; i += nth) {
        const uint2 v = ((const uint2*)src)[i];
        ((uint4*)dst)[i] = make_uint4(v.x << 16, v.x & 0xffff0000u, v.y << 16, v.y & 0xffff0000u);
    }
    for (size_t i = (n4 << 2) + tid; i < n; i += nth) dst[i] = __uint_as_float((uint32_t)src[i] << 16);
}

extern "C" int seraph_b200_load_safetensors(cuda_train_context_t* ctx, train_state_t* state, const char* path) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !state || !state->full_weights || !state->config || !path) return SB_ERR_ARG;
    if (sb_ensure_full_model(c, state)) return c->status ? c->status : SB_ERR_ARG;
    FILE* f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "ERROR: Cannot open %s\n", path); return SB_ERR_ARG; }
    uint64_t hsize = 0;
    if (fread(&hsize, sizeof hsize, 1, f) != 1 || fseek(f, (long)hsize, SEEK_CUR) != 0) { fclose(f); return SB_ERR_ARG; }
    const size_t nE = (size_t)c->V * c->d;
    struct { size_t begin, n; } seg[3] = {{0, nE}, {c->off[0].q, c->n_params - c->off[0].q}, {nE, (size_t)c->d}};
    size_t chunk = CK_CHUNK_DEFAULT;
    { const char* e = getenv("SERAPH_B200_CKPT_CHUNK"); if (e && atol(e) >= 1024) chunk = ((size_t)atol(e) + 3) & ~(size_t)3; }
    uint16_t* dbuf[2] = {NULL, NULL}; uint16_t* hbuf[2] = {NULL, NULL};
    cudaEvent_t ev[2] = {NULL, NULL};
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    int rc = SB_OK;
    for (int i = 0; i < 2 && rc == SB_OK; i++)
        if (cudaMalloc((void**)&dbuf[i], chunk * 2) != cudaSuccess || cudaMallocHost((void**)&hbuf[i], chunk * 2) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); rc = SB_ERR_OOM; }
    const int blocks = (c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148) * 8;
    int k = 0;
    for (int s = 0; s < 3 && rc == SB_OK; s++)
        for (size_t o = 0; o < seg[s].n && rc == SB_OK; o += chunk, k++) {
            const size_t n = seg[s].n - o < chunk ? seg[s].n - o : chunk;
            const int b = k & 1;
            if (k >= 2 && cudaEventSynchronize(ev[b]) != cudaSuccess) { rc = SB_ERR_CUDA; break; }     // the copy out of this pinned buffer two chunks ago
            if (fread(hbuf[b], 2, n, f) != n) { fprintf(stderr, "ERROR: Failed to read tensor data\n"); rc = SB_ERR_ARG; break; }
            cudaMemcpyAsync(dbuf[b], hbuf[b], n * 2, cudaMemcpyHostToDevice, st);
            cudaEventRecord(ev[b], st);
            unpack_bf16_kernel<<<blocks, 256, 0, st>>>(dbuf[b], c->W + seg[s].begin + o, n);
            c->launches++;
        }
    cudaStreamSynchronize(st);
    if (sb_check(c, cudaGetLastError(), "safetensors import")) rc = SB_ERR_CUDA;
    for (int i = 0; i < 2; i++) { if (dbuf[i]) cudaFree(dbuf[i]); if (hbuf[i]) cudaFreeHost(hbuf[i]); if (ev[i]) cudaEventDestroy(ev[i]); }
    fclose(f);
    if (rc != SB_OK) sb_set_status(c, rc);
    return rc;
}


// BF16 words in host memory (pageable: a memory-mapped safetensors file) widened into FP32 device memory: chunks go through
// two pinned buffers, 2 bytes per element over the bus, the 16-bit shift of bf16_to_f32 (src/train_cuda.c:19-23) on the GPU.
extern "C" int sb_upload_bf16(sb_ctx_t* c, const uint16_t* src, float* dst, size_t n) {
    size_t chunk = CK_CHUNK_DEFAULT;
    { const char* e = getenv("SERAPH_B200_CKPT_CHUNK"); if (e && atol(e) >= 1024) chunk = ((size_t)atol(e) + 3) & ~(size_t)3; }
    if (chunk > n) chunk = (n + 3) & ~(size_t)3;
    uint16_t* dbuf[2] = {NULL, NULL}; uint16_t* hbuf[2] = {NULL, NULL};
    cudaEvent_t ev[2] = {NULL, NULL};
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    int rc = SB_OK;
    for (int i = 0; i < 2 && rc == SB_OK; i++)
        if (cudaMalloc((void**)&dbuf[i], chunk * 2) != cudaSuccess || cudaMallocHost((void**)&hbuf[i], chunk * 2) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); rc = SB_ERR_OOM; }
    const int blocks = (c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148) * 8;
    int k = 0;
    for (size_t o = 0; o < n && rc == SB_OK; o += chunk, k++) {
        const size_t m = n - o < chunk ? n - o : chunk;
        const int b = k & 1;
        if (k >= 2 && cudaEventSynchronize(ev[b]) != cudaSuccess) { rc = SB_ERR_CUDA; break; }
        memcpy(hbuf[b], src + o, m * 2);
        cudaMemcpyAsync(dbuf[b], hbuf[b], m * 2, cudaMemcpyHostToDevice, st);
        cudaEventRecord(ev[b], st);
        unpack_bf16_kernel<<<blocks, 256, 0, st>>>(dbuf[b], dst + o, m);
        c->launches++;
    }
    cudaStreamSynchronize(st);
    if (sb_check(c, cudaGetLastError(), "BF16 weight upload")) rc = SB_ERR_CUDA;
    for (int i = 0; i < 2; i++) { if (dbuf[i]) cudaFree(dbuf[i]); if (hbuf[i]) cudaFreeHost(hbuf[i]); if (ev[i]) cudaEventDestroy(ev[i]); }
    return rc;
}
