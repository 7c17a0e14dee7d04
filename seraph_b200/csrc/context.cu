// context.cu - context lifetime, device buffers, scratch and status of libseraph_b200.
// Replaces the context/buffer half of the reference's src/cuda_train_context.cu
// (cuda_train_init :2246, cuda_train_free :2404, buffer functions :2568-2640).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

extern "C" {

int sb_check(sb_ctx_t* c, int err, const char* what) {
    if (err == (int)cudaSuccess) return 0;
    fprintf(stderr, "seraph_b200: CUDA error in %s: %s\n", what, cudaGetErrorString((cudaError_t)err));
    if (c) c->status = SB_ERR_CUDA;
    return 1;
}

void sb_set_status(sb_ctx_t* c, int st) { if (c && st != SB_OK) c->status = st; }

void* sb_scratch(sb_ctx_t* c, size_t bytes) {
    if (c->scratch_bytes >= bytes) return c->scratch;
    cudaStreamSynchronize((cudaStream_t)c->pub.stream);
    if (c->scratch) cudaFree(c->scratch);
    c->scratch = NULL; c->scratch_bytes = 0;
    size_t want = bytes + (bytes >> 2) + (1u << 20);
    if (sb_check(c, cudaMalloc(&c->scratch, want), "scratch alloc")) { c->status = SB_ERR_OOM; return NULL; }
    c->scratch_bytes = want;
    return c->scratch;
}

void* sb_gemm_stage(sb_ctx_t* c, int slot, size_t bytes) {
    if (c->gemm_stage_bytes[slot] >= bytes) return c->gemm_stage[slot];
    cudaStreamSynchronize((cudaStream_t)c->pub.stream);
    if (c->gemm_stage[slot]) cudaFree(c->gemm_stage[slot]);
    c->gemm_stage[slot] = NULL; c->gemm_stage_bytes[slot] = 0;
    size_t want = bytes + (1u << 20);
    if (sb_check(c, cudaMalloc(&c->gemm_stage[slot], want), "gemm staging alloc")) { c->status = SB_ERR_OOM; return NULL; }
    c->gemm_stage_bytes[slot] = want;
    return c->gemm_stage[slot];
}

void sb_memset(sb_ctx_t* c, void* p, int byte, size_t bytes) {
    int t = sb_tick_begin(c, SB_CLS_COPY);
    sb_check(c, cudaMemsetAsync(p, byte, bytes, (cudaStream_t)c->pub.stream), "memset");
    sb_tick_end(c, t, 0, (double)bytes);
}
void sb_copy(sb_ctx_t* c, void* dst, const void* src, size_t bytes) {
    int t = sb_tick_begin(c, SB_CLS_COPY);
    sb_check(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)c->pub.stream), "copy");
    sb_tick_end(c, t, 0, 2.0 * (double)bytes);
}

// ---------------------------------------------------------------------------
// Context management (reference: src/cuda_train_context.cu:2246-2402)
// ---------------------------------------------------------------------------
cuda_train_context_t* cuda_train_init(int device_id) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        fprintf(stderr, "seraph_b200: no CUDA device; this library has no CPU path\n");
        return NULL;
    }
    if (device_id < 0) device_id = 0;
    if (cudaSetDevice(device_id) != cudaSuccess) {
        fprintf(stderr, "seraph_b200: cannot select device %d\n", device_id);
        return NULL;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) return NULL;
    if (prop.major != 10) {
        fprintf(stderr, "seraph_b200: device %d is sm_%d%d; this build carries sm_100a code only\n",
                device_id, prop.major, prop.minor);
        return NULL;
    }
    sb_ctx_t* c = (sb_ctx_t*)calloc(1, sizeof(sb_ctx_t));
    if (!c) return NULL;
    cudaStream_t s;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { free(c); return NULL; }
    c->magic = SB_MAGIC;
    c->gemm_mode = SB_GEMM_FP16X3;
    { const char* e = getenv("SERAPH_B200_GEMM_PAIR"); c->gemm_pair = (e && e[0] == '0') ? 0 : 1; }
    { const char* e = getenv("SERAPH_B200_EVAL_BATCH_TOKENS"); c->eval_batch_tokens = (e && e[0]) ? atoi(e) : 8192; if (c->eval_batch_tokens < 0) c->eval_batch_tokens = 0; }
    { const char* e = getenv("SERAPH_B200_ATTN_FLASH"); c->attn_flash = (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 1; }
    { const char* e = getenv("SERAPH_B200_ATTN_FUSED"); c->attn_fused = (e && e[0] == '1') ? 1 : 0; }
    { const char* e = getenv("SERAPH_B200_GEMM_TAIL_SPLIT"); c->gemm_tail_split = (e && e[0] == '0') ? 0 : 1; }
    { const char* e = getenv("SERAPH_B200_PARTS_CACHE"); c->parts_cache = (e && e[0] == '0') ? 0 : 1; }
    c->dp_world = 1;
    { const char* e = getenv("SERAPH_B200_DP_TIMEOUT_MS"); c->dp_timeout_ms = (e && atoi(e) > 0) ? atoi(e) : 120000; }
    cuda_train_context_t* p = &c->pub;
    p->device_id = device_id; p->stream = s; p->initialized = 1;
    p->gpu_sm_count = prop.multiProcessorCount;
    p->gpu_max_threads_per_block = prop.maxThreadsPerBlock;
    p->gpu_shared_mem_per_block = (int)prop.sharedMemPerBlock;
    p->gpu_shared_mem_per_sm = (int)prop.sharedMemPerMultiprocessor;
    p->gpu_warp_size = prop.warpSize;
    p->gpu_compute_major = prop.major; p->gpu_compute_minor = prop.minor;
    p->gpu_l2_cache_bytes = prop.l2CacheSize;
    p->gpu_max_shared_per_block_optin = (int)prop.sharedMemPerBlockOptin;
    p->gpu_max_threads_per_sm = prop.maxThreadsPerMultiProcessor;
    p->gpu_regs_per_sm = prop.regsPerMultiprocessor;
    // informational only: the kernels here fix their own tile shapes
    p->matmul_tile_dim = 128; p->matmul_block_k = 32;
    p->parallel_block_size = 256; p->attention_block_size = 256; p->attention_num_warps = 8;
    if (cudaMalloc(&c->d_status, 4 * sizeof(int)) != cudaSuccess) { cudaStreamDestroy(s); free(c); return NULL; }
    cudaMemset(c->d_status, 0, 4 * sizeof(int));
    cudaMalloc(&c->d_loss, 16 * sizeof(float));
    c->d_gnorm = c->d_loss + 8;
    cudaMemset(c->d_loss, 0, 16 * sizeof(float));
    return p;
}

void cuda_train_get_gpu_info(cuda_train_context_t* ctx, char* name, int name_len, float* memory_gb) {
    if (name && name_len > 0) name[0] = '\0';
    if (memory_gb) *memory_gb = 0.0f;
    if (!ctx || !ctx->initialized) return;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ctx->device_id) != cudaSuccess) return;
    if (name && name_len > 0) { strncpy(name, prop.name, (size_t)name_len - 1); name[name_len - 1] = '\0'; }
    if (memory_gb) *memory_gb = (float)(prop.totalGlobalMem / (1024.0 * 1024.0 * 1024.0));
}

void cuda_train_sync(cuda_train_context_t* ctx) {
    if (!ctx || !ctx->stream) return;
    sb_check(sb_priv(ctx), cudaStreamSynchronize((cudaStream_t)ctx->stream), "stream sync");
}

// ---------------------------------------------------------------------------
// Buffers (reference: src/cuda_train_context.cu:2568-2640).  Uploads and the
// fill are stream-ordered, downloads synchronise, as in the reference.
// ---------------------------------------------------------------------------
cuda_buffer_t* cuda_train_buffer_create(cuda_train_context_t* ctx, size_t size) {
    (void)ctx;
    cuda_buffer_t* b = (cuda_buffer_t*)malloc(sizeof(cuda_buffer_t));
    if (!b) return NULL;
    void* p = NULL;
    cudaError_t e = cudaMalloc(&p, size ? size : 4);
    if (e != cudaSuccess) {
        fprintf(stderr, "seraph_b200: failed to allocate %zu bytes: %s\n", size, cudaGetErrorString(e));
        free(b);
        return NULL;
    }
    b->data = (float*)p; b->size = size;
    return b;
}

void cuda_train_buffer_free(cuda_train_context_t* ctx, cuda_buffer_t* buf) {
    (void)ctx;
    if (!buf) return;
    if (buf->data) cudaFree(buf->data);
    free(buf);
}

void cuda_train_buffer_upload(cuda_train_context_t* ctx, cuda_buffer_t* buf, const float* data, size_t count) {
    if (!ctx || !buf || !data) return;
    sb_check(sb_priv(ctx), cudaMemcpyAsync(buf->data, data, count * sizeof(float), cudaMemcpyHostToDevice,
                                           (cudaStream_t)ctx->stream), "upload");
}
void cuda_train_buffer_upload_u32(cuda_train_context_t* ctx, cuda_buffer_t* buf, const uint32_t* data, size_t count) {
    if (!ctx || !buf || !data) return;
    sb_check(sb_priv(ctx), cudaMemcpyAsync(buf->data, data, count * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                           (cudaStream_t)ctx->stream), "upload_u32");
}
void cuda_train_buffer_download_bytes(cuda_train_context_t* ctx, cuda_buffer_t* buf, void* data, size_t bytes) {
    if (!ctx || !buf || !data) return;
    sb_ctx_t* c = sb_priv(ctx);
    sb_check(c, cudaMemcpyAsync(data, buf->data, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)ctx->stream), "download");
    sb_check(c, cudaStreamSynchronize((cudaStream_t)ctx->stream), "download sync");
}
void cuda_train_buffer_download(cuda_train_context_t* ctx, cuda_buffer_t* buf, float* data, size_t count) {
    cuda_train_buffer_download_bytes(ctx, buf, data, count * sizeof(float));
}
// `value` is a byte value, as with cudaMemsetAsync in the reference
void cuda_train_fill_buffer_range(cuda_train_context_t* ctx, cuda_buffer_t* buf, size_t offset, uint32_t value, size_t bytes) {
    if (!ctx || !buf) return;
    sb_check(sb_priv(ctx), cudaMemsetAsync((char*)buf->data + offset, (int)value, bytes, (cudaStream_t)ctx->stream), "fill");
}
void cuda_train_fill_buffer(cuda_train_context_t* ctx, cuda_buffer_t* buf, uint32_t value, size_t bytes) {
    cuda_train_fill_buffer_range(ctx, buf, 0, value, bytes);
}
void cuda_train_copy_buffer(cuda_train_context_t* ctx, cuda_buffer_t* src, cuda_buffer_t* dst, size_t bytes) {
    if (!ctx || !src || !dst) return;
    sb_check(sb_priv(ctx), cudaMemcpyAsync(dst->data, src->data, bytes, cudaMemcpyDeviceToDevice,
                                           (cudaStream_t)ctx->stream), "copy_buffer");
}

// ---------------------------------------------------------------------------
// Per-class timer: one CUDA-event pair per launch, recorded on the context's
// stream, summed per kernel class on read-out.
// ---------------------------------------------------------------------------
// Names under which the class timer's launches appear in a cuda_profiler_t report; the reference's analysis sorts ops into its
// categories by substrings of these names (src/cuda_profiler.cu:159-178).
static const char* sb_prof_class_name(int cls) {
    static const char* names[SB_NCLS] = {"matmul", "matmul_operand_prep", "attention", "attention_bwd", "rmsnorm", "rmsnorm_bwd",
                                         "swiglu", "rope", "cross_entropy", "embedding", "adamw", "copy", "other"};
    return (cls >= 0 && cls < SB_NCLS) ? names[cls] : "other";
}
int sb_tick_begin(sb_ctx_t* c, int cls) {
    // every launcher passes through here, the training step's own launches included: with a profiler attached and no op-level
    // record open around this launch, the launch becomes a profiler op of its class
    c->tick_prof = 0;
    if (c->profiler && c->profiler->enabled && c->prof_depth == 0)
        c->tick_prof = 1 + cuda_profiler_begin_op(c->profiler, sb_prof_class_name(cls), c->pub.stream);
    if (!c->timing_on) return -1;
    if (c->tick_n >= c->tick_cap) {
        int ncap = c->tick_cap ? c->tick_cap * 2 : 4096;
        void** ev = (void**)realloc(c->tick_ev, sizeof(void*) * 2 * ncap);
        int* cl = (int*)realloc(c->tick_cls, sizeof(int) * ncap);
        double* fl = (double*)realloc(c->tick_flops, sizeof(double) * ncap);
        double* by = (double*)realloc(c->tick_bytes, sizeof(double) * ncap);
        if (ev) c->tick_ev = ev;
        if (cl) c->tick_cls = cl;
        if (fl) c->tick_flops = fl;
        if (by) c->tick_bytes = by;
        if (!ev || !cl || !fl || !by) return -1;
        for (int i = c->tick_cap; i < ncap; i++) {
            cudaEvent_t a, b;
            cudaEventCreate(&a); cudaEventCreate(&b);
            c->tick_ev[2 * i] = a; c->tick_ev[2 * i + 1] = b;
        }
        c->tick_cap = ncap;
    }
    int i = c->tick_n++;
    c->tick_cls[i] = cls; c->tick_flops[i] = 0; c->tick_bytes[i] = 0;
    cudaEventRecord((cudaEvent_t)c->tick_ev[2 * i], (cudaStream_t)c->pub.stream);
    return i;
}
void sb_tick_end(sb_ctx_t* c, int slot, double flops, double bytes) {
    if (c->tick_prof > 0 && c->profiler) {
        const int op = c->tick_prof - 1;
        cuda_profiler_end_op(c->profiler, op, c->pub.stream);
        cuda_profiler_set_flops(c->profiler, op, (size_t)flops); cuda_profiler_set_bytes(c->profiler, op, (size_t)bytes);
    }
    c->tick_prof = 0;
    if (slot < 0) return;
    cudaEventRecord((cudaEvent_t)c->tick_ev[2 * slot + 1], (cudaStream_t)c->pub.stream);
    c->tick_flops[slot] = flops; c->tick_bytes[slot] = bytes;
}
int seraph_b200_timing_enable(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->timing_on = on ? 1 : 0;
    if (on) c->tick_n = 0;
    return SB_OK;
}
int seraph_b200_timing_classes(void) { return SB_NCLS; }
const char* seraph_b200_timing_class_name(int cls) {
    static const char* names[SB_NCLS] = {"gemm", "gemm_operand_prep", "attention_fwd", "attention_bwd", "rmsnorm_fwd", "rmsnorm_bwd",
                                         "swiglu", "rope", "cross_entropy", "embedding", "adamw", "copy_fill", "other"};
    return (cls >= 0 && cls < SB_NCLS) ? names[cls] : "";
}
// out[cls*4 + {0: milliseconds, 1: algorithmic FLOPs, 2: algorithmic bytes, 3: launches}]; resets the record
int seraph_b200_timing_read(cuda_train_context_t* ctx, double* out) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !out) return SB_ERR_ARG;
    cudaStreamSynchronize((cudaStream_t)ctx->stream);
    for (int i = 0; i < SB_NCLS * 4; i++) out[i] = 0.0;
    for (int i = 0; i < c->tick_n; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, (cudaEvent_t)c->tick_ev[2 * i], (cudaEvent_t)c->tick_ev[2 * i + 1]) != cudaSuccess) continue;
        int k = c->tick_cls[i];
        out[k * 4 + 0] += ms; out[k * 4 + 1] += c->tick_flops[i]; out[k * 4 + 2] += c->tick_bytes[i]; out[k * 4 + 3] += 1.0;
    }
    c->tick_n = 0;
    return SB_OK;
}

// ---------------------------------------------------------------------------
// Extensions
// ---------------------------------------------------------------------------
int seraph_b200_last_status(cuda_train_context_t* ctx) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    int dev[4] = {0, 0, 0, 0};
    cudaStreamSynchronize((cudaStream_t)ctx->stream);
    if (cudaMemcpy(dev, c->d_status, sizeof dev, cudaMemcpyDeviceToHost) == cudaSuccess && dev[0] != 0) {
        c->status = dev[0];
        cudaMemset(c->d_status, 0, sizeof dev);
    }
    int s = c->status;
    c->status = SB_OK;
    return s;
}

int seraph_b200_set_gemm_mode(cuda_train_context_t* ctx, int mode) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || mode < 0 || mode > 4) return SB_ERR_ARG;
    c->gemm_mode = mode;
    return SB_OK;
}

int seraph_b200_set_gemm_pair(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->gemm_pair = on ? 1 : 0;
    return SB_OK;
}

int seraph_b200_set_eval_batch_tokens(cuda_train_context_t* ctx, int tokens) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || tokens < 0) return SB_ERR_ARG;
    c->eval_batch_tokens = tokens;
    return SB_OK;
}

int seraph_b200_set_attn_flash(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->attn_flash = (on >= 0 && on <= 3) ? on : 1;
    return SB_OK;
}

int seraph_b200_set_attn_fused(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->attn_fused = on ? 1 : 0;
    return SB_OK;
}

int seraph_b200_set_gemm_tail_split(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->gemm_tail_split = on ? 1 : 0;
    return SB_OK;
}

int seraph_b200_set_parts_cache(cuda_train_context_t* ctx, int on) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->parts_cache = on ? 1 : 0;
    return SB_OK;
}

int seraph_b200_set_lora_exact(cuda_train_context_t* ctx, int exact) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    c->lora_exact = exact ? 1 : 0;
    return SB_OK;
}

int seraph_b200_set_grad_clip(cuda_train_context_t* ctx, float max_norm) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || max_norm < 0) return SB_ERR_ARG;
    c->grad_clip = max_norm;
    return SB_OK;
}

// the NaN/Inf flags of the last step that ran with state->debug_nan_check (ctx->debug_nan_flags), copied to the host;
// returns the number of words written
int seraph_b200_nan_flags(cuda_train_context_t* ctx, uint32_t* out, int max_words) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || !out || max_words <= 0 || !c->pub.debug_nan_flags) return 0;
    int n = (int)(c->pub.debug_nan_flags->size / 4);
    if (n > max_words) n = max_words;
    cudaStreamSynchronize((cudaStream_t)ctx->stream);
    return cudaMemcpy(out, c->pub.debug_nan_flags->data, (size_t)n * 4, cudaMemcpyDeviceToHost) == cudaSuccess ? n : 0;
}

// category totals of an analysed cuda_profiler_t as floats: step, matmul, attention, attention_bwd, rmsnorm, rmsnorm_bwd,
// cross_entropy, adamw, copy, other (milliseconds); returns the number of recorded ops
int seraph_b200_profiler_totals(cuda_profiler_t* p, float* out10) {
    if (!p || !out10) return 0;
    out10[0] = p->total_step_ms; out10[1] = p->total_matmul_ms; out10[2] = p->total_attention_ms; out10[3] = p->total_attention_bwd_ms;
    out10[4] = p->total_rmsnorm_ms; out10[5] = p->total_rmsnorm_bwd_ms; out10[6] = p->total_cross_entropy_ms; out10[7] = p->total_adamw_ms;
    out10[8] = p->total_copy_ms; out10[9] = p->total_other_ms;
    return p->num_ops;
}

unsigned long long seraph_b200_launch_count(cuda_train_context_t* ctx, int reset) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return 0;
    unsigned long long n = c->launches;
    if (reset) c->launches = 0;
    return n;
}

}  // extern "C"
