// profiler.cu - per-op CUDA-event profiler with the reference's 13-symbol ABI
// (include/cuda_profiler.h:53-82, src/cuda_profiler.cu).  Each op records an
// event pair on the context's stream plus its algorithmic FLOPs and bytes, so
// the report can show achieved GB/s and TFLOP/s next to the time.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

extern "C" {

cuda_profiler_t* cuda_profiler_create(void) {
    cuda_profiler_t* p = (cuda_profiler_t*)calloc(1, sizeof(cuda_profiler_t));
    if (!p) return NULL;
    for (int i = 0; i < PROFILER_MAX_OPS; i++) {
        cudaEvent_t a, b;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) { free(p); return NULL; }
        p->ops[i].event_start = a; p->ops[i].event_end = b;
    }
    return p;
}
void cuda_profiler_destroy(cuda_profiler_t* p) {
    if (!p) return;
    for (int i = 0; i < PROFILER_MAX_OPS; i++) {
        if (p->ops[i].event_start) cudaEventDestroy((cudaEvent_t)p->ops[i].event_start);
        if (p->ops[i].event_end) cudaEventDestroy((cudaEvent_t)p->ops[i].event_end);
    }
    free(p);
}
void cuda_profiler_enable(cuda_profiler_t* p) { if (p) p->enabled = 1; }
void cuda_profiler_disable(cuda_profiler_t* p) { if (p) p->enabled = 0; }
void cuda_profiler_reset(cuda_profiler_t* p) {
    if (!p) return;
    p->num_ops = 0;
    p->total_step_ms = p->total_matmul_ms = p->total_attention_ms = p->total_attention_bwd_ms = 0.f;
    p->total_rmsnorm_ms = p->total_rmsnorm_bwd_ms = p->total_cross_entropy_ms = p->total_adamw_ms = 0.f;
    p->total_copy_ms = p->total_other_ms = 0.f;
}
int cuda_profiler_begin_op(cuda_profiler_t* p, const char* name, void* stream) {
    if (!p || !p->enabled || p->num_ops >= PROFILER_MAX_OPS) return -1;
    int i = p->num_ops++;
    profiler_op_t* o = &p->ops[i];
    strncpy(o->name, name ? name : "", sizeof(o->name) - 1); o->name[sizeof(o->name) - 1] = '\0';
    o->elapsed_ms = 0.f; o->flops = 0; o->bytes = 0; o->shared_mem = 0;
    o->grid_x = o->grid_y = o->grid_z = o->block_x = o->block_y = o->block_z = 0;
    cudaEventRecord((cudaEvent_t)o->event_start, (cudaStream_t)stream);
    return i;
}
void cuda_profiler_end_op(cuda_profiler_t* p, int i, void* stream) {
    if (!p || i < 0 || i >= p->num_ops) return;
    cudaEventRecord((cudaEvent_t)p->ops[i].event_end, (cudaStream_t)stream);
}
void cuda_profiler_set_launch(cuda_profiler_t* p, int i, int gx, int gy, int gz, int bx, int by, int bz, size_t smem) {
    if (!p || i < 0 || i >= p->num_ops) return;
    profiler_op_t* o = &p->ops[i];
    o->grid_x = gx; o->grid_y = gy; o->grid_z = gz; o->block_x = bx; o->block_y = by; o->block_z = bz; o->shared_mem = smem;
}
void cuda_profiler_set_flops(cuda_profiler_t* p, int i, size_t flops) { if (p && i >= 0 && i < p->num_ops) p->ops[i].flops = flops; }
void cuda_profiler_set_bytes(cuda_profiler_t* p, int i, size_t bytes) { if (p && i >= 0 && i < p->num_ops) p->ops[i].bytes = bytes; }

// categories by substring of the op name, as the reference does (src/cuda_profiler.cu:159-178)
void cuda_profiler_sync_and_analyze(cuda_profiler_t* p, void* stream) {
    if (!p) return;
    cudaStreamSynchronize((cudaStream_t)stream);
    float tot = 0.f;
    p->total_matmul_ms = p->total_attention_ms = p->total_attention_bwd_ms = p->total_rmsnorm_ms = 0.f;
    p->total_rmsnorm_bwd_ms = p->total_cross_entropy_ms = p->total_adamw_ms = p->total_copy_ms = p->total_other_ms = 0.f;
    for (int i = 0; i < p->num_ops; i++) {
        profiler_op_t* o = &p->ops[i];
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, (cudaEvent_t)o->event_start, (cudaEvent_t)o->event_end) != cudaSuccess) ms = 0.f;
        o->elapsed_ms = ms; tot += ms;
        const char* n = o->name;
        if (strstr(n, "matmul") || strstr(n, "lora")) p->total_matmul_ms += ms;
        else if (strstr(n, "attention_bwd") || strstr(n, "attn_bwd")) p->total_attention_bwd_ms += ms;
        else if (strstr(n, "attention") || strstr(n, "attn")) p->total_attention_ms += ms;
        else if (strstr(n, "rmsnorm_bwd")) p->total_rmsnorm_bwd_ms += ms;
        else if (strstr(n, "rmsnorm")) p->total_rmsnorm_ms += ms;
        else if (strstr(n, "cross_entropy")) p->total_cross_entropy_ms += ms;
        else if (strstr(n, "adamw")) p->total_adamw_ms += ms;
        else if (strstr(n, "copy") || strstr(n, "fill")) p->total_copy_ms += ms;
        else p->total_other_ms += ms;
    }
    p->total_step_ms = tot;
}

static void emit(cuda_profiler_t* p, const char* line) {
    fputs(line, stdout);
    if (p->log_file) fputs(line, (FILE*)p->log_file);
}
static void print_op(cuda_profiler_t* p, const profiler_op_t* o) {
    char line[256];
    double s = o->elapsed_ms * 1e-3;
    double tf = (s > 0 && o->flops) ? o->flops / s * 1e-12 : 0.0, gb = (s > 0 && o->bytes) ? o->bytes / s * 1e-9 : 0.0;
    snprintf(line, sizeof line, "  %-48s %9.4f ms  %8.2f TFLOP/s  %8.1f GB/s\n", o->name, o->elapsed_ms, tf, gb);
    emit(p, line);
}
void cuda_profiler_print(cuda_profiler_t* p) {
    if (!p) return;
    char line[256];
    snprintf(line, sizeof line, "# seraph_b200 profile: %d ops, %.3f ms\n", p->num_ops, p->total_step_ms); emit(p, line);
    for (int i = 0; i < p->num_ops; i++) print_op(p, &p->ops[i]);
    snprintf(line, sizeof line, "# matmul %.3f | attn %.3f | attn_bwd %.3f | rmsnorm %.3f | rmsnorm_bwd %.3f | ce %.3f | adamw %.3f | copy %.3f | other %.3f (ms)\n",
             p->total_matmul_ms, p->total_attention_ms, p->total_attention_bwd_ms, p->total_rmsnorm_ms, p->total_rmsnorm_bwd_ms,
             p->total_cross_entropy_ms, p->total_adamw_ms, p->total_copy_ms, p->total_other_ms);
    emit(p, line);
}
void cuda_profiler_print_top(cuda_profiler_t* p, int top_n) {
    if (!p || top_n <= 0) return;
    int n = p->num_ops;
    int* idx = (int*)malloc(sizeof(int) * (n > 0 ? n : 1));
    if (!idx) return;
    for (int i = 0; i < n; i++) idx[i] = i;
    for (int i = 0; i < n && i < top_n; i++) {          // partial selection sort
        int best = i;
        for (int j = i + 1; j < n; j++) if (p->ops[idx[j]].elapsed_ms > p->ops[idx[best]].elapsed_ms) best = j;
        int t = idx[i]; idx[i] = idx[best]; idx[best] = t;
    }
    char line[64]; snprintf(line, sizeof line, "# top %d ops\n", top_n < n ? top_n : n); emit(p, line);
    for (int i = 0; i < n && i < top_n; i++) print_op(p, &p->ops[idx[i]]);
    free(idx);
}
void cuda_profiler_set_log(cuda_profiler_t* p, void* file_ptr) { if (p) p->log_file = file_ptr; }

// op-level record around one call of the per-op C ABI; the launches inside it are not recorded a second time
int sb_prof_begin(sb_ctx_t* c, const char* name) {
    if (!c->profiler || !c->profiler->enabled) return -1;
    const int op = cuda_profiler_begin_op(c->profiler, name, c->pub.stream);
    if (op >= 0) c->prof_depth++;
    return op;
}
void sb_prof_end(sb_ctx_t* c, int op, size_t flops, size_t bytes) {
    if (op < 0 || !c->profiler) return;
    if (c->prof_depth > 0) c->prof_depth--;
    cuda_profiler_end_op(c->profiler, op, c->pub.stream);
    c->profiler->ops[op].flops = flops; c->profiler->ops[op].bytes = bytes;
}

}  // extern "C"
