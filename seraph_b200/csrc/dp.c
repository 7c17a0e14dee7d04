/*
 * dp.c - data parallelism for the training step: one process per GPU, every
 * rank holds the full model and runs the step on its own micro-batch; the
 * gradients are summed with NCCL all-reduce over NVLink.  The reference has no
 * multi-GPU code at all, so these entry points have no counterpart there.
 *
 * Gradients live in one arena, so a bucket is a plain range.  During backward
 * the step hands over each finished range (a layer, last the embedding and the
 * final norm); the all-reduce of a bucket runs on a second stream while the
 * next layer's backward computes.  AdamW waits for the last bucket and folds
 * 1/world into its gradient read.
 *
 * NCCL is loaded at run time (dlopen of libnccl.so.2), so single-GPU users do
 * not need it, and a process that already holds NCCL (for example through
 * torch) shares that copy.  Errors are reported through the status code; a
 * failed or timed-out communicator is aborted on the host, never waited on
 * forever.
 */
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include "sb_internal.h"

static struct {
    void* lib;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);      /* optional */
    ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, ncclConfig_t*);                 /* optional */
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    const char* (*GetErrorString)(ncclResult_t);
} N;

static int load_nccl(void) {
    if (N.lib) return 0;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { fprintf(stderr, "seraph_b200: cannot load NCCL: %s\n", dlerror()); return 1; }
#define SYM(f) do { *(void**)(&N.f) = dlsym(h, "nccl" #f); if (!N.f) { fprintf(stderr, "seraph_b200: NCCL lacks nccl" #f "\n"); dlclose(h); return 1; } } while (0)
    SYM(GetUniqueId); SYM(CommInitRank); SYM(AllReduce); SYM(CommDestroy); SYM(CommAbort); SYM(CommGetAsyncError); SYM(GetErrorString);
#undef SYM
    *(void**)(&N.CommInitRankConfig) = dlsym(h, "ncclCommInitRankConfig");
    *(void**)(&N.CommSplit) = dlsym(h, "ncclCommSplit");
    N.lib = h;
    return 0;
}

static int nccl_fail(sb_ctx_t* c, ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return 0;
    fprintf(stderr, "seraph_b200: NCCL error in %s: %s\n", what, N.GetErrorString ? N.GetErrorString(r) : "?");
    c->status = SB_ERR_NCCL;
    return 1;
}

/* 128-byte id made on rank 0 and carried to the other ranks by the caller */
int seraph_dp_get_unique_id(void* id_out_128) {
    if (!id_out_128 || load_nccl()) return SB_ERR_NCCL;
    ncclUniqueId id;
    if (N.GetUniqueId(&id) != ncclSuccess) return SB_ERR_NCCL;
    memcpy(id_out_128, &id, sizeof id);
    return SB_OK;
}

void sb_dp_finalize(sb_ctx_t* c);
int seraph_dp_init(cuda_train_context_t* ctx, int rank, int world, const void* nccl_unique_id) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || world < 1 || rank < 0 || rank >= world) return SB_ERR_ARG;
    if (c->nccl_comm || c->comm_stream) sb_dp_finalize(c);      /* a second init, or one after an aborted communicator */
    if (world == 1) { c->dp_world = 1; c->dp_rank = 0; return SB_OK; }
    if (!nccl_unique_id || load_nccl()) return SB_ERR_NCCL;
    if (cudaSetDevice(ctx->device_id) != cudaSuccess) return SB_ERR_CUDA;
    ncclUniqueId id; memcpy(&id, nccl_unique_id, sizeof id);
    ncclComm_t comm;
    /* The all-reduce kernels run beside the backward pass, whose GEMM launches are persistent grids of one CTA pair per SM pair:
       every SM a collective takes makes a straggler pair that runs its share of the tiles after the others, which can double
       a product's time.  The gradients of a whole step need well under a tenth of NVLink's bandwidth to finish inside the backward
       pass, so the communicator is held to a few CTAs (SERAPH_B200_NCCL_MAX_CTAS, default 8; 0 leaves NCCL's own choice), and
       while buckets are being reduced the GEMM grids are launched that many SMs smaller (gemm_reserve_sms). */
    int max_ctas = 8;
    { const char* e = getenv("SERAPH_B200_NCCL_MAX_CTAS"); if (e && e[0]) max_ctas = atoi(e); }
    ncclResult_t ir;
    if (N.CommInitRankConfig && max_ctas > 0) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.minCTAs = 1; cfg.maxCTAs = max_ctas;
        ir = N.CommInitRankConfig(&comm, world, id, rank, &cfg);
    } else ir = N.CommInitRank(&comm, world, id, rank);
    if (nccl_fail(c, ir, "ncclCommInitRank")) return SB_ERR_NCCL;
    /* The step's last bucket (embedding and final norm, a sixth of the gradients) is reduced after the backward pass, beside
       AdamW on the layers and no GEMM: a second communicator over the same ranks, without the cap, takes it at full NVLink
       bandwidth.  SERAPH_B200_NCCL_WIDE=0 switches it off. */
    ncclComm_t wide = NULL;
    { const char* e = getenv("SERAPH_B200_NCCL_WIDE");
      if (N.CommSplit && N.CommInitRankConfig && max_ctas > 0 && !(e && e[0] == '0')) {
          ncclConfig_t cfg2 = NCCL_CONFIG_INITIALIZER;
          cfg2.minCTAs = 1; cfg2.maxCTAs = 64;
          if (N.CommSplit(comm, 0, rank, &wide, &cfg2) != ncclSuccess) wide = NULL;
      } }
    cudaStream_t cs;
    if (cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking) != cudaSuccess) { if (wide) N.CommAbort(wide); N.CommAbort(comm); return SB_ERR_CUDA; }
    c->nccl_comm = comm; c->nccl_comm_wide = wide; c->comm_stream = cs; c->dp_rank = rank; c->dp_world = world;
    c->dp_ctas = (N.CommInitRankConfig && max_ctas > 0) ? max_ctas : 0; c->gemm_reserve_sms = 0;
    for (int i = 0; i < 64; i++) { cudaEvent_t e; cudaEventCreateWithFlags(&e, cudaEventDisableTiming); c->ev_bucket[i] = e; }
    return SB_OK;
}

/* The communicator is gone (destroyed or aborted): single-GPU from here on.  The stream and the events stay until
 * sb_dp_finalize, because work of the compute stream may still be ordered behind them. */
static void dp_drop_comm(sb_ctx_t* c, int status) {
    if (c->nccl_comm_wide) N.CommAbort((ncclComm_t)c->nccl_comm_wide);
    if (c->nccl_comm) N.CommAbort((ncclComm_t)c->nccl_comm);
    c->nccl_comm = NULL; c->nccl_comm_wide = NULL; c->dp_world = 1; c->dp_rank = 0; c->gemm_reserve_sms = 0;
    if (status) {
        c->status = status;
        fprintf(stderr, "seraph_b200: data parallelism is off for this context after the failure above; later steps run on this GPU alone\n");
    }
}

#define DP_FINALIZE_TIMEOUT_MS 30000
void sb_dp_finalize(sb_ctx_t* c) {
    if (!c) return;
    if (c->nccl_comm) {
        /* bounded: a peer that died leaves collectives of this rank unfinished for ever */
        if (seraph_dp_wait(&c->pub, DP_FINALIZE_TIMEOUT_MS) == SB_OK && c->nccl_comm) {
            if (c->nccl_comm_wide) N.CommDestroy((ncclComm_t)c->nccl_comm_wide);
            N.CommDestroy((ncclComm_t)c->nccl_comm);
            c->nccl_comm = NULL; c->nccl_comm_wide = NULL;
        }
    }
    if (c->comm_stream) {
        for (int i = 0; i < 64; i++) if (c->ev_bucket[i]) { cudaEventDestroy((cudaEvent_t)c->ev_bucket[i]); c->ev_bucket[i] = NULL; }
        cudaStreamDestroy((cudaStream_t)c->comm_stream);
        c->comm_stream = NULL;
    }
    c->nccl_comm = NULL; c->nccl_comm_wide = NULL; c->dp_world = 1; c->dp_rank = 0; c->n_buckets = 0; c->gemm_reserve_sms = 0;
}
void seraph_dp_finalize(cuda_train_context_t* ctx) { sb_dp_finalize(sb_priv(ctx)); }

/* Hand a finished gradient range to the communication stream.  Ordering: the
 * compute stream records an event, the communication stream waits for it. */
static int dp_bucket(sb_ctx_t* c, float* p, size_t n, int wide);
int sb_dp_bucket_ready(sb_ctx_t* c, float* p, size_t n) { return dp_bucket(c, p, n, 0); }
/* a bucket handed over when no GEMM follows it in the step: on the communicator without the CTA cap when there is one */
int sb_dp_bucket_ready_last(sb_ctx_t* c, float* p, size_t n) { return dp_bucket(c, p, n, 1); }
static int dp_bucket(sb_ctx_t* c, float* p, size_t n, int wide) {
    if (c->dp_world <= 1 || !n) return 0;
    cudaEvent_t e = (cudaEvent_t)c->ev_bucket[c->n_buckets % 62];      /* 62 and 63 are the join events */
    c->n_buckets++;
    /* whole SM pairs, until the join; not for buckets whose reduction is over in a fraction of one product's time (adapter gradients) */
    if (n * sizeof(float) >= ((size_t)32 << 20)) c->gemm_reserve_sms = (c->dp_ctas + 1) & ~1;
    if (sb_check(c, cudaEventRecord(e, (cudaStream_t)c->pub.stream), "bucket event")) return 1;
    if (sb_check(c, cudaStreamWaitEvent((cudaStream_t)c->comm_stream, e, 0), "bucket wait")) return 1;
    ncclComm_t comm = (ncclComm_t)((wide && c->nccl_comm_wide) ? c->nccl_comm_wide : c->nccl_comm);
    return nccl_fail(c, N.AllReduce(p, p, n, ncclFloat32, ncclSum, comm, (cudaStream_t)c->comm_stream), "ncclAllReduce");
}

/* A mark on the communication stream behind the buckets handed over so far, and the compute stream's wait for that mark.  Buckets
 * handed over between the two calls are not waited for: the step marks, hands over its last bucket and then waits, so that AdamW
 * on the layers runs while the last bucket is still being reduced. */
int sb_dp_mark_partial(sb_ctx_t* c) {
    if (c->dp_world <= 1) return 1;
    return sb_check(c, cudaEventRecord((cudaEvent_t)c->ev_bucket[62], (cudaStream_t)c->comm_stream), "partial join event");
}
int sb_dp_wait_partial(sb_ctx_t* c) {
    if (c->dp_world <= 1) return 1;
    return sb_check(c, cudaStreamWaitEvent((cudaStream_t)c->pub.stream, (cudaEvent_t)c->ev_bucket[62], 0), "partial join wait");
}

/* compute stream waits until every bucket handed over so far is reduced */
int sb_dp_join(sb_ctx_t* c) {
    if (c->dp_world <= 1) return 0;
    cudaEvent_t e = (cudaEvent_t)c->ev_bucket[63];
    if (sb_check(c, cudaEventRecord(e, (cudaStream_t)c->comm_stream), "join event")) return 1;
    if (sb_check(c, cudaStreamWaitEvent((cudaStream_t)c->pub.stream, e, 0), "join wait")) return 1;
    c->n_buckets = 0; c->gemm_reserve_sms = 0;
    ncclResult_t async = ncclSuccess;
    if (N.CommGetAsyncError((ncclComm_t)c->nccl_comm, &async) != ncclSuccess || async != ncclSuccess) {
        fprintf(stderr, "seraph_b200: NCCL reported an asynchronous error; aborting the communicator\n");
        dp_drop_comm(c, SB_ERR_NCCL);
        return 1;
    }
    return 0;
}

/* whole range at once, on the compute stream's order (used when no bucket was handed over during backward) */
int sb_dp_allreduce_range(sb_ctx_t* c, float* p, size_t n) {
    if (c->dp_world <= 1) return 0;
    if (sb_dp_bucket_ready(c, p, n)) return 1;
    return sb_dp_join(c);
}

int sb_dp_allreduce_scalar(sb_ctx_t* c, float* p) { return sb_dp_allreduce_range(c, p, 1); }

/* Host-side bounded wait for the communication stream: polls the stream and the
 * communicator's asynchronous error until done or `timeout_ms` passed; on
 * time-out or error the communicator is aborted and an error is returned. */
int seraph_dp_wait(cuda_train_context_t* ctx, int timeout_ms) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return SB_ERR_ARG;
    if (c->dp_world <= 1 || !c->nccl_comm) return SB_OK;
    struct timespec t0, t; clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        cudaError_t q = cudaStreamQuery((cudaStream_t)c->comm_stream);
        if (q == cudaSuccess) return SB_OK;
        ncclResult_t async = ncclSuccess;
        N.CommGetAsyncError((ncclComm_t)c->nccl_comm, &async);
        clock_gettime(CLOCK_MONOTONIC, &t);
        long ms = (t.tv_sec - t0.tv_sec) * 1000L + (t.tv_nsec - t0.tv_nsec) / 1000000L;
        if (q != cudaErrorNotReady || async != ncclSuccess || ms > timeout_ms) {
            fprintf(stderr, "seraph_b200: data-parallel wait failed (%s); aborting the communicator\n",
                    ms > timeout_ms ? "time-out" : "error");
            const int st = ms > timeout_ms ? SB_ERR_TIMEOUT : SB_ERR_NCCL;
            dp_drop_comm(c, st);
            return st;
        }
        struct timespec nap = {0, 200000}; nanosleep(&nap, NULL);
    }
}

/* The smallest `value` any rank passed (every rank must call it at the same point).  A trainer whose ranks may run out of
 * batches at different times calls it once per step with 1 = "I have a batch" and stops when it returns 0, so that no rank
 * enters a step whose collectives the others never join.  A world of one returns `value`; -1 on a communication failure. */
int seraph_dp_all_min(cuda_train_context_t* ctx, int value) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c) return -1;
    if (c->dp_world <= 1 || !c->nccl_comm) return value;
    int* d = (int*)sb_scratch(c, 64);
    if (!d) return -1;
    cudaStream_t cs = (cudaStream_t)c->comm_stream;
    cudaStreamSynchronize((cudaStream_t)c->pub.stream);            /* the scratch word may still be in use by the step */
    if (cudaMemcpyAsync(d, &value, sizeof value, cudaMemcpyHostToDevice, cs) != cudaSuccess) return -1;
    if (nccl_fail(c, N.AllReduce(d, d, 1, ncclInt32, ncclMin, (ncclComm_t)c->nccl_comm, cs), "ncclAllReduce(min)")) return -1;
    if (seraph_dp_wait(ctx, c->dp_timeout_ms) != SB_OK) return -1;
    int out = value;
    if (cudaMemcpy(&out, d, sizeof out, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return out;
}

int seraph_dp_world(cuda_train_context_t* ctx) { sb_ctx_t* c = sb_priv(ctx); return c ? c->dp_world : 0; }
