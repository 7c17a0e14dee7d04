/*
 * sb_internal.h - private state and kernel-launch entry points of libseraph_b200.
 *
 * The public cuda_train_context_t keeps the reference's layout; everything this
 * library adds lives in sb_ctx_t, which embeds the public struct as its first
 * member so the pointer handed to callers is also the pointer to the private
 * state.  All launchers take raw device pointers and run on ctx->stream.
 */
#ifndef SB_INTERNAL_H
#define SB_INTERNAL_H

#include "../../include/seraph_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define SB_MAGIC 0x53423230u   /* "SB20" */
#define SB_F16_KEPT 10          /* operand-part slots kept across the products of a keep region */
#define SB_F16_SLOTS 12         /* plus one per operand for products outside a region */

/* status codes (seraph_b200_last_status) */
enum {
    SB_OK = 0,
    SB_ERR_ARG = 1,          /* NULL / shape argument rejected */
    SB_ERR_CUDA = 2,         /* a CUDA runtime call failed */
    SB_ERR_OOM = 3,
    SB_ERR_TOKEN_RANGE = 4,  /* a token id >= vocab reached a kernel */
    SB_ERR_TIMEOUT = 5,      /* a bounded device-side wait ran out */
    SB_ERR_NCCL = 6,
    SB_ERR_SIZE = 7          /* size beyond a fixed capacity */
};

/* kernel classes of the built-in per-class timer (seraph_b200_timing_*) */
enum { SB_CLS_GEMM = 0, SB_CLS_GEMM_PREP, SB_CLS_ATTN_FWD, SB_CLS_ATTN_BWD, SB_CLS_NORM_FWD, SB_CLS_NORM_BWD,
       SB_CLS_SWIGLU, SB_CLS_ROPE, SB_CLS_CE, SB_CLS_EMBED, SB_CLS_ADAMW, SB_CLS_COPY, SB_CLS_OTHER, SB_NCLS };

/* GEMM arithmetic modes */
enum {
    SB_GEMM_FP32X3 = 0,  /* tcgen05 kind::tf32, hi/lo split, 3 MMAs per k-block: FP32-level accuracy */
    SB_GEMM_TF32   = 1,  /* tcgen05 kind::tf32, one MMA per k-block */
    SB_GEMM_BF16   = 2,  /* tcgen05 kind::f16 on BF16 copies (use_bf16) */
    SB_GEMM_SIMT   = 3,  /* FP32 FMA on CUDA cores */
    SB_GEMM_FP16X3 = 4   /* default: FP32-level accuracy from scaled FP16 hi/lo parts (kind::f16, half the MMA cycles of FP32X3) for the plain
                            products; attention's products and shapes the FP16 path does not take run as FP32X3 */
};

typedef struct { size_t q, k, v, o, gate, up, down, in_norm, post_norm; } sb_layer_off_t;

typedef struct {
    float *layer_in, *x_norm_attn, *q, *k, *v, *attn_out, *lse, *post_attn_in, *x_norm_ffn, *gate, *up, *ffn_hidden;
    float *q_rms, *k_rms;            /* per-token sqrt(mean(x^2)) of q and k before their whole-row normalisation (use_qk_norm) */
    float *q_pre, *k_pre;            /* q and k before the learned per-head RMSNorm (head_norm), kept for its backward */
} sb_layer_act_t;

typedef struct { const float* ptr; size_t n, cur, off; unsigned gen; int kind; float* amax_ptr; } sb_parts_entry_t;   /* n: registered floats, cur: floats of the parts held */

typedef struct sb_ctx {
    cuda_train_context_t pub;        /* MUST stay first */
    uint32_t magic;
    int status;                      /* last host-side status */
    int* d_status;                   /* device status word (bounds checks, bounded waits) */
    int gemm_mode;                   /* SB_GEMM_* (use_bf16 in pub overrides to BF16) */
    float* d_amax;                   /* FP16 split: max |x| of the operand held by each part slot */
    struct { void* h; size_t cap; const float* ptr; size_t n; unsigned stamp; int valid; float* amax; } f16_slot[SB_F16_SLOTS];   /* FP16 parts of GEMM operands: 0-9 kept across
                                        calls inside a keep region (train_step.c marks runs of GEMMs that share operands), 10-11 for one call */
    int f16_keep; unsigned f16_clock;
    /* FP16 parts of registered tensors (weights, saved activations), valid from their first use inside a training or
       evaluation step until that step returns: made once, then shared by every product of the step that reads the tensor */
    sb_parts_entry_t* parts_tab;
    int parts_n, parts_cap; int* parts_hash; int parts_hash_cap;
    size_t parts_total;              /* halves the registered tensors need */
    void* parts_arena; size_t parts_arena_halves; float* parts_amax; int parts_amax_cap;
    /* largest magnitudes left by the kernels that produce GEMM operands (announced by the step driver, valid inside one step):
       the operand preparation then skips its own pass over the tensor */
    struct { const float* ptr; size_t n; } *hint_tab; int hint_n, hint_cap; float* hint_pool;
    struct { const float* ptr; size_t n; } hint_pending[4]; int hint_npending;
    unsigned parts_gen; int parts_open; int parts_cache;   /* parts_cache 0: off (switch, or the arena did not fit) */
    int eval_batch_tokens;           /* cuda_evaluate packs samples up to this many tokens per forward pass; 0: one sample per pass */
    int attn_flash;                  /* 128-wide heads: 0 a launch per product over a score scratch; otherwise the forward is one kernel and the backward
                                        is 2: scores in one kernel and three long products, 3: dK/dV kept on chip, 1 (default): whichever of the two
                                        measured faster for the shape */
    int attn_fused;                  /* 1: P and dS of the attention backward come out of the score products' epilogues */
    int gemm_tail_split;             /* 1: tiles of the last partial wave are cut into k pieces */
    int gemm_pair;                   /* 1: plain GEMMs run on CTA pairs (cta_group::2), 0: one CTA per tile */
    int lora_exact;                  /* 0: reference behaviour (adapter dX term left out), 1: full chain rule */
    float grad_clip;                 /* 0 = off (the reference has none) */
    int nan_on; uint32_t nan_count;  /* a step with state->debug_nan_check is filling pub.debug_nan_flags (nan_count words) */
    int prof_depth; int tick_prof;   /* an op-level profiler record is open; 1 + the profiler record opened by the running class timer */
    cuda_profiler_t* profiler;
    size_t launches;                 /* kernels launched since the last reset */
    int timing_on;                   /* per-class CUDA-event timing of every launch */
    void** tick_ev; int tick_cap, tick_n;   /* event pairs: tick_ev[2*i], tick_ev[2*i+1] */
    int* tick_cls; double* tick_flops; double* tick_bytes;

    /* model geometry of the resident weights */
    int V, d, L, Hq, Hkv, hd, F, qd, kvd;
    size_t n_params;
    sb_layer_off_t* off;             /* [L] offsets into the arenas */
    float *W, *G, *M, *Vv;           /* parameter, gradient, Adam m, Adam v arenas (flat order) */
    int qk_norm;                     /* config->use_qk_norm of the step in flight */
    int frozen_base;                 /* 1: LoRA mode, G/M/Vv not allocated */
    /* model options the reference's trainable_weights_t has no tensors for (seraph_b200_set_model_extras): a learned RMSNorm over
       each head of q and k before RoPE (per layer q_norm [hd], k_norm [hd]) and a separate lm_head [V,d].  Flat order: the norms of
       layer 0, 1, ..., then lm_head.  h_extras is the host master copy (uploaded when the model becomes resident). */
    int head_norm, untied;
    float* h_extras; size_t n_extras_host;
    float *XW, *XG, *XM, *XV; size_t n_extras;
    float *g_q2, *g_k2;              /* gradients of q, k before the per-head norm */

    /* LoRA adapters: one arena per kind, same flat order as the oracle */
    int lora_rank, lora_mask; float lora_alpha;
    size_t n_lora;
    float *LW, *LG, *LM, *LV;
    /* The rank-r products are far too thin for the tensor-core kernel's tiles (and ran 40 times slower on the CUDA-core GEMM),
       so the step works on copies of A and B whose rank is padded with zero rows / columns to lora_R, a multiple of 128 (the
       narrow tile of the CTA-pair kernel):
       LWp [per adapter: A (R, in) then B (out, R)] is refreshed from LW before a step when the adapters changed, the gradient
       products accumulate into LGp and the live part is copied to LG layer by layer.  Padding changes no value: the extra rows of
       A and columns of B are zero, so the extra columns of X A^T are zero and the extra gradient rows / columns are never read. */
    int lora_R; size_t n_lora_pad; float *LWp, *LGp; int lora_pad_stale;
    float* lora_tmp; size_t lora_tmp_cap;

    /* activations */
    int T_cap;
    sb_layer_act_t* act;             /* [L] */
    float* act_arena; size_t act_arena_bytes;
    float *hidden, *hidden_norm, *final_in, *logits, *dlogits, *loss_rows;
    float *g_hidden, *g_tmp, *g_xnorm, *g_q, *g_k, *g_v, *g_attn, *g_ffn, *g_gate, *g_up, *attn_delta;
    uint32_t *tokens, *targets, *seq_starts, *pos_ids, *seq_ids;
    int seq_cap, seq_starts_cap;
    int* h_seq; int h_seq_n, h_seq_cap;   /* host copy of the current batch's sequence starts (h_seq_n + 1 entries); 0 = unknown */
    int res_T, res_B, res_max_seq;   /* geometry of the batch currently resident on the device */
    float* d_loss;                   /* device scalar */
    float* d_gnorm;                  /* device scalar: sum of squares of all gradients */
    void* h_pinned; size_t h_pinned_bytes;   /* pinned staging for tokens/targets/seq_starts/loss */

    /* scratch shared by kernels (partials of deterministic reductions, sort tables) */
    void* scratch; size_t scratch_bytes;
    /* operand staging of the tensor-core GEMM (hi/lo, transposed copies) */
    void* gemm_stage[5]; size_t gemm_stage_bytes[5];
    /* rope cos/sin table */
    float* rope_tab; int rope_tab_pos, rope_tab_hd; float rope_tab_theta;

    /* data parallel */
    void* nccl_comm; int dp_rank, dp_world;
    void* nccl_comm_wide;            /* second communicator over the same ranks without the CTA cap, for the step's last bucket (NULL: none) */
    int dp_ctas;                     /* CTA cap of the communicator (0: NCCL's own choice) */
    int gemm_reserve_sms;            /* SMs the persistent GEMM grids leave free: set while gradient buckets are being reduced */
    int dp_timeout_ms;               /* host-side limit for a step's collectives (SERAPH_B200_DP_TIMEOUT_MS, default 120 s) */
    void* comm_stream; void* ev_bucket[64]; int n_buckets;
    void* side_stream[4]; void* side_ev[5]; int side_ready;   /* side streams of the attention path (sequences run side by side) */
    size_t bucket_begin[64], bucket_end[64];
} sb_ctx_t;

static inline sb_ctx_t* sb_priv(cuda_train_context_t* c) {
    sb_ctx_t* p = (sb_ctx_t*)c;
    return (p && p->magic == SB_MAGIC) ? p : (sb_ctx_t*)0;
}

/* ---- helpers (context.cu) ---- */
void* sb_scratch(sb_ctx_t* c, size_t bytes);                 /* grow-only device scratch; NULL on failure */
void* sb_gemm_stage(sb_ctx_t* c, int slot, size_t bytes);
int   sb_check(sb_ctx_t* c, int cuda_err, const char* what); /* records + prints, returns nonzero on error */
void  sb_set_status(sb_ctx_t* c, int st);

/* per-class timer: returns a slot (or -1 when timing is off) */
int  sb_tick_begin(sb_ctx_t* c, int cls);
void sb_tick_end(sb_ctx_t* c, int slot, double flops, double bytes);

/* ---- kernel launchers (raw pointers) ---- */
void sb_embed_lookup(sb_ctx_t*, const uint32_t* tok, const float* E, float* out, int T, int d, int V);
void sb_rmsnorm(sb_ctx_t*, const float* x, const float* w, float* y, int rows, int cols, float eps);
/* dx = rmsnorm'(x; dy); if resid != NULL, dx_out = resid + dx (fused residual-gradient add) */
void sb_qk_norm(sb_ctx_t*, float* x, float* rms_out, int rows, int cols, float eps);
void sb_qk_norm_backward(sb_ctx_t*, const float* y, const float* rms, const float* dy, float* dx, int rows, int cols, float eps);
void sb_rmsnorm_backward(sb_ctx_t*, const float* x, const float* w, const float* dy, const float* resid,
                         float* dx_out, float* dscale, int rows, int cols, float eps);
void sb_add(sb_ctx_t*, const float* a, const float* b, float* c, size_t n);
void sb_mul(sb_ctx_t*, const float* a, const float* b, float* c, size_t n);
void sb_scale(sb_ctx_t*, float* a, size_t n, float alpha);
void sb_silu(sb_ctx_t*, const float* x, float* y, size_t n);
void sb_softmax(sb_ctx_t*, const float* x, float* y, int rows, int cols);
void sb_silu_backward(sb_ctx_t*, const float* x, const float* dy, float* dx, size_t n);
void sb_mul_backward(sb_ctx_t*, const float* A, const float* B, const float* dC, float* dA, float* dB, size_t n);
void sb_swiglu(sb_ctx_t*, const float* gate, const float* up, float* out, size_t n);
void sb_swiglu_backward(sb_ctx_t*, const float* gate, const float* up, const float* dout, float* dgate, float* dup, size_t n);
/* The same two, writing `out` (dgate, dup) only as the FP16 parts of registered tensors, scaled by bounds formed from the largest
   magnitudes their producers left for the inputs; 1 = done, 0 = not possible here (no parts, no hints): call the plain one */
int  sb_swiglu_parts(sb_ctx_t*, const float* gate, const float* up, float* out, size_t n);
int  sb_rmsnorm_parts(sb_ctx_t*, const float* x, const float* w, float* y, int rows, int cols, float eps);      /* bound: sqrt(cols) max|w| */
int  sb_swiglu_backward_parts(sb_ctx_t*, const float* gate, const float* up, const float* dout, float* dgate, float* dup, size_t n);
void sb_amax_forget(sb_ctx_t*, const float* x);      /* x is written by something that leaves no maximum: earlier hints for it are void */
void sb_seq_index(sb_ctx_t*, const uint32_t* seq_starts, int B, int T, uint32_t* pos_ids, uint32_t* seq_ids);
/* Between begin and end the FP16 parts of GEMM operands are kept and reused by later calls on the same array; the caller
 * guarantees that no operand array is written inside the region. */
int sb_ensure_full_model(sb_ctx_t*, const train_state_t* st);
void sb_gemm_keep_begin(sb_ctx_t*);
void sb_gemm_keep_end(sb_ctx_t*);
void sb_gemm_keep_forget(sb_ctx_t*, const float* p);      /* p is about to be rewritten inside the region */
/* step-scoped FP16 parts of registered tensors: kind 0 = weights, 1 = saved activations */
void sb_parts_register(sb_ctx_t*, int kind, const float* p, size_t n);
void sb_parts_unregister(sb_ctx_t*, int kind);
void sb_parts_open(sb_ctx_t*);
void sb_parts_close(sb_ctx_t*);
void sb_parts_free(sb_ctx_t*);
/* sb_amax_announce: the next kernel that writes out[n] should leave max |out| behind (step driver).  sb_amax_take: called by that
   kernel's launcher with its output; returns the zeroed device word to raise with atomicMax on float bits, or NULL.
   sb_amax_lookup: the word of the latest producer of x[n] in this step, or NULL. */
void sb_amax_announce(sb_ctx_t*, const float* out, size_t n);
unsigned* sb_amax_take(sb_ctx_t*, const float* out, size_t n);
float* sb_amax_lookup(sb_ctx_t*, const float* x, size_t n);
void sb_parts_set_amax(sb_ctx_t*, const float* x, float* word);
/* 1: x[n] is registered and the step is open; *h = its two parts (h, h + n), *amax its scale word, *fresh = parts must be made now */
int sb_parts_find(sb_ctx_t*, const float* x, size_t n, void** h, float** amax, int* fresh);
void sb_parts_invalidate(sb_ctx_t*, const float* x);      /* x is rewritten as plain FP32: parts held for it are stale */
void sb_rope2(sb_ctx_t*, float* q, float* k, const uint32_t* pos_ids, int T, int Hq, int Hkv, int hd, float theta, int max_pos, int backward);
void sb_rope(sb_ctx_t*, const float* in, float* out, const uint32_t* pos_ids, int T, int H, int hd, float theta,
             int max_pos, int backward);
void sb_attention(sb_ctx_t*, const float* Q, const float* K, const float* V, float* out, float* lse,
                  const uint32_t* seq_starts_dev, const uint32_t* seq_ids, int T, int Hq, int Hkv, int hd);
void sb_attention_backward(sb_ctx_t*, const float* Q, const float* K, const float* V, const float* O, const float* lse,
                           const float* dO, float* dQ, float* dK, float* dV, int accumulate_kv,
                           const uint32_t* seq_starts_dev, const uint32_t* seq_ids, int B, int T, int Hq, int Hkv, int hd);
void sb_cross_entropy(sb_ctx_t*, const float* logits, const uint32_t* targets, float* grad, float* loss_rows,
                      const uint32_t* pos_ids, const uint32_t* seq_ids, const uint32_t* seq_starts,
                      int T, int V, int num_valid);
int  sb_cross_entropy_parts(sb_ctx_t*, const float* logits, const uint32_t* targets, float* grad, float* loss_rows,
                            const uint32_t* pos_ids, const uint32_t* seq_ids, const uint32_t* seq_starts, int T, int V, int num_valid);
void sb_reduce_sum(sb_ctx_t*, const float* in, float* out, size_t n);          /* deterministic; out[0] = sum */
void sb_embedding_backward(sb_ctx_t*, const uint32_t* tok, const float* g, float* dE, int T, int d, int V);
void sb_adamw(sb_ctx_t*, float* w, const float* g, float* m, float* v, size_t n, float lr, float b1, float b2,
              float wd, float eps, int step, float grad_scale, const float* d_sumsq, float clip);
void sb_sumsq(sb_ctx_t*, const float* g, size_t n, float* d_out);               /* deterministic sum of squares */
void sb_nan_check(sb_ctx_t*, const float* x, size_t n, uint32_t* flags, uint32_t idx);
/* C[M,N] (+)= op(A) op(B); same semantics as the reference's matmul_dispatch */
void sb_gemm(sb_ctx_t*, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc);
int  sb_gemm_reads_f16_parts(sb_ctx_t*, int M, int N, int K, int tA, int tB);      /* 1: that product takes prepared FP16 parts of its operands */
void sb_gemm_simt(sb_ctx_t*, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc);
/* returns 0 if the tensor-core path took the call, nonzero if the shape is not eligible */
int  sb_gemm_tc(sb_ctx_t*, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc, int mode);
void sb_lora_backward(sb_ctx_t*, const float* dY, const float* X, const float* A, const float* B, float* gA, float* gB,
                      float* tmp, int T, int in, int out, int r, float s);
void sb_memset(sb_ctx_t*, void* p, int byte, size_t bytes);
void sb_copy(sb_ctx_t*, void* dst, const void* src, size_t bytes);

/* host copy of the sequence boundaries of the batch the index tables describe */
int  sb_set_host_seq(sb_ctx_t* c, const int* starts, int B);
/* tensor-core attention (attention_tc.cu); nonzero = not eligible, caller uses the CUDA-core kernels */
int  sb_attention_fused_forward(sb_ctx_t*, const void* q1, const void* q2, const void* k1, const void* k2, const void* v1, const void* v2,
                                const float* amax_q, const float* amax_k, const float* amax_v, float* O, float* lse, int T, int Hq, int Hkv, int hd);
int  sb_attention_fused_scores(sb_ctx_t*, const void* q1, const void* q2, const void* do1, const void* do2, const void* k1, const void* k2,
                               const void* v1, const void* v2, const float* amax_q, const float* amax_k, const float* amax_v, const float* amax_do,
                               const float* ds_bound, const float* lse, const float* D, void* P1, void* P2, void* dS1, void* dS2,
                               int t0, int S, int Sp, int T, int Hq, int Hkv, int hd, int head0, int head_step, int nb);
int  sb_attention_fused_dkv(sb_ctx_t*, const void* q1, const void* q2, const void* do1, const void* do2, const void* k1, const void* k2,
                            const void* v1, const void* v2, const float* amax_q, const float* amax_k, const float* amax_v, const float* amax_do,
                            const float* ds_bound, const float* lse, const float* D, void* dS1, void* dS2, float* lse_rows, float* d_rows, float* dK, float* dV,
                            int Sp, int T, int Hq, int Hkv, int hd);     /* lse_rows, d_rows: scratch of sequences x Hq x Sp floats each */
int  sb_attention_tc_forward(sb_ctx_t*, const float* Q, const float* K, const float* V, float* O, float* lse, int T, int Hq, int Hkv, int hd);
int  sb_attention_tc_backward(sb_ctx_t*, const float* Q, const float* K, const float* V, const float* O, const float* lse, const float* dO,
                              float* dQ, float* dK, float* dV, int accumulate_kv, int T, int Hq, int Hkv, int hd);

/* profiler hooks used around launches */
int  sb_prof_begin(sb_ctx_t*, const char* name);
void sb_prof_end(sb_ctx_t*, int op, size_t flops, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif

#ifdef __CUDACC__
/* Largest magnitude seen by a CTA (each thread passes its own maximum, >= 0) raised into *out with an integer atomicMax on the
   float bits; every thread of the CTA must call it, CTAs of at most 1024 threads.  out == NULL: nothing happens. */
static __device__ __forceinline__ void sb_block_amax(float v, unsigned* out) {
    if (!out) return;
    __shared__ float sb_amax_red[32];
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sb_amax_red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nw ? sb_amax_red[lane] : 0.f;
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0 && v > 0.f) atomicMax(out, __float_as_uint(v));
    }
}
static __device__ __forceinline__ float sb_amax4(float m, float4 v) {
    return fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
}
/* FP16 operand parts: an operand whose largest magnitude (or a bound of it) is `amax` is scaled by 2^s with amax 2^s in
   [2^14, 2^15) (s = 0 for an all-zero operand) and every scaled value x is stored as hi = fp16(x), lo = fp16(x - hi).  Both parts
   are floating point, so a bound that is loose by 2^k only moves the few values below 2^-(18-k) of the largest into fp16's
   subnormal range; the bound must be a true upper bound, or hi overflows. */
static __device__ __forceinline__ int sb_f16_shift(float amax) {
    const int e = (int)((__float_as_uint(amax) >> 23) & 255u) - 127;
    if (amax == 0.f || e < -100) return 0;
    const int sh = 14 - e;
    return sh < -100 ? -100 : (sh > 100 ? 100 : sh);
}
static __device__ __forceinline__ float sb_pow2(int sh) { return __uint_as_float((unsigned)(127 + sh) << 23); }
/* two scaled values as packed parts (x0 in the low half); x - hi by the mixed-precision fma hi * -1 + x, exact */
static __device__ __forceinline__ void sb_split2(float x0, float x1, unsigned& hi, unsigned& lo) {
    asm("{\n\t.reg .b16 h0, h1, m1;\n\t.reg .f32 l0, l1;\n\t"
        "cvt.rn.f16x2.f32 %0, %3, %2;\n\t"
        "mov.b32 {h0, h1}, %0;\n\t"
        "mov.b16 m1, 0xBC00;\n\t"
        "fma.rn.f32.f16 l0, h0, m1, %2;\n\t"
        "fma.rn.f32.f16 l1, h1, m1, %3;\n\t"
        "cvt.rn.f16x2.f32 %1, l1, l0;\n\t}"
        : "=&r"(hi), "=r"(lo) : "f"(x0), "f"(x1));
}
#endif
