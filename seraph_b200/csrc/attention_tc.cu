// attention_tc.cu - causal attention forward and backward on the tcgen05 GEMM kernel.
//
// FP32-accurate attention does not fit one SM's on-chip memory as a single fused kernel at
// head_dim 128 (every operand needs a hi and a lo copy, and five products share them), so the
// score-sized matrices of a few heads at a time go through a scratch area that is sized to
// stay resident in the 126 MB L2; the five contractions run on the tensor cores with TMA-staged
// operand tiles, whole tiles above the causal diagonal are skipped, and the k range of the
// products with P or dS is cut at the diagonal.  Per sequence and per group of G heads:
//
//   forward    S = Q K^T  ->  rows: p = exp(s*scale - lse), lse kept  ->  O = P V
//   backward   query-major:  S = Q K^T, dP = dO V^T  ->  dS = P o (dP - D) * scale  ->  dQ = dS K
//              key-major:    S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO, dK += dS^T Q
//   (P is recomputed from the forward's log-sum-exp, nothing score-sized is kept between passes;
//    D[t,h] = sum_d dO*O.)  dK/dV of a GQA group are accumulated head after head in stream
//   order, so results are bit-reproducible.
//
// Reference kernels replaced: src/cuda_train_context.cu batch_attention[_packed] :712/:921,
// flash_attention_fwd[_packed] :1145/:1289, batch_attention_backward[_packed] :792/:1013,
// flash_attention_bwd[_packed] :1859/:2012.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include "gemm_tc.cuh"

#define AT_ROWTILE 128
#define AT_SCRATCH_BUDGET (512.0 * 1024 * 1024)   // causal part of the score scratch per launch; measured: fewer, larger launches beat L2 residency

static inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

__device__ __forceinline__ float warp_sum_f(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }
__device__ __forceinline__ float warp_max_f(float v) { for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }

// Forward rows: S[i][q][0..q] (raw dot products) -> P hi (in place) and P lo, normalised; lse written.
// Columns (q, end of q's 128-row tile) are zeroed: the P V product reads them.
__global__ void __launch_bounds__(256) at_softmax_rows(float* __restrict__ Sb, float* __restrict__ Plo, float* __restrict__ lse,
                                                       int S, int Sp, int Hq, int head0, int head_step, int tok0, float scale) {
    __shared__ float red[16];
    const int q = blockIdx.x, i = blockIdx.y, h = head0 + i * head_step;
    float* row = Sb + ((size_t)i * Sp + q) * Sp;
    float* lrow = Plo + ((size_t)i * Sp + q) * Sp;
    const int n = q + 1, zend = min(Sp, (q / AT_ROWTILE + 1) * AT_ROWTILE);
    float m = -INFINITY;
    for (int k = threadIdx.x; k < n; k += blockDim.x) m = fmaxf(m, row[k] * scale);
    m = warp_max_f(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
    float s = 0.f;
    for (int k = threadIdx.x; k < n; k += blockDim.x) s += expf(row[k] * scale - m);
    s = warp_sum_f(s);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[8 + (threadIdx.x >> 5)] = s;
    __syncthreads();
    s = 0.f;
    for (int w = 0; w < 8; w++) s += red[8 + w];
    const float L = m + logf(s);
    if (threadIdx.x == 0 && lse) lse[(size_t)(tok0 + q) * Hq + h] = L;
    for (int k = threadIdx.x; k < zend; k += blockDim.x) {
        float p = k < n ? expf(row[k] * scale - L) : 0.f;
        row[k] = p; lrow[k] = tf32_lo(p);
    }
}

// D[t,h] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (t,h)
__global__ void at_delta_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ D, int n_th, int hd) {
    int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= n_th) return;
    const float* a = dO + (size_t)w * hd; const float* b = O + (size_t)w * hd;
    float s = 0.f;
    for (int d = lane; d < hd; d += 32) s += a[d] * b[d];
    s = warp_sum_f(s);
    if (lane == 0) D[w] = s;
}

// Backward, query-major rows: S (buf_s) and dP (buf_dp) -> dS hi (into buf_dp) and dS lo (into buf_s)
__global__ void __launch_bounds__(256) at_ds_rows(float* __restrict__ buf_s, float* __restrict__ buf_dp, const float* __restrict__ lse,
                                                  const float* __restrict__ D, int S, int Sp, int Hq, int head0, int head_step,
                                                  int tok0, float scale) {
    const int q = blockIdx.x, i = blockIdx.y, h = head0 + i * head_step;
    float* srow = buf_s + ((size_t)i * Sp + q) * Sp;
    float* drow = buf_dp + ((size_t)i * Sp + q) * Sp;
    const float L = lse[(size_t)(tok0 + q) * Hq + h], Dq = D[(size_t)(tok0 + q) * Hq + h];
    const int zend = min(Sp, (q / AT_ROWTILE + 1) * AT_ROWTILE);
    for (int k = threadIdx.x; k < zend; k += blockDim.x) {
        float ds = 0.f;
        if (k <= q) { float p = expf(srow[k] * scale - L); ds = p * (drow[k] - Dq) * scale; }
        drow[k] = ds; srow[k] = tf32_lo(ds);
    }
}

// Backward, key-major rows: S^T (b0) and dP^T (b1), row = key k, column = query q >= k.
// Writes P^T hi -> b0, dS^T hi -> b1, P^T lo -> b2, dS^T lo -> b3; columns from the start of k's tile up to k-1 are zeroed.
__global__ void __launch_bounds__(256) at_pds_cols(float* __restrict__ b0, float* __restrict__ b1, float* __restrict__ b2, float* __restrict__ b3,
                                                   const float* __restrict__ lse, const float* __restrict__ D, int S, int Sp, int Hq,
                                                   int head0, int head_step, int tok0, float scale) {
    const int k = blockIdx.x, i = blockIdx.y, h = head0 + i * head_step;
    const size_t o = ((size_t)i * Sp + k) * Sp;
    const int q0 = (k / AT_ROWTILE) * AT_ROWTILE;
    for (int q = q0 + threadIdx.x; q < S; q += blockDim.x) {
        float p = 0.f, ds = 0.f;
        if (q >= k) {
            const float L = lse[(size_t)(tok0 + q) * Hq + h], Dq = D[(size_t)(tok0 + q) * Hq + h];
            p = expf(b0[o + q] * scale - L);
            ds = p * (b1[o + q] - Dq) * scale;
        }
        b0[o + q] = p; b2[o + q] = tf32_lo(p);
        b1[o + q] = ds; b3[o + q] = tf32_lo(ds);
    }
}

// ---------------------------------------------------------------------------------------------
struct AtPlan {
    int T, Hq, Hkv, hd, qd, kvd, g;
    const int* seq; int nseq;
};

static bool at_eligible(sb_ctx_t* c, int T, int Hq, int Hkv, int hd) {
    int mode = c->pub.use_bf16 ? SB_GEMM_BF16 : c->gemm_mode;
    if (mode == SB_GEMM_SIMT) return false;
    if (c->h_seq_n <= 0 || !c->h_seq) return false;
    if (hd % 4 || hd < 16 || hd > 256 || Hkv <= 0 || Hq % Hkv) return false;
    if (T < 128) return false;
    if (c->h_seq[c->h_seq_n] != T) return false;
    return tc_load_encode();
}

static TcOperand op_tokens(const float* hi, const float* lo, int tok0, int S, int row_pitch, int nheads, int hd, int slot_base, int slot_step) {
    TcOperand o;
    o.hi = hi + (size_t)tok0 * row_pitch; o.lo = lo ? lo + (size_t)tok0 * row_pitch : nullptr;
    o.mn = 0; o.rows = S; o.pitch = row_pitch; o.c2_dim = nheads; o.c2_stride = hd; o.c2_base = slot_base; o.c2_step = slot_step;
    return o;
}
static TcOperand op_scratch(const float* hi, const float* lo, int S, int Sp, int nb) {
    TcOperand o;
    o.hi = hi; o.lo = lo; o.mn = 0; o.rows = S; o.pitch = Sp; o.c2_dim = nb; o.c2_stride = (long)Sp * Sp; o.c2_base = 0; o.c2_step = 1;
    return o;
}
// transposed per-sequence copy X^T [nheads*hd rows][Sp]: rows of one head are hd consecutive rows
static TcOperand op_transposed(const float* hi, const float* lo, int S, int Sp, int nheads, int hd, int slot_base, int slot_step) {
    TcOperand o;
    o.hi = hi; o.lo = lo; o.mn = 0; o.rows = hd; o.pitch = Sp; o.c2_dim = nheads; o.c2_stride = (long)hd * Sp; o.c2_base = slot_base; o.c2_step = slot_step;
    return o;
}

static bool at_gemm(sb_ctx_t* c, const TcOperand& A, const TcOperand& B, float* C, long ldc, long cbs, int M, int N, int K,
                    int acc, int nb, int causal) {
    TcProblem p; p.A = A; p.B = B; p.C = C; p.ldc = ldc; p.c_batch_stride = cbs; p.M = M; p.N = N; p.K = K; p.acc = acc; p.nbatch = nb; p.causal = causal;
    return tc_launch(c, p, 3);
}

static void at_split(sb_ctx_t* c, const float* x, float* lo, size_t n) {
    split_lo_kernel<<<tc_ew_blocks(c, n / 4), 256, 0, (cudaStream_t)c->pub.stream>>>(x, lo, n / 4);
    c->launches++;
}
// X[tok0 .. tok0+S) x cols  ->  hi/lo [cols][Sp]
static void at_transpose(sb_ctx_t* c, const float* x, int tok0, int S, int cols, float* hi, float* lo, int Sp) {
    dim3 grid((cols + 31) / 32, (Sp + 31) / 32);
    transpose_split_kernel<<<grid, 256, 0, (cudaStream_t)c->pub.stream>>>(x + (size_t)tok0 * cols, hi, lo, S, cols, Sp, 1);
    c->launches++;
}

// heads per launch: as many as keep the causal part of their score scratch inside the budget
// (SERAPH_B200_ATTN_SCRATCH_MB overrides the default, which is sized to stay in L2)
static int at_group(int S_pad, int nbuf, int Hkv) {
    static double budget = 0;
    if (budget == 0) {
        const char* e = getenv("SERAPH_B200_ATTN_SCRATCH_MB");
        budget = (e && atof(e) > 0) ? atof(e) * 1024 * 1024 : AT_SCRATCH_BUDGET;
    }
    double per_head = (double)nbuf * S_pad * (double)S_pad * 4.0 * 0.55;
    int G = (int)(budget / per_head);
    if (G < 1) G = 1;
    if (G > Hkv) G = Hkv;
    return G;
}

extern "C" int sb_attention_tc_forward(sb_ctx_t* c, const float* Q, const float* K, const float* V, float* O, float* lse,
                                       int T, int Hq, int Hkv, int hd) {
    if (!at_eligible(c, T, Hq, Hkv, hd)) return 1;
    const int qd = Hq * hd, kvd = Hkv * hd, g = Hq / Hkv;
    const float scale = 1.0f / sqrtf((float)hd);
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    int Smax = 0;
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    const int Sp_max = round_up(Smax, 256), Spv = round_up(Smax, 4);
    const int G = at_group(Sp_max, 2, Hkv);
    // staging: lo parts of Q and K; V^T hi/lo of one sequence; score scratch
    size_t n_q = (size_t)T * qd, n_kv = (size_t)T * kvd, n_vt = (size_t)kvd * Spv, n_s = (size_t)G * Sp_max * Sp_max;
    float* st0 = (float*)sb_gemm_stage(c, 2, (n_q + n_kv + 2 * n_vt) * sizeof(float));
    float* st1 = (float*)sb_gemm_stage(c, 3, 2 * n_s * sizeof(float));
    if (!st0 || !st1) return 1;
    float *Qlo = st0, *Klo = Qlo + n_q, *Vt = Klo + n_kv, *Vtlo = Vt + n_vt;
    float *Sb = st1, *Plo = Sb + n_s;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_FWD);
    at_split(c, Q, Qlo, n_q);
    at_split(c, K, Klo, n_kv);
    bool ok = true;
    double flops = 0;
    for (int b = 0; b < c->h_seq_n && ok; b++) {
        const int t0 = c->h_seq[b], S = c->h_seq[b + 1] - t0;
        if (S <= 0) continue;
        const int Sp = Sp_max;                                          // one pitch for all sequences of the call
        at_transpose(c, V, t0, S, kvd, Vt, Vtlo, Spv);
        flops += 2.0 * Hq * (double)S * S * hd;
        for (int r = 0; r < g && ok; r++)
            for (int i0 = 0; i0 < Hkv && ok; i0 += G) {
                const int nb = min(G, Hkv - i0), qh0 = r + i0 * g;
                TcOperand Aq = op_tokens(Q, Qlo, t0, S, qd, Hq, hd, qh0, g);
                TcOperand Bk = op_tokens(K, Klo, t0, S, kvd, Hkv, hd, i0, 1);
                ok = ok && at_gemm(c, Aq, Bk, Sb, Sp, (long)Sp * Sp, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER);
                at_softmax_rows<<<dim3(S, nb), 256, 0, s>>>(Sb, Plo, lse, S, Sp, Hq, qh0, g, t0, scale);
                c->launches++;
                TcOperand Ap = op_scratch(Sb, Plo, S, Sp, nb);
                TcOperand Bv = op_transposed(Vt, Vtlo, S, Spv, Hkv, hd, i0, 1);
                Bv.rows = hd;
                ok = ok && at_gemm(c, Ap, Bv, O + (size_t)t0 * qd + (size_t)qh0 * hd, qd, (long)g * hd, S, hd, S, 0, nb, TC_CAUSAL_K_UPTO_M);
            }
    }
    sb_tick_end(c, tk, flops, 0.0);
    if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
    return 0;
}

extern "C" int sb_attention_tc_backward(sb_ctx_t* c, const float* Q, const float* K, const float* V, const float* O, const float* lse,
                                        const float* dO, float* dQ, float* dK, float* dV, int accumulate_kv,
                                        int T, int Hq, int Hkv, int hd) {
    if (!at_eligible(c, T, Hq, Hkv, hd)) return 1;
    const int qd = Hq * hd, kvd = Hkv * hd, g = Hq / Hkv;
    const float scale = 1.0f / sqrtf((float)hd);
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    int Smax = 0;
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    const int Sp = round_up(Smax, 256), Spt = round_up(Smax, 4);
    const int G = at_group(Sp, 4, Hkv);
    size_t n_q = (size_t)T * qd, n_kv = (size_t)T * kvd, n_s = (size_t)G * Sp * Sp;
    size_t n_qt = (size_t)qd * Spt, n_kt = (size_t)kvd * Spt;
    // lo parts: Q, K, V, dO;  D;  per-sequence transposes hi/lo: Q^T, dO^T, K^T
    size_t need0 = (2 * n_q + 2 * n_kv + (size_t)T * Hq + 4 * n_qt + 2 * n_kt + 64) * sizeof(float);
    float* st0 = (float*)sb_gemm_stage(c, 2, need0);
    float* st1 = (float*)sb_gemm_stage(c, 3, 4 * n_s * sizeof(float));
    if (!st0 || !st1) return 1;
    float *Qlo = st0, *dOlo = Qlo + n_q, *Klo = dOlo + n_q, *Vlo = Klo + n_kv, *D = Vlo + n_kv;
    float *Qt = D + (((size_t)T * Hq + 3) & ~(size_t)3), *Qtlo = Qt + n_qt, *dOt = Qtlo + n_qt, *dOtlo = dOt + n_qt, *Kt = dOtlo + n_qt, *Ktlo = Kt + n_kt;
    float *b0 = st1, *b1 = b0 + n_s, *b2 = b1 + n_s, *b3 = b2 + n_s;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_BWD);
    at_split(c, Q, Qlo, n_q); at_split(c, dO, dOlo, n_q); at_split(c, K, Klo, n_kv); at_split(c, V, Vlo, n_kv);
    at_delta_kernel<<<(T * Hq * 32 + 255) / 256, 256, 0, s>>>(dO, O, D, T * Hq, hd);
    c->launches++;
    bool ok = true;
    double flops = 0;
    for (int b = 0; b < c->h_seq_n && ok; b++) {
        const int t0 = c->h_seq[b], S = c->h_seq[b + 1] - t0;
        if (S <= 0) continue;
        flops += 5.0 * Hq * (double)S * S * hd;
        at_transpose(c, Q, t0, S, qd, Qt, Qtlo, Spt);
        at_transpose(c, dO, t0, S, qd, dOt, dOtlo, Spt);
        at_transpose(c, K, t0, S, kvd, Kt, Ktlo, Spt);
        for (int r = 0; r < g && ok; r++)
            for (int i0 = 0; i0 < Hkv && ok; i0 += G) {
                const int nb = min(G, Hkv - i0), qh0 = r + i0 * g;
                TcOperand q_tok = op_tokens(Q, Qlo, t0, S, qd, Hq, hd, qh0, g);
                TcOperand do_tok = op_tokens(dO, dOlo, t0, S, qd, Hq, hd, qh0, g);
                TcOperand k_tok = op_tokens(K, Klo, t0, S, kvd, Hkv, hd, i0, 1);
                TcOperand v_tok = op_tokens(V, Vlo, t0, S, kvd, Hkv, hd, i0, 1);
                const long sb = (long)Sp * Sp;
                // ---- query-major: dQ ----
                ok = ok && at_gemm(c, q_tok, k_tok, b0, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER);       // S
                ok = ok && at_gemm(c, do_tok, v_tok, b1, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER);      // dP
                at_ds_rows<<<dim3(S, nb), 256, 0, s>>>(b0, b1, lse, D, S, Sp, Hq, qh0, g, t0, scale);         // dS hi -> b1, lo -> b0
                c->launches++;
                {
                    TcOperand Ads = op_scratch(b1, b0, S, Sp, nb);
                    TcOperand Bkt = op_transposed(Kt, Ktlo, S, Spt, Hkv, hd, i0, 1);
                    ok = ok && at_gemm(c, Ads, Bkt, dQ + (size_t)t0 * qd + (size_t)qh0 * hd, qd, (long)g * hd, S, hd, S, 0, nb, TC_CAUSAL_K_UPTO_M);
                }
                // ---- key-major: dV, dK ----
                ok = ok && at_gemm(c, k_tok, q_tok, b0, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_LOWER);       // S^T
                ok = ok && at_gemm(c, v_tok, do_tok, b1, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_LOWER);      // dP^T
                at_pds_cols<<<dim3(S, nb), 256, 0, s>>>(b0, b1, b2, b3, lse, D, S, Sp, Hq, qh0, g, t0, scale);
                c->launches++;
                {
                    const int acc = (r > 0 || accumulate_kv) ? 1 : 0;
                    TcOperand Ap = op_scratch(b0, b2, S, Sp, nb), Ads = op_scratch(b1, b3, S, Sp, nb);
                    TcOperand Bdot = op_transposed(dOt, dOtlo, S, Spt, Hq, hd, qh0, g);
                    TcOperand Bqt = op_transposed(Qt, Qtlo, S, Spt, Hq, hd, qh0, g);
                    float* dv = dV + (size_t)t0 * kvd + (size_t)i0 * hd; float* dk = dK + (size_t)t0 * kvd + (size_t)i0 * hd;
                    ok = ok && at_gemm(c, Ap, Bdot, dv, kvd, hd, S, hd, S, acc, nb, TC_CAUSAL_K_FROM_M);
                    ok = ok && at_gemm(c, Ads, Bqt, dk, kvd, hd, S, hd, S, acc, nb, TC_CAUSAL_K_FROM_M);
                }
            }
    }
    sb_tick_end(c, tk, flops, 0.0);
    if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
    return 0;
}
