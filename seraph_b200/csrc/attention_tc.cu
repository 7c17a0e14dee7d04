// attention_tc.cu - causal attention forward and backward on the tcgen05 GEMM kernel.
//
// The general path (any head size that is a multiple of 4, either FP32-accurate mode).  For 128-wide heads in the
// default mode the forward pass and the backward's score products run in the fused kernels of attention_fused.cu
// instead; the drivers below choose, prepare the operand parts for both, and run the backward's three long products.
// FP32-accurate attention does not fit one SM's on-chip memory as a single fused kernel at
// head_dim 128 (every operand needs a hi and a lo part, and five products share them), so here the
// score-sized matrices of a few heads at a time go through a scratch area; the five contractions
// run on the tensor cores (CTA-pair kernel: operands taken as they lie in memory, lo parts made in
// the kernel), whole tiles above the causal diagonal are skipped, and the k range of the products
// with P or dS is cut at the diagonal.  Per sequence and per group of G heads:
//
//   forward    S = Q K^T  ->  rows: p = exp(s*scale - lse), lse kept  ->  O = P V
//   backward   S = Q K^T, dP = dO V^T  ->  P, dS = P o (dP - D) * scale
//              ->  dQ = dS K,  dV += P^T dO,  dK += dS^T Q
//   (P is recomputed from the forward's log-sum-exp, nothing score-sized is kept between passes;
//    D[t,h] = sum_d dO*O.)  V, K, Q and dO enter the last four products as [token, head_dim]
//   matrices read MN-major in place, P and dS enter dV and dK transposed the same way, so nothing
//   is transposed or copied.  dK/dV of a GQA group are accumulated head after head in stream
//   order, so results are bit-reproducible.
//
// Reference kernels replaced: src/cuda_train_context.cu batch_attention[_packed] :712/:921,
// flash_attention_fwd[_packed] :1145/:1289, batch_attention_backward[_packed] :792/:1013,
// flash_attention_bwd[_packed] :1859/:2012.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include "gemm_tc.cuh"

#define AT_ROWTILE 256                            // rows of a CTA pair's tile: P and dS are zeroed up to this boundary past the diagonal
#define AT_ALL_SCORES_BYTES ((size_t)0)           // > 0: the backward scores of all sequences and heads in one launch when their parts fit this many bytes
                                                  // (measured slower than a launch per sequence and head group, whose idle SMs the long products of other sequences fill)
#define AT_SCRATCH_BUDGET (512.0 * 1024 * 1024)   // causal part of the score scratch per launch; measured: fewer, larger launches beat L2 residency

static inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

__device__ __forceinline__ float warp_sum_f(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }
__device__ __forceinline__ float warp_max_f(float v) { for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }

// Forward rows: S[i][q][0..q] (raw dot products) -> P (in place), normalised; lse written.
// Columns (q, end of q's row tile) are zeroed: the P V product reads them.  A row of up to
// 256*AT_SM_REGS scores is read once and kept in registers; longer rows are read three times.
#define AT_SM_REGS 16
__device__ __forceinline__ float at_block_max(float v, float* red) {
    v = warp_max_f(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
    __syncthreads();
    return m;
}
__device__ __forceinline__ float at_block_sum(float v, float* red) {
    v = warp_sum_f(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < 8; w++) s += red[w];
    __syncthreads();
    return s;
}
// x * 2^14 (P lies in [0, 1]) or x * sc as two FP16 parts: h1 = fp16(x'), h2 = fp16(x' - h1)
__device__ __forceinline__ void at_put_parts(__half* __restrict__ h1, __half* __restrict__ h2, size_t idx, float xs) {
    const __half a = __float2half_rn(xs);
    h1[idx] = a; h2[idx] = __float2half_rn(xs - __half2float(a));
}
#define AT_P_SCALE 16384.0f

// P1/P2 given: P is written as its two FP16 parts (scale 2^14) to those arrays instead of in place
__global__ void __launch_bounds__(256) at_softmax_rows(float* __restrict__ Sb, float* __restrict__ lse,
                                                       int S, int Sp, int Hq, int head0, int head_step, int tok0, float scale,
                                                       __half* __restrict__ P1, __half* __restrict__ P2) {
    __shared__ float red[8];
    const int q = blockIdx.x, i = blockIdx.y, h = head0 + i * head_step;
    float* row = Sb + ((size_t)i * Sp + q) * Sp;
    const size_t rbase = ((size_t)i * Sp + q) * Sp;
    const int n = q + 1, zend = min(Sp, (q / AT_ROWTILE + 1) * AT_ROWTILE);
    if (n <= 256 * AT_SM_REGS) {
        const int nj = (n + 255) >> 8, zj = (zend + 255) >> 8;      // passes of 256 columns that hold scores / that are written
        float v[AT_SM_REGS];
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < AT_SM_REGS; j++) {
            v[j] = -INFINITY;
            if (j < nj) {
                const int k = threadIdx.x + 256 * j;
                if (k < n) v[j] = row[k] * scale;
                m = fmaxf(m, v[j]);
            }
        }
        m = at_block_max(m, red);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < AT_SM_REGS; j++)
            if (j < nj) { v[j] = expf(v[j] - m); s += v[j]; }                               // exp(-inf) = 0 beyond the row
        s = at_block_sum(s, red);
        if (threadIdx.x == 0 && lse) lse[(size_t)(tok0 + q) * Hq + h] = m + logf(s);
        const float inv = 1.0f / s;
#pragma unroll
        for (int j = 0; j < AT_SM_REGS; j++)
            if (j < zj) {
                const int k = threadIdx.x + 256 * j;
                if (k < zend) {                                                             // 0 past the diagonal
                    const float pv = j < nj ? v[j] * inv : 0.f;
                    if (P1) at_put_parts(P1, P2, rbase + k, pv * AT_P_SCALE); else row[k] = pv;
                }
            }
        return;
    }
    float m = -INFINITY;
    for (int k = threadIdx.x; k < n; k += blockDim.x) m = fmaxf(m, row[k] * scale);
    m = at_block_max(m, red);
    float s = 0.f;
    for (int k = threadIdx.x; k < n; k += blockDim.x) s += expf(row[k] * scale - m);
    s = at_block_sum(s, red);
    const float L = m + logf(s);
    if (threadIdx.x == 0 && lse) lse[(size_t)(tok0 + q) * Hq + h] = L;
    for (int k = threadIdx.x; k < zend; k += blockDim.x) {
        const float pv = k < n ? expf(row[k] * scale - L) : 0.f;
        if (P1) at_put_parts(P1, P2, rbase + k, pv * AT_P_SCALE); else row[k] = pv;
    }
}

// Backward rows: S (buf_s) and dP (buf_dp) -> P (into buf_s) and dS (into buf_dp); zero past the diagonal up to the row tile's end
// P1..dS2 given: both are written as FP16 parts (P with scale 2^14, dS with the power of two that brings *ds_bound to [2^14, 2^15))
__global__ void __launch_bounds__(256) at_ds_rows(float* __restrict__ buf_s, float* __restrict__ buf_dp, const float* __restrict__ lse,
                                                  const float* __restrict__ D, int S, int Sp, int Hq, int head0, int head_step,
                                                  int tok0, float scale, __half* __restrict__ P1, __half* __restrict__ P2,
                                                  __half* __restrict__ dS1, __half* __restrict__ dS2, const float* __restrict__ ds_bound) {
    const int q = blockIdx.x, i = blockIdx.y, h = head0 + i * head_step;
    float* srow = buf_s + ((size_t)i * Sp + q) * Sp;
    float* drow = buf_dp + ((size_t)i * Sp + q) * Sp;
    const float L = lse[(size_t)(tok0 + q) * Hq + h], Dq = D[(size_t)(tok0 + q) * Hq + h];
    const int zend = min(Sp, (q / AT_ROWTILE + 1) * AT_ROWTILE);
    const size_t rbase = ((size_t)i * Sp + q) * Sp;
    const float dsc = P1 ? tc_pow2(tc_f16_shift(*ds_bound)) : 1.f;
    for (int k = threadIdx.x; k < zend; k += blockDim.x) {
        float p = 0.f, ds = 0.f;
        if (k <= q) { p = expf(srow[k] * scale - L); ds = p * (drow[k] - Dq) * scale; }
        if (P1) { at_put_parts(P1, P2, rbase + k, p * AT_P_SCALE); at_put_parts(dS1, dS2, rbase + k, ds * dsc); }
        else { srow[k] = p; drow[k] = ds; }
    }
}

// largest row norm of x[n_rows, hd] (one warp per row), as float bits through an integer atomicMax; out zeroed before
__global__ void at_rownorm_max_kernel(const float* __restrict__ x, int n_rows, int hd, unsigned* __restrict__ out) {
    const int lane = threadIdx.x & 31, nwarps = (gridDim.x * blockDim.x) >> 5;
    int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    float best = 0.f;
    if (hd == 128) {
        // four rows of 32 float4 per pass and warp, all loads in flight together
        for (int r0 = w * 4; r0 < n_rows; r0 += nwarps * 4) {
            float s[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s[i] = 0.f;
                if (r0 + i < n_rows) {
                    const float4 v = __ldg((const float4*)(x + (size_t)(r0 + i) * 128) + lane);
                    s[i] = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) best = fmaxf(best, warp_sum_f(s[i]));
        }
    } else {
        for (; w < n_rows; w += nwarps) {
            const float* a = x + (size_t)w * hd;
            float s = 0.f;
            for (int d = lane; d < hd; d += 32) s += a[d] * a[d];
            best = fmaxf(best, warp_sum_f(s));
        }
    }
    if (lane == 0 && best > 0.f) atomicMax(out, __float_as_uint(sqrtf(best)));
}
static inline int at_rn_blocks(sb_ctx_t* c, int n_rows) {
    const int want = (n_rows + 31) / 32;                      // 8 warps x 4 rows per pass
    const int cap = c->pub.gpu_sm_count * 8;
    return want < 1 ? 1 : (want < cap ? want : cap);
}
// consts[0] = 1 (the largest possible P); consts[1] = 2 * max|dO row| * max|V row| * scale >= |dS| everywhere:
// |dP| = |dO_q . V_k| <= the product of the norms, D_q is a convex combination of the dP_qk, P <= 1
__global__ void at_consts_kernel(float* consts, const float* norms, float scale) {
    consts[0] = 1.0f;
    consts[1] = 2.0f * norms[0] * norms[1] * scale;
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

// The same D for 128-wide heads, together with what the FP16 split of dO and the bound of dS need from the same rows:
// the largest |dO| (amax) and the largest row norm of dO (norm_max), both raised with integer atomicMax on the float
// bits (order-free; zeroed before).  One warp per four (t,h) rows, a float4 per lane and row.
__global__ void __launch_bounds__(256) at_bwd_prep128_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ D,
                                                             int n_th, unsigned* __restrict__ norm_max, unsigned* __restrict__ amax) {
    const int lane = threadIdx.x & 31, nwarps = (gridDim.x * blockDim.x) >> 5;
    float bn = 0.f, ba = 0.f;
    for (int r0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 4; r0 < n_th; r0 += nwarps * 4) {
        float d[4], n2[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            d[i] = 0.f; n2[i] = 0.f;
            if (r0 + i < n_th) {
                const float4 g = __ldg((const float4*)(dO + (size_t)(r0 + i) * 128) + lane);
                const float4 o = __ldg((const float4*)(O + (size_t)(r0 + i) * 128) + lane);
                d[i] = g.x * o.x + g.y * o.y + g.z * o.z + g.w * o.w;
                n2[i] = g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
                ba = sb_amax4(ba, g);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float ds = warp_sum_f(d[i]);
            bn = fmaxf(bn, warp_sum_f(n2[i]));
            if (lane == 0 && r0 + i < n_th) D[r0 + i] = ds;
        }
    }
    sb_block_amax(sqrtf(bn), norm_max);
    __syncthreads();
    sb_block_amax(ba, amax);
}

// ---------------------------------------------------------------------------------------------

// FP16 parts for the attention products: the default GEMM mode, head sizes that fill whole 32-element k blocks
static bool at_f16(sb_ctx_t* c, int hd) {
    int mode = c->pub.use_bf16 ? SB_GEMM_BF16 : c->gemm_mode;
    return mode == SB_GEMM_FP16X3 && (hd % 32) == 0 && !c->attn_fused;
}
static bool at_eligible(sb_ctx_t* c, int T, int Hq, int Hkv, int hd) {
    int mode = c->pub.use_bf16 ? SB_GEMM_BF16 : c->gemm_mode;
    if (mode == SB_GEMM_SIMT || !c->gemm_pair) return false;
    if (c->h_seq_n <= 0 || !c->h_seq) return false;
    if (hd % 4 || hd < 16 || hd > 256 || Hkv <= 0 || Hq % Hkv) return false;
    if (T < 128) return false;
    if (c->h_seq[c->h_seq_n] != T) return false;
    return tc_load_encode();
}

// FP16 parts of a token-major tensor (made once per attention call), or of a score matrix
struct AtParts { const __half* h1; const __half* h2; const float* amax; };
static const AtParts AT_NOPARTS = {nullptr, nullptr, nullptr};

// K-major view of [token, heads*hd] rows: rows = tokens of the sequence, k = the head's hd columns, slot = head
static TcOperand op_tokens(const float* x, const AtParts& pt, int tok0, int S, int row_pitch, int nheads, int hd, int slot_base, int slot_step) {
    TcOperand o;
    o.hi = x + (size_t)tok0 * row_pitch; o.lo = nullptr;
    o.h1 = pt.h1 ? pt.h1 + (size_t)tok0 * row_pitch : nullptr; o.h2 = pt.h2 ? pt.h2 + (size_t)tok0 * row_pitch : nullptr;
    o.mn = 0; o.rows = S; o.pitch = row_pitch; o.c2_dim = nheads; o.c2_stride = hd; o.c2_base = slot_base; o.c2_step = slot_step;
    return o;
}
// MN-major view of the same rows: k = tokens of the sequence, rows = the head's hd columns (contiguous), slot = head
static TcOperand op_tokens_mn(const float* x, const AtParts& pt, int tok0, int row_pitch, int nheads, int hd, int slot_base, int slot_step) {
    TcOperand o = op_tokens(x, pt, tok0, hd, row_pitch, nheads, hd, slot_base, slot_step);
    o.mn = 1;
    return o;
}
// score scratch [head][query][key]: K-major = rows are queries, k runs over keys; mn = rows are keys, k runs over queries
static TcOperand op_scratch(const float* x, const AtParts& pt, int S, int Sp, int nb, int mn) {
    TcOperand o;
    o.hi = x; o.lo = nullptr; o.h1 = pt.h1; o.h2 = pt.h2; o.mn = mn; o.rows = S; o.pitch = Sp; o.c2_dim = nb; o.c2_stride = (long)Sp * Sp; o.c2_base = 0; o.c2_step = 1;
    return o;
}

static bool at_gemm(sb_ctx_t* c, const TcOperand& A, const TcOperand& B, float* C, long ldc, long cbs, int M, int N, int K,
                    int acc, int nb, int causal, const TcEpi* epi = nullptr, const float* amax_a = nullptr, const float* amax_b = nullptr) {
    TcProblem p; p.A = A; p.B = B; p.C = C; p.ldc = ldc; p.c_batch_stride = cbs; p.M = M; p.N = N; p.K = K; p.acc = acc; p.nbatch = nb; p.causal = causal;
    if (epi) p.epi = *epi; else memset(&p.epi, 0, sizeof p.epi);
    p.amax_a = amax_a; p.amax_b = amax_b;
    return tc_launch(c, p, 3);
}
// FP16 parts of x[n] into h[0..n) and h[n..2n), its largest magnitude into *amax
static AtParts at_make_parts(sb_ctx_t* c, const float* x, size_t n, __half* h, float* amax, bool amax_known = false) {
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    void* kept; float* kept_amax; int fresh;
    if (sb_parts_find(c, x, n, &kept, &kept_amax, &fresh)) {          // q, k, v of a training step: made in the forward pass, read again here
        h = (__half*)kept; amax = kept_amax;
        if (!fresh) { AtParts p = {h, h + n, amax}; return p; }
    }
    const dim3 pg(tc_ew_blocks(c, n / 4), 1);
    float* left = sb_amax_lookup(c, x, n);                            // the kernel that wrote x may have left its largest magnitude
    if (left) { amax = left; sb_parts_set_amax(c, x, left); }
    else if (!amax_known) {
        cudaMemsetAsync(amax, 0, sizeof(float), st);
        tc_amax_kernel<<<pg, 256, 0, st>>>(x, n / 4, (unsigned*)amax, nullptr, 0, nullptr);
        c->launches++;
    }
    tc_split_f16_kernel<<<pg, 256, 0, st>>>(x, n / 4, h, h + n, amax, nullptr, 0, nullptr, nullptr, nullptr);
    c->launches++;
    AtParts p = {h, h + n, amax};
    return p;
}
// per-(token, head) vector (lse or D, laid out [token][Hq]) as seen by a launch over heads head0, head0+step, ...
static TcEpi at_epi(int mode, float scale, const float* vec, int tok0, int Hq, int head0, int head_step, const float* aux) {
    TcEpi e; e.mode = mode; e.scale = scale; e.vec = vec + (size_t)tok0 * Hq + head0; e.vec_row_stride = Hq; e.vec_batch_stride = head_step; e.aux = aux;
    return e;
}

// heads per launch: as many as keep the causal part of their score scratch inside the budget
// (SERAPH_B200_ATTN_SCRATCH_MB overrides the default)
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

// Sequences are independent, and each of their launches ends in a partly filled wave (causal tiles differ
// in length): up to four sequences run side by side on side streams, each with its own scratch slice, so
// the tails of one fill with the tiles of another.  Fork: the side streams wait for the work queued so far;
// join: the main stream waits for all of them.
#define AT_SIDE 4
static int at_fork(sb_ctx_t* c, int want) {
    if (want < 2) return 1;
    if (!c->side_ready) {
        for (int i = 0; i < AT_SIDE; i++) { cudaStream_t st; if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) return 1; c->side_stream[i] = st; }
        for (int i = 0; i < AT_SIDE + 1; i++) { cudaEvent_t e; if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return 1; c->side_ev[i] = e; }
        c->side_ready = 1;
    }
    const int ns = want < AT_SIDE ? want : AT_SIDE;
    cudaEventRecord((cudaEvent_t)c->side_ev[AT_SIDE], (cudaStream_t)c->pub.stream);
    for (int i = 0; i < ns; i++) cudaStreamWaitEvent((cudaStream_t)c->side_stream[i], (cudaEvent_t)c->side_ev[AT_SIDE], 0);
    return ns;
}
static void at_join(sb_ctx_t* c, int ns, void* main_stream) {
    c->pub.stream = main_stream;
    if (ns < 2) return;
    for (int i = 0; i < ns; i++) {
        cudaEventRecord((cudaEvent_t)c->side_ev[i], (cudaStream_t)c->side_stream[i]);
        cudaStreamWaitEvent((cudaStream_t)main_stream, (cudaEvent_t)c->side_ev[i], 0);
    }
}

extern "C" int sb_attention_tc_forward(sb_ctx_t* c, const float* Q, const float* K, const float* V, float* O, float* lse,
                                       int T, int Hq, int Hkv, int hd) {
    if (!at_eligible(c, T, Hq, Hkv, hd)) return 1;
    const int qd = Hq * hd, kvd = Hkv * hd, g = Hq / Hkv;
    const float scale = 1.0f / sqrtf((float)hd);
    int Smax = 0;
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    const int Sp = round_up(Smax, AT_ROWTILE);                       // one pitch for all sequences of the call
    // FP16 parts (the default GEMM mode): Q, K, V are split once here, P is written as parts by the softmax kernel
    const bool f16 = at_f16(c, hd);
    const int G = at_group(Sp, f16 ? 2 : 1, Hkv);
    const size_t n_s = (size_t)G * Sp * Sp;
    const size_t per_stream = f16 ? 2 * n_s : n_s;                   // floats: S, then (FP16) the two parts of P
    const bool one_kernel = f16 && c->attn_flash && hd == 128 && c->h_seq_n <= 240;      // no score scratch at all
    float* Sb0 = one_kernel ? nullptr : (float*)sb_gemm_stage(c, 3, AT_SIDE * per_stream * sizeof(float));
    if (!Sb0 && !one_kernel) return 1;
    const size_t n_q = (size_t)T * qd, n_kv = (size_t)T * kvd;
    AtParts pq = AT_NOPARTS, pk = AT_NOPARTS, pv = AT_NOPARTS;
    float* consts = nullptr;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_FWD);
    if (f16) {
        float* st0 = (float*)sb_gemm_stage(c, 2, (n_q + 2 * n_kv) * 2 * sizeof(__half) + 64 * sizeof(float));
        if (!st0) return 1;
        consts = st0;                                            // [0] 1.0, [1] dS bound, [2..] norms, [8..] amax of Q, K, V, dO
        __half* hb = (__half*)(st0 + 64);
        pq = at_make_parts(c, Q, n_q, hb, consts + 8);
        pk = at_make_parts(c, K, n_kv, hb + 2 * n_q, consts + 9);
        pv = at_make_parts(c, V, n_kv, hb + 2 * n_q + 2 * n_kv, consts + 10);
        if (one_kernel) {
            double fl = 0;
            for (int b = 0; b < c->h_seq_n; b++) { const double S = c->h_seq[b + 1] - c->h_seq[b]; fl += 2.0 * Hq * S * S * hd; }
            if (sb_attention_fused_forward(c, pq.h1, pq.h2, pk.h1, pk.h2, pv.h1, pv.h2, pq.amax, pk.amax, pv.amax, O, lse, T, Hq, Hkv, hd) == 0) {
                sb_tick_end(c, tk, fl, 0.0);
                return 0;
            }
            Sb0 = (float*)sb_gemm_stage(c, 3, AT_SIDE * per_stream * sizeof(float));
            if (!Sb0) { sb_tick_end(c, tk, 0.0, 0.0); return 1; }
        }
        at_consts_kernel<<<1, 1, 0, (cudaStream_t)c->pub.stream>>>(consts, consts + 2, scale);       // only consts[0] is used here
        c->launches++;
    }
    bool ok = true;
    double flops = 0;
    void* main_stream = c->pub.stream;
    const int ns = at_fork(c, c->h_seq_n);
    for (int b = 0; b < c->h_seq_n && ok; b++) {
        const int t0 = c->h_seq[b], S = c->h_seq[b + 1] - t0;
        if (S <= 0) continue;
        flops += 2.0 * Hq * (double)S * S * hd;
        if (ns > 1) c->pub.stream = c->side_stream[b % ns];
        cudaStream_t s = (cudaStream_t)c->pub.stream;
        float* Sb = Sb0 + (size_t)(b % ns) * per_stream;
        __half* P1 = f16 ? (__half*)(Sb + n_s) : nullptr; __half* P2 = f16 ? P1 + n_s : nullptr;
        const AtParts pp = {P1, P2, consts};
        for (int r = 0; r < g && ok; r++)
            for (int i0 = 0; i0 < Hkv && ok; i0 += G) {
                const int nb = min(G, Hkv - i0), qh0 = r + i0 * g;
                ok = ok && at_gemm(c, op_tokens(Q, pq, t0, S, qd, Hq, hd, qh0, g), op_tokens(K, pk, t0, S, kvd, Hkv, hd, i0, 1),
                                   Sb, Sp, (long)Sp * Sp, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER, nullptr, pq.amax, pk.amax);
                at_softmax_rows<<<dim3(S, nb), 256, 0, s>>>(Sb, lse, S, Sp, Hq, qh0, g, t0, scale, P1, P2);
                c->launches++;
                ok = ok && at_gemm(c, op_scratch(Sb, pp, S, Sp, nb, 0), op_tokens_mn(V, pv, t0, kvd, Hkv, hd, i0, 1),
                                   O + (size_t)t0 * qd + (size_t)qh0 * hd, qd, (long)g * hd, S, hd, S, 0, nb, TC_CAUSAL_K_UPTO_M,
                                   nullptr, f16 ? consts : nullptr, pv.amax);
            }
    }
    at_join(c, ns, main_stream);
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
    int Smax = 0;
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    const int Sp = round_up(Smax, AT_ROWTILE);
    // FP16 parts (the default GEMM mode): Q, K, V, dO are split once here, P and dS are written as parts by at_ds_rows
    const bool f16 = at_f16(c, hd);
    const int G = at_group(Sp, f16 ? 4 : 2, Hkv);
    const size_t n_s = (size_t)G * Sp * Sp;
    const size_t per_stream = f16 ? 4 * n_s : 2 * n_s;               // floats: S, dP, then (FP16) the parts of P and of dS
    const size_t n_q = (size_t)T * qd, n_kv = (size_t)T * kvd;
    const size_t d_floats = ((size_t)T * Hq + 63) & ~(size_t)63;
    float* st0 = (float*)sb_gemm_stage(c, 2, (d_floats + 64) * sizeof(float) + (f16 ? (2 * n_q + 2 * n_kv) * 2 * sizeof(__half) : 0));
    // 128-wide heads, default mode: S, dP, P, dS of every sequence and head come from one launch that leaves only the FP16
    // parts of P and dS ([sequence][group member][K-V head][Sp][Sp], 8 bytes per score) when they fit the scratch limit
    const size_t n_all = (size_t)c->h_seq_n * Hq * Sp * Sp;
    size_t all_limit = AT_ALL_SCORES_BYTES;                          // SERAPH_B200_ATTN_ALL_SCORES_MB overrides (0, the default: one launch per sequence and head group)
    { const char* e = getenv("SERAPH_B200_ATTN_ALL_SCORES_MB"); if (e && e[0]) all_limit = (size_t)atol(e) << 20; }
    const bool all_scores = f16 && c->attn_flash && !c->attn_fused && hd == 128 && c->h_seq_n <= 240 && n_all * 8 <= all_limit;
    const size_t group_bytes = AT_SIDE * per_stream * sizeof(float);
    // 128-wide heads, default mode: dK and dV accumulate on chip in one launch over all sequences and K/V heads that leaves only
    // the FP16 parts of dS^T (4 bytes per score, [sequence][K-V head][group member][key][query]); dQ is then one product per
    // sequence over all its query heads.  seraph_b200_set_attn_flash(ctx, 2) or SERAPH_B200_ATTN_FLASH=2 selects the older
    // score-materialising path, 3 this one, for every shape.
    // attn_flash 1 (default) and 3 take this path (it measured faster at every shape tried: 16 % at 2048 tokens with two query heads
    // per K/V head, 30 % without head grouping)
    const bool dkv_fused = f16 && (c->attn_flash == 3 || c->attn_flash == 1) && !c->attn_fused && hd == 128 &&
                           c->h_seq_n <= 240 && !all_scores;
    size_t need = all_scores ? (n_all * 8 > group_bytes ? n_all * 8 : group_bytes) : group_bytes;
    const size_t n_rows = (size_t)c->h_seq_n * Hq * Sp;             // log-sum-exp and D by [sequence][head][query] for the on-chip kernel
    if (dkv_fused && n_all * 4 + 2 * n_rows * sizeof(float) > need) need = n_all * 4 + 2 * n_rows * sizeof(float);
    float* bb = (float*)sb_gemm_stage(c, 3, need);
    if (!st0 || !bb) return 1;
    float* D = st0;
    float* consts = st0 + d_floats;                                  // [0] 1.0, [1] dS bound, [2] max |dO row|, [3] max |V row|, [8..11] amax of Q, K, V, dO
    AtParts pq = AT_NOPARTS, pk = AT_NOPARTS, pv = AT_NOPARTS, pdo = AT_NOPARTS;
    cudaStream_t s0 = (cudaStream_t)c->pub.stream;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_BWD);
    const bool prep128 = f16 && hd == 128 && tc_aligned16(dO) && tc_aligned16(O);      // D, max |dO| and its largest row norm in one pass
    if (prep128) {
        cudaMemsetAsync(consts + 2, 0, 10 * sizeof(float), s0);
        at_bwd_prep128_kernel<<<at_rn_blocks(c, T * Hq), 256, 0, s0>>>(dO, O, D, T * Hq, (unsigned*)(consts + 2), (unsigned*)(consts + 11));
    } else
    at_delta_kernel<<<(T * Hq * 32 + 255) / 256, 256, 0, s0>>>(dO, O, D, T * Hq, hd);
    c->launches++;
    if (f16) {
        __half* hb = (__half*)(consts + 64);
        pq = at_make_parts(c, Q, n_q, hb, consts + 8);
        pk = at_make_parts(c, K, n_kv, hb + 2 * n_q, consts + 9);
        pv = at_make_parts(c, V, n_kv, hb + 2 * n_q + 2 * n_kv, consts + 10);
        pdo = at_make_parts(c, dO, n_q, hb + 2 * n_q + 4 * n_kv, consts + 11, prep128);
        if (!prep128) {
            cudaMemsetAsync(consts + 2, 0, 2 * sizeof(float), s0);
            at_rownorm_max_kernel<<<at_rn_blocks(c, T * Hq), 256, 0, s0>>>(dO, T * Hq, hd, (unsigned*)(consts + 2));
            c->launches++;
        }
        at_rownorm_max_kernel<<<at_rn_blocks(c, T * Hkv), 256, 0, s0>>>(V, T * Hkv, hd, (unsigned*)(consts + 3));
        at_consts_kernel<<<1, 1, 0, s0>>>(consts, consts + 2, scale);
        c->launches += 2;
    }
    bool ok = true;
    double flops = 0;
    void* main_stream = c->pub.stream;
    bool have_all = false;
    if (all_scores) {
        __half* a = (__half*)bb;
        have_all = sb_attention_fused_scores(c, pq.h1, pq.h2, pdo.h1, pdo.h2, pk.h1, pk.h2, pv.h1, pv.h2, pq.amax, pk.amax, pv.amax, pdo.amax,
                                             consts + 1, lse, D, a, a + n_all, a + 2 * n_all, a + 3 * n_all, 0, 0, Sp, T, Hq, Hkv, hd, 0, 0, 0) == 0;
    }
    if (dkv_fused) {
        __half* a = (__half*)bb;
        if (!accumulate_kv) {
            cudaMemsetAsync(dK, 0, n_kv * sizeof(float), s0);
            cudaMemsetAsync(dV, 0, n_kv * sizeof(float), s0);
        }
        if (sb_attention_fused_dkv(c, pq.h1, pq.h2, pdo.h1, pdo.h2, pk.h1, pk.h2, pv.h1, pv.h2, pq.amax, pk.amax, pv.amax, pdo.amax,
                                   consts + 1, lse, D, a, a + n_all, (float*)(a + 2 * n_all), (float*)(a + 2 * n_all) + n_rows, dK, dV, Sp, T, Hq, Hkv, hd) == 0) {
            const int ns2 = at_fork(c, c->h_seq_n);
            const long sb = (long)Sp * Sp;
            for (int b = 0; b < c->h_seq_n && ok; b++) {
                const int t0 = c->h_seq[b], S = c->h_seq[b + 1] - t0;
                if (S <= 0) continue;
                flops += 5.0 * Hq * (double)S * S * hd;
                if (ns2 > 1) c->pub.stream = c->side_stream[b % ns2];
                {
                    // all query heads of the sequence in one launch: head h reads slot b Hq + h of dS^T and K/V head h / g
                    __half* d1 = a + ((size_t)b * Hq) * (size_t)sb;
                    const AtParts pds = {d1, d1 + n_all, consts + 1};
                    TcOperand kop = op_tokens_mn(K, pk, t0, kvd, Hkv, hd, 0, 1);
                    kop.c2_div = g;
                    ok = ok && at_gemm(c, op_scratch(bb, pds, S, Sp, Hq, 1), kop, dQ + (size_t)t0 * qd, qd, (long)hd, S, hd, S, 0, Hq,
                                       TC_CAUSAL_K_UPTO_M, nullptr, pds.amax, pk.amax);                                       // dQ = dS K
                }
            }
            at_join(c, ns2, main_stream);
            sb_tick_end(c, tk, flops, 0.0);
            if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
            return 0;
        }
    }
    const int Gl = have_all ? Hkv : G;                               // K-V heads per launch of the long products
    const int ns = at_fork(c, c->h_seq_n);
    for (int b = 0; b < c->h_seq_n && ok; b++) {
        const int t0 = c->h_seq[b], S = c->h_seq[b + 1] - t0;
        if (S <= 0) continue;
        flops += 5.0 * Hq * (double)S * S * hd;
        if (ns > 1) c->pub.stream = c->side_stream[b % ns];
        cudaStream_t s = (cudaStream_t)c->pub.stream;
        float* b0 = have_all ? bb : bb + (size_t)(b % ns) * per_stream; float* b1 = have_all ? bb : b0 + n_s;
        for (int r = 0; r < g && ok; r++)
            for (int i0 = 0; i0 < Hkv && ok; i0 += Gl) {
                const int nb = min(Gl, Hkv - i0), qh0 = r + i0 * g;
                const long sb = (long)Sp * Sp;
                __half* P1 = f16 ? (__half*)(b0 + 2 * n_s) : nullptr; __half* P2 = f16 ? P1 + n_s : nullptr;
                __half* dS1 = f16 ? P2 + n_s : nullptr; __half* dS2 = f16 ? dS1 + n_s : nullptr;
                if (have_all) {
                    P1 = (__half*)bb + ((size_t)(b * g + r) * Hkv) * (size_t)sb; P2 = P1 + n_all; dS1 = P2 + n_all; dS2 = dS1 + n_all;
                }
                const AtParts pp = {P1, P2, consts}, pds = {dS1, dS2, f16 ? consts + 1 : nullptr};
                if (have_all) {
                    // scores already made
                } else if (c->attn_fused) {
                    // P = exp(S*scale - lse) and dS = P o (dP - D) * scale come straight out of the two products' epilogues (TF32 parts)
                    const TcEpi e_p = at_epi(TC_EPI_EXP, scale, lse, t0, Hq, qh0, g, nullptr);
                    const TcEpi e_ds = at_epi(TC_EPI_DS, scale, D, t0, Hq, qh0, g, b0);
                    ok = ok && at_gemm(c, op_tokens(Q, AT_NOPARTS, t0, S, qd, Hq, hd, qh0, g), op_tokens(K, AT_NOPARTS, t0, S, kvd, Hkv, hd, i0, 1),
                                       b0, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER, &e_p);                          // P
                    ok = ok && at_gemm(c, op_tokens(dO, AT_NOPARTS, t0, S, qd, Hq, hd, qh0, g), op_tokens(V, AT_NOPARTS, t0, S, kvd, Hkv, hd, i0, 1),
                                       b1, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER, &e_ds);                         // dS
                } else if (f16 && c->attn_flash && hd == 128 &&
                           sb_attention_fused_scores(c, pq.h1, pq.h2, pdo.h1, pdo.h2, pk.h1, pk.h2, pv.h1, pv.h2, pq.amax, pk.amax, pv.amax, pdo.amax,
                                                     consts + 1, lse, D, P1, P2, dS1, dS2, t0, S, Sp, T, Hq, Hkv, hd, qh0, g, nb) == 0) {
                    // S, dP, P and dS in one kernel: only the parts of P and dS reach memory
                } else {
                    ok = ok && at_gemm(c, op_tokens(Q, pq, t0, S, qd, Hq, hd, qh0, g), op_tokens(K, pk, t0, S, kvd, Hkv, hd, i0, 1),
                                       b0, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER, nullptr, pq.amax, pk.amax);     // S
                    ok = ok && at_gemm(c, op_tokens(dO, pdo, t0, S, qd, Hq, hd, qh0, g), op_tokens(V, pv, t0, S, kvd, Hkv, hd, i0, 1),
                                       b1, Sp, sb, S, S, hd, 0, nb, TC_CAUSAL_SKIP_UPPER, nullptr, pdo.amax, pv.amax);    // dP
                    at_ds_rows<<<dim3(S, nb), 256, 0, s>>>(b0, b1, lse, D, S, Sp, Hq, qh0, g, t0, scale, P1, P2, dS1, dS2, consts + 1);   // P, dS
                    c->launches++;
                }
                const int acc = (r > 0 || accumulate_kv) ? 1 : 0;
                ok = ok && at_gemm(c, op_scratch(b1, pds, S, Sp, nb, 0), op_tokens_mn(K, pk, t0, kvd, Hkv, hd, i0, 1),
                                   dQ + (size_t)t0 * qd + (size_t)qh0 * hd, qd, (long)g * hd, S, hd, S, 0, nb, TC_CAUSAL_K_UPTO_M,
                                   nullptr, pds.amax, pk.amax);                                                                       // dQ = dS K
                ok = ok && at_gemm(c, op_scratch(b0, pp, S, Sp, nb, 1), op_tokens_mn(dO, pdo, t0, qd, Hq, hd, qh0, g),
                                   dV + (size_t)t0 * kvd + (size_t)i0 * hd, kvd, hd, S, hd, S, acc, nb, TC_CAUSAL_K_FROM_M,
                                   nullptr, f16 ? consts : nullptr, pdo.amax);                                                        // dV += P^T dO
                ok = ok && at_gemm(c, op_scratch(b1, pds, S, Sp, nb, 1), op_tokens_mn(Q, pq, t0, qd, Hq, hd, qh0, g),
                                   dK + (size_t)t0 * kvd + (size_t)i0 * hd, kvd, hd, S, hd, S, acc, nb, TC_CAUSAL_K_FROM_M,
                                   nullptr, pds.amax, pq.amax);                                                                       // dK += dS^T Q
            }
    }
    at_join(c, ns, main_stream);
    sb_tick_end(c, tk, flops, 0.0);
    if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
    return 0;
}
