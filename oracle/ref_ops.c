/*
 * ref_ops.c - CPU restatement of Seraph's GPU training arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library,
 * never a code path of it: nothing in the product links or calls it.
 *
 * Every function restates, op for op, what the reference's CUDA backend
 * computes (reference file:line given at each function).  Storage is FP32 as
 * in the reference; sums are carried in double when ref_set_acc64(1) (the
 * default) so that the result is the "FP64-accumulate" value the FP32 GPU
 * kernels are compared with, and in float when ref_set_acc64(0) so that the
 * rounding gap of a plain FP32 implementation can be measured.
 *
 * Parity status: the reference ships no golden vectors for this path.  The
 * pins used instead are (1) the reference's own CPU forward/loss/AdamW/LoRA
 * code compiled from its sources (oracle/_ref) and (2) the reference's CUDA
 * backend run on a B200, whose outputs are committed under tests/golden.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static int g_acc64 = 1;
void ref_set_acc64(int on) { g_acc64 = on; }

/* dot product with the configured accumulator width; 8 partial sums so the
 * compiler can vectorise without -ffast-math */
static double dotp(const float* a, const float* b, long n, long sa, long sb) {
    if (g_acc64) {
        double acc[8] = {0};
        long i = 0;
        if (sa == 1 && sb == 1) {
            for (; i + 8 <= n; i += 8)
                for (int j = 0; j < 8; j++) acc[j] += (double)a[i + j] * (double)b[i + j];
        }
        double s = 0;
        for (; i < n; i++) s += (double)a[i * sa] * (double)b[i * sb];
        for (int j = 0; j < 8; j++) s += acc[j];
        return s;
    } else {
        float s = 0.f;
        for (long i = 0; i < n; i++) s += a[i * sa] * b[i * sb];
        return (double)s;
    }
}

/* which packed sequence a global row belongs to
 * (src/cuda_train_context.cu:641-650, find_seq_idx) */
static int seq_of(const uint32_t* ss, int B, int pos) {
    int lo = 0, hi = B;
    while (lo < hi) {
        int mid = (lo + hi) / 2;
        if ((int)ss[mid + 1] <= pos) lo = mid + 1; else hi = mid;
    }
    return lo;
}

/* src/cuda_train_context.cu:119-128 embed_lookup_kernel */
void ref_embed_lookup(const uint32_t* tok, const float* E, float* out, int T, int d) {
    for (int t = 0; t < T; t++)
        memcpy(out + (size_t)t * d, E + (size_t)tok[t] * d, (size_t)d * sizeof(float));
}

/* src/cuda_train_context.cu:148-204 rmsnorm_kernel */
void ref_rmsnorm(const float* x, const float* w, float* y, int rows, int cols, float eps) {
#pragma omp parallel for
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * cols;
        double ss = dotp(xr, xr, cols, 1, 1);
        if (g_acc64) {
            double inv = 1.0 / sqrt(ss / cols + (double)eps);
            for (int i = 0; i < cols; i++) y[(size_t)r * cols + i] = (float)(xr[i] * inv * w[i]);
        } else {
            float inv = 1.0f / sqrtf((float)ss / cols + eps);
            for (int i = 0; i < cols; i++) y[(size_t)r * cols + i] = xr[i] * inv * w[i];
        }
    }
}

/* src/cuda_train_context.cu:2645-2709 matmul_dispatch:
 *   tA=0,tB=0: C[M,N] = A[M,K] B[K,N]
 *   tA=1,tB=0: C[M,N] = A[K,M]^T B[K,N]
 *   tA=0,tB=1: C[M,N] = A[M,K] B[N,K]^T
 *   tA=1,tB=1 falls through to the first form, as the reference's dispatch does.
 *   acc: C += instead of C = */
void ref_matmul(const float* A, const float* B, float* C, int M, int N, int K,
                int tA, int tB, int acc) {
    long sa_m, sa_k, sb_k, sb_n;
    if (tA && !tB)      { sa_m = 1; sa_k = M; sb_k = N; sb_n = 1; }
    else if (!tA && tB) { sa_m = K; sa_k = 1; sb_k = 1; sb_n = K; }
    else                { sa_m = K; sa_k = 1; sb_k = N; sb_n = 1; }
    /* make B contiguous along k once so the inner loop streams */
    float* Bt = NULL;
    if (sb_k != 1) {
        Bt = (float*)malloc((size_t)N * K * sizeof(float));
#pragma omp parallel for
        for (int n = 0; n < N; n++)
            for (int k = 0; k < K; k++) Bt[(size_t)n * K + k] = B[(size_t)k * sb_k + (size_t)n * sb_n];
    }
    float* At = NULL;
    if (sa_k != 1) {
        At = (float*)malloc((size_t)M * K * sizeof(float));
#pragma omp parallel for
        for (int m = 0; m < M; m++)
            for (int k = 0; k < K; k++) At[(size_t)m * K + k] = A[(size_t)k * sa_k + (size_t)m * sa_m];
    }
    const float* Ak = At ? At : A;
    const float* Bk = Bt ? Bt : B;
#pragma omp parallel for
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            double s = dotp(Ak + (size_t)m * K, Bk + (size_t)n * K, K, 1, 1);
            size_t o = (size_t)m * N + n;
            if (acc) C[o] = g_acc64 ? (float)((double)C[o] + s) : C[o] + (float)s;
            else C[o] = (float)s;
        }
    }
    free(At); free(Bt);
}

/* src/cuda_train_context.cu:652-704 rope_packed_kernel / rope_backward_packed_kernel:
 * interleaved pairs (x[2i], x[2i+1]), angle = local_pos / theta^(2i/hd); the
 * backward applies the transposed rotation.  B=1 with ss={0,T} gives the
 * unpacked kernels (:616, :1831).  The angle is formed in FP32 exactly as the
 * kernels do (powf, then pos*freq) so cos/sin see the same argument. */
void ref_rope(const float* in, float* out, const uint32_t* ss, int T, int B, int H, int hd,
              float theta, int backward) {
#pragma omp parallel for
    for (int t = 0; t < T; t++) {
        int s = seq_of(ss, B, t);
        int lp = t - (int)ss[s];
        for (int h = 0; h < H; h++)
            for (int p = 0; p < hd / 2; p++) {
                size_t o = (size_t)t * H * hd + (size_t)h * hd + 2 * p;
                float freq = 1.0f / powf(theta, (float)(p * 2) / hd);
                float ang = lp * freq;
                double c = cos((double)ang), sn = sin((double)ang);
                double x0 = in[o], x1 = in[o + 1];
                if (!backward) { out[o] = (float)(x0 * c - x1 * sn); out[o + 1] = (float)(x0 * sn + x1 * c); }
                else           { out[o] = (float)(x0 * c + x1 * sn); out[o + 1] = (float)(-x0 * sn + x1 * c); }
            }
    }
}

/* src/cuda_train_context.cu:921-1011 batch_attention_packed_kernel (softmax form) and
 * :1289-1438 flash_attention_fwd_packed_kernel (lse[t*Hq+h] = max + log sum, :1435).
 * Causal inside each packed sequence; kv head = h*Hkv/Hq (:728); scale 1/sqrt(hd). */
void ref_attention(const float* Q, const float* K, const float* V, float* out, float* lse,
                   const uint32_t* ss, int T, int B, int Hq, int Hkv, int hd) {
    double scale = 1.0 / sqrt((double)hd);
    if (!g_acc64) scale = (double)(1.0f / sqrtf((float)hd));
#pragma omp parallel for collapse(2)
    for (int t = 0; t < T; t++)
        for (int h = 0; h < Hq; h++) {
            int s0 = (int)ss[seq_of(ss, B, t)];
            int kvh = h * Hkv / Hq;
            int n = t - s0 + 1;
            double* p = (double*)malloc((size_t)n * sizeof(double));
            const float* q = Q + (size_t)t * Hq * hd + (size_t)h * hd;
            double mx = -1e300;
            for (int j = 0; j < n; j++) {
                const float* k = K + (size_t)(s0 + j) * Hkv * hd + (size_t)kvh * hd;
                p[j] = dotp(q, k, hd, 1, 1) * scale;
                if (p[j] > mx) mx = p[j];
            }
            double sum = 0;
            for (int j = 0; j < n; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
            for (int d = 0; d < hd; d++) {
                double a = 0;
                for (int j = 0; j < n; j++)
                    a += p[j] * (double)V[(size_t)(s0 + j) * Hkv * hd + (size_t)kvh * hd + d];
                out[(size_t)t * Hq * hd + (size_t)h * hd + d] = (float)(a / sum);
            }
            if (lse) lse[(size_t)t * Hq + h] = (float)(mx + log(sum));
            free(p);
        }
}

/* src/cuda_train_context.cu:1013-1138 batch_attention_backward_packed_kernel and
 * :2012-2172 flash_attention_bwd_packed_kernel (same maths, P from lse).
 * dQ is written; dK and dV are accumulated into what the caller passes (the
 * reference zero-fills them first, src/train_cuda.c:2234-2237). */
void ref_attention_backward(const float* Q, const float* K, const float* V, const float* dO,
                            float* dQ, float* dK, float* dV,
                            const uint32_t* ss, int T, int B, int Hq, int Hkv, int hd) {
    double scale = 1.0 / sqrt((double)hd);
    size_t nkv = (size_t)T * Hkv * hd;
    double* aK = (double*)calloc(nkv, sizeof(double));
    double* aV = (double*)calloc(nkv, sizeof(double));
    /* parallel over kv heads so each thread owns its dK/dV slice */
#pragma omp parallel for
    for (int kvh = 0; kvh < Hkv; kvh++) {
        for (int h = 0; h < Hq; h++) {
            if (h * Hkv / Hq != kvh) continue;
            for (int t = 0; t < T; t++) {
                int s0 = (int)ss[seq_of(ss, B, t)];
                int n = t - s0 + 1;
                double* p = (double*)malloc((size_t)n * 2 * sizeof(double));
                double* dp = p + n;
                const float* q = Q + (size_t)t * Hq * hd + (size_t)h * hd;
                const float* g = dO + (size_t)t * Hq * hd + (size_t)h * hd;
                double mx = -1e300, sum = 0;
                for (int j = 0; j < n; j++) {
                    p[j] = dotp(q, K + (size_t)(s0 + j) * Hkv * hd + (size_t)kvh * hd, hd, 1, 1) * scale;
                    if (p[j] > mx) mx = p[j];
                }
                for (int j = 0; j < n; j++) { p[j] = exp(p[j] - mx); sum += p[j]; }
                double dsum = 0;
                for (int j = 0; j < n; j++) {
                    p[j] /= sum;
                    size_t kvo = (size_t)(s0 + j) * Hkv * hd + (size_t)kvh * hd;
                    dp[j] = dotp(g, V + kvo, hd, 1, 1);
                    for (int d = 0; d < hd; d++) aV[kvo + d] += p[j] * (double)g[d];
                    dsum += p[j] * dp[j];
                }
                double* dq = (double*)calloc((size_t)hd, sizeof(double));
                for (int j = 0; j < n; j++) {
                    double ds = p[j] * (dp[j] - dsum) * scale;
                    size_t kvo = (size_t)(s0 + j) * Hkv * hd + (size_t)kvh * hd;
                    for (int d = 0; d < hd; d++) {
                        dq[d] += ds * (double)K[kvo + d];
                        aK[kvo + d] += ds * (double)q[d];
                    }
                }
                for (int d = 0; d < hd; d++) dQ[(size_t)t * Hq * hd + (size_t)h * hd + d] = (float)dq[d];
                free(dq); free(p);
            }
        }
    }
    for (size_t i = 0; i < nkv; i++) { dK[i] = (float)((double)dK[i] + aK[i]); dV[i] = (float)((double)dV[i] + aV[i]); }
    free(aK); free(aV);
}

/* src/cuda_train_context.cu:1442-1475 add / silu / mul / scale kernels */
void ref_add(const float* a, const float* b, float* c, size_t n) { for (size_t i = 0; i < n; i++) c[i] = a[i] + b[i]; }
void ref_mul(const float* a, const float* b, float* c, size_t n) { for (size_t i = 0; i < n; i++) c[i] = a[i] * b[i]; }
void ref_scale(float* a, size_t n, float alpha) { for (size_t i = 0; i < n; i++) a[i] *= alpha; }
void ref_silu(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; i++)
        y[i] = g_acc64 ? (float)((double)x[i] / (1.0 + exp(-(double)x[i]))) : x[i] / (1.0f + expf(-x[i]));
}

/* src/cuda_train_context.cu:1486-1551 softmax_kernel */
void ref_softmax(const float* x, float* y, int rows, int cols) {
#pragma omp parallel for
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * cols;
        double mx = -1e300, sum = 0;
        for (int i = 0; i < cols; i++) if (xr[i] > mx) mx = xr[i];
        for (int i = 0; i < cols; i++) sum += exp((double)xr[i] - mx);
        for (int i = 0; i < cols; i++) y[(size_t)r * cols + i] = (float)(exp((double)xr[i] - mx) / sum);
    }
}

/* src/cuda_train_context.cu:1657-1741 cross_entropy_grad_packed_kernel.
 * The last token of each sequence predicts nothing: zero row, zero loss.
 * Otherwise loss = -log softmax[target], grad = (softmax - onehot)/num_valid.
 * With B=1, ss={0,rows+1} this is the unpacked kernel (:1566) on rows rows. */
void ref_cross_entropy_grad(const float* logits, const uint32_t* targets, float* grad, float* loss_rows,
                            const uint32_t* ss, int T, int B, int V, int num_valid) {
#pragma omp parallel for
    for (int r = 0; r < T; r++) {
        int s = seq_of(ss, B, r);
        int lp = r - (int)ss[s], sl = (int)ss[s + 1] - (int)ss[s];
        float* gr = grad + (size_t)r * V;
        const float* lr = logits + (size_t)r * V;
        if (lp >= sl - 1) { memset(gr, 0, (size_t)V * sizeof(float)); loss_rows[r] = 0.f; continue; }
        uint32_t tg = targets[r];
        double mx = -1e300, sum = 0;
        for (int i = 0; i < V; i++) if (lr[i] > mx) mx = lr[i];
        for (int i = 0; i < V; i++) sum += exp((double)lr[i] - mx);
        loss_rows[r] = (float)(-(((double)lr[tg] - mx) - log(sum)));
        for (int i = 0; i < V; i++) {
            double g = exp((double)lr[i] - mx) / sum;
            if ((uint32_t)i == tg) g -= 1.0;
            gr[i] = (float)(g / (double)num_valid);
        }
    }
}

/* src/cuda_train_context.cu:2209-2224 reduce_sum_kernel (+ host loop src/train_cuda.c:2168-2179) */
float ref_reduce_sum(const float* x, size_t n) {
    double s = 0; for (size_t i = 0; i < n; i++) s += x[i]; return (float)s;
}

/* src/cuda_train_context.cu:1744-1753 silu_backward_kernel */
void ref_silu_backward(const float* x, const float* dy, float* dx, size_t n) {
    for (size_t i = 0; i < n; i++) {
        double v = x[i], sg = 1.0 / (1.0 + exp(-v));
        dx[i] = (float)((double)dy[i] * (sg + v * sg * (1.0 - sg)));
    }
}

/* src/cuda_train_context.cu:1756-1764 elementwise_mul_backward_kernel */
void ref_mul_backward(const float* A, const float* Bm, const float* dC, float* dA, float* dB, size_t n) {
    for (size_t i = 0; i < n; i++) { float g = dC[i]; dA[i] = g * Bm[i]; dB[i] = g * A[i]; }
}

/* src/cuda_train_context.cu:1767-1828 rmsnorm_backward_kernel:
 *   inv = 1/sqrt(mean(x^2)+eps); dscale[i] += g*x*inv (accumulates);
 *   dx = g*s*inv - x*inv^3/cols * sum(g*s*x).
 * (The GLSL twin shaders/rmsnorm_backward_batch.comp clamps rms >= 0.01; the
 * CUDA backend, which is the parity target, does not.) */
void ref_rmsnorm_backward(const float* x, const float* scale, const float* dy, float* dx, float* dscale,
                          int rows, int cols, float eps) {
    double* acc = (double*)calloc((size_t)cols, sizeof(double));
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * cols;
        const float* gr = dy + (size_t)r * cols;
        double ssq = dotp(xr, xr, cols, 1, 1);
        double inv = 1.0 / sqrt(ssq / cols + (double)eps);
        double coupled = 0;
        for (int i = 0; i < cols; i++) coupled += (double)gr[i] * scale[i] * xr[i];
        double inv3 = inv * inv * inv;
        for (int i = 0; i < cols; i++) {
            acc[i] += (double)gr[i] * xr[i] * inv;
            dx[(size_t)r * cols + i] = (float)((double)gr[i] * scale[i] * inv - xr[i] * inv3 / cols * coupled);
        }
    }
    for (int i = 0; i < cols; i++) dscale[i] = (float)((double)dscale[i] + acc[i]);
    free(acc);
}

/* shaders/qk_norm.comp:30-76 (called on Q and on K after RoPE, src/train.c:4688-4689): every token row of
 * [seq_len, num_heads*head_dim] is divided by max(sqrt(mean(x^2)), eps), in place; use_qk_norm == 0 leaves it alone.
 * rms_out (may be NULL) receives the row's sqrt(mean(x^2)) before the clamp: what a backward pass needs, since the
 * in-place forward overwrites x. */
void ref_qk_norm(float* qk, float* rms_out, int seq_len, int num_heads, int head_dim, int use_qk_norm, float eps) {
    if (!use_qk_norm) return;
    int n = num_heads * head_dim;
    for (int t = 0; t < seq_len; t++) {
        float* r = qk + (size_t)t * n;
        double rms = sqrt(dotp(r, r, n, 1, 1) / n);
        if (rms_out) rms_out[t] = (float)rms;
        double inv = 1.0 / (rms > (double)eps ? rms : (double)eps);
        for (int i = 0; i < n; i++) r[i] = (float)(r[i] * inv);
    }
}

/* The reference has no backward for qk_norm (its training passes the gradient through unchanged).  This is the derivative of
 * the forward above: with y = x / r, r = sqrt(mean(x^2)) > eps:  dx = (dy - y * mean(dy o y)) / r;  with the clamp active
 * (r <= eps, y = x / eps):  dx = dy / eps.  y is the forward's output, rms its saved statistic. */
void ref_qk_norm_backward(const float* y, const float* rms, const float* dy, float* dx, int seq_len, int num_heads, int head_dim,
                          int use_qk_norm, float eps) {
    int n = num_heads * head_dim;
    for (int t = 0; t < seq_len; t++) {
        const float* yr = y + (size_t)t * n; const float* gr = dy + (size_t)t * n; float* o = dx + (size_t)t * n;
        if (!use_qk_norm) { for (int i = 0; i < n; i++) o[i] = gr[i]; continue; }
        if (!(rms[t] > eps)) { for (int i = 0; i < n; i++) o[i] = (float)((double)gr[i] / (double)eps); continue; }
        double m = dotp(gr, yr, n, 1, 1) / n, inv = 1.0 / (double)rms[t];
        for (int i = 0; i < n; i++) o[i] = (float)(((double)gr[i] - (double)yr[i] * m) * inv);
    }
}

/* src/cuda_train_context.cu:2175-2184 embedding_backward_kernel: dE[tok[t],:] += g[t,:] */
void ref_embedding_backward(const uint32_t* tok, const float* g, float* dE, int T, int d) {
    for (int t = 0; t < T; t++)
        for (int i = 0; i < d; i++) dE[(size_t)tok[t] * d + i] += g[(size_t)t * d + i];
}

/* src/cuda_train_context.cu:2187-2206 adamw_kernel (FP32 arithmetic as written there;
 * CPU twin src/train.c:1710-1732).  No clipping exists in the reference. */
void ref_adamw(float* w, const float* g, float* m, float* v, size_t n,
               float lr, float b1, float b2, float wd, float eps, int t) {
    float c1 = 1.0f - powf(b1, (float)t), c2 = 1.0f - powf(b2, (float)t);
    for (size_t i = 0; i < n; i++) {
        float gi = g[i];
        m[i] = b1 * m[i] + (1.0f - b1) * gi;
        v[i] = b2 * v[i] + (1.0f - b2) * gi * gi;
        float mh = m[i] / c1, vh = v[i] / c2;
        w[i] = w[i] * (1.0f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
}

/* src/cuda_train_context.cu:3240-3290 cuda_train_lora_backward, equal to
 * src/train.c:5803-5845 lora_gpu_backward with grad_input=NULL and to
 * src/lora.c:150-211 lora_backward:
 *   h = X A^T ; gB += dY^T (s h) ; gh = s (dY B) ; gA += gh^T X.
 * A [r,in], B [out,r], X [T,in], dY [T,out].  tmp holds T*r floats. */
void ref_lora_backward(const float* dY, const float* X, const float* A, const float* Bm,
                       float* gA, float* gB, float* tmp, int T, int in, int out, int r, float s) {
    ref_matmul(X, A, tmp, T, r, in, 0, 1, 0);
    ref_scale(tmp, (size_t)T * r, s);
    ref_matmul(dY, tmp, gB, out, r, T, 1, 0, 1);
    ref_matmul(dY, Bm, tmp, T, r, out, 0, 0, 0);
    ref_scale(tmp, (size_t)T * r, s);
    ref_matmul(tmp, X, gA, r, in, T, 1, 0, 1);
}

/* src/train.c:5778-5796 lora_gpu_forward_add: Y += (s X A^T) B^T */
void ref_lora_forward_add(const float* X, float* Y, const float* A, const float* Bm, float* tmp,
                          int T, int in, int out, int r, float s) {
    ref_matmul(X, A, tmp, T, r, in, 0, 1, 0);
    ref_scale(tmp, (size_t)T * r, s);
    ref_matmul(tmp, Bm, Y, T, out, r, 0, 1, 1);
}
