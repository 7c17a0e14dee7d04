// kernels_attention.cu - tiled causal attention over packed sequences, FP32.
// Forward keeps the log-sum-exp per (token, head); backward recomputes the
// probabilities from it (flash style) and is deterministic: dQ is owned by the
// query tile, dK/dV by the key tile (which walks the query heads of its GQA
// group and the query tiles that can see it), so nothing is added atomically.
//
// Reference kernels replaced (src/cuda_train_context.cu):
//   batch_attention[_packed] :712/:921, flash_attention_fwd[_packed] :1145/:1289,
//   batch_attention_backward[_packed] :792/:1013 and flash_attention_bwd[_packed]
//   :1859/:2012 (float atomicAdd on dK/dV in both).
// Layout: Q,dO,O,dQ [T, Hq*hd]; K,V,dK,dV [T, Hkv*hd]; lse, delta [T, Hq];
// kv head of query head h is h*Hkv/Hq (:728).
//
// Arithmetic here is FP32 FMA on CUDA cores in 64x64 tiles (4x4 register
// blocks); it is the parity baseline for the tensor-core attention path.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "sb_internal.h"

#define AT 64            // tile edge (queries and keys)
#define AT_THREADS 256   // 16 x 16 threads, each a 4x4 block of the score tile
#define PLD 68           // leading dimension of the probability tile in smem

// acc[i][j] += sum_d At[d][r0+i] * Bt[d][c0+j]   (both operands stored transposed, ld = AT)
__device__ __forceinline__ void tile_dot(float acc[4][4], const float* __restrict__ At, const float* __restrict__ Bt,
                                         int r0, int c0, int hd) {
#pragma unroll 4
    for (int d = 0; d < hd; d++) {
        float4 a = *(const float4*)(At + d * AT + r0);
        float4 b = *(const float4*)(Bt + d * AT + c0);
        acc[0][0] += a.x * b.x; acc[0][1] += a.x * b.y; acc[0][2] += a.x * b.z; acc[0][3] += a.x * b.w;
        acc[1][0] += a.y * b.x; acc[1][1] += a.y * b.y; acc[1][2] += a.y * b.z; acc[1][3] += a.y * b.w;
        acc[2][0] += a.z * b.x; acc[2][1] += a.z * b.y; acc[2][2] += a.z * b.z; acc[2][3] += a.z * b.w;
        acc[3][0] += a.w * b.x; acc[3][1] += a.w * b.y; acc[3][2] += a.w * b.z; acc[3][3] += a.w * b.w;
    }
}

// out[i][c] += sum_j P[r0+i][j] * Bm[j][tx + 16c]   (P row-major ld PLD, Bm row-major ld hd)
template <int CPT>
__device__ __forceinline__ void tile_pv(float out[4][CPT], const float* __restrict__ P, const float* __restrict__ Bm,
                                        int r0, int tx, int hd) {
    for (int j = 0; j < AT; j += 4) {
        float4 p0 = *(const float4*)(P + (r0 + 0) * PLD + j), p1 = *(const float4*)(P + (r0 + 1) * PLD + j);
        float4 p2 = *(const float4*)(P + (r0 + 2) * PLD + j), p3 = *(const float4*)(P + (r0 + 3) * PLD + j);
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            int col = tx + 16 * c;
            if (col < hd) {
                float b0 = Bm[(j + 0) * hd + col], b1 = Bm[(j + 1) * hd + col], b2 = Bm[(j + 2) * hd + col], b3 = Bm[(j + 3) * hd + col];
                out[0][c] += p0.x * b0 + p0.y * b1 + p0.z * b2 + p0.w * b3;
                out[1][c] += p1.x * b0 + p1.y * b1 + p1.z * b2 + p1.w * b3;
                out[2][c] += p2.x * b0 + p2.y * b1 + p2.z * b2 + p2.w * b3;
                out[3][c] += p3.x * b0 + p3.y * b1 + p3.z * b2 + p3.w * b3;
            }
        }
    }
}

// Load rows [row0, row0+AT) x hd of one head into smem, row-major (sR, ld hd)
// and/or transposed (sT, ld AT).  Rows outside [0,T) read as zero.
__device__ __forceinline__ void load_tile(const float* __restrict__ g, size_t row_stride, int row0, int T, int hd,
                                          float* sR, float* sT) {
    for (int idx = threadIdx.x; idx < AT * hd; idx += AT_THREADS) {
        int r = idx / hd, d = idx - r * hd;
        int gr = row0 + r;
        float v = (gr >= 0 && gr < T) ? g[(size_t)gr * row_stride + d] : 0.f;
        if (sR) sR[r * hd + d] = v;
        if (sT) sT[d * AT + r] = v;
    }
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <int CPT>
__global__ void __launch_bounds__(AT_THREADS) attn_fwd_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                              const float* __restrict__ V, float* __restrict__ O,
                                                              float* __restrict__ lse, const uint32_t* __restrict__ seq_starts,
                                                              const uint32_t* __restrict__ seq_ids,
                                                              int T, int Hq, int Hkv, int hd, float scale) {
    extern __shared__ float smem[];
    float* sQt = smem;                 // [hd][AT]
    float* sKt = sQt + hd * AT;        // [hd][AT]
    float* sV = sKt + hd * AT;         // [AT][hd]
    float* sP = sV + AT * hd;          // [AT][PLD]
    const int h = blockIdx.y, kvh = h * Hkv / Hq, q0 = blockIdx.x * AT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, r0 = ty * 4, c0 = tx * 4;
    const size_t qs = (size_t)Hq * hd, ks = (size_t)Hkv * hd;

    load_tile(Q + (size_t)h * hd, qs, q0, T, hd, nullptr, sQt);
    int row_start[4];
#pragma unroll
    for (int i = 0; i < 4; i++) { int r = q0 + r0 + i; row_start[i] = r < T ? (int)seq_starts[seq_ids[r]] : 0x7fffffff; }
    int q_last = min(q0 + AT, T) - 1;
    int k_begin = ((int)seq_starts[seq_ids[q0]] / AT) * AT;   // first row of the tile is in the earliest sequence
    float m[4], l[4], o[4][CPT];
#pragma unroll
    for (int i = 0; i < 4; i++) { m[i] = -INFINITY; l[i] = 0.f; for (int c = 0; c < CPT; c++) o[i][c] = 0.f; }

    for (int k0 = k_begin; k0 <= q_last; k0 += AT) {
        __syncthreads();
        load_tile(K + (size_t)kvh * hd, ks, k0, T, hd, nullptr, sKt);
        load_tile(V + (size_t)kvh * hd, ks, k0, T, hd, sV, nullptr);
        __syncthreads();
        float s[4][4] = {};
        tile_dot(s, sQt, sKt, r0, c0, hd);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int qi = q0 + r0 + i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int kj = k0 + c0 + j;
                bool ok = (kj <= qi) && (kj >= row_start[i]) && (qi < T);
                s[i][j] = ok ? s[i][j] * scale : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
            for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float mn = fmaxf(m[i], mx);
            float corr = (m[i] == -INFINITY) ? 0.f : expf(m[i] - mn);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) { float p = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - mn); s[i][j] = p; rs += p; }
            for (int off = 8; off > 0; off >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, off);
            l[i] = l[i] * corr + rs; m[i] = mn;
#pragma unroll
            for (int c = 0; c < CPT; c++) o[i][c] *= corr;
            *(float4*)(sP + (r0 + i) * PLD + c0) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
        }
        __syncthreads();
        tile_pv<CPT>(o, sP, sV, r0, tx, hd);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int qi = q0 + r0 + i;
        if (qi >= T) continue;
        float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
        for (int c = 0; c < CPT; c++) { int col = tx + 16 * c; if (col < hd) O[(size_t)qi * qs + (size_t)h * hd + col] = o[i][c] * inv; }
        if (tx == 0 && lse) lse[(size_t)qi * Hq + h] = m[i] + logf(l[i] > 0.f ? l[i] : 1.0f);
    }
}

// delta[t,h] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (t,h)
__global__ void attn_delta_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ delta,
                                  int T, int Hq, int hd) {
    int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= T * Hq) return;
    const float* a = dO + (size_t)w * hd; const float* b = O + (size_t)w * hd;
    float s = 0.f;
    for (int d = lane; d < hd; d += 32) s += a[d] * b[d];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) delta[w] = s;
}

// ---------------------------------------------------------------------------
// Backward, dQ: one CTA per (query tile, query head)
// ---------------------------------------------------------------------------
template <int CPT>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_dq_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                                 const float* __restrict__ V, const float* __restrict__ dO,
                                                                 const float* __restrict__ lse, const float* __restrict__ delta,
                                                                 float* __restrict__ dQ, const uint32_t* __restrict__ seq_starts,
                                                                 const uint32_t* __restrict__ seq_ids,
                                                                 int T, int Hq, int Hkv, int hd, float scale) {
    extern __shared__ float smem[];
    float* sQt = smem;                  // [hd][AT]
    float* sdOt = sQt + hd * AT;        // [hd][AT]
    float* sKt = sdOt + hd * AT;        // [hd][AT]
    float* sVt = sKt + hd * AT;         // [hd][AT]
    float* sK = sVt + hd * AT;          // [AT][hd]
    float* sS = sK + AT * hd;           // [AT][PLD]
    const int h = blockIdx.y, kvh = h * Hkv / Hq, q0 = blockIdx.x * AT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, r0 = ty * 4, c0 = tx * 4;
    const size_t qs = (size_t)Hq * hd, ks = (size_t)Hkv * hd;
    load_tile(Q + (size_t)h * hd, qs, q0, T, hd, nullptr, sQt);
    load_tile(dO + (size_t)h * hd, qs, q0, T, hd, nullptr, sdOt);
    int row_start[4]; float L[4], D[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int r = q0 + r0 + i;
        row_start[i] = r < T ? (int)seq_starts[seq_ids[r]] : 0x7fffffff;
        L[i] = r < T ? lse[(size_t)r * Hq + h] : 0.f;
        D[i] = r < T ? delta[(size_t)r * Hq + h] : 0.f;
    }
    int q_last = min(q0 + AT, T) - 1;
    int k_begin = ((int)seq_starts[seq_ids[q0]] / AT) * AT;
    float acc[4][CPT];
#pragma unroll
    for (int i = 0; i < 4; i++) for (int c = 0; c < CPT; c++) acc[i][c] = 0.f;
    for (int k0 = k_begin; k0 <= q_last; k0 += AT) {
        __syncthreads();
        load_tile(K + (size_t)kvh * hd, ks, k0, T, hd, sK, sKt);
        load_tile(V + (size_t)kvh * hd, ks, k0, T, hd, nullptr, sVt);
        __syncthreads();
        float s[4][4] = {}, dp[4][4] = {};
        tile_dot(s, sQt, sKt, r0, c0, hd);
        tile_dot(dp, sdOt, sVt, r0, c0, hd);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int qi = q0 + r0 + i;
            float ds[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int kj = k0 + c0 + j;
                bool ok = (kj <= qi) && (kj >= row_start[i]) && (qi < T);
                float p = ok ? expf(s[i][j] * scale - L[i]) : 0.f;
                ds[j] = p * (dp[i][j] - D[i]) * scale;
            }
            *(float4*)(sS + (r0 + i) * PLD + c0) = make_float4(ds[0], ds[1], ds[2], ds[3]);
        }
        __syncthreads();
        tile_pv<CPT>(acc, sS, sK, r0, tx, hd);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int qi = q0 + r0 + i;
        if (qi >= T) continue;
#pragma unroll
        for (int c = 0; c < CPT; c++) { int col = tx + 16 * c; if (col < hd) dQ[(size_t)qi * qs + (size_t)h * hd + col] = acc[i][c]; }
    }
}

// ---------------------------------------------------------------------------
// Backward, dK and dV: one CTA per (key tile, kv head).  It walks every query
// head of the GQA group and every query tile that can attend to these keys.
// ---------------------------------------------------------------------------
template <int CPT>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_dkv_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                                  const float* __restrict__ V, const float* __restrict__ dO,
                                                                  const float* __restrict__ lse, const float* __restrict__ delta,
                                                                  float* __restrict__ dK, float* __restrict__ dV, int accumulate,
                                                                  const uint32_t* __restrict__ seq_starts,
                                                                  const uint32_t* __restrict__ seq_ids,
                                                                  int T, int Hq, int Hkv, int hd, float scale) {
    extern __shared__ float smem[];
    float* sKt = smem;                  // [hd][AT]
    float* sVt = sKt + hd * AT;         // [hd][AT]
    float* sQt = sVt + hd * AT;         // [hd][AT]
    float* sdOt = sQt + hd * AT;        // [hd][AT]
    float* sQ = sdOt + hd * AT;         // [AT][hd]
    float* sdO = sQ + AT * hd;          // [AT][hd]
    float* sS = sdO + AT * hd;          // [AT][PLD]  (P^T, then dS^T)
    __shared__ float sL[AT], sD[AT]; __shared__ int sRS[AT];
    const int kvh = blockIdx.y, k0 = blockIdx.x * AT;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, r0 = ty * 4, c0 = tx * 4;   // rows = keys, cols = queries
    const size_t qs = (size_t)Hq * hd, ks = (size_t)Hkv * hd;
    load_tile(K + (size_t)kvh * hd, ks, k0, T, hd, nullptr, sKt);
    load_tile(V + (size_t)kvh * hd, ks, k0, T, hd, nullptr, sVt);
    // queries that can see a key of this tile: same sequence as the tile's last key, up to its end
    int k_last = min(k0 + AT, T) - 1;
    int q_end = (int)seq_starts[seq_ids[k_last] + 1];      // exclusive
    float aK[4][CPT], aV[4][CPT];
#pragma unroll
    for (int i = 0; i < 4; i++) for (int c = 0; c < CPT; c++) { aK[i][c] = 0.f; aV[i][c] = 0.f; }
    const int group = Hq / Hkv;
    for (int h = 0; h < Hq; h++) {
        if (h * Hkv / Hq != kvh) continue;
        (void)group;
        for (int q0 = k0; q0 < q_end; q0 += AT) {
            __syncthreads();
            load_tile(Q + (size_t)h * hd, qs, q0, T, hd, sQ, sQt);
            load_tile(dO + (size_t)h * hd, qs, q0, T, hd, sdO, sdOt);
            if (threadIdx.x < AT) {
                int r = q0 + threadIdx.x;
                sL[threadIdx.x] = r < T ? lse[(size_t)r * Hq + h] : 0.f;
                sD[threadIdx.x] = r < T ? delta[(size_t)r * Hq + h] : 0.f;
                sRS[threadIdx.x] = r < T ? (int)seq_starts[seq_ids[r]] : 0x7fffffff;
            }
            __syncthreads();
            float st[4][4] = {}, dpt[4][4] = {};
            tile_dot(st, sKt, sQt, r0, c0, hd);       // S^T[key][query]
            tile_dot(dpt, sVt, sdOt, r0, c0, hd);     // dP^T[key][query]
            float ds[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int kj = k0 + r0 + i;
                float p[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int qi = q0 + c0 + j;
                    bool ok = (kj <= qi) && (kj >= sRS[c0 + j]) && (qi < T) && (kj < T);
                    p[j] = ok ? expf(st[i][j] * scale - sL[c0 + j]) : 0.f;
                    ds[i][j] = p[j] * (dpt[i][j] - sD[c0 + j]) * scale;
                }
                *(float4*)(sS + (r0 + i) * PLD + c0) = make_float4(p[0], p[1], p[2], p[3]);
            }
            __syncthreads();
            tile_pv<CPT>(aV, sS, sdO, r0, tx, hd);    // dV += P^T dO
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 4; i++) *(float4*)(sS + (r0 + i) * PLD + c0) = make_float4(ds[i][0], ds[i][1], ds[i][2], ds[i][3]);
            __syncthreads();
            tile_pv<CPT>(aK, sS, sQ, r0, tx, hd);     // dK += dS^T Q
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int kj = k0 + r0 + i;
        if (kj >= T) continue;
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            int col = tx + 16 * c;
            if (col < hd) {
                size_t o = (size_t)kj * ks + (size_t)kvh * hd + col;
                if (accumulate) { dK[o] += aK[i][c]; dV[o] += aV[i][c]; } else { dK[o] = aK[i][c]; dV[o] = aV[i][c]; }
            }
        }
    }
}

template <typename F>
static bool set_smem(sb_ctx_t* c, F kernel, size_t bytes) {
    if (bytes > (size_t)c->pub.gpu_max_shared_per_block_optin) { sb_set_status(c, SB_ERR_SIZE); return false; }
    if (bytes > 48 * 1024) return !sb_check(c, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), "attention smem");
    return true;
}

#define DISPATCH_CPT(hd, CALL) \
    do { int cpt_ = ((hd) + 15) / 16; \
         if (cpt_ <= 1) { CALL(1) } else if (cpt_ <= 2) { CALL(2) } else if (cpt_ <= 4) { CALL(4) } \
         else if (cpt_ <= 8) { CALL(8) } else { CALL(16) } } while (0)

extern "C" {

void sb_attention(sb_ctx_t* c, const float* Q, const float* K, const float* V, float* out, float* lse,
                  const uint32_t* seq_starts, const uint32_t* seq_ids, int T, int Hq, int Hkv, int hd) {
    if (T <= 0 || Hq <= 0 || Hkv <= 0 || hd <= 0) return;
    if (hd > 256 || Hq < Hkv) { sb_set_status(c, SB_ERR_SIZE); return; }
    if (sb_attention_tc_forward(c, Q, K, V, out, lse, T, Hq, Hkv, hd) == 0) return;      // tensor-core path took it
    float scale = 1.0f / sqrtf((float)hd);
    dim3 grid((T + AT - 1) / AT, Hq);
    size_t smem = ((size_t)3 * hd * AT + (size_t)AT * PLD) * sizeof(float);
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_FWD);
#define CALL(N) if (set_smem(c, attn_fwd_kernel<N>, smem)) attn_fwd_kernel<N><<<grid, AT_THREADS, smem, s>>>(Q, K, V, out, lse, seq_starts, seq_ids, T, Hq, Hkv, hd, scale);
    DISPATCH_CPT(hd, CALL);
#undef CALL
    // causal: about half of the T x S score matrix per head is live; counted as 2*T*T/B... reported per call as 2 matmuls
    sb_tick_end(c, tk, 0.0, 4.0 * ((double)T * Hq * hd * 2 + (double)T * Hkv * hd * 2));
    c->launches++;
}

void sb_attention_backward(sb_ctx_t* c, const float* Q, const float* K, const float* V, const float* O, const float* lse,
                           const float* dO, float* dQ, float* dK, float* dV, int accumulate_kv,
                           const uint32_t* seq_starts, const uint32_t* seq_ids, int B, int T, int Hq, int Hkv, int hd) {
    (void)B;
    if (T <= 0 || Hq <= 0 || Hkv <= 0 || hd <= 0) return;
    if (hd > 256) { sb_set_status(c, SB_ERR_SIZE); return; }
    if (sb_attention_tc_backward(c, Q, K, V, O, lse, dO, dQ, dK, dV, accumulate_kv, T, Hq, Hkv, hd) == 0) return;
    float scale = 1.0f / sqrtf((float)hd);
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    float* delta = (float*)sb_scratch(c, (size_t)T * Hq * sizeof(float));
    if (!delta) return;
    int warps = T * Hq;
    int tk = sb_tick_begin(c, SB_CLS_ATTN_BWD);
    attn_delta_kernel<<<(warps * 32 + 255) / 256, 256, 0, s>>>(dO, O, delta, T, Hq, hd);
    dim3 gq((T + AT - 1) / AT, Hq), gk((T + AT - 1) / AT, Hkv);
    size_t smem_q = ((size_t)5 * hd * AT + (size_t)AT * PLD) * sizeof(float);
    size_t smem_k = ((size_t)6 * hd * AT + (size_t)AT * PLD) * sizeof(float);
#define CALL(N) if (set_smem(c, attn_bwd_dq_kernel<N>, smem_q)) attn_bwd_dq_kernel<N><<<gq, AT_THREADS, smem_q, s>>>(Q, K, V, dO, lse, delta, dQ, seq_starts, seq_ids, T, Hq, Hkv, hd, scale);
    DISPATCH_CPT(hd, CALL);
#undef CALL
#define CALL(N) if (set_smem(c, attn_bwd_dkv_kernel<N>, smem_k)) attn_bwd_dkv_kernel<N><<<gk, AT_THREADS, smem_k, s>>>(Q, K, V, dO, lse, delta, dK, dV, accumulate_kv, seq_starts, seq_ids, T, Hq, Hkv, hd, scale);
    DISPATCH_CPT(hd, CALL);
#undef CALL
    sb_tick_end(c, tk, 0.0, 4.0 * ((double)T * Hq * hd * 4 + (double)T * Hkv * hd * 4));
    c->launches += 3;
}

}  // extern "C"
