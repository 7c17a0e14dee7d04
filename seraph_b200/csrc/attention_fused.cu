// attention_fused.cu - causal attention forward in one kernel (head size 128, FP16 hi/lo parts, FP32-level accuracy).
//
// One CTA owns 128 consecutive queries of one (sequence, query head) and walks over that sequence's keys in
// blocks of 64, up to the diagonal.  Nothing of size S x S ever reaches memory:
//
//   S_j  = Q K_j^T          tcgen05.mma kind::f16, M 128 x N 64 x K 128, three passes (q1 k1 + q2 k1 + q1 k2) on the
//                           prepared parts of Q and K (x * 2^s = h1 + h2), accumulator in tensor memory: the two halves
//                           of the head dimension go to two accumulators of twelve instructions each, added in FP32
//   P_j  = exp(S_j/sqrt(hd) - m)   by the softmax warps, one query row per thread, running maximum m and sum l;
//                           written to shared memory as two FP16 parts of P * 2^14 in the K-major 128-byte swizzle
//   O    = O * alpha + P_j V_j     M 128 x N 128 x K 64, three passes on the parts of P and V (V read in place,
//                           MN-major), twelve instructions into a fresh accumulator that the O warps add into
//                           registers (round-to-nearest FP32) after scaling by alpha = exp(m_old - m_new)
//   out  = O / l,  lse = m + log l
//
// Warps: 0 TMA producer, 1 MMA issuer (owns the tensor-memory allocation), 4-7 softmax, 8-15 O accumulation
// (two warps per lane quarter, 64 columns each).  Shared memory: Q parts 64 KB, K and V parts 2 x 32 KB each
// (double buffered), P parts 32 KB.  Tensor memory: 2 x (64 + 64) columns for S, 2 x 128 for P V.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA drains and frees its
// tensor memory.
#include "attention_fused.cuh"

__global__ void __launch_bounds__(AF_THREADS, 1)
at_fused_fwd_kernel(const __grid_constant__ CUtensorMap mQ1, const __grid_constant__ CUtensorMap mQ2,
                    const __grid_constant__ CUtensorMap mK1, const __grid_constant__ CUtensorMap mK2,
                    const __grid_constant__ CUtensorMap mV1, const __grid_constant__ CUtensorMap mV2,
                    const __grid_constant__ AfSeqs seqs, float* __restrict__ O, float* __restrict__ lse,
                    const float* __restrict__ amax_q, const float* __restrict__ amax_k, const float* __restrict__ amax_v,
                    int Hq, int g, int nqb_max, float scale, int* status, unsigned* amax_o) {
    // which (query block, sequence, head): blocks with the most keys first, the query heads of one K/V head side by side
    const int per_i = seqs.n * Hq;
    const int qb = nqb_max - 1 - (int)blockIdx.x / per_i;
    const int rem = (int)blockIdx.x % per_i;
    const int b = rem / Hq, h = rem % Hq;
    const int t0 = seqs.start[b], S = seqs.start[b + 1] - t0;
    if (qb * AF_BQ >= S) return;
    if (*(volatile int*)status != 0) return;                 // an earlier CTA gave up: do not queue behind its cause
    const int nkv = min((S + AF_BKV - 1) / AF_BKV, 2 * qb + 2);
    const int kvh = h / g;
    const int qd = Hq * AF_HD;

    extern __shared__ uint8_t af_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)af_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + AF_OFF_BAR);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* k_empty = bars + 3;       // 2
    uint64_t* v_full = bars + 5;        // 2
    uint64_t* v_empty = bars + 7;       // 2
    uint64_t* s_full = bars + 9;        // 2
    uint64_t* s_empty = bars + 11;      // 2
    uint64_t* p_full = bars + 13;       // 1
    uint64_t* p_empty = bars + 14;      // 1
    uint64_t* pv_full = bars + 15;      // 2
    uint64_t* pv_empty = bars + 17;     // 2
    uint64_t* a_full = bars + 19;       // 2
    uint64_t* fin_full = bars + 21;     // 1
    uint32_t* tmem_slot = (uint32_t*)(bars + 24);
    float* alpha_s = (float*)(smem + AF_OFF_BAR + 256);          // [2][128]
    float* fin_s = alpha_s + 256;                                 // [128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&pv_full[i], 1); mbar_init(&pv_empty[i], 8);
            mbar_init(&a_full[i], 4);
        }
        mbar_init(p_full, 4); mbar_init(p_empty, 1); mbar_init(fin_full, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            mbar_expect_tx(q_full, AF_Q_BYTES);
            for (int p = 0; p < 2; p++) {
                af_tma_2d(smem + p * 16384, &mQ1, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
                af_tma_2d(smem + 32768 + p * 16384, &mQ2, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
            }
            // order of need: K_0, K_1, V_0, K_2, V_1, ...
            for (int jj = -1; jj < nkv && ok; jj++) {
                const int jk = jj + 1;
                if (jk < nkv) {
                    const int s = jk & 1, u = jk >> 1;
                    ok = mbar_wait(&k_empty[s], (u & 1) ^ 1);
                    if (!ok) break;
                    uint8_t* dst = smem + AF_OFF_K + s * AF_KV_STAGE;
                    mbar_expect_tx(&k_full[s], AF_KV_STAGE);
                    for (int p = 0; p < 2; p++) {
                        af_tma_2d(dst + p * 8192, &mK1, &k_full[s], kvh * AF_HD + p * 64, t0 + jk * AF_BKV);
                        af_tma_2d(dst + 16384 + p * 8192, &mK2, &k_full[s], kvh * AF_HD + p * 64, t0 + jk * AF_BKV);
                    }
                }
                if (jj >= 0) {
                    const int s = jj & 1, u = jj >> 1;
                    ok = mbar_wait(&v_empty[s], (u & 1) ^ 1);
                    if (!ok) break;
                    uint8_t* dst = smem + AF_OFF_V + s * AF_KV_STAGE;
                    mbar_expect_tx(&v_full[s], AF_KV_STAGE);
                    for (int p = 0; p < 2; p++) {
                        af_tma_2d(dst + p * 8192, &mV1, &v_full[s], kvh * AF_HD + p * 64, t0 + jj * AF_BKV);
                        af_tma_2d(dst + 16384 + p * 8192, &mV2, &v_full[s], kvh * AF_HD + p * 64, t0 + jj * AF_BKV);
                    }
                }
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            const uint32_t idesc_s = (1u << 4) | ((uint32_t)(AF_BKV >> 3) << 17) | ((uint32_t)(AF_BQ >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(AF_HD >> 3) << 17) | ((uint32_t)(AF_BQ >> 4) << 24);
            const uint32_t sq = smem_u32(smem);
            ok = mbar_wait(q_full, 0);
            for (int jj = -1; jj < nkv && ok; jj++) {
                const int js = jj + 1;
                if (js < nkv) {
                    // S_js = Q K_js^T: head-dimension half p into accumulator p of S buffer js & 1
                    const int s = js & 1, u = js >> 1;
                    ok = mbar_wait(&k_full[s], u & 1) && mbar_wait(&s_empty[s], (u & 1) ^ 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sk = smem_u32(smem + AF_OFF_K + s * AF_KV_STAGE);
#pragma unroll
                    for (int p = 0; p < 2; p++) {
                        const uint64_t a1 = make_kmajor_desc<128>(sq + p * 16384), a2 = make_kmajor_desc<128>(sq + 32768 + p * 16384);
                        const uint64_t b1 = make_kmajor_desc<128>(sk + p * 8192), b2 = make_kmajor_desc<128>(sk + 16384 + p * 8192);
                        const uint32_t d = tmem_base + (uint32_t)(s * 128 + p * 64);
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {
                            const uint64_t adv = (uint64_t)(kk * 2);
                            af_mma_f16(d, a1 + adv, b1 + adv, idesc_s, kk ? 1u : 0u);
                            af_mma_f16(d, a2 + adv, b1 + adv, idesc_s, 1);
                            af_mma_f16(d, a1 + adv, b2 + adv, idesc_s, 1);
                        }
                    }
                    tc_commit(&s_full[s]);
                    tc_commit(&k_empty[s]);
                }
                if (jj >= 0) {
                    // O contribution of block jj: P_jj V_jj into P V buffer jj & 1
                    const int s = jj & 1, u = jj >> 1;
                    ok = mbar_wait(p_full, jj & 1) && mbar_wait(&v_full[s], u & 1) && mbar_wait(&pv_empty[s], (u & 1) ^ 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sp = smem_u32(smem + AF_OFF_P), sv = smem_u32(smem + AF_OFF_V + s * AF_KV_STAGE);
                    const uint64_t a1 = make_kmajor_desc<128>(sp), a2 = make_kmajor_desc<128>(sp + 16384);
                    const uint64_t b1 = make_mn16_desc<AF_BKV>(sv), b2 = make_mn16_desc<AF_BKV>(sv + 16384);
                    const uint32_t d = tmem_base + (uint32_t)(256 + s * 128);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t adva = (uint64_t)(kk * 2), advb = (uint64_t)(kk * 128);
                        af_mma_f16(d, a1 + adva, b1 + advb, idesc_o, kk ? 1u : 0u);
                        af_mma_f16(d, a2 + adva, b1 + advb, idesc_o, 1);
                        af_mma_f16(d, a1 + adva, b2 + advb, idesc_o, 1);
                    }
                    tc_commit(&pv_full[s]);
                    tc_commit(&v_empty[s]);
                    tc_commit(p_empty);
                }
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------- softmax: one query row per thread ----------------
        const int q = warp & 3, r = q * 32 + lane;
        const int qi = qb * AF_BQ + r;                        // position of this row inside the sequence
        const float cs = tc_pow2(-tc_f16_shift(__ldg(amax_q))) * tc_pow2(-tc_f16_shift(__ldg(amax_k))) * (scale * 1.4426950408889634f);
        float m = -INFINITY, l = 0.f;
        uint8_t* prow = smem + AF_OFF_P + r * 128;
        for (int j = 0; j < nkv && ok; j++) {
            const int s = j & 1, u = j >> 1;
            ok = mbar_wait(&s_full[s], u & 1);
            if (!ok) break;
            tc_fence_after();
            float y[64];                                        // raw scores (the two accumulators added)
            {
                const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * 128);
                uint32_t a[32], c[32];
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    af_ld32_issue(ta + hh * 32, a);
                    af_ld32_issue(ta + 64 + hh * 32, c);
                    af_ld_wait(a); af_ld_dep(c);
#pragma unroll
                    for (int i = 0; i < 32; i++) y[hh * 32 + i] = __uint_as_float(a[i]) + __uint_as_float(c[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) af_arrive(&s_empty[s]);
            if (j >= 2 * qb) {                                 // blocks that reach the diagonal: keys after the query do not count
                const int k0 = j * AF_BKV;
#pragma unroll
                for (int i = 0; i < 64; i++) if (k0 + i > qi) y[i] = -INFINITY;
            }
            float mx4[4] = {y[0], y[1], y[2], y[3]};
#pragma unroll
            for (int i = 4; i < 64; i++) mx4[i & 3] = fmaxf(mx4[i & 3], y[i]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * cs;      // cs > 0
            const float m_new = fmaxf(m, mx);                 // finite from block 0 on: key 0 counts for every row
            const float alpha = af_ex2(m - m_new);
            const float off = 14.f - m_new;                   // P leaves as P * 2^14
            float sm4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 64; i++) { y[i] = af_ex2(fmaf(y[i], cs, off)); sm4[i & 3] += y[i]; }
            l = l * alpha + ((sm4[0] + sm4[1]) + (sm4[2] + sm4[3]));          // in units of 2^-14
            m = m_new;
            // alpha to the O warps (the slot was last read for block j - 2)
            ok = mbar_wait(&pv_empty[s], (u & 1) ^ 1);
            if (!ok) break;
            alpha_s[s * 128 + r] = alpha;
            __syncwarp();
            if (lane == 0) af_arrive(&a_full[s]);
            // P * 2^14 as two FP16 parts, K-major rows of 128 bytes, 16-byte chunks swizzled by the row
            ok = mbar_wait(p_empty, (j & 1) ^ 1);
            if (!ok) break;
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
                uint32_t w1[4], w2[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    af_split2(y[c8 * 8 + 2 * e], y[c8 * 8 + 2 * e + 1], w1[e], w2[e]);
                }
                const int off = ((c8 ^ (r & 7)) << 4);
                *(uint4*)(prow + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
                *(uint4*)(prow + 16384 + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) af_arrive(p_full);
        }
        if (ok) {
            fin_s[r] = l > 0.f ? 1.0f / l : 0.f;
            if (lse && qi < S) lse[(size_t)(t0 + qi) * Hq + h] = (m + log2f(l) - 14.f) * 0.6931471805599453f;
        }
        __syncwarp();
        if (lane == 0) af_arrive(fin_full);
        if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
    } else if (warp >= 8) {
        // ---------------- O accumulation: one row and 64 columns per thread ----------------
        const int q = warp & 3, r = q * 32 + lane, ch = (warp - 8) >> 2;
        const int qi = qb * AF_BQ + r;
        float o[64];
#pragma unroll
        for (int i = 0; i < 64; i++) o[i] = 0.f;
        for (int j = 0; j < nkv && ok; j++) {
            const int s = j & 1, u = j >> 1;
            ok = mbar_wait(&a_full[s], u & 1) && mbar_wait(&pv_full[s], u & 1);
            if (!ok) break;
            tc_fence_after();
            const float alpha = alpha_s[s * 128 + r];
            const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(256 + s * 128 + ch * 64);
            {
                uint32_t t[32], t2[32];
                af_ld32_issue(ta, t);
                af_ld32_issue(ta + 32, t2);
                af_ld_wait(t); af_ld_dep(t2);
#pragma unroll
                for (int i = 0; i < 32; i++) { o[i] = fmaf(o[i], alpha, __uint_as_float(t[i])); o[32 + i] = fmaf(o[32 + i], alpha, __uint_as_float(t2[i])); }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) af_arrive(&pv_empty[s]);
        }
        if (ok) ok = mbar_wait(fin_full, 0);
        float am = 0.f;
        if (ok && qi < S) {
            const float f = fin_s[r] * tc_pow2(-tc_f16_shift(__ldg(amax_v)));      // fin = 1 / l with l in units of 2^-14, O holds (P * 2^14) V' products
            float4* dst = (float4*)(O + (size_t)(t0 + qi) * qd + (size_t)h * AF_HD + ch * 64);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float4 v = make_float4(o[4 * i] * f, o[4 * i + 1] * f, o[4 * i + 2] * f, o[4 * i + 3] * f);
                dst[i] = v;
                am = sb_amax4(am, v);
            }
        }
        if (amax_o) {                                          // largest |O|, for the split of the output projection's operand
            for (int d = 16; d > 0; d >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, d));
            if (lane == 0 && am > 0.f) atomicMax(amax_o, __float_as_uint(am));
        }
        if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Backward scores in one kernel: for 128 queries of one (sequence, head) and every block of 64 keys up to the diagonal
//   S = Q K^T, dP = dO V^T   (three FP16 passes each, two twelve-instruction accumulators per product, in tensor memory)
//   P = exp(S/sqrt(hd) - lse),  dS = P o (dP - D) / sqrt(hd)
// and P, dS leave as the FP16 parts the three long products of the backward pass read (P * 2^14; dS times the power
// of two that brings its bound to [2^14, 2^15)), laid out [head][Sp][Sp] like the score scratch.  Columns past the
// diagonal are written as zeros up to the end of the row's 256-column tile, which is as far as those products read.
// Warps: 0 TMA producer, 1 MMA issuer, 4-11 elementwise (two per lane quarter, 32 of the 64 columns each).
// Shared memory: Q and dO parts 2 x 64 KB, K parts 2 x 32 KB (double buffered), V parts 32 KB.
#define AS_OFF_DO 65536
#define AS_OFF_K 131072
#define AS_OFF_V (AS_OFF_K + 2 * AF_KV_STAGE)
#define AS_OFF_BAR (AS_OFF_V + AF_KV_STAGE)
#define AS_SMEM (AS_OFF_BAR + 1024 + 1024)
#define AS_THREADS 384

__global__ void __launch_bounds__(AS_THREADS, 1)
at_score_bwd_kernel(const __grid_constant__ CUtensorMap mQ1, const __grid_constant__ CUtensorMap mQ2,
                    const __grid_constant__ CUtensorMap mD1, const __grid_constant__ CUtensorMap mD2,
                    const __grid_constant__ CUtensorMap mK1, const __grid_constant__ CUtensorMap mK2,
                    const __grid_constant__ CUtensorMap mV1, const __grid_constant__ CUtensorMap mV2,
                    const float* __restrict__ lse, const float* __restrict__ D,
                    __half* __restrict__ P1, __half* __restrict__ P2, __half* __restrict__ dS1, __half* __restrict__ dS2,
                    const float* __restrict__ amax_q, const float* __restrict__ amax_k, const float* __restrict__ amax_v,
                    const float* __restrict__ amax_do, const float* __restrict__ ds_bound,
                    const __grid_constant__ AfSeqs seqs, int Sp, int Hq, int g, int head0, int head_step, int nb, int nqb, float scale, int* status) {
    // nb > 0: one sequence, heads head0 + i * head_step, output slot i.  nb == 0: every sequence and head of the call,
    // output slot ((sequence * g + head % g) * Hkv + head / g), i.e. the Hkv heads of one (sequence, group member) side by side
    const int nheads = nb > 0 ? nb : Hq;
    const int per_i = seqs.n * nheads;
    const int qb = nqb - 1 - (int)blockIdx.x / per_i;
    const int rem = (int)blockIdx.x % per_i;
    const int b = rem / nheads, hi = rem % nheads;
    const int h = nb > 0 ? head0 + hi * head_step : hi;
    const int hb = nb > 0 ? hi : (b * g + h % g) * (Hq / g) + h / g;
    const int t0 = seqs.start[b], S = seqs.start[b + 1] - t0;
    if (qb * AF_BQ >= S) return;
    if (*(volatile int*)status != 0) return;
    const int nkv = min((S + AF_BKV - 1) / AF_BKV, 2 * qb + 2);           // key blocks that hold scores
    const int nz = min(Sp / AF_BKV, 4 * (qb / 2 + 1));                    // key blocks that are written
    const int kvh = h / g;

    extern __shared__ uint8_t af_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)af_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + AS_OFF_BAR);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* k_empty = bars + 3;       // 2
    uint64_t* v_full = bars + 5;        // 1
    uint64_t* v_empty = bars + 6;       // 1
    uint64_t* acc_full = bars + 7;      // 2
    uint64_t* acc_empty = bars + 9;     // 2
    uint32_t* tmem_slot = (uint32_t*)(bars + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
        for (int i = 0; i < 2; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (elect_one()) {
            mbar_expect_tx(q_full, 2 * AF_Q_BYTES);
            for (int p = 0; p < 2; p++) {
                af_tma_2d(smem + p * 16384, &mQ1, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
                af_tma_2d(smem + 32768 + p * 16384, &mQ2, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
                af_tma_2d(smem + AS_OFF_DO + p * 16384, &mD1, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
                af_tma_2d(smem + AS_OFF_DO + 32768 + p * 16384, &mD2, q_full, h * AF_HD + p * 64, t0 + qb * AF_BQ);
            }
            for (int j = 0; j < nkv && ok; j++) {
                const int s = j & 1, u = j >> 1;
                ok = mbar_wait(&k_empty[s], (u & 1) ^ 1);
                if (!ok) break;
                uint8_t* dk = smem + AS_OFF_K + s * AF_KV_STAGE;
                mbar_expect_tx(&k_full[s], AF_KV_STAGE);
                for (int p = 0; p < 2; p++) {
                    af_tma_2d(dk + p * 8192, &mK1, &k_full[s], kvh * AF_HD + p * 64, t0 + j * AF_BKV);
                    af_tma_2d(dk + 16384 + p * 8192, &mK2, &k_full[s], kvh * AF_HD + p * 64, t0 + j * AF_BKV);
                }
                ok = mbar_wait(v_empty, (j & 1) ^ 1);
                if (!ok) break;
                uint8_t* dv = smem + AS_OFF_V;
                mbar_expect_tx(v_full, AF_KV_STAGE);
                for (int p = 0; p < 2; p++) {
                    af_tma_2d(dv + p * 8192, &mV1, v_full, kvh * AF_HD + p * 64, t0 + j * AF_BKV);
                    af_tma_2d(dv + 16384 + p * 8192, &mV2, v_full, kvh * AF_HD + p * 64, t0 + j * AF_BKV);
                }
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(AF_BKV >> 3) << 17) | ((uint32_t)(AF_BQ >> 4) << 24);
            const uint32_t sq = smem_u32(smem), sdo = smem_u32(smem + AS_OFF_DO), sv = smem_u32(smem + AS_OFF_V);
            ok = mbar_wait(q_full, 0);
            for (int j = 0; j < nkv && ok; j++) {
                const int s = j & 1, u = j >> 1;
                ok = mbar_wait(&acc_empty[s], (u & 1) ^ 1) && mbar_wait(&k_full[s], u & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sk = smem_u32(smem + AS_OFF_K + s * AF_KV_STAGE);
#pragma unroll
                for (int p = 0; p < 2; p++) {
                    const uint64_t a1 = make_kmajor_desc<128>(sq + p * 16384), a2 = make_kmajor_desc<128>(sq + 32768 + p * 16384);
                    const uint64_t b1 = make_kmajor_desc<128>(sk + p * 8192), b2 = make_kmajor_desc<128>(sk + 16384 + p * 8192);
                    const uint32_t d = tmem_base + (uint32_t)(s * 256 + p * 64);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t adv = (uint64_t)(kk * 2);
                        af_mma_f16(d, a1 + adv, b1 + adv, idesc, kk ? 1u : 0u);
                        af_mma_f16(d, a2 + adv, b1 + adv, idesc, 1);
                        af_mma_f16(d, a1 + adv, b2 + adv, idesc, 1);
                    }
                }
                tc_commit(&k_empty[s]);
                ok = mbar_wait(v_full, j & 1);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int p = 0; p < 2; p++) {
                    const uint64_t a1 = make_kmajor_desc<128>(sdo + p * 16384), a2 = make_kmajor_desc<128>(sdo + 32768 + p * 16384);
                    const uint64_t b1 = make_kmajor_desc<128>(sv + p * 8192), b2 = make_kmajor_desc<128>(sv + 16384 + p * 8192);
                    const uint32_t d = tmem_base + (uint32_t)(s * 256 + 128 + p * 64);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t adv = (uint64_t)(kk * 2);
                        af_mma_f16(d, a1 + adv, b1 + adv, idesc, kk ? 1u : 0u);
                        af_mma_f16(d, a2 + adv, b1 + adv, idesc, 1);
                        af_mma_f16(d, a1 + adv, b2 + adv, idesc, 1);
                    }
                }
                tc_commit(v_empty);
                tc_commit(&acc_full[s]);
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else if (warp >= 4) {
        // ---------------- elementwise: one query row and 32 of the block's 64 keys per thread ----------------
        const int q = warp & 3, r = q * 32 + lane, half = (warp - 4) >> 2;
        const int qi = qb * AF_BQ + r;
        const bool live = qi < S;
        const float cs = tc_pow2(-tc_f16_shift(__ldg(amax_q))) * tc_pow2(-tc_f16_shift(__ldg(amax_k))) * (scale * 1.4426950408889634f);
        const float cp = tc_pow2(-tc_f16_shift(__ldg(amax_do))) * tc_pow2(-tc_f16_shift(__ldg(amax_v)));
        const float dsc = tc_pow2(tc_f16_shift(__ldg(ds_bound))) * scale * (1.0f / 16384.f);      // pr holds P * 2^14
        const float L2 = live ? lse[(size_t)(t0 + qi) * Hq + h] * 1.4426950408889634f : 0.f;
        const float Dq = live ? D[(size_t)(t0 + qi) * Hq + h] : 0.f;
        // after the transpose: lane (a, c) = (lane / 4, lane % 4) writes chunk c of the warp's rows 4a + t, t = 0..3
        const size_t qrowbase = ((size_t)hb * Sp + (size_t)(qb * AF_BQ + q * 32 + 4 * (lane >> 2))) * Sp + half * 32 + (lane & 3) * 8;
        for (int j = 0; j < nz && ok; j++) {
            uint4 w[4][4];                                      // P1, P2, dS1, dS2: 32 halfs each
            if (j < nkv) {
                const int s = j & 1, u = j >> 1;
                ok = mbar_wait(&acc_full[s], u & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * 256 + half * 32);
                float pr[32];
                {
                    uint32_t a[32], c[32];
                    uint32_t a2[32], c2[32];
                    af_ld32_issue(ta, a);
                    af_ld32_issue(ta + 64, c);
                    af_ld32_issue(ta + 128, a2);
                    af_ld32_issue(ta + 192, c2);
                    af_ld_wait(a); af_ld_dep(c); af_ld_dep(a2); af_ld_dep(c2);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) af_arrive(&acc_empty[s]);
                    const int k0 = j * AF_BKV + half * 32;
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const float y = fmaf(__uint_as_float(a[i]) + __uint_as_float(c[i]), cs, 14.f - L2);
                        pr[i] = (live && k0 + i <= qi) ? af_ex2(y) : 0.f;                   // P * 2^14
                    }
                    uint32_t* w0 = (uint32_t*)&w[0][0]; uint32_t* w1 = (uint32_t*)&w[1][0];
                    uint32_t* w2 = (uint32_t*)&w[2][0]; uint32_t* w3 = (uint32_t*)&w[3][0];
#pragma unroll
                    for (int e = 0; e < 16; e++) {
                        const float p0 = pr[2 * e], p1 = pr[2 * e + 1];
                        const float d0 = p0 * ((__uint_as_float(a2[2 * e]) + __uint_as_float(c2[2 * e])) * cp - Dq) * dsc;
                        const float d1 = p1 * ((__uint_as_float(a2[2 * e + 1]) + __uint_as_float(c2[2 * e + 1])) * cp - Dq) * dsc;
                        af_split2(p0, p1, w0[e], w1[e]);
                        af_split2(d0, d1, w2[e], w3[e]);
                    }
                }
            } else {
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int i = 0; i < 4; i++) w[a][i] = make_uint4(0, 0, 0, 0);
            }
            // A lane holds 64 bytes of its own row per array; lanes 4a..4a+3 transpose their 4 x 4 chunks of 16 bytes so that one
            // store instruction writes whole 64-byte row pieces (8 rows) instead of one chunk in each of 32 rows.
            if (j < nkv) {
#pragma unroll
                for (int a = 0; a < 4; a++) af_quad_transpose(w[a], lane);
            }
            const size_t o = qrowbase + (size_t)j * AF_BKV;
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const size_t ot = o + (size_t)t * Sp;
                *(uint4*)(P1 + ot) = w[0][t]; *(uint4*)(P2 + ot) = w[1][t]; *(uint4*)(dS1 + ot) = w[2][t]; *(uint4*)(dS2 + ot) = w[3][t];
            }
        }
        if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// q1/q2, k1/k2, v1/v2: the FP16 parts of Q [T, Hq*128], K and V [T, Hkv*128]; amax_*: the device words their scales derive from.
// Returns 0 when the kernel was launched, 1 when this path does not take the call.
extern "C" int sb_attention_fused_forward(sb_ctx_t* c, const void* q1, const void* q2, const void* k1, const void* k2,
                                          const void* v1, const void* v2, const float* amax_q, const float* amax_k, const float* amax_v,
                                          float* O, float* lse, int T, int Hq, int Hkv, int hd) {
    if (hd != AF_HD || c->h_seq_n <= 0 || c->h_seq_n > AF_MAXSEQ || Hq % Hkv) return 1;
    if (!tc_aligned16(O) || !tc_load_encode()) return 1;
    static bool attr_done = false;
    if (!attr_done) {
        if (cudaFuncSetAttribute(at_fused_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AF_SMEM) != cudaSuccess) { cudaGetLastError(); return 1; }
        attr_done = true;
    }
    AfSeqs seqs;
    seqs.n = c->h_seq_n;
    int Smax = 0;
    for (int b = 0; b <= c->h_seq_n; b++) seqs.start[b] = c->h_seq[b];
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    if (Smax <= 0) return 1;
    const int nqb = (Smax + AF_BQ - 1) / AF_BQ;
    const int qd = Hq * hd, kvd = Hkv * hd;
    CUtensorMap mQ1, mQ2, mK1, mK2, mV1, mV2;
    if (!af_make_map(&mQ1, q1, T, qd, AF_BQ) || !af_make_map(&mQ2, q2, T, qd, AF_BQ) ||
        !af_make_map(&mK1, k1, T, kvd, AF_BKV) || !af_make_map(&mK2, k2, T, kvd, AF_BKV) ||
        !af_make_map(&mV1, v1, T, kvd, AF_BKV) || !af_make_map(&mV2, v2, T, kvd, AF_BKV)) return 1;
    const long blocks = (long)nqb * seqs.n * Hq;
    if (blocks > 0x7fffffffL) return 1;
    at_fused_fwd_kernel<<<(unsigned)blocks, AF_THREADS, AF_SMEM, (cudaStream_t)c->pub.stream>>>(
        mQ1, mQ2, mK1, mK2, mV1, mV2, seqs, O, lse, amax_q, amax_k, amax_v, Hq, Hq / Hkv, nqb, 1.0f / sqrtf((float)hd), c->d_status,
        sb_amax_take(c, O, (size_t)T * qd));
    c->launches++;
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// The backward score kernel.  nb > 0: one sequence [t0, t0 + S) and the heads head0, head0 + head_step, ... (nb of them), the
// parts P1..dS2 laid out [nb][Sp][Sp].  nb == 0: every sequence and head of the batch in one launch, parts laid out
// [sequence][group member][K-V head][Sp][Sp] (t0, S, head0, head_step unused).  Returns 0 when launched.
extern "C" int sb_attention_fused_scores(sb_ctx_t* c, const void* q1, const void* q2, const void* do1, const void* do2,
                                         const void* k1, const void* k2, const void* v1, const void* v2,
                                         const float* amax_q, const float* amax_k, const float* amax_v, const float* amax_do, const float* ds_bound,
                                         const float* lse, const float* D, void* P1, void* P2, void* dS1, void* dS2,
                                         int t0, int S, int Sp, int T, int Hq, int Hkv, int hd, int head0, int head_step, int nb) {
    if (hd != AF_HD || (Sp % 256) || nb < 0 || !tc_load_encode()) return 1;
    if (nb > 0 && S <= 0) return 1;
    if (nb == 0 && (c->h_seq_n <= 0 || c->h_seq_n > AF_MAXSEQ)) return 1;
    static bool attr_done = false;
    if (!attr_done) {
        if (cudaFuncSetAttribute(at_score_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AS_SMEM) != cudaSuccess) { cudaGetLastError(); return 1; }
        attr_done = true;
    }
    AfSeqs seqs;
    int Smax = S;
    if (nb > 0) { seqs.n = 1; seqs.start[0] = t0; seqs.start[1] = t0 + S; }
    else {
        seqs.n = c->h_seq_n; Smax = 0;
        for (int b = 0; b <= c->h_seq_n; b++) seqs.start[b] = c->h_seq[b];
        for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
        if (Smax <= 0) return 1;
    }
    const int qd = Hq * hd, kvd = Hkv * hd, nqb = (Smax + AF_BQ - 1) / AF_BQ;
    CUtensorMap mQ1, mQ2, mD1, mD2, mK1, mK2, mV1, mV2;
    if (!af_make_map(&mQ1, q1, T, qd, AF_BQ) || !af_make_map(&mQ2, q2, T, qd, AF_BQ) ||
        !af_make_map(&mD1, do1, T, qd, AF_BQ) || !af_make_map(&mD2, do2, T, qd, AF_BQ) ||
        !af_make_map(&mK1, k1, T, kvd, AF_BKV) || !af_make_map(&mK2, k2, T, kvd, AF_BKV) ||
        !af_make_map(&mV1, v1, T, kvd, AF_BKV) || !af_make_map(&mV2, v2, T, kvd, AF_BKV)) return 1;
    const long blocks = (long)nqb * seqs.n * (nb > 0 ? nb : Hq);
    if (blocks > 0x7fffffffL) return 1;
    at_score_bwd_kernel<<<(unsigned)blocks, AS_THREADS, AS_SMEM, (cudaStream_t)c->pub.stream>>>(
        mQ1, mQ2, mD1, mD2, mK1, mK2, mV1, mV2, lse, D, (__half*)P1, (__half*)P2, (__half*)dS1, (__half*)dS2,
        amax_q, amax_k, amax_v, amax_do, ds_bound, seqs, Sp, Hq, Hq / Hkv, head0, head_step, nb, nqb, 1.0f / sqrtf((float)hd), c->d_status);
    c->launches++;
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
