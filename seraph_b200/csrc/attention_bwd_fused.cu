// attention_bwd_fused.cu - causal attention backward with dK and dV kept on chip (head size 128, FP16 hi/lo parts,
// FP32-level accuracy).  Replaces batch_attention_backward_packed_kernel / flash_attention_bwd_packed_kernel of the
// reference (src/cuda_train_context.cu:1013, :2012), which add into dK and dV with float atomics from every query tile.
//
// One CTA owns 128 consecutive keys of one (sequence, K/V head) for its whole life: the FP16 parts of those rows of V
// stay in shared memory (64 KB), those of K in tensor memory (128 columns), where they are the A operand of the S^T
// product: an MMA of 32 queries then reads 1 KB instead of 5 KB from shared memory, which is what its time went by.
// The CTA walks over the query heads of the K/V head's group and, for each, over the sequence's queries from the
// diagonal to the end in blocks of 32 (Q and dO parts, 32 KB per block, three stages):
//
//   S^T  = K Q_j^T,  dP^T = V dO_j^T     tcgen05.mma kind::f16, M 128 (keys) x N 32 (queries) x K 128, three passes each
//                                        (k1 q1 + k2 q1 + k1 q2), accumulators in tensor memory, two buffers
//   P^T  = exp(S^T/sqrt(hd) - lse),  dS^T = P^T o (dP^T - D)/sqrt(hd)      by the elementwise warps, one key row per
//                                        thread; both go BACK INTO TENSOR MEMORY as FP16 hi/lo parts, over the very
//                                        columns S^T and dP^T came from (tcgen05.st), to be the A operand of
//   dV  += P^T dO_j,  dK += dS^T Q_j     M 128 (keys) x N 128 (head dim) x K 32 (queries), A from tensor memory, B = the
//                                        same Q / dO tiles read in place MN-major; accumulators of 128 columns each in
//                                        tensor memory, summed over the query blocks and heads
//
// The tensor core adds into its accumulator with truncation, so a chain of accumulation is cut after AB_DRAIN query
// blocks: four drain warps read dK and dV out of tensor memory and add them into the output (round to nearest,
// performed in L2).  A dK/dV element is only ever touched by the one CTA that owns its key, one chain's additions have
// been performed before the next chain's are issued, and the output is zeroed (or holds the caller's values) before the
// launch: the result does not depend on scheduling and is the same bits on every run.
// dS^T also leaves the chip, as FP16 parts laid out [head slot = (sequence, K/V head, group member)][key][query]: dQ = dS K is one more product on the
// GEMM kernel (M = queries, K = keys up to the diagonal, A read MN-major).  P never reaches memory, dS is written once
// and read once: 8 bytes per score element instead of the 20 of the score-materialising path.
//
// Everything that leaves the CTA goes through shared memory and the TMA unit.  With one key row per thread (the layout
// tensor memory gives), a warp's direct stores and reductions touch 32 different rows per instruction, 32 memory
// transactions each; cycle counters in the warps showed the load/store unit busy two thirds of a step with them and the
// elementwise warps, which bound the step, waiting on it.  So the elementwise warps stage a step's dS^T parts in shared memory
// and one thread stores them as two tiles of 128 keys x 32 queries (a store per warp cost the issuing lane 500 cycles a step: the
// TMA unit takes few, large requests), each drain warp stages 32 rows x 32 columns of a chain at a time
// (128-byte swizzle, conflict-free for row-per-lane writes) and adds it with a TMA reduction, and the log-sum-exp and the row
// dot products D are read from copies transposed to [sequence][head][query] (at_lse_d_rows_kernel), 16 consecutive queries as
// four 16-byte loads from one address for the whole warp.  A key block that reaches past its sequence's end keeps the
// per-thread reductions, so that no CTA ever adds (even a zero) into a row of the next sequence.
//
// Warps (16): 0 TMA producer, 1 MMA issuer (owns the tensor-memory allocation), 4-11 elementwise (a lane quarter and half of
// a step's queries each), 12-15 drain.  Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA drains
// and frees its tensor memory.
#include <type_traits>
#include "attention_fused.cuh"

#define AB_BK 128                 // keys per CTA
#define AB_BQ 32                  // queries per step
#define AB_STAGES 3
#define AB_THREADS 512
#define AB_DRAIN 8                // steps per accumulation chain in tensor memory (8 x 12 instructions: 3e-6 of one-sided truncation)
#define AB_KV_BYTES 65536         // the parts of 128 rows of V: 2 parts x 2 halves of the head dimension x 128 x 128 B
#define AB_OFF_V 0
#define AB_OFF_ST AB_KV_BYTES
#define AB_STAGE_BYTES 32768      // Q parts 16 KB, dO parts 16 KB
#define AB_OFF_EWS (AB_OFF_ST + AB_STAGES * AB_STAGE_BYTES)      // dS^T staging: 2 buffers x (hi tile 8 KB, lo tile 8 KB); a tile is 128 keys x 32 queries (64-byte rows)
#define AB_OFF_DRS (AB_OFF_EWS + 2 * 16384)                      // per drain warp 2 buffers x 4 KB: 32 rows x 32 floats, 128-byte swizzle
                                                                 // (before the first step these 64 KB receive the parts of K on their way to tensor memory)
#define AB_OFF_BAR (AB_OFF_DRS + 4 * 8192)
#define AB_SMEM (AB_OFF_BAR + 1024 + 1024)
#define AB_REGS_LIGHT 72          // producer / MMA issuer warpgroup
#define AB_REGS_EW 120             // the two elementwise warpgroups
#define AB_REGS_DRAIN 200          // the drain warpgroup holds 128 accumulator values at a time   (128*72 + 256*120 + 128*200 = 65536)
// tensor-memory columns: dK 0..127, dV 128..255, the parts of K 256..383 (for each k-step of 16 head-dimension elements, 8 columns
// of hi parts then 8 of lo parts, two halfs per column), then per buffer e: S^T at 384 + 64 e (32 columns, one per query), dP^T 32
// further.  The FP16 parts of P^T and dS^T replace them in place: for each k-step of 16 queries, 8 columns of hi parts then 8 of lo parts.
#define AB_COL_DK 0
#define AB_COL_DV 128
#define AB_COL_K 256
#define AB_COL_S(e) (384 + 64 * (e))
#define AB_COL_DP(e) (384 + 64 * (e) + 32)

// A from tensor memory (M 128 lanes, 16 halfs of k = 8 columns), B from shared memory
__device__ __forceinline__ void ab_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ab_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
#define AB_REGS16(r) "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), \
                     "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
__device__ __forceinline__ void ab_ld_wait2(uint32_t (&a)[16], uint32_t (&b)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : AB_REGS16(a), AB_REGS16(b) :: "memory");
}
__device__ __forceinline__ void ab_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void ab_red4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void ab_sts4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// tile in shared memory -> global memory through a tensor map, as a store or as an FP32 addition; completion by bulk group
__device__ __forceinline__ void ab_tma_store(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}
__device__ __forceinline__ void ab_tma_add(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}
#define AB_BULK_COMMIT() asm volatile("cp.async.bulk.commit_group;" ::: "memory")
#define AB_BULK_WAIT_READ(n) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(n) : "memory")
#define AB_BULK_WAIT(n) asm volatile("cp.async.bulk.wait_group %0;" ::"n"(n) : "memory")
#define AB_FENCE_ASYNC() asm volatile("fence.proxy.async.shared::cta;" ::: "memory")

// lse and D, [token][head], as [sequence][head][Sp queries] (zeros past the sequence's end), in the form the elementwise warps use:
// 14 - lse log2(e) (the probabilities are formed times 2^14) and D times the factor that takes P 2^14 (dP - D) to the scaled dS
__global__ void at_lse_d_rows_kernel(const float* __restrict__ lse, const float* __restrict__ D, float* __restrict__ LT, float* __restrict__ DT,
                                     const __grid_constant__ AfSeqs seqs, int Hq, int Sp, const float* __restrict__ ds_bound, float scale) {
    const size_t n = (size_t)seqs.n * Hq * Sp;
    const float dsc = tc_pow2(tc_f16_shift(__ldg(ds_bound))) * scale * (1.0f / 16384.f);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int q = (int)(i % Sp), h = (int)((i / Sp) % Hq), b = (int)(i / ((size_t)Sp * Hq));
        const int t0 = seqs.start[b], S = seqs.start[b + 1] - t0;
        float l = 0.f, d = 0.f;
        if (q < S) { l = 14.f - __ldg(&lse[(size_t)(t0 + q) * Hq + h]) * 1.4426950408889634f; d = __ldg(&D[(size_t)(t0 + q) * Hq + h]) * dsc; }
        LT[i] = l; DT[i] = d;
    }
}

__global__ void __launch_bounds__(AB_THREADS, 1)
at_dkv_bwd_kernel(const __grid_constant__ CUtensorMap mQ1, const __grid_constant__ CUtensorMap mQ2,
                  const __grid_constant__ CUtensorMap mD1, const __grid_constant__ CUtensorMap mD2,
                  const __grid_constant__ CUtensorMap mK1, const __grid_constant__ CUtensorMap mK2,
                  const __grid_constant__ CUtensorMap mV1, const __grid_constant__ CUtensorMap mV2,
                  const __grid_constant__ CUtensorMap mS1, const __grid_constant__ CUtensorMap mS2,
                  const __grid_constant__ CUtensorMap mdK, const __grid_constant__ CUtensorMap mdV,
                  const float* __restrict__ LT, const float* __restrict__ DT,
                  __half* __restrict__ dS1, __half* __restrict__ dS2, float* __restrict__ dK, float* __restrict__ dV,
                  const float* __restrict__ amax_q, const float* __restrict__ amax_k, const float* __restrict__ amax_v,
                  const float* __restrict__ amax_do, const float* __restrict__ ds_bound,
                  const __grid_constant__ AfSeqs seqs, int Sp, int Hq, int g, int nkb, int chunk, float scale, int* status) {
    // which (key block, sequence, K/V head).  Key blocks from the start of the sequences have the most queries, so the launch runs
    // in up to four phases over ranges of key blocks, the longest first, and ends on CTAs of a few steps that fill the last wave.
    // Inside a phase the (sequence, head) pairs are taken `chunk` at a time, so that the Q and dO parts the CTAs in flight read
    // again and again (once per key block) stay in L2.
    const int Hkv = Hq / g;
    const int pairs = seqs.n * Hkv;
    const int nph = min(4, nkb);
    int bid = (int)blockIdx.x, ph = 0;
    while (ph + 1 < nph && bid >= pairs * ((ph + 1) * nkb / nph - ph * nkb / nph)) { bid -= pairs * ((ph + 1) * nkb / nph - ph * nkb / nph); ph++; }
    const int kb_lo = ph * nkb / nph, nk = (ph + 1) * nkb / nph - kb_lo;
    const int ci = bid / (chunk * nk);
    const int in_chunk = min(chunk, pairs - ci * chunk);
    const int cr = bid - ci * chunk * nk;
    const int kb = kb_lo + cr / in_chunk;
    const int rem = ci * chunk + cr % in_chunk;
    const int b = rem / Hkv, kvh = rem % Hkv;
    const int t0 = seqs.start[b], S = seqs.start[b + 1] - t0;
    const int k0 = kb * AB_BK;
    if (kb >= nkb || k0 >= S) return;
    if (*(volatile int*)status != 0) return;
    const int nq = (S + AB_BQ - 1) / AB_BQ, j0 = k0 / AB_BQ, per_head = nq - j0;
    const int nsteps = g * per_head;
    const int nchains = (nsteps + AB_DRAIN - 1) / AB_DRAIN;
    const int kvd = Hkv * AF_HD;

    extern __shared__ uint8_t af_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)af_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + AB_OFF_BAR);
    uint64_t* kv_full = bars;                          // 1: V in shared memory
    uint64_t* full = bars + 1;                         // AB_STAGES
    uint64_t* empty = full + AB_STAGES;                // AB_STAGES
    uint64_t* sdp_full = empty + AB_STAGES;            // 2
    uint64_t* p_full = sdp_full + 2;                   // 2
    uint64_t* acc_ready = p_full + 2;                  // 1
    uint64_t* acc_free = acc_ready + 1;                // 1
    uint64_t* k_ready = acc_free + 1;                  // 1: K in tensor memory
    uint64_t* k_full = k_ready + 1;                    // 1: K in shared memory, on its way there
    uint64_t* ew_sync = k_full + 1;                    // 1: the elementwise warps have staged their rows of a step's dS^T tiles
    uint32_t* tmem_slot = (uint32_t*)(ew_sync + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1); mbar_init(acc_ready, 1); mbar_init(acc_free, 4); mbar_init(k_ready, 8); mbar_init(k_full, 1); mbar_init(ew_sync, 8);
        for (int i = 0; i < AB_STAGES; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&sdp_full[i], 1); mbar_init(&p_full[i], 8); }
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

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(AB_REGS_LIGHT));
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            if (elect_one()) {
                mbar_expect_tx(k_full, AB_KV_BYTES);
                for (int p = 0; p < 2; p++) {
                    af_tma_2d(smem + AB_OFF_EWS + p * 16384, &mK1, k_full, kvh * AF_HD + p * 64, t0 + k0);
                    af_tma_2d(smem + AB_OFF_EWS + 32768 + p * 16384, &mK2, k_full, kvh * AF_HD + p * 64, t0 + k0);
                }
                mbar_expect_tx(kv_full, AB_KV_BYTES);
                for (int p = 0; p < 2; p++) {
                    af_tma_2d(smem + AB_OFF_V + p * 16384, &mV1, kv_full, kvh * AF_HD + p * 64, t0 + k0);
                    af_tma_2d(smem + AB_OFF_V + 32768 + p * 16384, &mV2, kv_full, kvh * AF_HD + p * 64, t0 + k0);
                }
                for (int t = 0; t < nsteps && ok; t++) {
                    const int s = t % AB_STAGES, u = t / AB_STAGES;
                    const int h = kvh * g + t / per_head, j = j0 + t % per_head;
                    ok = mbar_wait(&empty[s], (u & 1) ^ 1);
                    if (!ok) break;
                    uint8_t* st = smem + AB_OFF_ST + s * AB_STAGE_BYTES;
                    mbar_expect_tx(&full[s], AB_STAGE_BYTES);
                    for (int p = 0; p < 2; p++) {
                        af_tma_2d(st + p * 4096, &mQ1, &full[s], h * AF_HD + p * 64, t0 + j * AB_BQ);
                        af_tma_2d(st + 8192 + p * 4096, &mQ2, &full[s], h * AF_HD + p * 64, t0 + j * AB_BQ);
                        af_tma_2d(st + 16384 + p * 4096, &mD1, &full[s], h * AF_HD + p * 64, t0 + j * AB_BQ);
                        af_tma_2d(st + 24576 + p * 4096, &mD2, &full[s], h * AF_HD + p * 64, t0 + j * AB_BQ);
                    }
                }
                if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (elect_one()) {
                const uint32_t idesc_s = (1u << 4) | ((uint32_t)(AB_BQ >> 3) << 17) | ((uint32_t)(AB_BK >> 4) << 24);
                const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(AF_HD >> 3) << 17) | ((uint32_t)(AB_BK >> 4) << 24);
                const uint32_t sv = smem_u32(smem + AB_OFF_V), tk = tmem_base + AB_COL_K;
                ok = mbar_wait(kv_full, 0) && mbar_wait(k_ready, 0);
                for (int t = 0; t <= nsteps && ok; t++) {
                    if (t < nsteps) {
                        // S^T and dP^T of step t into buffer t & 1 (its parts of step t - 2 were consumed by instructions issued before these)
                        const int s = t % AB_STAGES, e = t & 1;
                        ok = mbar_wait(&full[s], (t / AB_STAGES) & 1);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t st = smem_u32(smem + AB_OFF_ST + s * AB_STAGE_BYTES);
                        {                                          // S^T: K parts from tensor memory
                            const uint32_t d = tmem_base + (uint32_t)AB_COL_S(e);
#pragma unroll
                            for (int p = 0; p < 2; p++) {
                                const uint64_t b1 = make_kmajor_desc<128>(st + p * 4096), b2 = make_kmajor_desc<128>(st + 8192 + p * 4096);
#pragma unroll
                                for (int kk = 0; kk < 4; kk++) {
                                    const uint64_t adv = (uint64_t)(kk * 2);
                                    const uint32_t ta = tk + (uint32_t)((p * 4 + kk) * 16);
                                    ab_mma_ts(d, ta, b1 + adv, idesc_s, (p | kk) ? 1u : 0u);
                                    ab_mma_ts(d, ta + 8, b1 + adv, idesc_s, 1);
                                    ab_mma_ts(d, ta, b2 + adv, idesc_s, 1);
                                }
                            }
                        }
                        {                                          // dP^T: V parts from shared memory
                            const uint32_t sb = st + 16384;
                            const uint32_t d = tmem_base + (uint32_t)AB_COL_DP(e);
#pragma unroll
                            for (int p = 0; p < 2; p++) {
                                const uint64_t a1 = make_kmajor_desc<128>(sv + p * 16384), a2 = make_kmajor_desc<128>(sv + 32768 + p * 16384);
                                const uint64_t b1 = make_kmajor_desc<128>(sb + p * 4096), b2 = make_kmajor_desc<128>(sb + 8192 + p * 4096);
#pragma unroll
                                for (int kk = 0; kk < 4; kk++) {
                                    const uint64_t adv = (uint64_t)(kk * 2);
                                    af_mma_f16(d, a1 + adv, b1 + adv, idesc_s, (p | kk) ? 1u : 0u);
                                    af_mma_f16(d, a2 + adv, b1 + adv, idesc_s, 1);
                                    af_mma_f16(d, a1 + adv, b2 + adv, idesc_s, 1);
                                }
                            }
                        }
                        tc_commit(&sdp_full[e]);
                    }
                    if (t >= 1) {
                        // dV += P^T dO and dK += dS^T Q of step t - 1
                        const int u = t - 1, e = u & 1, s = u % AB_STAGES;
                        ok = mbar_wait(&p_full[e], (u >> 1) & 1);
                        if (!ok) break;
                        const bool first = (u % AB_DRAIN) == 0;
                        if (first && u > 0) {                        // the drain warps have read the previous chain out
                            ok = mbar_wait(acc_free, (u / AB_DRAIN - 1) & 1);
                            if (!ok) break;
                        }
                        tc_fence_after();
                        const uint32_t st = smem_u32(smem + AB_OFF_ST + s * AB_STAGE_BYTES);
#pragma unroll
                        for (int prod = 0; prod < 2; prod++) {
                            const uint32_t ta = tmem_base + (uint32_t)(prod ? AB_COL_DP(e) : AB_COL_S(e));      // per k-step of 16 queries: hi part 8 columns, lo part the next 8
                            const uint32_t sb = st + (prod ? 0 : 16384);                                       // dK takes Q, dV takes dO
                            const uint64_t b1 = make_mn16_desc<AB_BQ>(sb), b2 = make_mn16_desc<AB_BQ>(sb + 8192);
                            const uint32_t d = tmem_base + (uint32_t)(prod ? AB_COL_DK : AB_COL_DV);
#pragma unroll
                            for (int kk = 0; kk < 2; kk++) {
                                const uint64_t advb = (uint64_t)(kk * 128);
                                ab_mma_ts(d, ta + kk * 16, b1 + advb, idesc_o, (first && kk == 0) ? 0u : 1u);
                                ab_mma_ts(d, ta + kk * 16 + 8, b1 + advb, idesc_o, 1);
                                ab_mma_ts(d, ta + kk * 16, b2 + advb, idesc_o, 1);
                            }
                        }
                        tc_commit(&empty[s]);
                        if (((u + 1) % AB_DRAIN) == 0 || u == nsteps - 1) tc_commit(acc_ready);
                    }
                }
                if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
            }
        }
    } else if (warp >= 12) {
        // ---------------- drain: dK and dV chains out of tensor memory, added into the output ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(AB_REGS_DRAIN));
        {
            const int q = warp & 3, r = q * 32 + lane, kg = k0 + r;
            const bool live = kg < S;
            // dV accumulates (P 2^14) (dO 2^s_do), dK accumulates (dS 2^s_ds) (Q 2^s_q)
            const float fv = tc_pow2(-14) * tc_pow2(-tc_f16_shift(__ldg(amax_do)));
            const float fk = tc_pow2(-tc_f16_shift(__ldg(ds_bound))) * tc_pow2(-tc_f16_shift(__ldg(amax_q)));
            float* rowk = dK + (size_t)(t0 + (live ? kg : 0)) * kvd + (size_t)kvh * AF_HD;
            float* rowv = dV + (size_t)(t0 + (live ? kg : 0)) * kvd + (size_t)kvh * AF_HD;
            const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16);
            const bool whole = k0 + AB_BK <= S;                // all 128 keys belong to this sequence: tiles through the TMA unit
            ok = mbar_wait(k_ready, 0);                         // the staging area held the parts of K until now
            const uint32_t stg = smem_u32(smem + AB_OFF_DRS + q * 8192);
            const int row0 = t0 + k0 + q * 32, col0 = kvh * AF_HD;
            int pieces = 0;                                     // tiles this warp has handed to the TMA unit
            for (int c = 0; c < nchains && ok; c++) {
                ok = mbar_wait(acc_ready, c & 1);
                if (!ok) break;
                tc_fence_after();
                if (whole && c > 0) {                           // the previous chain's additions have been performed: one order per element
                    if (lane == 0) AB_BULK_WAIT(0);
                    __syncwarp();
                }
#pragma unroll
                for (int which = 0; which < 2; which++) {          // dK (columns 0..127), then dV (128..255): four loads in flight, one wait
                    uint32_t v0[32], v1[32], v2[32], v3[32];
                    af_ld32_issue(ta + (uint32_t)(which * 128), v0);
                    af_ld32_issue(ta + (uint32_t)(which * 128 + 32), v1);
                    af_ld32_issue(ta + (uint32_t)(which * 128 + 64), v2);
                    af_ld32_issue(ta + (uint32_t)(which * 128 + 96), v3);
                    af_ld_wait(v0); af_ld_dep(v1); af_ld_dep(v2); af_ld_dep(v3);
                    if (which == 1) {                               // everything is in registers: the next chain may overwrite the accumulators
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) af_arrive(acc_free);
                    }
                    const float f = which ? fv : fk;
                    if (whole) {
#define AB_STAGE_PIECE(v, pc)                                                                                                              \
                        {                                                                                                                  \
                            const uint32_t buf = stg + (uint32_t)((pieces & 1) * 4096);                                                    \
                            if (pieces >= 2) { if (lane == 0) AB_BULK_WAIT_READ(1); __syncwarp(); }     /* the tile staged here two pieces ago has been read */ \
                            _Pragma("unroll")                                                                                              \
                            for (int i = 0; i < 8; i++)                                                                                    \
                                ab_sts4(buf + (uint32_t)(lane * 128 + ((i ^ (lane & 7)) << 4)),                                            \
                                        __float_as_uint(__uint_as_float(v[4 * i]) * f), __float_as_uint(__uint_as_float(v[4 * i + 1]) * f), \
                                        __float_as_uint(__uint_as_float(v[4 * i + 2]) * f), __float_as_uint(__uint_as_float(v[4 * i + 3]) * f)); \
                            AB_FENCE_ASYNC();                                                                                              \
                            __syncwarp();                                                                                                  \
                            if (lane == 0) { ab_tma_add(which ? &mdV : &mdK, buf, col0 + (pc) * 32, row0); AB_BULK_COMMIT(); }             \
                            pieces++;                                                                                                      \
                        }
                        AB_STAGE_PIECE(v0, 0) AB_STAGE_PIECE(v1, 1) AB_STAGE_PIECE(v2, 2) AB_STAGE_PIECE(v3, 3)
#undef AB_STAGE_PIECE
                    } else if (live) {
                        float* dst = which ? rowv : rowk;
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            ab_red4(dst + 4 * i, __uint_as_float(v0[4 * i]) * f, __uint_as_float(v0[4 * i + 1]) * f, __uint_as_float(v0[4 * i + 2]) * f, __uint_as_float(v0[4 * i + 3]) * f);
                            ab_red4(dst + 32 + 4 * i, __uint_as_float(v1[4 * i]) * f, __uint_as_float(v1[4 * i + 1]) * f, __uint_as_float(v1[4 * i + 2]) * f, __uint_as_float(v1[4 * i + 3]) * f);
                            ab_red4(dst + 64 + 4 * i, __uint_as_float(v2[4 * i]) * f, __uint_as_float(v2[4 * i + 1]) * f, __uint_as_float(v2[4 * i + 2]) * f, __uint_as_float(v2[4 * i + 3]) * f);
                            ab_red4(dst + 96 + 4 * i, __uint_as_float(v3[4 * i]) * f, __uint_as_float(v3[4 * i + 1]) * f, __uint_as_float(v3[4 * i + 2]) * f, __uint_as_float(v3[4 * i + 3]) * f);
                        }
                    }
                }
            }
            if (lane == 0) AB_BULK_WAIT_READ(0);               // the staging buffers are read out before the CTA gives its shared memory back
            if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else {
        // ---------------- elementwise: one key row and 16 of the step's 32 queries per thread (warps 4-7: queries 0..15, 8-11: 16..31) ----------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(AB_REGS_EW));
        const int ch = (warp - 4) >> 2, q = warp & 3, r = q * 32 + lane, kg = k0 + r;
        const float cs = tc_pow2(-tc_f16_shift(__ldg(amax_q))) * tc_pow2(-tc_f16_shift(__ldg(amax_k))) * (scale * 1.4426950408889634f);
        const float cp = tc_pow2(-tc_f16_shift(__ldg(amax_do))) * tc_pow2(-tc_f16_shift(__ldg(amax_v)));
        const float cpd = cp * (tc_pow2(tc_f16_shift(__ldg(ds_bound))) * scale * (1.0f / 16384.f));      // p holds P * 2^14
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        // This key row's parts of K from shared memory (four 128-byte-swizzled tiles: hi and lo part of each half of the head
        // dimension) into tensor memory: head-dimension k-steps ch*4 .. ch*4+3 are half `ch`, two consecutive halfs per column
        ok = mbar_wait(k_full, 0);
        {
            const uint32_t kt = smem_u32(smem + AB_OFF_EWS + ch * 16384) + (uint32_t)(r * 128);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                uint32_t h8[8], l8[8];
                const uint32_t c0 = (uint32_t)(((2 * kk) ^ (r & 7)) << 4), c1 = (uint32_t)(((2 * kk + 1) ^ (r & 7)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(h8[0]), "=r"(h8[1]), "=r"(h8[2]), "=r"(h8[3]) : "r"(kt + c0) : "memory");
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(h8[4]), "=r"(h8[5]), "=r"(h8[6]), "=r"(h8[7]) : "r"(kt + c1) : "memory");
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(l8[0]), "=r"(l8[1]), "=r"(l8[2]), "=r"(l8[3]) : "r"(kt + 32768 + c0) : "memory");
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(l8[4]), "=r"(l8[5]), "=r"(l8[6]), "=r"(l8[7]) : "r"(kt + 32768 + c1) : "memory");
                ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_K + (ch * 4 + kk) * 16), h8);
                ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_K + (ch * 4 + kk) * 16 + 8), l8);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) af_arrive(k_ready);
        }
        ok = ok && mbar_wait(k_ready, 0);                       // every warp has its rows of K out of the staging area
        const uint32_t ews = smem_u32(smem + AB_OFF_EWS);
        const bool issuer = warp == 4 && lane == 0;            // hands the staged tiles to the TMA unit
        // Columns before this key block that the dQ product reads together with it (its query tiles are 256 wide): zeros, stored
        // from a tile of zeros that sits where the second step will stage its hi parts
        // ew_sync counts one phase per hand-over: a warp arrives when its rows are staged; the issuing thread waits for all eight, and
        // before it arrives it makes sure that everything it handed over earlier has been read.  So a completed phase n tells every
        // warp that the tiles handed over in phases < n are read out: a buffer is written again one phase after the next.
        int sync_n = 0;
        if ((k0 & 255) != 0 && ok) {
            ab_sts4(ews + 16384 + (uint32_t)((warp - 4) * 1024 + lane * 32), 0, 0, 0, 0);
            ab_sts4(ews + 16384 + (uint32_t)((warp - 4) * 1024 + lane * 32 + 16), 0, 0, 0, 0);
            AB_FENCE_ASYNC();
            __syncwarp();
            if (lane == 0) af_arrive(ew_sync);
            if (warp == 4) {
                ok = mbar_wait(ew_sync, 0);
                if (issuer && ok) {
                    for (int hi = 0; hi < g; hi++) {
                        const int y = (int)(((size_t)(b * Hkv + kvh) * g + hi) * Sp) + k0;
                        for (int i = 0; i < 4; i++) { ab_tma_store(&mS1, ews + 16384, k0 - 128 + i * 32, y); ab_tma_store(&mS2, ews + 16384, k0 - 128 + i * 32, y); }
                    }
                    AB_BULK_COMMIT();
                }
            }
            sync_n = 1;
        }
        int hi = 0, j = j0;                                     // query head within the group, query block
        for (int t = 0; t < nsteps && ok; t++) {
            const int e = t & 1;
            const int q0 = j * AB_BQ;
            ok = mbar_wait(&sdp_full[e], (t >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const size_t hb = (size_t)(b * Hkv + kvh) * g + hi;
            uint32_t sr[16], dr[16];
            ab_ld16(tmem_base + lane_addr + (uint32_t)(AB_COL_S(e) + ch * 16), sr);
            ab_ld16(tmem_base + lane_addr + (uint32_t)(AB_COL_DP(e) + ch * 16), dr);
            // log-sum-exp (times log2 e) and D of this warp's 16 queries: the same addresses for every lane
            float4 L4[4], D4[4];
            {
                const size_t o = ((size_t)(b * Hq + kvh * g + hi)) * Sp + q0 + ch * 16;
                const float4* lp = (const float4*)(LT + o); const float4* dp = (const float4*)(DT + o);
#pragma unroll
                for (int i = 0; i < 4; i++) { L4[i] = __ldg(lp + i); D4[i] = __ldg(dp + i); }
            }
            ab_ld_wait2(sr, dr);
            uint32_t p1[8], p2[8], d1[8], d2[8];
            // away from the diagonal and from the sequence's end no element of the step is masked
            const bool nomask = q0 >= k0 + AB_BK && q0 + AB_BQ <= S && k0 + AB_BK <= S;
            auto columns = [&](auto masked) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    float pv[2], dv[2];
#pragma unroll
                    for (int w = 0; w < 2; w++) {
                        const int c = 2 * i + w;
                        const float4 l4 = L4[c >> 2], dq4 = D4[c >> 2];
                        const float Lq = (c & 3) == 0 ? l4.x : (c & 3) == 1 ? l4.y : (c & 3) == 2 ? l4.z : l4.w;      // 14 - lse log2 e
                        const float Dq = (c & 3) == 0 ? dq4.x : (c & 3) == 1 ? dq4.y : (c & 3) == 2 ? dq4.z : dq4.w;  // D dsc
                        const int qi = q0 + ch * 16 + c;
                        const bool valid = !decltype(masked)::value || (kg <= qi && qi < S && kg < S);
                        const float y = fmaf(__uint_as_float(sr[c]), cs, Lq);
                        pv[w] = valid ? af_ex2(y) : 0.f;                                             // P * 2^14
                        dv[w] = pv[w] * fmaf(__uint_as_float(dr[c]), cpd, -Dq);
                    }
                    af_split2(pv[0], pv[1], p1[i], p2[i]);
                    af_split2(dv[0], dv[1], d1[i], d2[i]);
                }
            };
            if (nomask) columns(std::false_type{}); else columns(std::true_type{});
            // The parts of these 16 queries go back over the 16 columns their scores came from (all of them are in registers by now):
            // hi part in the first 8 columns, lo part in the next 8, which is where the MMA issuer looks for k-step `ch`.
            ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_S(e) + ch * 16), p1);
            ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_S(e) + ch * 16 + 8), p2);
            ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_DP(e) + ch * 16), d1);
            ab_st8(tmem_base + lane_addr + (uint32_t)(AB_COL_DP(e) + ch * 16 + 8), d2);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) af_arrive(&p_full[e]);
            // dS^T parts of this key row, 16 queries = 32 bytes per part, into the step's two tiles (64-byte rows).  The issuing thread
            // first makes sure that everything it handed over earlier has been read (the other buffer is written in the next step),
            // then all eight warps meet and it hands this step's tiles to the TMA unit.
            {
                const uint32_t buf = ews + (uint32_t)(e * 16384);
                const uint32_t row = buf + (uint32_t)(r * 64 + ch * 32);
                if (warp != 4 && sync_n > 0) {                  // (the issuer's warp waited for this phase when it handed the tiles over)
                    ok = mbar_wait(ew_sync, (sync_n - 1) & 1);
                    if (!ok) break;
                }
                ab_sts4(row, d1[0], d1[1], d1[2], d1[3]); ab_sts4(row + 16, d1[4], d1[5], d1[6], d1[7]);
                ab_sts4(row + 8192, d2[0], d2[1], d2[2], d2[3]); ab_sts4(row + 8192 + 16, d2[4], d2[5], d2[6], d2[7]);
                AB_FENCE_ASYNC();
                __syncwarp();
                if (issuer) AB_BULK_WAIT_READ(0);
                if (lane == 0) af_arrive(ew_sync);
                if (warp == 4) {
                    ok = mbar_wait(ew_sync, sync_n & 1);
                    if (!ok) break;
                    if (issuer) {
                        const int y = (int)(hb * Sp) + k0;
                        ab_tma_store(&mS1, buf, q0, y); ab_tma_store(&mS2, buf + 8192, q0, y);
                        AB_BULK_COMMIT();
                    }
                }
                sync_n++;
            }
            if (++j == nq) { j = j0; hi++; }
        }
        if (issuer) AB_BULK_WAIT_READ(0);                      // the staging tiles are read out before the CTA gives its shared memory back
        if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// q, do, k, v: the FP16 parts of Q, dO [T, Hq*128] and K, V [T, Hkv*128]; amax_*: the device words their scales derive from;
// ds_bound: the device word that bounds |dS|.  dS1/dS2: the parts of dS^T, laid out [sequence][K-V head][group member][Sp][Sp]
// (key rows, query columns).  dK and dV are added into (the caller zeroes them when they do not accumulate).
// Returns 0 when the kernel was launched, 1 when this path does not take the call.
extern "C" int sb_attention_fused_dkv(sb_ctx_t* c, const void* q1, const void* q2, const void* do1, const void* do2,
                                      const void* k1, const void* k2, const void* v1, const void* v2,
                                      const float* amax_q, const float* amax_k, const float* amax_v, const float* amax_do, const float* ds_bound,
                                      const float* lse, const float* D, void* dS1, void* dS2, float* LT, float* DT, float* dK, float* dV,
                                      int Sp, int T, int Hq, int Hkv, int hd) {
    if (hd != AF_HD || (Sp % 256) || Hkv <= 0 || Hq % Hkv || !tc_load_encode()) return 1;
    if (c->h_seq_n <= 0 || c->h_seq_n > AF_MAXSEQ) return 1;
    if (!tc_aligned16(dK) || !tc_aligned16(dV)) return 1;
    static bool attr_done = false;
    if (!attr_done) {
        if (cudaFuncSetAttribute(at_dkv_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_SMEM) != cudaSuccess) { cudaGetLastError(); return 1; }
        attr_done = true;
    }
    AfSeqs seqs;
    seqs.n = c->h_seq_n;
    int Smax = 0;
    for (int b = 0; b <= c->h_seq_n; b++) seqs.start[b] = c->h_seq[b];
    for (int b = 0; b < c->h_seq_n; b++) Smax = max(Smax, c->h_seq[b + 1] - c->h_seq[b]);
    if (Smax <= 0 || Smax > Sp) return 1;
    const int qd = Hq * hd, kvd = Hkv * hd, nkb = (Smax + AB_BK - 1) / AB_BK;
    CUtensorMap mQ1, mQ2, mD1, mD2, mK1, mK2, mV1, mV2, mS1, mS2, mdK, mdV;
    if (!af_make_map(&mQ1, q1, T, qd, AB_BQ) || !af_make_map(&mQ2, q2, T, qd, AB_BQ) ||
        !af_make_map(&mD1, do1, T, qd, AB_BQ) || !af_make_map(&mD2, do2, T, qd, AB_BQ) ||
        !af_make_map(&mK1, k1, T, kvd, AB_BK) || !af_make_map(&mK2, k2, T, kvd, AB_BK) ||
        !af_make_map(&mV1, v1, T, kvd, AB_BK) || !af_make_map(&mV2, v2, T, kvd, AB_BK)) return 1;
    {
        // dS^T parts: [head slots x Sp keys][Sp queries] halfs, tiles of 32 queries x 128 keys, plain rows of 64 bytes in shared memory;
        // dK, dV: [T][kvd] floats, tiles of 32 columns x 32 keys, 128-byte swizzle
        const cuuint64_t slots = (cuuint64_t)seqs.n * Hq;
        cuuint64_t sd[2] = {(cuuint64_t)Sp, slots * (cuuint64_t)Sp}, ss[1] = {(cuuint64_t)Sp * 2};
        cuuint32_t sbx[2] = {32u, 128u}, est[2] = {1, 1};
        cuuint64_t gd[2] = {(cuuint64_t)kvd, (cuuint64_t)T}, gs[1] = {(cuuint64_t)kvd * 4};
        cuuint32_t gbx[2] = {32u, 32u};
        if (slots * (cuuint64_t)Sp > 0x7fffffffull || !tc_aligned16(dS1) || !tc_aligned16(dS2) ||
            g_tc_encode(&mS1, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dS1, sd, ss, sbx, est, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            g_tc_encode(&mS2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dS2, sd, ss, sbx, est, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            g_tc_encode(&mdK, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dK, gd, gs, gbx, est, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            g_tc_encode(&mdV, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dV, gd, gs, gbx, est, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 1;
    }
    const long blocks = (long)nkb * seqs.n * Hkv;
    // pairs per chunk: their Q and dO parts (8 bytes per element) within about a third of the L2
    const size_t pair_bytes = (size_t)(Hq / Hkv) * Smax * hd * 8;
    int chunk = (int)((size_t)(40u << 20) / pair_bytes);
    chunk = max(1, min(chunk, seqs.n * Hkv));
    if (blocks > 0x7fffffffL) return 1;
    {
        const size_t n = (size_t)seqs.n * Hq * Sp;
        at_lse_d_rows_kernel<<<(unsigned)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184), 256, 0, (cudaStream_t)c->pub.stream>>>(lse, D, LT, DT, seqs, Hq, Sp, ds_bound, 1.0f / sqrtf((float)hd));
        c->launches++;
    }
    at_dkv_bwd_kernel<<<(unsigned)blocks, AB_THREADS, AB_SMEM, (cudaStream_t)c->pub.stream>>>(
        mQ1, mQ2, mD1, mD2, mK1, mK2, mV1, mV2, mS1, mS2, mdK, mdV, LT, DT, (__half*)dS1, (__half*)dS2, dK, dV,
        amax_q, amax_k, amax_v, amax_do, ds_bound, seqs, Sp, Hq, Hq / Hkv, nkb, chunk, 1.0f / sqrtf((float)hd), c->d_status);
    c->launches++;
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
