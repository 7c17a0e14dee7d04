// gemm_tc.cuh - the tcgen05 GEMM kernel and its launcher, shared by the plain GEMM
// (gemm_tc.cu) and the attention path (attention_tc.cu).
//
//   C_b[M,N] (+)= A_b[M,K] * B_b[N,K]^T      for b in [0, nbatch)
//
// Both operands are K-major (rows of K contiguous floats, any 16-byte-multiple pitch) and are
// fetched by TMA through 3-D tensor maps {K, rows, batch-slot}; the slot of batch b is
// c2_base + b*c2_step, so one launch can walk over attention heads (and share one K/V head
// between the query heads of a GQA group).
//
// Arithmetic: tcgen05.mma kind::tf32, accumulator in tensor memory.
//   NTERMS = 3: FP32-accurate.  x = hi + lo, hi = the 19 leading bits the tensor core reads
//               from an FP32 word, lo = x - hi; the kernel issues hi*hi + lo*hi + hi*lo.
//   NTERMS = 1: single-pass TF32.
// The tensor core adds into its FP32 accumulator with truncation, so a long chain of
// accumulating MMAs drifts by about half an ulp per instruction, always towards zero (measured:
// 3e-5 relative after K = 4096 in one chain; 1.4e-6 per product with 48-instruction chains, which
// the layers of a model amplify to 1e-5 in the deepest gradients; 12-instruction chains bring the
// whole model to 3e-6).  The k range is therefore cut into chunks of TC_CHUNK_K floats: each chunk is accumulated
// in one of two TMEM buffers and the epilogue warps add the finished chunk into register
// accumulators with round-to-nearest FP32 adds while the next chunk is already being
// multiplied into the other buffer.
//
// CTA: tile 128 x BN, ring of STAGES shared-memory stages of BK floats of k (one swizzle span).
// Warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane each; warp 1 owns the TMEM
// allocation), warps 2-9 = epilogue: two warps per TMEM lane quarter, BN/2 columns each.
// The finished tile is staged in the (by then idle) operand stages and leaves row by row
// through bulk copies (cp.async.bulk, or its f32 add form when accumulating into C).  Every mbarrier wait is bounded: a wait that runs out sets the status word, the
// CTA drains, frees its TMEM and returns, and the host reports SB_ERR_TIMEOUT.
//
// Causal modes (attention; rows/columns are positions inside one sequence):
//   TC_CAUSAL_NONE
//   TC_CAUSAL_SKIP_UPPER   M = queries, N = keys   : tiles with every key after every query are not computed
//   TC_CAUSAL_SKIP_LOWER   M = keys,    N = queries: tiles with every query before every key are not computed
//   TC_CAUSAL_K_UPTO_M     M = queries, K = keys   : k runs over [0, m_tile_end)
//   TC_CAUSAL_K_FROM_M     M = keys,    K = queries: k runs over [m_tile_start, K)
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "sb_internal.h"

#define TC_BM 128
#define TC_EPI_WARPS 8
#define TC_THREADS (64 + 32 * TC_EPI_WARPS)
#define TC_CONV_WARPS 4                   // converter warps of the FP32-accurate CTA-pair kernel
// Warp roles.  Without converters: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (10 warps).
// With converters the CTA has four warpgroups of four warps, so that registers can be moved between them
// (setmaxnreg works on aligned groups of four warps): warps 0/1 producer and MMA issuer, 2-3 and 12-13
// converters, 4-11 epilogue, 14-15 idle; the epilogue warpgroups take the registers the others give up.
#define TC_CONV_THREADS 512
#define TC_REGS_LIGHT 72
#define TC_REGS_EPI 184
#define TC_GROUP_M 16
#define TC_CHUNK_K 32
#define TC_SPIN_CYCLES 4000000000ll      // ~2 s at 2 GHz: far beyond any legitimate wait

enum { TC_CAUSAL_NONE = 0, TC_CAUSAL_SKIP_UPPER, TC_CAUSAL_SKIP_LOWER, TC_CAUSAL_K_UPTO_M, TC_CAUSAL_K_FROM_M };

struct TcOperand {
    const float* hi; const float* lo;   // lo may be NULL when nterms == 1, or when the kernel makes it (CTA pairs)
    int rows;                            // M or N
    long pitch;                          // floats between rows (mn: between k-rows)
    int mn;                              // 1: the array is [K, rows], rows contiguous (CTA-pair kernel only)
    const void* h1; const void* h2;      // prepared FP16 parts (same layout as hi), or NULL
    int c2_dim; long c2_stride;          // third tensor-map dimension (floats); c2_dim = 1 for a plain matrix
    int c2_base, c2_step;                // slot of batch b = c2_base + (b / c2_div)*c2_step
    int c2_div = 1;                      // batch entries that share a slot (query heads of one K/V head)
};
// What the epilogue writes for an accumulator value x at (row, col) of batch b (attention's score-sized products):
//   TC_EPI_EXP  col <= row ? exp(x*scale - vec[row*vec_row_stride + b*vec_batch_stride]) : 0      (P from S and the log-sum-exp)
//   TC_EPI_DS   aux[row][col] * (x - vec[...]) * scale, aux laid out like C                        (dS from dP, P and D)
enum { TC_EPI_PLAIN = 0, TC_EPI_EXP, TC_EPI_DS };
struct TcEpi {
    int mode; float scale;
    const float* vec; long vec_row_stride, vec_batch_stride;
    const float* aux;
};
struct TcProblem {
    TcOperand A, B;
    float* C; long ldc; long c_batch_stride;
    int M, N, K, acc, nbatch, causal;
    TcEpi epi;
    const float* amax_a; const float* amax_b;      // FP16 split: device floats max |A|, max |B|; NULL = TF32 split
    unsigned* out_amax = nullptr;                  // when set (plain stores only, no accumulation into C): max |C| is left there as float bits
};

// --------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded wait; returns false when `limit` clock cycles passed without the phase completing
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, long long limit) {
    uint32_t addr = smem_u32(bar), done = 0;
    long long t0 = clock64();
    for (;;) {
        asm volatile("{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.u32 %0, 1, 0, P;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() - t0 > limit) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return mbar_wait_limit(bar, parity, TC_SPIN_CYCLES); }
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// ---- CTA-pair (cta_group::2) forms: the two CTAs of a cluster issue one 256-row MMA; rank 0 leads
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// load into this CTA's shared memory, byte count credited to the barrier at cluster address `bar_cluster` (the leader's)
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// arrives on the barrier at the same offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// FP16 split: power-of-two exponent s with amax * 2^s in [2^14, 2^15) (0 for an all-zero operand); 2^s as a float
__device__ __forceinline__ int tc_f16_shift(float amax) { return sb_f16_shift(amax); }
__device__ __forceinline__ float tc_pow2(int sh) { return sb_pow2(sh); }
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
template <bool PAIRBAR>
__device__ __forceinline__ void tc_load_box(void* dst, const CUtensorMap* map, uint64_t* bar, uint32_t bar_cluster, int c0, int c1, int c2) {
    if (PAIRBAR) tma_load_3d_pair(dst, map, bar_cluster, c0, c1, c2); else tma_load_3d(dst, map, bar, c0, c1, c2);
}
// one operand tile of a stage: K-major = one box {BK, rows}; MN-major = boxes {128 bytes of rows, BK} of BK*128 bytes each
// (32 rows of FP32, 64 rows of FP16); BK = k elements per stage
template <bool PAIRBAR, bool MN, int BK, int ROWS, int ELT = 4>
__device__ __forceinline__ void tc_load_operand(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, uint32_t bar_cluster,
                                                int kb, int row0, int c2, bool swapped) {
    if (MN) {
        // {row, k, slot}, or {row, slot, k} when the slot stride is smaller than the k-row pitch
        constexpr int RPB = 128 / ELT;
#pragma unroll
        for (int j = 0; j < ROWS / RPB; j++)
            tc_load_box<PAIRBAR>(dst + j * BK * 128, map, bar, bar_cluster, row0 + RPB * j, swapped ? c2 : kb * BK, swapped ? kb * BK : c2);
    } else {
        // a map whose slot stride is smaller than its row pitch is encoded as {k, slot, row}
        tc_load_box<PAIRBAR>(dst, map, bar, bar_cluster, kb * BK, swapped ? c2 : row0, swapped ? row0 : c2);
    }
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// shared-memory matrix descriptor, K-major operand, rows of SWZ bytes (64 or 128), 8-row groups contiguous
template <int SWZ>
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);                 // start address
    d |= (uint64_t)1 << 16;                                      // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(((8 * SWZ) >> 4) & 0x3fff) << 32;            // stride byte offset: one 8-row group
    d |= (uint64_t)1 << 46;                                      // descriptor version for sm_100
    d |= (uint64_t)(SWZ == 128 ? 2 : (SWZ == 64 ? 4 : 6)) << 61; // swizzle mode: 128B = 2, 64B = 4, 32B = 6
    return d;
}

// Tile order: groups of `group` row tiles; inside a group the row tile runs fastest, so CTAs
// resident together share a few A row tiles and a few B row tiles and both operands are re-read
// from L2 even when one of them (the embedding table) is far larger than L2.
__device__ __forceinline__ void tc_raster(int tile_id, int tiles_m, int tiles_n, int group, int* m_tile, int* n_tile) {
    const int per_group = group * tiles_n;
    const int gid = tile_id / per_group, in_g = tile_id % per_group;
    const int first_m = gid * group;
    const int gsize = min(group, tiles_m - first_m);
    *m_tile = first_m + in_g % gsize;
    *n_tile = in_g / gsize;
}

// shared-memory matrix descriptor, MN-major 32-bit operand: atoms of 4 k-rows x 128 bytes (32 floats of M or N) in
// the 128-byte swizzle with 32-byte granularity (the only MN-major form for TF32; TMA writes it as
// SWIZZLE_128B_ATOM_32B); the next 4 k-rows follow 512 bytes later, the atoms of the next 32 rows BK*128 bytes later
template <int BK>
__device__ __forceinline__ uint64_t make_mnmajor_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)(((BK * 128) >> 4) & 0x3fff) << 16;           // leading byte offset: next 32 rows
    d |= (uint64_t)((512 >> 4) & 0x3fff) << 32;                  // stride byte offset: next 4 k-rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;                                      // 128-byte swizzle, 32-byte base
    return d;
}
// shared-memory matrix descriptor, MN-major 16-bit operand: atoms of 8 k-rows x 128 bytes (64 halfs of M or N) in the
// 128-byte swizzle (TMA: SWIZZLE_128B); the next 8 k-rows follow 1024 bytes later, the atoms of the next 64 rows BKE*128 bytes later
template <int BKE>
__device__ __forceinline__ uint64_t make_mn16_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)(((BKE * 128) >> 4) & 0x3fff) << 16;          // leading byte offset: next 64 rows
    d |= (uint64_t)((1024 >> 4) & 0x3fff) << 32;                 // stride byte offset: next 8 k-rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                                      // 128-byte swizzle
    return d;
}
// lo part of the hi/lo split: x minus the 19 leading bits the tensor core reads, plus half a TF32 ulp
// of the result.  The tensor core truncates the word it is given, so the half ulp turns its truncation
// into rounding to nearest and the cross terms carry no one-sided error.
__device__ __forceinline__ float tf32_lo(float x) {
    float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    float lo = x - hi;
    return __uint_as_float(__float_as_uint(lo) + 0x00001000u);
}

// --------------------------------------------------------------------------- the kernel
// CTAS = 2: the CTA pair of a cluster computes a 256 x BN tile with cta_group::2 MMAs issued by the
// pair's rank-0 CTA.  Each CTA loads its own 128 rows of A and BN/2 rows of B, so per flop it takes a
// third less from L2 and the tensor core reads a third less shared memory than two independent CTAs
// would; each CTA's tensor memory holds its 128 rows of the tile and its own epilogue warps drain them.
// In this form the kernel takes the caller's FP32 matrices as they are:
//   * an operand stored [K, rows] (rows contiguous, "MN-major") is fetched in boxes of 32 floats x BK
//     k-rows (128-byte swizzle of 32-byte units) and read by the MMA through an MN-major descriptor, so no
//     transposed copy is made;
//   * the lo parts of the FP32-accurate mode are computed in the kernel: four converter warps per CTA
//     read each landed hi stage, write x - trunc_tf32(x) (rounded to nearest at TF32 precision) beside
//     it at the same offsets - the layout, whatever its swizzle, carries over - and release the stage to
//     the MMA warp.  TMA moves 4 bytes per operand element instead of 8 and nothing is prepared in HBM.
//
// Tail split: the tiles beyond the last full wave (tile ids >= split_full) are each cut into split_s
// pieces of the k range, one CTA (pair) per piece, so the last wave fills the machine with short
// pieces instead of leaving most SMs idle behind a few whole tiles.  A piece writes its 128 x BN
// block to `partial`; tc_splitk_fixup_kernel adds the pieces in piece order, so the result does not
// depend on timing.
// One unit of work of a launch: a tile of one batch entry, or one k piece of a split tile.
struct TcWork {
    int m0, n0, nb0;            // this CTA's first row of A and C, the tile's first column, this CTA's first row of B
    int kb_begin, num_kb;       // k range in blocks of BK
    int batch, slot;            // batch entry; index of the piece's block in the split workspace
    bool split;
};

// Decodes work item `item` (identically in every thread of the pair); false = nothing to compute (a tile above the
// causal diagonal).  Items are ordered tile-major, batch entry fastest, so that with causal k ranges the longest
// tiles of all batch entries come first.  tri: the tiles on or below the diagonal of a square tile grid are
// enumerated directly (row m holds m+1 tiles).
template <int BN, int BK, int CTAS>
__device__ __forceinline__ bool tc_work(int item, int rank, int M, int N, int K, int causal, int nbatch, int split_full, int split_s,
                                        int tri, TcWork& w) {
    constexpr int TILE_M = TC_BM * CTAS, BROWS = BN / CTAS;
    constexpr int KB_PER_CHUNK = TC_CHUNK_K / BK > 0 ? TC_CHUNK_K / BK : 1;
    const int tiles_m = (M + TILE_M - 1) / TILE_M, tiles_n = (N + BN - 1) / BN;
    const int gt = item / nbatch;
    w.batch = item - gt * nbatch;
    int tile_id = gt, piece = 0;
    w.split = split_s > 1 && gt >= split_full;
    w.slot = 0;
    if (w.split) { const int t = gt - split_full; piece = t % split_s; tile_id = split_full + t / split_s; w.slot = t; }
    int m_tile, n_tile;
    if (tri) {
        m_tile = (int)((sqrtf(8.0f * (float)tile_id + 1.0f) - 1.0f) * 0.5f);
        while ((m_tile + 1) * (m_tile + 2) / 2 <= tile_id) m_tile++;
        while (m_tile * (m_tile + 1) / 2 > tile_id) m_tile--;
        n_tile = tile_id - m_tile * (m_tile + 1) / 2;
    } else {
        tc_raster(tile_id, tiles_m, tiles_n, TC_GROUP_M / CTAS, &m_tile, &n_tile);
    }
    if (causal == TC_CAUSAL_K_UPTO_M) m_tile = tiles_m - 1 - m_tile;      // longest k ranges first
    const int tm0 = m_tile * TILE_M;
    w.m0 = tm0 + rank * TC_BM; w.n0 = n_tile * BN; w.nb0 = w.n0 + rank * BROWS;
    int kb_begin = 0, kb_end = (K + BK - 1) / BK;
    // causal structure: whole-tile skips and the k range, the same for both CTAs of a pair
    if (causal == TC_CAUSAL_SKIP_UPPER && w.n0 > tm0 + TILE_M - 1) return false;
    if (causal == TC_CAUSAL_SKIP_LOWER && w.n0 + BN - 1 < tm0) return false;
    if (causal == TC_CAUSAL_K_UPTO_M) kb_end = min(kb_end, (tm0 + TILE_M + BK - 1) / BK);
    if (causal == TC_CAUSAL_K_FROM_M) kb_begin = min(kb_end, tm0 / BK);
    if (w.split) {
        const int per = ((kb_end + split_s - 1) / split_s + KB_PER_CHUNK - 1) / KB_PER_CHUNK * KB_PER_CHUNK;
        kb_begin = min(kb_end, piece * per);
        kb_end = min(kb_end, kb_begin + per);
    }
    w.kb_begin = kb_begin; w.num_kb = kb_end - kb_begin;
    return true;
}
// item of cluster `cid` in round k of a launch with G clusters; snake: odd rounds run backwards, so a cluster that
// got a long item in one round gets a short one in the next (items are ordered longest first)
__device__ __forceinline__ int tc_item(int k, int cid, int G, int snake) { return k * G + ((snake && (k & 1)) ? G - 1 - cid : cid); }

#define TC_STG_ROWS 64          // rows of the output staging buffer: two TMEM lane quarters at a time

// The kernel is persistent: a launch has at most one CTA (pair) per SM (pair), and each walks over its work items.
// Barriers, tensor memory and the operand ring live across items, so while the epilogue warps write one tile out
// (through a small dedicated staging buffer, 32 rows at a time) the producer, the converters and the MMA warp are
// already working on the next item: only the epilogue itself is left of the per-tile overhead.
// F16 + PREP (FP32-accurate pair kernel): the hi/lo parts are FP16 instead of TF32.  Each operand is scaled by a power
// of two that brings its largest magnitude to [2^14, 2^15) (amax[0] for A, amax[1] for B, from tc_amax_kernel),
// h1 = fp16(x'), h2 = fp16(x' - h1): 22+ significant bits like the TF32 split, but the three MMAs per 16 k are kind::f16,
// half the tensor-core cycles; the epilogue undoes the scales.  Converting in the kernel (tried: converter warps writing
// the 16-bit tiles from the landed FP32 stage) is bound by the converter warps and no faster than the TF32 split.
// PREP (with F16): the two FP16 parts of both operands were written to memory beforehand (tc_split_f16_kernel, same
// layouts as the FP32 arrays) and TMA brings them in directly, 32 k elements per stage; no warp converts anything, the
// tensor pipe is the only consumer of the stages.  Either operand may be K-major or MN-major.
template <int BN, int BK, int NTERMS, int STAGES, int CTAS, bool AMN, bool BMN, bool F16 = false, bool PREP = false>
__global__ void __launch_bounds__((CTAS == 2 && NTERMS == 3) ? TC_CONV_THREADS : TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
               const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
               float* __restrict__ Cbase, long ldc, long c_batch_stride, int M, int N, int K, int acc, int causal,
               int a_c2_base, int a_c2_step, int b_c2_base, int b_c2_step, int b_c2_div, int swap_mask,
               int split_full, int split_s, float* __restrict__ partial, const TcEpi epi,
               int nbatch, int total_items, int snake, int tri, int store_warps, const float* __restrict__ amax_a, const float* __restrict__ amax_b,
               unsigned* __restrict__ out_amax, int* status) {
    constexpr int SWZ = BK * 4;
    constexpr int BROWS = BN / CTAS;                             // B rows this CTA loads
    constexpr int TILE_M = TC_BM * CTAS;
    constexpr int A_BYTES = TC_BM * BK * 4, B_BYTES = BROWS * BK * 4;
    constexpr int HI_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGE_BYTES = (NTERMS == 3 ? 2 : 1) * HI_BYTES;
    constexpr bool CONV = (CTAS == 2 && NTERMS == 3);            // lo parts made in the kernel
    static_assert(F16 == PREP, "the FP16 split works on prepared parts");
    static_assert(!F16 || (CONV && BK == 16), "FP16 split: FP32-accurate pair kernel");
    constexpr bool CONVERT = CONV && !PREP;                      // converter warps at work
    constexpr int BKE = PREP ? 2 * BK : BK;                      // k elements per stage (PREP: 64-byte rows of halfs)
    static_assert(CTAS == 2 || (!AMN && !BMN), "MN-major operands: CTA-pair kernel only");
    static_assert(BROWS % 32 == 0, "an MN-major tile is made of boxes of 32 rows");
    constexpr uint32_t TMEM_COLS = 2 * BN;                       // two accumulator buffers
    constexpr int KB_PER_CHUNK = (F16 ? 2 : 1) * TC_CHUNK_K / BKE;    // twelve MMAs per accumulation chunk either way
    constexpr int COLS_PER_WARP = BN / (TC_EPI_WARPS / 4);       // 128 or 64 register accumulators per epilogue thread
    constexpr int SLD = BN + 4;                                  // padded row pitch of the staging buffer (floats)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* stg = (float*)(smem + STAGES * STAGE_BYTES);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES + TC_STG_ROWS * SLD * 4);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;          // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;           // [2] epilogue -> MMA
    uint64_t* conv = acc_empty + 2;               // [STAGES] converter warps -> MMA (leader's copy is the one used)
    uint64_t* stg_full = conv + STAGES;           // [2] epilogue warps -> store warps: a 32-row half of the staging buffer is written
    uint64_t* stg_go = stg_full + 2;              // [4] store warps -> the epilogue warps of one lane quarter: its half is free for it
    uint32_t* tmem_slot = (uint32_t*)(stg_go + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    const int cid = blockIdx.x / CTAS, G = gridDim.x / CTAS;
    const int rounds = (total_items + G - 1) / G;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], TC_EPI_WARPS * CTAS); }
        if (CONV) for (int s = 0; s < STAGES; s++) mbar_init(&conv[s], TC_CONV_WARPS * CTAS);
        for (int b = 0; b < 2; b++) mbar_init(&stg_full[b], TC_EPI_WARPS / 4);
        for (int b = 0; b < 4; b++) mbar_init(&stg_go[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (CTAS == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();          // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    constexpr int EPI0 = CONV ? 4 : 2;            // first epilogue warp
    const bool is_epi = warp >= EPI0 && warp < EPI0 + TC_EPI_WARPS;
    // converter index of this warp (CONV only): warps 2, 3, 12, 13 -> 0..3; -1 otherwise
    const int cw = !CONV ? -1 : (warp == 2 || warp == 3) ? warp - 2 : (warp == 12 || warp == 13) ? warp - 10 : -1;

    if (!is_epi) {
    if (CONV) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_REGS_LIGHT));      // whole warpgroups 0 and 3
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            const bool swa = (swap_mask & 1) != 0, swb = (swap_mask & 2) != 0;
            uint32_t git = 0;                      // k blocks issued so far, over all items
            for (int k = 0; k < rounds && ok; k++) {
                const int item = tc_item(k, cid, G, snake);
                TcWork w;
                if (item >= total_items || !tc_work<BN, BKE, CTAS>(item, (int)rank, M, N, K, causal, nbatch, split_full, split_s, tri, w)) continue;
                const int a_c2 = a_c2_base + w.batch * a_c2_step, b_c2 = b_c2_base + (b_c2_div > 1 ? w.batch / b_c2_div : w.batch) * b_c2_step;
                for (int it = 0; it < w.num_kb && ok; it++, git++) {
                    const int s = git % STAGES, kb = w.kb_begin + it;
                    ok = mbar_wait(&empty[s], ((git / STAGES) & 1) ^ 1);
                    if (!ok) break;
                    uint8_t* st = smem + s * STAGE_BYTES;
                    if (PREP) {
                        // four 16-bit tiles per CTA (h1 A, h1 B, h2 A, h2 B), the pair's bytes all land on the leader's barrier
                        if (leader) mbar_expect_tx(&full[s], STAGE_BYTES * CTAS);
                        const uint32_t fb = mapa_u32(smem_u32(&full[s]), 0);
                        tc_load_operand<true, AMN, BKE, TC_BM, 2>(st, &tmAh, nullptr, fb, kb, w.m0, a_c2, swa);
                        tc_load_operand<true, BMN, BKE, BROWS, 2>(st + A_BYTES, &tmBh, nullptr, fb, kb, w.nb0, b_c2, swb);
                        tc_load_operand<true, AMN, BKE, TC_BM, 2>(st + HI_BYTES, &tmAl, nullptr, fb, kb, w.m0, a_c2, swa);
                        tc_load_operand<true, BMN, BKE, BROWS, 2>(st + HI_BYTES + A_BYTES, &tmBl, nullptr, fb, kb, w.nb0, b_c2, swb);
                    } else if (CONV) {
                        // each CTA's hi tiles land on its own barrier; its converter warps take it from there
                        mbar_expect_tx(&full[s], HI_BYTES);
                        tc_load_operand<false, AMN, BK, TC_BM>(st, &tmAh, &full[s], 0, kb, w.m0, a_c2, swa);
                        tc_load_operand<false, BMN, BK, BROWS>(st + A_BYTES, &tmBh, &full[s], 0, kb, w.nb0, b_c2, swb);
                    } else if (CTAS == 2) {
                        if (leader) mbar_expect_tx(&full[s], STAGE_BYTES * CTAS);      // the pair's bytes all land on the leader's barrier
                        const uint32_t fb = mapa_u32(smem_u32(&full[s]), 0);
                        tc_load_operand<true, AMN, BK, TC_BM>(st, &tmAh, nullptr, fb, kb, w.m0, a_c2, swa);
                        tc_load_operand<true, BMN, BK, BROWS>(st + A_BYTES, &tmBh, nullptr, fb, kb, w.nb0, b_c2, swb);
                    } else {
                        mbar_expect_tx(&full[s], STAGE_BYTES);
                        tc_load_operand<false, false, BK, TC_BM>(st, &tmAh, &full[s], 0, kb, w.m0, a_c2, swa);
                        tc_load_operand<false, false, BK, BROWS>(st + A_BYTES, &tmBh, &full[s], 0, kb, w.nb0, b_c2, swb);
                        if (NTERMS == 3) {
                            tc_load_operand<false, false, BK, TC_BM>(st + HI_BYTES, &tmAl, &full[s], 0, kb, w.m0, a_c2, swa);
                            tc_load_operand<false, false, BK, BROWS>(st + HI_BYTES + A_BYTES, &tmBl, &full[s], 0, kb, w.nb0, b_c2, swb);
                        }
                    }
                }
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (leader && elect_one()) {
            // instruction descriptor: D = F32, A = B = TF32, majors of the operands, N and M of the tile
            // (kind::f16: A = B = F16, format code 0)
            const uint32_t idesc = (1u << 4) | ((F16 ? 0u : 2u) << 7) | ((F16 ? 0u : 2u) << 10) | ((AMN ? 1u : 0u) << 15) | ((BMN ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
            uint32_t git = 0, gch = 0;             // k blocks and chunks consumed so far, over all items
            for (int k = 0; k < rounds && ok; k++) {
                const int item = tc_item(k, cid, G, snake);
                TcWork w;
                if (item >= total_items || !tc_work<BN, BKE, CTAS>(item, (int)rank, M, N, K, causal, nbatch, split_full, split_s, tri, w)) continue;
                int it = 0;
                const int num_chunks = (w.num_kb + KB_PER_CHUNK - 1) / KB_PER_CHUNK;
                for (int ch = 0; ch < num_chunks && ok; ch++, gch++) {
                    const int buf = gch & 1;
                    ok = mbar_wait(&acc_empty[buf], ((gch >> 1) & 1) ^ 1);      // epilogue has drained this buffer
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    const int it_end = min(it + KB_PER_CHUNK, w.num_kb);
                    bool first = true;
                    for (; it < it_end && ok; it++, git++) {
                        const int s = git % STAGES;
                        ok = mbar_wait(CONVERT ? &conv[s] : &full[s], (git / STAGES) & 1);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                        if (PREP) {
                            // stage = h1 A, h1 B, h2 A, h2 B (the FP32 tiles' sizes and places); two K = 16 MMAs per term
                            const uint64_t a1 = AMN ? make_mn16_desc<BKE>(sa) : make_kmajor_desc<SWZ>(sa);
                            const uint64_t b1 = BMN ? make_mn16_desc<BKE>(sa + A_BYTES) : make_kmajor_desc<SWZ>(sa + A_BYTES);
                            const uint64_t a2 = AMN ? make_mn16_desc<BKE>(sa + HI_BYTES) : make_kmajor_desc<SWZ>(sa + HI_BYTES);
                            const uint64_t b2 = BMN ? make_mn16_desc<BKE>(sa + HI_BYTES + A_BYTES) : make_kmajor_desc<SWZ>(sa + HI_BYTES + A_BYTES);
#pragma unroll
                            for (int kk = 0; kk < BKE / 16; kk++) {
                                // 16 halfs of k, in 16-byte units: 32 bytes along a K-major row, 16 k-rows of 128 bytes in an MN-major tile
                                const uint64_t adva = (uint64_t)(AMN ? kk * 128 : kk * 2), advb = (uint64_t)(BMN ? kk * 128 : kk * 2);
                                tc_mma_f16_pair(tmem_d, a1 + adva, b1 + advb, idesc, first ? 0u : 1u);
                                tc_mma_f16_pair(tmem_d, a2 + adva, b1 + advb, idesc, 1);
                                tc_mma_f16_pair(tmem_d, a1 + adva, b2 + advb, idesc, 1);
                                first = false;
                            }
                            tc_commit_pair(&empty[s]);
                            continue;
                        }
                        const uint64_t ah = AMN ? make_mnmajor_desc<BK>(sa) : make_kmajor_desc<SWZ>(sa);
                        const uint64_t bh = BMN ? make_mnmajor_desc<BK>(sa + A_BYTES) : make_kmajor_desc<SWZ>(sa + A_BYTES);
                        const uint64_t al = AMN ? make_mnmajor_desc<BK>(sa + HI_BYTES) : make_kmajor_desc<SWZ>(sa + HI_BYTES);
                        const uint64_t bl = BMN ? make_mnmajor_desc<BK>(sa + HI_BYTES + A_BYTES) : make_kmajor_desc<SWZ>(sa + HI_BYTES + A_BYTES);
#pragma unroll
                        for (int kk = 0; kk < BK / 8; kk++) {
                            // 8 floats of k, in 16-byte units: 32 bytes along a K-major row, 8 k-rows of 128 bytes in an MN-major tile
                            const uint64_t adva = (uint64_t)(AMN ? kk * 64 : kk * 2), advb = (uint64_t)(BMN ? kk * 64 : kk * 2);
                            if (CTAS == 2) {
                                tc_mma_tf32_pair(tmem_d, ah + adva, bh + advb, idesc, first ? 0u : 1u);
                                if (NTERMS == 3) {
                                    tc_mma_tf32_pair(tmem_d, al + adva, bh + advb, idesc, 1);
                                    tc_mma_tf32_pair(tmem_d, ah + adva, bl + advb, idesc, 1);
                                }
                            } else {
                                tc_mma_tf32(tmem_d, ah + adva, bh + advb, idesc, first ? 0u : 1u);
                                if (NTERMS == 3) {
                                    tc_mma_tf32(tmem_d, al + adva, bh + advb, idesc, 1);
                                    tc_mma_tf32(tmem_d, ah + adva, bl + advb, idesc, 1);
                                }
                            }
                            first = false;
                        }
                        if (CTAS == 2) tc_commit_pair(&empty[s]); else tc_commit(&empty[s]);      // stage reusable once these MMAs have read it
                    }
                    if (CTAS == 2) tc_commit_pair(&acc_full[buf]); else tc_commit(&acc_full[buf]); // chunk complete (also releases the epilogue on a time-out)
                }
            }
            if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
        }
    } else {
        // ---------------- converter (CTA-pair FP32-accurate kernel): lo = x - trunc_tf32(x) beside each landed hi stage ----------------
        if (CONVERT && cw >= 0) {
            constexpr int N4 = HI_BYTES / 16;
            constexpr int PER = N4 / (32 * TC_CONV_WARPS);
            constexpr int UNR = PER % 8 == 0 ? 8 : (PER % 6 == 0 ? 6 : 4);
            static_assert(N4 % (32 * TC_CONV_WARPS) == 0 && PER % UNR == 0, "stage size against the converter's unroll");
            const uint32_t cb_base = mapa_u32(smem_u32(&conv[0]), 0);
            uint32_t git = 0;
            for (int k = 0; k < rounds && ok; k++) {
                const int item = tc_item(k, cid, G, snake);
                TcWork w;
                if (item >= total_items || !tc_work<BN, BKE, CTAS>(item, (int)rank, M, N, K, causal, nbatch, split_full, split_s, tri, w)) continue;
                for (int it = 0; it < w.num_kb && ok; it++, git++) {
                    const int s = git % STAGES;
                    ok = mbar_wait(&full[s], (git / STAGES) & 1);
                    if (!ok) break;
                    const float4* src = (const float4*)(smem + s * STAGE_BYTES);
                    float4* dst = (float4*)(smem + s * STAGE_BYTES + HI_BYTES);
#pragma unroll
                    for (int b = 0; b < PER; b += UNR) {
                        float4 v[UNR];
#pragma unroll
                        for (int j = 0; j < UNR; j++) v[j] = src[(cw * PER + b + j) * 32 + lane];
#pragma unroll
                        for (int j = 0; j < UNR; j++)
                            dst[(cw * PER + b + j) * 32 + lane] = make_float4(tf32_lo(v[j].x), tf32_lo(v[j].y), tf32_lo(v[j].z), tf32_lo(v[j].w));
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the MMA reads these writes through the async proxy
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(cb_base + (uint32_t)(s * 8));
                }
            }
            if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
        }
        // ---------------- store warps (warps 14 and 15 of the FP32-accurate pair kernel, plain tiles only) ----------------
        // Each owns one 32-row half of the staging buffer, used in turn by lane quarters b and b+2: when the two epilogue warps
        // of a quarter have written it, every lane sends one row to memory with a bulk copy, and once the copies have read it
        // the half is handed to the other quarter (one barrier per quarter, so a waiter is never more than one phase behind).
        // The epilogue warps thus only write their registers out and go back to the next tile's accumulator chunks.
        if (CONV && store_warps && warp >= 14) {
            const int b = warp - 14;
            uint32_t tcount = 0;
            bool issued = false;
            for (int k = 0; k < rounds && ok; k++) {
                const int item = tc_item(k, cid, G, snake);
                TcWork w;
                if (item >= total_items || !tc_work<BN, BKE, CTAS>(item, (int)rank, M, N, K, causal, nbatch, split_full, split_s, tri, w)) continue;
                float* C = Cbase + (size_t)w.batch * c_batch_stride;
                float* dst = w.split ? partial + ((size_t)w.slot * CTAS + rank) * (size_t)(TC_BM * BN) : C + (size_t)w.m0 * ldc + w.n0;
                const long ld = w.split ? (long)BN : ldc;
                const int rows_valid = w.split ? TC_BM : M - w.m0, cols_valid = w.split ? BN : N - w.n0;
                const int accf = w.split ? 0 : acc;
                const uint32_t bytes = (uint32_t)min(cols_valid, BN) * 4u;
                for (int qq = b; qq < 4 && ok; qq += 2) {
                    const uint32_t u = (tcount * 4 + (uint32_t)qq) >> 1;           // how many times this half has been used before
                    ok = mbar_wait(&stg_full[b], u & 1);
                    if (!ok) break;
                    const int r = qq * 32 + lane;
                    if (r < rows_valid) {
                        const uint32_t src = smem_u32(stg + (size_t)(b * 32 + lane) * SLD);
                        float* gp = dst + (size_t)r * ld;
                        if (accf) asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gp), "r"(src), "r"(bytes) : "memory");
                        else      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gp), "r"(src), "r"(bytes) : "memory");
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    issued = true;
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&stg_go[qq ^ 2])) : "memory");
                }
                tcount++;
            }
            if (issued) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // every row has reached memory
            if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
        }
    }
    } else {
        // ---------------- epilogue: TMEM chunks -> register accumulators -> staging -> global ----------------
        if (CONV) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_REGS_EPI));          // whole warpgroups 1 and 2
        const int ew = warp - EPI0;                   // 0..7
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int col0 = (ew >> 2) * COLS_PER_WARP;   // which half of the tile's columns
        constexpr int RPP = TC_STG_ROWS / TC_EPI_WARPS;      // rows per warp and pass in the row-wise work (8)
        constexpr int RB = 4;                                // of which this many are in flight together in the dS transform
        constexpr int NH = (BN + 127) / 128;                 // float4 per lane and row
        uint32_t gch = 0, tcount = 0;           // chunks drained and tiles written so far, over all items
        bool issued = false;
        for (int k = 0; k < rounds && ok; k++) {
            const int item = tc_item(k, cid, G, snake);
            TcWork w;
            if (item >= total_items || !tc_work<BN, BKE, CTAS>(item, (int)rank, M, N, K, causal, nbatch, split_full, split_s, tri, w)) continue;
            const int num_chunks = (w.num_kb + KB_PER_CHUNK - 1) / KB_PER_CHUNK;
            float accr[COLS_PER_WARP];
#pragma unroll
            for (int j = 0; j < COLS_PER_WARP; j++) accr[j] = 0.f;
            for (int ch = 0; ch < num_chunks && ok; ch++, gch++) {
                const int buf = gch & 1;
                ok = mbar_wait(&acc_full[buf], (gch >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + col0);
#pragma unroll
                for (int g = 0; g < COLS_PER_WARP / 32; g++) {
                    uint32_t r[32];
                    tc_ld32(taddr + (uint32_t)(g * 32), r);
                    if (g == COLS_PER_WARP / 32 - 1) {
                        // the buffer is in registers: hand it back to the MMA warp before the adds
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (CTAS == 2) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[buf]), 0));
                            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) accr[g * 32 + j] += __uint_as_float(r[j]);
                }
            }
            if (F16) {
                // undo the operands' power-of-two scales (two exact multiplications: the product of both may leave the float range)
                const float ua = tc_pow2(-tc_f16_shift(*amax_a)), ub = tc_pow2(-tc_f16_shift(*amax_b));
#pragma unroll
                for (int j = 0; j < COLS_PER_WARP; j++) accr[j] = accr[j] * ua * ub;
            }
            if (out_amax && !w.split) {
                // largest magnitude of the tile for whoever splits C into FP16 parts next (rows and columns past the edge are zero)
                float m = 0.f;
#pragma unroll
                for (int j = 0; j < COLS_PER_WARP; j++) m = fmaxf(m, fabsf(accr[j]));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                if (lane == 0 && m > 0.f) atomicMax(out_amax, __float_as_uint(m));
            }
            if (CONV && store_warps) {
                // plain tile: write this warp's rows into its quarter's half of the staging buffer and hand it to the store warp
                const int b = q & 1;
                // quarters 0 and 1 use their half first in every tile (free once quarter q+2 of the previous tile has left it),
                // quarters 2 and 3 after quarter q-2 of the same tile
                ok = ok && mbar_wait(&stg_go[q], q < 2 ? ((tcount & 1) ^ 1) : (tcount & 1));
                if (!ok) break;
                float* srow = stg + (size_t)(b * 32 + lane) * SLD + col0;
#pragma unroll
                for (int j = 0; j < COLS_PER_WARP; j += 4)
                    *(float4*)(srow + j) = make_float4(accr[j], accr[j + 1], accr[j + 2], accr[j + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");              // the bulk copies read these writes
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&stg_full[b])) : "memory");
                tcount++;
                continue;
            }
            {
                // a bounded wait may have run out in some warps only: all eight agree before the barriers of the store passes
                int okall, okin = ok ? 1 : 0;
                asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.s32 pin, %1, 0;\n\tbar.red.and.pred pout, 1, %2, pin;\n\tselp.s32 %0, 1, 0, pout;\n\t}"
                             : "=r"(okall) : "r"(okin), "n"(32 * TC_EPI_WARPS) : "memory");
                if (!okall) { if (ok) ok = false; break; }
            }
            // The tile leaves 32 rows (one TMEM lane quarter) at a time through the staging buffer: the two warps that hold
            // the quarter write it (with the exp transform if asked), all eight warps do the row-wise work on it (the dS
            // transform, which reads a second matrix), and whole rows go out as bulk copies (an f32 add into C when
            // accumulating: every element of C is touched by one CTA, so the sum does not depend on timing).
            // Measured: warps storing the tile themselves took 16 us per tile, the bulk copies 2 us.
            float* C = Cbase + (size_t)w.batch * c_batch_stride;
            // destination: the tile's place in C, or (a piece of a split tile) its own block of `partial`
            float* dst = w.split ? partial + ((size_t)w.slot * CTAS + rank) * (size_t)(TC_BM * BN) : C + (size_t)w.m0 * ldc + w.n0;
            const long ld = w.split ? (long)BN : ldc;
            const int rows_valid = w.split ? TC_BM : M - w.m0, cols_valid = w.split ? BN : N - w.n0;
            const int accf = w.split ? 0 : acc;
            const int emode = w.split ? TC_EPI_PLAIN : epi.mode;
            const bool vec = ((ld & 3) == 0) && ((((uintptr_t)dst) & 15) == 0) && (emode != TC_EPI_DS || (((uintptr_t)epi.aux) & 15) == 0);
            const bool bulk = vec && (cols_valid >= BN || (cols_valid & 3) == 0);      // rows are 16-byte multiples at 16-byte addresses
            const uint32_t bytes = (uint32_t)min(cols_valid, BN) * 4u;
            const float* abase = emode == TC_EPI_DS ? epi.aux + (size_t)w.batch * c_batch_stride + (size_t)w.m0 * ldc + w.n0 : nullptr;
#pragma unroll 1
            for (int p = 0; p < TC_BM / TC_STG_ROWS; p++) {
                // the copies of the previous pass must have read the staging buffer before it is written again
                if (issued && lane < RPP) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                asm volatile("bar.sync 1, %0;" ::"n"(32 * TC_EPI_WARPS) : "memory");                                  // epilogue warps only
                if ((q >> 1) == p) {
                    // each thread holds one row of the tile; TC_EPI_EXP: P = exp(S*scale - lse[row]), zero past the diagonal
                    const int r = q * 32 + lane, grow = w.m0 + r;
                    float* srow = stg + (size_t)((q & 1) * 32 + lane) * SLD + col0;
                    if (emode == TC_EPI_EXP) {
                        const float rv = r < rows_valid ? epi.vec[(size_t)grow * epi.vec_row_stride + (size_t)w.batch * epi.vec_batch_stride] : 0.f;
                        const int kmax = grow - (w.n0 + col0);        // columns j <= kmax are on or below the diagonal
#pragma unroll
                        for (int j = 0; j < COLS_PER_WARP; j += 4) {
                            float4 v;
                            v.x = j <= kmax ? expf(accr[j] * epi.scale - rv) : 0.f;         v.y = j + 1 <= kmax ? expf(accr[j + 1] * epi.scale - rv) : 0.f;
                            v.z = j + 2 <= kmax ? expf(accr[j + 2] * epi.scale - rv) : 0.f; v.w = j + 3 <= kmax ? expf(accr[j + 3] * epi.scale - rv) : 0.f;
                            *(float4*)(srow + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < COLS_PER_WARP; j += 4)
                            *(float4*)(srow + j) = make_float4(accr[j], accr[j + 1], accr[j + 2], accr[j + 3]);
                    }
                    if (bulk && emode != TC_EPI_DS) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the bulk copies read these writes
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * TC_EPI_WARPS) : "memory");                                  // epilogue warps only
                const int i0 = ew * RPP;                    // this warp's rows of the staged rows
                const int prow = p * TC_STG_ROWS;           // first tile row of this pass
                if (emode == TC_EPI_DS) {
                    // dS = P o (dP - D[row]) * scale, row-wise in the staged rows (P is read with whole-row accesses)
#pragma unroll
                    for (int ib = 0; ib < RPP; ib += RB) {
                        float4 av[RB][NH];
                        float rowv[RB];
#pragma unroll
                        for (int ii = 0; ii < RB; ii++) {
                            const int r = prow + i0 + ib + ii;
                            rowv[ii] = r < rows_valid ? epi.vec[(size_t)(w.m0 + r) * epi.vec_row_stride + (size_t)w.batch * epi.vec_batch_stride] : 0.f;
#pragma unroll
                            for (int h = 0; h < NH; h++) {
                                const int col = (h * 32 + lane) * 4;
                                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (r < rows_valid && col < BN) {
                                    const float* ap = abase + (size_t)r * ldc + col;
                                    if (vec && col + 3 < cols_valid) t = *(const float4*)ap;
                                    else { if (col < cols_valid) t.x = ap[0]; if (col + 1 < cols_valid) t.y = ap[1]; if (col + 2 < cols_valid) t.z = ap[2]; if (col + 3 < cols_valid) t.w = ap[3]; }
                                }
                                av[ii][h] = t;
                            }
                        }
#pragma unroll
                        for (int ii = 0; ii < RB; ii++) {
                            const float rv = rowv[ii];
#pragma unroll
                            for (int h = 0; h < NH; h++) {
                                const int col = (h * 32 + lane) * 4;
                                if (col < BN) {
                                    float4* sp = (float4*)(stg + (size_t)(i0 + ib + ii) * SLD + col);
                                    float4 v = *sp; const float4 pv = av[ii][h];
                                    v.x = pv.x * (v.x - rv) * epi.scale; v.y = pv.y * (v.y - rv) * epi.scale;
                                    v.z = pv.z * (v.z - rv) * epi.scale; v.w = pv.w * (v.w - rv) * epi.scale;
                                    *sp = v;
                                }
                            }
                        }
                    }
                    if (bulk) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();                          // a warp copies out the rows it has just transformed
                }
                if (bulk) {
                    if (lane < RPP) {
                        const int r = prow + i0 + lane;
                        if (r < rows_valid) {
                            const uint32_t src = smem_u32(stg + (size_t)(i0 + lane) * SLD);
                            float* gp = dst + (size_t)r * ld;
                            if (accf) asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gp), "r"(src), "r"(bytes) : "memory");
                            else      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gp), "r"(src), "r"(bytes) : "memory");
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");       // one group per pass and lane, also when the row is outside C
                        issued = true;
                    }
                } else {
                    // ragged or unaligned rows: the warps store the (already transformed) rows themselves
                    for (int ii = 0; ii < RPP; ii++) {
                        const int r = prow + i0 + ii;
                        if (r >= rows_valid) break;
                        const float* srow = stg + (size_t)(i0 + ii) * SLD;
                        float* crow = dst + (size_t)r * ld;
                        for (int col = lane; col < BN && col < cols_valid; col += 32)
                            crow[col] = accf ? crow[col] + srow[col] : srow[col];
                    }
                }
            }
        }
        if (!ok && lane == 0) atomicExch(status, SB_ERR_TIMEOUT);
        if (issued) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");              // every row has reached memory
        tc_fence_before();
    }
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();          // neither CTA leaves while the other may still signal it or read its operands
    if (warp == 1) {
        tc_fence_after();
        if (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
        else           asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

// Adds the pieces of the split tiles into C in piece order.  One thread per four columns of one row
// (the loads of a thread are independent, and a grid of many small CTAs keeps the latency hidden).
static __global__ void __launch_bounds__(256) tc_splitk_fixup_kernel(const float* __restrict__ partial, float* __restrict__ C, long ldc,
                                                                     int M, int N, int acc, int BN, int ctas, int split_full, int split_s,
                                                                     int nblocks, unsigned* __restrict__ out_amax) {
    const int bn4 = BN >> 2;
    const long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int blk = (int)(item / (TC_BM * bn4)), i = (int)(item % (TC_BM * bn4));
    if (blk >= nblocks) return;
    const int t = blk / ctas, rank = blk % ctas;
    const int tile_m = TC_BM * ctas;
    const int tiles_m = (M + tile_m - 1) / tile_m, tiles_n = (N + BN - 1) / BN;
    int m_tile, n_tile;
    tc_raster(split_full + t, tiles_m, tiles_n, TC_GROUP_M / ctas, &m_tile, &n_tile);
    const int m0 = m_tile * tile_m + rank * TC_BM, n0 = n_tile * BN;
    const size_t block = (size_t)TC_BM * BN;
    const float* p0 = partial + ((size_t)t * split_s * ctas + rank) * block;
    const size_t piece_stride = (size_t)ctas * block;
    const bool vec = ((ldc & 3) == 0) && ((((uintptr_t)C) & 15) == 0);
    {
        const int r = i / bn4, col = (i % bn4) * 4;
        if (m0 + r >= M || n0 + col >= N) return;
        float* crow = C + (size_t)(m0 + r) * ldc + n0 + col;
        const bool whole = vec && n0 + col + 3 < N;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (acc) {
            if (whole) v = *(const float4*)crow;
            else { v.x = crow[0]; if (n0 + col + 1 < N) v.y = crow[1]; if (n0 + col + 2 < N) v.z = crow[2]; if (n0 + col + 3 < N) v.w = crow[3]; }
        }
        float4 o[8];
#pragma unroll
        for (int p = 0; p < 8; p++) if (p < split_s) o[p] = *(const float4*)(p0 + (size_t)p * piece_stride + (size_t)r * BN + col);
#pragma unroll
        for (int p = 0; p < 8; p++) if (p < split_s) { v.x += o[p].x; v.y += o[p].y; v.z += o[p].z; v.w += o[p].w; }
        if (whole) *(float4*)crow = v;
        else { crow[0] = v.x; if (n0 + col + 1 < N) crow[1] = v.y; if (n0 + col + 2 < N) crow[2] = v.z; if (n0 + col + 3 < N) crow[3] = v.w; }
        if (out_amax) {
            float m = fabsf(v.x);
            if (whole) m = fmaxf(fmaxf(m, fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
            else { if (n0 + col + 1 < N) m = fmaxf(m, fabsf(v.y)); if (n0 + col + 2 < N) m = fmaxf(m, fabsf(v.z)); if (n0 + col + 3 < N) m = fmaxf(m, fabsf(v.w)); }
            // one atomic per warp: among the lanes still here, non-negative floats order like their bits
            const unsigned live = __activemask();
            const unsigned wm = __reduce_max_sync(live, __float_as_uint(m));
            if ((int)(threadIdx.x & 31) == __ffs(live) - 1 && wm != 0u) atomicMax(out_amax, wm);
        }
    }
}

// max |x| of up to two operands (blockIdx.y selects), as float bits through an integer atomicMax (order-free); outputs zeroed before
static __global__ void __launch_bounds__(256) tc_amax_kernel(const float* __restrict__ a, size_t na4, unsigned* __restrict__ oa,
                                                             const float* __restrict__ b, size_t nb4, unsigned* __restrict__ ob) {
    const float4* x = (const float4*)(blockIdx.y ? b : a);
    const size_t n4 = blockIdx.y ? nb4 : na4;
    float m = 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = x[i];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float red[8];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
        atomicMax(blockIdx.y ? ob : oa, __float_as_uint(m));
    }
}

// FP16 parts of up to two operands (blockIdx.y selects): x' = x * 2^shift(amax), h1 = fp16(x'), h2 = fp16(x' - h1); layout kept
static __global__ void __launch_bounds__(256) tc_split_f16_kernel(const float* __restrict__ a, size_t na4, __half* __restrict__ a1, __half* __restrict__ a2,
                                                                  const float* __restrict__ amax_a,
                                                                  const float* __restrict__ b, size_t nb4, __half* __restrict__ b1, __half* __restrict__ b2,
                                                                  const float* __restrict__ amax_b) {
    const float4* x = (const float4*)(blockIdx.y ? b : a);
    const size_t n4 = blockIdx.y ? nb4 : na4;
    uint2* o1 = (uint2*)(blockIdx.y ? b1 : a1); uint2* o2 = (uint2*)(blockIdx.y ? b2 : a2);
    const float sc = tc_pow2(tc_f16_shift(blockIdx.y ? *amax_b : *amax_a));
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = x[i];
        const float p0 = v.x * sc, p1 = v.y * sc, p2 = v.z * sc, p3 = v.w * sc;
        const __half2 ha = __floats2half2_rn(p0, p1), hb = __floats2half2_rn(p2, p3);
        const float2 fa = __half22float2(ha), fb = __half22float2(hb);
        const __half2 la = __floats2half2_rn(p0 - fa.x, p1 - fa.y), lb = __floats2half2_rn(p2 - fb.x, p3 - fb.y);
        uint2 u1, u2;
        u1.x = *(const uint32_t*)&ha; u1.y = *(const uint32_t*)&hb; u2.x = *(const uint32_t*)&la; u2.y = *(const uint32_t*)&lb;
        o1[i] = u1; o2[i] = u2;
    }
}

// --------------------------------------------------------------------------- operand preparation kernels
// lo[i] = x[i] - tf32_trunc(x[i]);  8 bytes per element
static __global__ void __launch_bounds__(256) split_lo_kernel(const float* __restrict__ x, float* __restrict__ lo, size_t n4) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < n4; i += nth) {
        float4 v = ((const float4*)x)[i];
        ((float4*)lo)[i] = make_float4(tf32_lo(v.x), tf32_lo(v.y), tf32_lo(v.z), tf32_lo(v.w));
    }
}
// in [R, C] row-major -> hi [C, Rp] = in^T, lo [C, Rp] = lo(in^T); Rp = row pitch of the outputs (>= R, multiple of 4)
static __global__ void __launch_bounds__(256) transpose_split_kernel(const float* __restrict__ in, float* __restrict__ hi, float* __restrict__ lo,
                                                                     int R, int C, int Rp, int want_lo) {
    __shared__ float tile[32][33];
    int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
    for (int i = ty; i < 32; i += 8) {
        int r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < R && c < C) ? in[(size_t)r * C + c] : 0.f;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        int c = c0 + i, r = r0 + tx;
        if (c < C && r < Rp) {
            float v = tile[tx][i];
            hi[(size_t)c * Rp + r] = v;
            if (want_lo) lo[(size_t)c * Rp + r] = tf32_lo(v);
        }
    }
}

// --------------------------------------------------------------------------- host side
typedef CUresult (*tc_encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tc_encode_fn_t g_tc_encode = nullptr;

static bool tc_load_encode() {
    if (g_tc_encode) return true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    g_tc_encode = (tc_encode_fn_t)fn;
    return true;
}

// slot stride below the row pitch (heads interleaved inside a token row): dimensions are ordered {k, slot, row}
// (MN-major: {row, slot, k})
static inline bool tc_swapped(const TcOperand& op) { return op.c2_dim > 1 && op.c2_stride < op.pitch; }

// Encoding a tensor map costs a few microseconds on the host and a training step re-issues the same
// (pointer, shape) combinations every layer and every step, so encoded maps are kept in a small
// direct-mapped cache keyed by everything that goes into the encoding.
struct TcMapKey { const void* base; long pitch, c2_stride; int K, rows, c2_dim, BK, box_rows, mn, elt; };
struct TcMapEntry { TcMapKey key; CUtensorMap map; bool valid; };
#define TC_MAP_CACHE 8192
static TcMapEntry* g_tc_map_cache = nullptr;

// 3-D FP32 tensor {K, rows, slots} (or {K, slots, rows}); box = BK x box_rows x 1; reads beyond the extents give zero
// elt = 2: the same for an FP16 array of the same shape (BK halfs per box; MN-major boxes are 64 rows, plain 128-byte swizzle)
static bool tc_make_map(CUtensorMap* m, const void* base, const TcOperand& op, int K, int BK, int box_rows, int elt = 4) {
    TcMapKey key;
    memset(&key, 0, sizeof key);
    key.elt = elt;
    const CUtensorMapDataType dt = elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    key.base = base; key.pitch = op.pitch; key.c2_stride = op.c2_dim > 1 ? op.c2_stride : 0; key.K = K; key.rows = op.rows;
    key.c2_dim = op.c2_dim > 1 ? op.c2_dim : 1; key.BK = BK; key.box_rows = box_rows; key.mn = op.mn;
    if (!g_tc_map_cache) g_tc_map_cache = (TcMapEntry*)calloc(TC_MAP_CACHE, sizeof(TcMapEntry));
    TcMapEntry* e = nullptr;
    if (g_tc_map_cache) {
        uint64_t h = 1469598103934665603ull;
        const unsigned char* kb = (const unsigned char*)&key;
        for (size_t i = 0; i < sizeof key; i++) { h ^= kb[i]; h *= 1099511628211ull; }
        e = &g_tc_map_cache[h % TC_MAP_CACHE];
        if (e->valid && memcmp(&e->key, &key, sizeof key) == 0) { *m = e->map; return true; }
    }
    if (op.mn) {
        // the array is [K, rows] with rows contiguous: {rows, K, 1}, boxes of 32 floats x BK k-rows, 128-byte swizzle of 32-byte units
        const bool swm = tc_swapped(op);
        const cuuint64_t nsl = (cuuint64_t)(op.c2_dim > 1 ? op.c2_dim : 1);
        const cuuint64_t krow = (cuuint64_t)op.pitch * elt;
        const cuuint64_t sl = op.c2_dim > 1 ? (cuuint64_t)op.c2_stride * elt : krow * (cuuint64_t)K;
        cuuint64_t dims[3] = {(cuuint64_t)op.rows, swm ? nsl : (cuuint64_t)K, swm ? (cuuint64_t)K : nsl};
        cuuint64_t strides[2] = {swm ? sl : krow, swm ? krow : sl};
        cuuint32_t box[3] = {(cuuint32_t)(128 / elt), swm ? 1u : (cuuint32_t)BK, swm ? (cuuint32_t)BK : 1u};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = g_tc_encode(m, dt, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 elt == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
        if (e) { e->key = key; e->map = *m; e->valid = true; }
        return true;
    }
    const bool sw = tc_swapped(op);
    const cuuint64_t nslot = (cuuint64_t)(op.c2_dim > 0 ? op.c2_dim : 1);
    const cuuint64_t slot_stride = (cuuint64_t)(op.c2_dim > 1 ? op.c2_stride : (long)op.pitch * op.rows) * elt;
    cuuint64_t dims[3] = {(cuuint64_t)K, sw ? nslot : (cuuint64_t)op.rows, sw ? (cuuint64_t)op.rows : nslot};
    cuuint64_t strides[2] = {sw ? slot_stride : (cuuint64_t)op.pitch * elt, sw ? (cuuint64_t)op.pitch * elt : slot_stride};
    cuuint32_t box[3] = {(cuuint32_t)BK, sw ? 1u : (cuuint32_t)box_rows, sw ? (cuuint32_t)box_rows : 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_tc_encode(m, dt, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             BK * elt == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (e) { e->key = key; e->map = *m; e->valid = true; }
    return true;
}

static inline bool tc_aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

template <int BN, int BK, int NTERMS, int STAGES, int CTAS = 1, bool AMN = false, bool BMN = false, bool F16 = false, bool PREP = false>
static bool tc_launch_t(sb_ctx_t* c, const TcProblem& p) {
    CUtensorMap mAh, mAl, mBh, mBl;
    constexpr int BROWS = BN / CTAS;
    constexpr bool CONV = (CTAS == 2 && NTERMS == 3);
    constexpr int BKE = PREP ? 2 * BK : BK;
    if (PREP) {
        if (!tc_make_map(&mAh, p.A.h1, p.A, p.K, BKE, TC_BM, 2) || !tc_make_map(&mBh, p.B.h1, p.B, p.K, BKE, BROWS, 2) ||
            !tc_make_map(&mAl, p.A.h2, p.A, p.K, BKE, TC_BM, 2) || !tc_make_map(&mBl, p.B.h2, p.B, p.K, BKE, BROWS, 2)) return false;
    } else
    if (!tc_make_map(&mAh, p.A.hi, p.A, p.K, BK, TC_BM) || !tc_make_map(&mBh, p.B.hi, p.B, p.K, BK, BROWS)) return false;
    if (!PREP && NTERMS == 3 && !CONV) { if (!tc_make_map(&mAl, p.A.lo, p.A, p.K, BK, TC_BM) || !tc_make_map(&mBl, p.B.lo, p.B, p.K, BK, BROWS)) return false; }
    else if (!PREP) { mAl = mAh; mBl = mBh; }
    constexpr int STAGE_BYTES = (NTERMS == 3 ? 2 : 1) * (TC_BM + BROWS) * BK * 4;
    constexpr size_t stg_bytes = (size_t)TC_STG_ROWS * (BN + 4) * 4;
    constexpr size_t ring_bytes = (size_t)STAGES * STAGE_BYTES;
    constexpr size_t smem = ring_bytes + stg_bytes + 1024 + 512;      // ring, output staging, alignment slack, barriers
    static_assert(smem <= 232448, "shared memory of one CTA");
    auto kern = gemm_tc_kernel<BN, BK, NTERMS, STAGES, CTAS, AMN, BMN, F16, PREP>;
    constexpr int THREADS = CONV ? TC_CONV_THREADS : TC_THREADS;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
        attr_set = true;
    }
    const int tiles_m = (p.M + TC_BM * CTAS - 1) / (TC_BM * CTAS), tiles_n = (p.N + BN - 1) / BN;
    // square tile grid with everything above the diagonal skipped: only the tiles on or below it are enumerated
    const int tri = (p.causal == TC_CAUSAL_SKIP_UPPER && BN == TC_BM * CTAS && tiles_m == tiles_n) ? 1 : 0;
    const int tiles = tri ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
    // one CTA (pair) per SM (pair); while gradient buckets are being reduced beside the backward pass the grid leaves the
    // collective's SMs free, or the CTAs that found no SM would run their share of the tiles after all the others
    const int sms = (c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148);
    const int slots = max(1, (sms - (c->gemm_reserve_sms < sms ? c->gemm_reserve_sms : 0)) / CTAS);
    // tail split: cut the tiles of the last, partly filled wave into k pieces that fill it
    int split_full = tiles, split_s = 1;
    float* partial = nullptr;
    if (c->gemm_tail_split && p.nbatch <= 1 && p.causal == TC_CAUSAL_NONE) {
        const int full = tiles / slots * slots, rem = tiles - full;
        constexpr int KB_PER_CHUNK = TC_CHUNK_K / BKE > 0 ? TC_CHUNK_K / BKE : 1;
        const int num_kb = (p.K + BKE - 1) / BKE;
        // an item's epilogue costs about as much as 160 floats of k (5.3 us against 0.52 us per 16 floats, measured with a
        // K sweep), the fix-up pass about as much as 256; costs below are in tile times
        // (FP16 parts: a stage of 32 k takes 0.27 us, so the same epilogue is worth 20 stages)
        const double ovh = (F16 ? 20.0 : 10.0 * 16 / BKE) / num_kb, fix = (F16 ? 30.0 : 16.0 * 16 / BKE) / num_kb;
        double best = rem > 0 ? 1.0 + ovh : 0.0;
        for (int s = 2; s <= 8 && rem > 0; s++) {
            const int per = ((num_kb + s - 1) / s + KB_PER_CHUNK - 1) / KB_PER_CHUNK * KB_PER_CHUNK;
            if (per * (s - 1) >= num_kb || per * BKE < 128) continue;     // an empty or very short piece
            const int waves = (rem * s + slots - 1) / slots;
            const double cost = waves * ((double)per / num_kb + ovh) + fix;
            if (cost < best - 0.05) { best = cost; split_s = s; }
        }
        if (split_s > 1) {
            split_full = full;
            partial = (float*)sb_gemm_stage(c, 4, (size_t)rem * split_s * CTAS * TC_BM * BN * sizeof(float));
            if (!partial) return false;
        }
    }
    const int grid_tiles = split_full + (tiles - split_full) * split_s;
    const int nbatch = p.nbatch > 0 ? p.nbatch : 1;
    const int total_items = grid_tiles * nbatch;
    // causal k ranges: items are ordered longest first and dealt to half as many clusters in snake order
    static int snake_on = -1;
    if (snake_on < 0) { const char* e = getenv("SERAPH_B200_GEMM_SNAKE"); snake_on = (e && e[0] == '0') ? 0 : 1; }
    const int snake = (snake_on && (p.causal == TC_CAUSAL_K_UPTO_M || p.causal == TC_CAUSAL_K_FROM_M)) ? 1 : 0;
    int G = snake ? (total_items + 1) / 2 : total_items;
    if (G > slots) G = slots;
    if (G < 1) G = 1;
    dim3 grid((unsigned)(G * CTAS), 1u);
    const int swap_mask = (tc_swapped(p.A) ? 1 : 0) | (tc_swapped(p.B) ? 2 : 0);
    // plain tiles whose rows are 16-byte multiples at 16-byte addresses leave through the store warps
    const int store_warps = (CONV && p.epi.mode == TC_EPI_PLAIN && (p.ldc & 3) == 0 && (p.N & 3) == 0 && (p.c_batch_stride & 3) == 0 &&
                             tc_aligned16(p.C)) ? 1 : 0;
    if (CTAS == 2) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof cfg);
        cfg.gridDim = grid; cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)c->pub.stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, kern, mAh, mAl, mBh, mBl, p.C, p.ldc, p.c_batch_stride, p.M, p.N, p.K, p.acc, p.causal,
                               p.A.c2_base, p.A.c2_step, p.B.c2_base, p.B.c2_step, p.B.c2_div, swap_mask, split_full, split_s, partial, p.epi,
                               nbatch, total_items, snake, tri, store_warps, p.amax_a, p.amax_b, p.out_amax, c->d_status) != cudaSuccess) return false;
    } else {
        kern<<<grid, THREADS, smem, (cudaStream_t)c->pub.stream>>>(mAh, mAl, mBh, mBl, p.C, p.ldc, p.c_batch_stride, p.M, p.N, p.K, p.acc,
                                                                     p.causal, p.A.c2_base, p.A.c2_step, p.B.c2_base, p.B.c2_step, p.B.c2_div,
                                                                     swap_mask, split_full, split_s, partial, p.epi,
                                                                     nbatch, total_items, snake, tri, store_warps, p.amax_a, p.amax_b, p.out_amax, c->d_status);
    }
    c->launches++;
    if (split_s > 1) {
        const int nblocks = (tiles - split_full) * CTAS;
        const long items = (long)nblocks * TC_BM * (BN / 4);
        tc_splitk_fixup_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)c->pub.stream>>>(partial, p.C, p.ldc, p.M, p.N, p.acc, BN, CTAS,
                                                                                                        split_full, split_s, nblocks, p.acc ? nullptr : p.out_amax);
        c->launches++;
    }
    return cudaGetLastError() == cudaSuccess;
}

// picks the tile width from N; nterms: 3 = FP32-accurate, 1 = TF32
static bool tc_launch(sb_ctx_t* c, const TcProblem& p, int nterms) {
    if (!tc_load_encode()) return false;
    const bool raw = nterms == 1 || (p.A.lo == nullptr && p.B.lo == nullptr);      // the pair kernel makes the lo parts itself
    if (c->gemm_pair && raw) {
        const int lay = (p.A.mn ? 1 : 0) | (p.B.mn ? 2 : 0);
        if (p.N > 128) {
            if (nterms == 3 && p.amax_a && p.amax_b && p.A.h1 && p.B.h1) switch (lay) {
                case 0: return tc_launch_t<256, 16, 3, 5, 2, false, false, true, true>(c, p);
                case 1: return tc_launch_t<256, 16, 3, 5, 2, true, false, true, true>(c, p);
                case 2: return tc_launch_t<256, 16, 3, 5, 2, false, true, true, true>(c, p);
                default: return tc_launch_t<256, 16, 3, 5, 2, true, true, true, true>(c, p);
            }
            if (nterms == 3) switch (lay) {
                case 0: return tc_launch_t<256, 16, 3, 5, 2, false, false>(c, p);
                case 1: return tc_launch_t<256, 16, 3, 5, 2, true, false>(c, p);
                case 2: return tc_launch_t<256, 16, 3, 5, 2, false, true>(c, p);
                default: return tc_launch_t<256, 16, 3, 5, 2, true, true>(c, p);
            }
            switch (lay) {
                case 0: return tc_launch_t<256, 32, 1, 5, 2, false, false>(c, p);
                case 1: return tc_launch_t<256, 32, 1, 5, 2, true, false>(c, p);
                case 2: return tc_launch_t<256, 32, 1, 5, 2, false, true>(c, p);
                default: return tc_launch_t<256, 32, 1, 5, 2, true, true>(c, p);
            }
        }
        // narrow outputs (attention's products with V, K, Q, dO: N = head_dim): 256 x 128 tiles
        if (nterms == 3 && p.amax_a && p.amax_b && p.A.h1 && p.B.h1) switch (lay) {
            case 0: return tc_launch_t<128, 16, 3, 8, 2, false, false, true, true>(c, p);
            case 1: return tc_launch_t<128, 16, 3, 8, 2, true, false, true, true>(c, p);
            case 2: return tc_launch_t<128, 16, 3, 8, 2, false, true, true, true>(c, p);
            default: return tc_launch_t<128, 16, 3, 8, 2, true, true, true, true>(c, p);
        }
        if (nterms == 3) switch (lay) {
            case 0: return tc_launch_t<128, 16, 3, 8, 2, false, false>(c, p);
            case 1: return tc_launch_t<128, 16, 3, 8, 2, true, false>(c, p);
            case 2: return tc_launch_t<128, 16, 3, 8, 2, false, true>(c, p);
            default: return tc_launch_t<128, 16, 3, 8, 2, true, true>(c, p);
        }
        switch (lay) {
            case 0: return tc_launch_t<128, 32, 1, 8, 2, false, false>(c, p);
            case 1: return tc_launch_t<128, 32, 1, 8, 2, true, false>(c, p);
            case 2: return tc_launch_t<128, 32, 1, 8, 2, false, true>(c, p);
            default: return tc_launch_t<128, 32, 1, 8, 2, true, true>(c, p);
        }
    }
    if (p.A.mn || p.B.mn || (nterms == 3 && (!p.A.lo || !p.B.lo))) return false;    // only the pair kernel takes these
    if (p.N > 128) return nterms == 3 ? tc_launch_t<256, 16, 3, 3>(c, p) : tc_launch_t<256, 32, 1, 3>(c, p);
    return nterms == 3 ? tc_launch_t<128, 16, 3, 5>(c, p) : tc_launch_t<128, 32, 1, 5>(c, p);
}

static inline int tc_ew_blocks(sb_ctx_t* c, size_t items) {
    size_t b = (items + 255) / 256, cap = (size_t)(c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148) * 8;
    return (int)(b > cap ? cap : (b ? b : 1));
}
