// gemm_tc.cu - the reference's matmul entry points on the tcgen05 kernel of gemm_tc.cuh.
//
// The reference's three layouts (src/cuda_train_context.cu:2645-2709: NN, TN, NT, optional
// accumulate) map onto C (+)= A^[M,K] B^[N,K]^T:
//   * large, 16-byte-aligned products go to the CTA-pair kernel as they are: it reads either
//     operand in either layout and makes the lo parts of the FP32-accurate mode itself, so
//     nothing is prepared in HBM;
//   * the rest are brought to the single-CTA kernel's one form (both operands K-major) by an
//     operand-preparation pass: an operand that already is K-major is used in place (only its lo
//     part is written, 8 bytes per element); an operand that is not gets a transposed hi copy and
//     a transposed lo copy (12 bytes per element).
#include <stdio.h>
#include "gemm_tc.cuh"

// Bring one operand to K-major [rows, K].  `kmajor`: the caller's array already is [rows, K] row-major.
static bool prep_operand(sb_ctx_t* c, const float* src, int rows, int K, bool kmajor, bool want_lo, int slot, TcOperand* op) {
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    op->mn = 0; op->h1 = op->h2 = nullptr; op->rows = rows; op->c2_dim = 1; op->c2_stride = 0; op->c2_base = 0; op->c2_step = 0; op->lo = nullptr;
    if (kmajor) {
        op->hi = src; op->pitch = K;
        if (want_lo) {
            size_t n = (size_t)rows * K;
            float* l = (float*)sb_gemm_stage(c, slot, n * sizeof(float));
            if (!l) return false;
            split_lo_kernel<<<tc_ew_blocks(c, n / 4), 256, 0, s>>>(src, l, n / 4);     // K % 4 == 0, 16-byte aligned: checked by the caller
            c->launches++;
            op->lo = l;
        }
        return true;
    }
    // src is [K, rows] row-major: write the transpose (and its lo part)
    int Kp = (K + 3) & ~3;
    size_t n = (size_t)rows * Kp;
    float* h = (float*)sb_gemm_stage(c, slot, n * sizeof(float) * (want_lo ? 2 : 1));
    if (!h) return false;
    float* l = want_lo ? h + n : nullptr;
    dim3 grid((rows + 31) / 32, (Kp + 31) / 32);
    transpose_split_kernel<<<grid, 256, 0, s>>>(src, h, l, K, rows, Kp, want_lo ? 1 : 0);
    c->launches++;
    op->hi = h; op->lo = l; op->pitch = Kp;
    return true;
}

// Slot holding (or about to hold) the FP16 parts of operand x[n].  Inside a keep region the kept slots are searched
// first and the least recently used one is taken on a miss; outside, the call's own slot `own` is used.  *fresh: the
// parts must be made.  Returns the slot index, -1 on allocation failure.
static int f16_slot(sb_ctx_t* c, const float* x, size_t n, int own, bool* fresh) {
    if (!c->d_amax && sb_check(c, cudaMalloc(&c->d_amax, SB_F16_SLOTS * sizeof(float)), "amax alloc")) return -1;
    int s = own;
    *fresh = true;
    if (c->f16_keep) {
        int lru = 0;
        for (int i = 0; i < SB_F16_KEPT; i++) {
            if (c->f16_slot[i].valid && c->f16_slot[i].ptr == x && c->f16_slot[i].n == n) { c->f16_slot[i].stamp = ++c->f16_clock; *fresh = false; return i; }
            if (!c->f16_slot[i].valid) { lru = i; break; }
            if (c->f16_slot[i].stamp < c->f16_slot[lru].stamp) lru = i;
        }
        s = lru;
    }
    const size_t need = n * 2 * sizeof(__half);
    if (c->f16_slot[s].cap < need) {
        cudaStreamSynchronize((cudaStream_t)c->pub.stream);
        if (c->f16_slot[s].h) cudaFree(c->f16_slot[s].h);
        c->f16_slot[s].h = NULL; c->f16_slot[s].cap = 0;
        if (sb_check(c, cudaMalloc(&c->f16_slot[s].h, need), "FP16 parts alloc")) { c->status = SB_ERR_OOM; return -1; }
        c->f16_slot[s].cap = need;
    }
    c->f16_slot[s].ptr = x; c->f16_slot[s].n = n; c->f16_slot[s].valid = c->f16_keep ? 1 : 0; c->f16_slot[s].stamp = ++c->f16_clock;
    return s;
}

// ---- step-scoped parts of registered tensors --------------------------------------------------------------------
// Weights and the activations the forward pass saves for the backward pass are read by several products of one step
// (a weight by its forward product and by the input gradient; a saved activation by the forward product and by the
// weight gradient).  The step driver registers them; their parts live in one arena at fixed offsets and are made at
// the first use inside a step.  Nothing is valid across steps: the caller may write any of these tensors between calls.
static size_t parts_hash_of(const float* p, int cap) { return (size_t)(((uintptr_t)p >> 8) * 0x9E3779B97F4A7C15ull >> 20) & (size_t)(cap - 1); }
static void parts_rehash(sb_ctx_t* c) {
    for (int i = 0; i < c->parts_hash_cap; i++) c->parts_hash[i] = -1;
    for (int i = 0; i < c->parts_n; i++) {
        size_t h = parts_hash_of(c->parts_tab[i].ptr, c->parts_hash_cap);
        while (c->parts_hash[h] >= 0) h = (h + 1) & (size_t)(c->parts_hash_cap - 1);
        c->parts_hash[h] = i;
    }
}
static void parts_drop_arena(sb_ctx_t* c) {
    if (c->parts_arena || c->parts_amax) cudaStreamSynchronize((cudaStream_t)c->pub.stream);
    if (c->parts_arena) cudaFree(c->parts_arena);
    if (c->parts_amax) cudaFree(c->parts_amax);
    c->parts_arena = NULL; c->parts_arena_halves = 0; c->parts_amax = NULL; c->parts_amax_cap = 0;
    c->parts_gen++;
}
extern "C" void sb_parts_register(sb_ctx_t* c, int kind, const float* p, size_t n) {
    if (!p || !n || (n & 7)) return;
    if (c->parts_n == c->parts_cap) {
        int cap = c->parts_cap ? 2 * c->parts_cap : 256;
        sb_parts_entry_t* t = (sb_parts_entry_t*)realloc(c->parts_tab, (size_t)cap * sizeof *t);
        if (!t) return;
        c->parts_tab = t; c->parts_cap = cap;
    }
    if (2 * (c->parts_n + 1) > c->parts_hash_cap) {
        int cap = c->parts_hash_cap ? 2 * c->parts_hash_cap : 1024;
        int* h = (int*)realloc(c->parts_hash, (size_t)cap * sizeof(int));
        if (!h) return;
        c->parts_hash = h; c->parts_hash_cap = cap;
        parts_rehash(c);
    }
    sb_parts_entry_t* e = &c->parts_tab[c->parts_n];
    e->ptr = p; e->n = n; e->cur = 0; e->off = c->parts_total; e->gen = 0; e->kind = kind;
    c->parts_total += (2 * n + 63) & ~(size_t)63;                    // every tensor's parts start on a 128-byte boundary
    size_t h = parts_hash_of(p, c->parts_hash_cap);
    while (c->parts_hash[h] >= 0) h = (h + 1) & (size_t)(c->parts_hash_cap - 1);
    c->parts_hash[h] = c->parts_n++;
    if (c->parts_arena) parts_drop_arena(c);                          // laid out again at the next use
}
extern "C" void sb_parts_unregister(sb_ctx_t* c, int kind) {
    int m = 0; size_t total = 0;
    for (int i = 0; i < c->parts_n; i++) {
        if (c->parts_tab[i].kind == kind) continue;
        c->parts_tab[m] = c->parts_tab[i];
        c->parts_tab[m].off = total; total += (2 * c->parts_tab[m].n + 63) & ~(size_t)63;
        m++;
    }
    if (m == c->parts_n) return;
    c->parts_n = m; c->parts_total = total;
    if (c->parts_hash) parts_rehash(c);
    parts_drop_arena(c);
}
#define SB_HINT_CAP 4096
extern "C" void sb_parts_open(sb_ctx_t* c) {
    c->parts_gen++; c->parts_open = 1;
    c->hint_n = 0; c->hint_npending = 0;
    if (c->parts_cache && !c->hint_pool) {
        c->hint_tab = (decltype(c->hint_tab))calloc(SB_HINT_CAP, sizeof *c->hint_tab);
        if (!c->hint_tab || cudaMalloc((void**)&c->hint_pool, SB_HINT_CAP * sizeof(float)) != cudaSuccess) { cudaGetLastError(); c->hint_pool = NULL; }
        c->hint_cap = c->hint_pool ? SB_HINT_CAP : 0;
    }
    if (c->hint_pool) cudaMemsetAsync(c->hint_pool, 0, SB_HINT_CAP * sizeof(float), (cudaStream_t)c->pub.stream);
}
extern "C" void sb_parts_close(sb_ctx_t* c) { c->parts_gen++; c->parts_open = 0; c->hint_n = 0; c->hint_npending = 0; }
extern "C" void sb_amax_announce(sb_ctx_t* c, const float* out, size_t n) {
    if (!c->parts_open || !c->parts_cache || !c->hint_pool) return;
    if (c->hint_npending >= 4) {                       // announcements nobody took (a launcher without the feature): the oldest goes
        for (int i = 1; i < 4; i++) c->hint_pending[i - 1] = c->hint_pending[i];
        c->hint_npending = 3;
    }
    c->hint_pending[c->hint_npending].ptr = out; c->hint_pending[c->hint_npending].n = n; c->hint_npending++;
}
extern "C" unsigned* sb_amax_take(sb_ctx_t* c, const float* out, size_t n) {
    for (int i = 0; i < c->hint_npending; i++)
        if (c->hint_pending[i].ptr == out && c->hint_pending[i].n == n) {
            c->hint_pending[i] = c->hint_pending[--c->hint_npending];
            if (c->hint_n >= c->hint_cap) return NULL;
            c->hint_tab[c->hint_n].ptr = out; c->hint_tab[c->hint_n].n = n;
            return (unsigned*)(c->hint_pool + c->hint_n++);
        }
    return NULL;
}
extern "C" void sb_amax_forget(sb_ctx_t* c, const float* x) {
    if (!c->parts_open || !c->hint_n) return;
    for (int i = c->hint_n - 1; i >= 0; i--)
        if (c->hint_tab[i].ptr == x) { c->hint_tab[i].n = 0; return; }      // the latest writer decides: a length nobody asks for
}
extern "C" float* sb_amax_lookup(sb_ctx_t* c, const float* x, size_t n) {
    if (!c->parts_open) return NULL;
    for (int i = c->hint_n - 1; i >= 0; i--)
        if (c->hint_tab[i].ptr == x) return c->hint_tab[i].n == n ? c->hint_pool + i : NULL;      // the latest writer decides
    return NULL;
}
extern "C" void sb_parts_set_amax(sb_ctx_t* c, const float* x, float* word) {
    if (!c->parts_cache || !c->parts_open || !c->parts_n) return;
    size_t h = parts_hash_of(x, c->parts_hash_cap);
    int idx;
    while ((idx = c->parts_hash[h]) >= 0 && c->parts_tab[idx].ptr != x) h = (h + 1) & (size_t)(c->parts_hash_cap - 1);
    if (idx >= 0) c->parts_tab[idx].amax_ptr = word;
}
// x is being rewritten as a plain FP32 array: parts held for it in this step are stale
extern "C" void sb_parts_invalidate(sb_ctx_t* c, const float* x) {
    if (!c->parts_cache || !c->parts_open || !c->parts_n) return;
    size_t h = parts_hash_of(x, c->parts_hash_cap);
    int idx;
    while ((idx = c->parts_hash[h]) >= 0 && c->parts_tab[idx].ptr != x) h = (h + 1) & (size_t)(c->parts_hash_cap - 1);
    if (idx >= 0) c->parts_tab[idx].cur = 0;
}
extern "C" void sb_parts_free(sb_ctx_t* c) {
    parts_drop_arena(c);
    free(c->parts_tab); free(c->parts_hash); free(c->hint_tab);
    if (c->hint_pool) cudaFree(c->hint_pool);
    c->hint_tab = NULL; c->hint_pool = NULL; c->hint_cap = c->hint_n = 0;
    c->parts_tab = NULL; c->parts_hash = NULL; c->parts_n = c->parts_cap = c->parts_hash_cap = 0; c->parts_total = 0;
}
extern "C" int sb_parts_find(sb_ctx_t* c, const float* x, size_t n, void** hout, float** amax, int* fresh) {
    if (!c->parts_cache || !c->parts_open || !c->parts_n) return 0;
    size_t h = parts_hash_of(x, c->parts_hash_cap);
    int idx;
    while ((idx = c->parts_hash[h]) >= 0 && c->parts_tab[idx].ptr != x) h = (h + 1) & (size_t)(c->parts_hash_cap - 1);
    if (idx < 0 || c->parts_tab[idx].n < n || (n & 7)) return 0;          // n below the registered size: a step on fewer tokens
    if (!c->parts_arena) {
        // the arena must leave an eighth of the device for the scratch areas that are sized later
        size_t fr = 0, tot = 0;
        const size_t bytes = c->parts_total * sizeof(__half);
        cudaStreamSynchronize((cudaStream_t)c->pub.stream);
        if (cudaMemGetInfo(&fr, &tot) != cudaSuccess || fr < bytes || fr - bytes < tot / 8 ||
            cudaMalloc(&c->parts_arena, bytes) != cudaSuccess ||
            cudaMalloc((void**)&c->parts_amax, (size_t)c->parts_n * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            if (c->parts_arena) cudaFree(c->parts_arena);
            c->parts_arena = NULL; c->parts_amax = NULL;
            c->parts_cache = 0;                                       // does not fit: every product prepares its own operands
            return 0;
        }
        c->parts_arena_halves = c->parts_total; c->parts_amax_cap = c->parts_n;
    }
    sb_parts_entry_t* e = &c->parts_tab[idx];
    *hout = (__half*)c->parts_arena + e->off;
    *fresh = e->gen != c->parts_gen || e->cur != n;
    if (*fresh) e->amax_ptr = c->parts_amax + idx;
    *amax = e->amax_ptr;
    e->gen = c->parts_gen; e->cur = n;
    return 1;
}

extern "C" void sb_gemm_keep_begin(sb_ctx_t* c) { c->f16_keep = 1; }
// the array at `p` is about to be rewritten inside a keep region: parts kept for it are stale
extern "C" void sb_gemm_keep_forget(sb_ctx_t* c, const float* p) {
    for (int i = 0; i < SB_F16_SLOTS; i++) if (c->f16_slot[i].valid && c->f16_slot[i].ptr == p) c->f16_slot[i].valid = 0;
}
extern "C" void sb_gemm_keep_end(sb_ctx_t* c) {
    c->f16_keep = 0;
    for (int i = 0; i < SB_F16_SLOTS; i++) c->f16_slot[i].valid = 0;
}

// 1 when sb_gemm(A, B, ..., M, N, K, tA, tB) in the context's present mode reads its operands as prepared FP16 parts (so that a
// producer may hand over the parts of a registered operand instead of its FP32 array); the same conditions as in sb_gemm_tc below
static bool tc_f16_direct(const sb_ctx_t* c, int mode, int M, int N, int K, bool a_kmajor, bool b_kmajor) {
    return c->gemm_pair && M >= 128 && N >= 128 && (a_kmajor ? (K & 3) == 0 : (M & 3) == 0) && (b_kmajor ? (K & 3) == 0 : (N & 3) == 0) &&
           mode == SB_GEMM_FP16X3 && (a_kmajor ? (K & 7) == 0 : (M & 7) == 0) && (b_kmajor ? (K & 7) == 0 : (N & 7) == 0);
}
extern "C" int sb_gemm_reads_f16_parts(sb_ctx_t* c, int M, int N, int K, int tA, int tB) {
    const int mode = c->pub.use_bf16 ? SB_GEMM_BF16 : c->gemm_mode;
    if (K <= 0 || M < 32 || N < 32 || (double)M * N * K < (double)(1 << 21)) return 0;
    if (tA && tB) { tA = 0; tB = 0; }
    const bool a_kmajor = !tA, b_kmajor = tB != 0;
    if ((a_kmajor || b_kmajor) && (K & 3)) return 0;
    return tc_f16_direct(c, mode, M, N, K, a_kmajor, b_kmajor) ? 1 : 0;
}

// SERAPH_B200_GEMM_OUT_AMAX=0: the epilogue never leaves max |C| (the kernels that would form bounds from it fall back to plain outputs)
static bool tc_out_amax_on() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("SERAPH_B200_GEMM_OUT_AMAX"); on = (e && e[0] == '0') ? 0 : 1; }
    return on != 0;
}
extern "C" int sb_gemm_tc(sb_ctx_t* c, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc, int mode) {
    if (K <= 0 || M < 32 || N < 32) return 1;
    if ((double)M * N * K < (double)(1 << 21)) return 1;                 // too small to pay for the pipeline
    if (!tc_aligned16(A) || !tc_aligned16(B) || !tc_aligned16(C)) return 1;
    if (!tc_load_encode()) { sb_set_status(c, SB_ERR_CUDA); return 1; }
    if (tA && tB) { tA = 0; tB = 0; }                                     // as the reference's dispatch does
    bool a_kmajor = !tA;       // tA: A is [K,M]
    bool b_kmajor = tB != 0;   // !tB: B is [K,N]
    if ((a_kmajor || b_kmajor) && (K & 3)) return 1;                     // in-place K-major rows need a 16-byte pitch
    const bool x3 = (mode == SB_GEMM_FP32X3 || mode == SB_GEMM_FP16X3);
    TcProblem p;
    memset(&p.epi, 0, sizeof p.epi);
    p.amax_a = p.amax_b = nullptr;
    p.C = C; p.ldc = N; p.c_batch_stride = 0; p.M = M; p.N = N; p.K = K; p.acc = acc; p.nbatch = 1; p.causal = TC_CAUSAL_NONE;
    // direct path: the pair kernel on the caller's arrays (rows of either layout must be 16-byte multiples)
    if (c->gemm_pair && M >= 128 && N >= 128 && (a_kmajor ? (K & 3) == 0 : (M & 3) == 0) && (b_kmajor ? (K & 3) == 0 : (N & 3) == 0)) {
        p.A.hi = A; p.A.lo = nullptr; p.A.rows = M; p.A.mn = a_kmajor ? 0 : 1; p.A.pitch = a_kmajor ? K : M;
        p.B.hi = B; p.B.lo = nullptr; p.B.rows = N; p.B.mn = b_kmajor ? 0 : 1; p.B.pitch = b_kmajor ? K : N;
        p.A.c2_dim = p.B.c2_dim = 1; p.A.c2_stride = p.B.c2_stride = 0; p.A.c2_base = p.B.c2_base = 0; p.A.c2_step = p.B.c2_step = 0;
        p.A.h1 = p.A.h2 = p.B.h1 = p.B.h2 = nullptr;
        if (tc_f16_direct(c, mode, M, N, K, a_kmajor, b_kmajor)) {
            // FP16 split: each operand's largest magnitude, then its two FP16 parts (skipped for an operand whose parts are kept)
            const size_t na = (size_t)M * K, nb = (size_t)N * K;
            bool fa = false, fb = false;
            __half *ha, *hb; float *ma, *mb;
            void* hv; int fr; int sa = -1, sb = -1;
            if (sb_parts_find(c, A, na, &hv, &ma, &fr)) { ha = (__half*)hv; fa = fr != 0; }
            else { sa = f16_slot(c, A, na, SB_F16_KEPT, &fa); if (sa < 0) return 1; ha = (__half*)c->f16_slot[sa].h; if (fa) c->f16_slot[sa].amax = c->d_amax + sa; ma = c->f16_slot[sa].amax; }
            if (sb_parts_find(c, B, nb, &hv, &mb, &fr)) { hb = (__half*)hv; fb = fr != 0; }
            else { sb = f16_slot(c, B, nb, SB_F16_KEPT + 1, &fb); if (sb < 0) return 1; hb = (__half*)c->f16_slot[sb].h; if (fb) c->f16_slot[sb].amax = c->d_amax + sb; mb = c->f16_slot[sb].amax; }
            if (fa || fb) {
                cudaStream_t st = (cudaStream_t)c->pub.stream;
                int tp = sb_tick_begin(c, SB_CLS_GEMM_PREP);
                // a producer may have left the operand's largest magnitude behind: then only the split runs for it
                bool ka = false, kb = false;
                if (fa) { float* w = sb_amax_lookup(c, A, na); if (w) { ma = w; ka = true; if (sa >= 0) c->f16_slot[sa].amax = w; else sb_parts_set_amax(c, A, w); } }
                if (fb) { float* w = sb_amax_lookup(c, B, nb); if (w) { mb = w; kb = true; if (sb >= 0) c->f16_slot[sb].amax = w; else sb_parts_set_amax(c, B, w); } }
                const bool xa = fa && !ka, xb = fb && !kb;             // operands whose amax pass is needed
                if (xa) cudaMemsetAsync(ma, 0, sizeof(float), st);
                if (xb) cudaMemsetAsync(mb, 0, sizeof(float), st);
                if (xa || xb) {
                    const float* x0 = xa ? A : B; const size_t n0 = xa ? na : nb; float* m0 = xa ? ma : mb;
                    const bool two = xa && xb;
                    const dim3 pg(tc_ew_blocks(c, (two ? (na > nb ? na : nb) : n0) / 4), two ? 2 : 1);
                    tc_amax_kernel<<<pg, 256, 0, st>>>(x0, n0 / 4, (unsigned*)m0, B, nb / 4, (unsigned*)mb);
                    c->launches++;
                }
                {
                    const float* x0 = fa ? A : B; const size_t n0 = fa ? na : nb; __half* h0 = fa ? ha : hb; float* m0 = fa ? ma : mb;
                    const bool two = fa && fb;
                    const dim3 pg(tc_ew_blocks(c, (two ? (na > nb ? na : nb) : n0) / 4), two ? 2 : 1);
                    tc_split_f16_kernel<<<pg, 256, 0, st>>>(x0, n0 / 4, h0, h0 + n0, m0, B, nb / 4, hb, hb + nb, mb);
                    c->launches++;
                }
                sb_tick_end(c, tp, 0.0, 8.0 * (double)((fa ? na : 0) + (fb ? nb : 0)) + 4.0 * (double)((xa ? na : 0) + (xb ? nb : 0)));
            }
            p.amax_a = ma; p.amax_b = mb;
            p.A.h1 = ha; p.A.h2 = ha + na; p.B.h1 = hb; p.B.h2 = hb + nb;
        }
        int tg = sb_tick_begin(c, SB_CLS_GEMM);
        if (!acc && tc_out_amax_on()) p.out_amax = sb_amax_take(c, C, (size_t)M * N);      // an announced output: the epilogue leaves max |C| for the next operand split
        bool ok = tc_launch(c, p, x3 ? 3 : 1);
        sb_tick_end(c, tg, 2.0 * M * N * K, 4.0 * ((double)M * K + (double)N * K + (double)M * N * (acc ? 2 : 1)));
        if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
        return 0;
    }
    int tp = sb_tick_begin(c, SB_CLS_GEMM_PREP);
    if (!prep_operand(c, A, M, K, a_kmajor, x3, 0, &p.A)) return 1;
    if (!prep_operand(c, B, N, K, b_kmajor, x3, 1, &p.B)) return 1;
    double prep_bytes = (double)M * K * (a_kmajor ? (x3 ? 8 : 0) : (x3 ? 12 : 8)) + (double)N * K * (b_kmajor ? (x3 ? 8 : 0) : (x3 ? 12 : 8));
    sb_tick_end(c, tp, 0.0, prep_bytes);
    int tg = sb_tick_begin(c, SB_CLS_GEMM);
    if (!acc && tc_out_amax_on()) p.out_amax = sb_amax_take(c, C, (size_t)M * N);
    bool ok = tc_launch(c, p, x3 ? 3 : 1);
    sb_tick_end(c, tg, 2.0 * M * N * K, 4.0 * ((double)M * K + (double)N * K + (double)M * N * (acc ? 2 : 1)));
    if (!ok) { sb_set_status(c, SB_ERR_CUDA); return 1; }
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Self-test of the bounded-wait rule every tensor-core kernel of this library follows: one warp waits, with a limit of
// `limit_cycles` clock cycles, on an mbarrier phase that nothing completes; the wait gives up, the kernel records
// SB_ERR_TIMEOUT in the context's device status word and returns normally (no trap, the context stays usable).
__global__ void tc_bounded_wait_selftest_kernel(long long limit_cycles, int* status, long long* waited) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const long long t0 = clock64();
        const bool ok = mbar_wait_limit(&bar, 0, limit_cycles);
        if (waited) *waited = clock64() - t0;
        if (!ok) atomicExch(status, SB_ERR_TIMEOUT);
    }
}
extern "C" int seraph_b200_selftest_bounded_wait(cuda_train_context_t* ctx, long long limit_cycles, long long* waited_cycles_out) {
    sb_ctx_t* c = sb_priv(ctx);
    if (!c || limit_cycles <= 0 || limit_cycles > 2000000000ll) return SB_ERR_ARG;      // at most about a second
    long long* d_w = (long long*)sb_scratch(c, 64);
    if (!d_w) return SB_ERR_OOM;
    tc_bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)c->pub.stream>>>(limit_cycles, c->d_status, d_w);
    c->launches++;
    if (sb_check(c, cudaStreamSynchronize((cudaStream_t)c->pub.stream), "bounded-wait self-test")) return SB_ERR_CUDA;
    if (waited_cycles_out && cudaMemcpy(waited_cycles_out, d_w, sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) return SB_ERR_CUDA;
    return SB_OK;
}
