/*
 * dp_cli.c - what a command-line trainer needs to run data parallel, one process per GPU: who am I (environment of the
 * launcher), the communicator id carried from rank 0 to the others through a file, this rank's share of the samples, and
 * an agreement on whether every rank still has a batch (ranks must issue the same number of steps, because every step
 * ends in collectives).  The reference has no multi-GPU code (tools/seraph_train_cuda.c runs one process on one GPU), so
 * these entry points have no counterpart there; they are written against its data layout: train_load_data leaves
 * state->train_tokens, state->sample_offsets[num_samples] (start of every sample) and state->num_train_tokens
 * (src/train.c:812), and the trainer's loop takes sample i as [offsets[i], offsets[i+1]) with the last one ending at
 * num_train_tokens (tools/seraph_train_cuda.c:395-403).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>
#include "sb_internal.h"

static int env_int(const char* a, const char* b, int dflt) {
    const char* e = getenv(a);
    if (!e || !e[0]) e = getenv(b);
    return (e && e[0]) ? atoi(e) : dflt;
}

/* rank and world size from SERAPH_DP_RANK / SERAPH_DP_WORLD, else RANK / WORLD_SIZE as torchrun and most launchers set them;
 * (0, 1) when neither is set.  Returns 0, or 1 for an inconsistent pair. */
int seraph_dp_env(int* rank, int* world) {
    int r = env_int("SERAPH_DP_RANK", "RANK", 0), w = env_int("SERAPH_DP_WORLD", "WORLD_SIZE", 1);
    if (rank) *rank = r;
    if (world) *world = w;
    return (w < 1 || r < 0 || r >= w) ? 1 : 0;
}

/* seraph_dp_init for the rank the environment names.  Rank 0 makes the communicator id and writes it to the file
 * SERAPH_DP_ID_FILE (default /tmp/seraph_dp_id.<MASTER_PORT>); the other ranks wait up to two minutes for it.
 * A world of one does nothing.  Returns SB_OK or an SB_ERR_* code. */
int seraph_dp_init_from_env(cuda_train_context_t* ctx) {
    int rank = 0, world = 1;
    if (seraph_dp_env(&rank, &world)) return SB_ERR_ARG;
    if (world == 1) return seraph_dp_init(ctx, 0, 1, NULL);
    char path[600], tmp[640];
    const char* e = getenv("SERAPH_DP_ID_FILE");
    if (e && e[0]) snprintf(path, sizeof path, "%s", e);
    else { const char* port = getenv("MASTER_PORT"); snprintf(path, sizeof path, "/tmp/seraph_dp_id.%s", (port && port[0]) ? port : "0"); }
    unsigned char id[128];
    if (rank == 0) {
        if (seraph_dp_get_unique_id(id) != SB_OK) return SB_ERR_NCCL;
        snprintf(tmp, sizeof tmp, "%s.tmp.%d", path, (int)getpid());
        FILE* f = fopen(tmp, "wb");
        if (!f || fwrite(id, 1, sizeof id, f) != sizeof id) { if (f) fclose(f); return SB_ERR_ARG; }
        fclose(f);
        if (rename(tmp, path)) return SB_ERR_ARG;
    } else {
        struct timespec t0, t; clock_gettime(CLOCK_MONOTONIC, &t0);
        for (;;) {
            FILE* f = fopen(path, "rb");
            if (f) { size_t n = fread(id, 1, sizeof id, f); fclose(f); if (n == sizeof id) break; }
            clock_gettime(CLOCK_MONOTONIC, &t);
            if (t.tv_sec - t0.tv_sec > 120) { fprintf(stderr, "seraph_b200: rank %d never saw the communicator id at %s\n", rank, path); return SB_ERR_TIMEOUT; }
            struct timespec nap = {0, 20000000}; nanosleep(&nap, NULL);
        }
    }
    int rc = seraph_dp_init(ctx, rank, world, id);
    if (rank == 0 && rc == SB_OK && !(e && e[0])) { /* the default file is left for late joiners of this launch; the next launch overwrites it */ }
    return rc;
}

/* This rank's share of the samples: a contiguous run of num_samples / world samples (the remainder at the end is left out so
 * that every rank holds the same count), moved to the front of sample_offsets; *num_train_tokens becomes the end of the run's
 * last sample, so that the trainer's "last sample ends at num_train_tokens" rule stays right.  The token array is not touched.
 * Returns the index of the first sample of the share in the original numbering, or -1 for bad arguments. */
int seraph_dp_shard_samples(int* sample_offsets, int* num_samples, int* num_train_tokens, int rank, int world) {
    if (!sample_offsets || !num_samples || !num_train_tokens || world < 1 || rank < 0 || rank >= world) return -1;
    const int n = *num_samples, per = n / world;
    if (world == 1) return 0;
    const int first = rank * per;
    const int end_tok = (first + per < n) ? sample_offsets[first + per] : *num_train_tokens;
    memmove(sample_offsets, sample_offsets + first, (size_t)per * sizeof(int));
    *num_samples = per;
    *num_train_tokens = end_tok;
    return first;
}
