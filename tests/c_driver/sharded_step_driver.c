/* One rank of a data-parallel optimizer step, as a plain C caller of libane_cuda's multi-GPU group would write it:
 *
 *     sharded_step_driver <nranks> <rank> <id file> <output file> <nccl|peer> [steps]
 *
 * Rank 0 creates the group id and leaves it in <id file>; every rank joins, fills its flat buffers from a
 * stateless integer hash (parameters equal on all ranks, gradients different per rank -- the Python test
 * regenerates the same values), runs ane_cuda_sharded_adam_step `steps` times with a host-side deadline
 * after each, and writes  w[n_padded] | m[slice] | v[slice] | squared norm of the last step  to <output file>.
 * The reference is a single-process program (training_dynamic/train.m:750-869 is its optimizer step);
 * this is the caller a multi-GPU version of that loop would contain.
 *
 * Build: gcc sharded_step_driver.c -I<include> -L<libdir> -lane_cuda -o sharded_step_driver */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "ane_cuda.h"

#define CALL(expr) do { int rc__ = (expr); if (rc__ != ANE_CUDA_OK) { fprintf(stderr, "rank %d: %s failed (%d): %s\n", rank, #expr, rc__, ane_cuda_last_error()); return 10; } } while (0)

enum { N_PARAMS = 100003, N_DECAY = 90000 };

/* value i of stream `seed`: uniform in [-scale/2, scale/2), the same bits in C and in numpy */
static float hashed(uint32_t i, uint32_t seed, float scale) {
    uint32_t x = i * 2654435761u + seed * 40503u + 12345u;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13; x *= 3266489917u; x ^= x >> 16;
    return ((float)(x >> 8) * (1.0f / 16777216.0f) - 0.5f) * scale;
}

int main(int argc, char **argv) {
    if (argc < 6) { fprintf(stderr, "usage: %s nranks rank id_file out_file nccl|peer [steps]\n", argv[0]); return 2; }
    const int nranks = atoi(argv[1]), rank = atoi(argv[2]);
    const char *id_file = argv[3], *out_file = argv[4];
    const int peer = strcmp(argv[5], "peer") == 0;
    const int steps = argc > 6 ? atoi(argv[6]) : 2;
    CALL(ane_cuda_init(rank));

    unsigned char id[ANE_CUDA_COMM_ID_BYTES];
    if (rank == 0) {
        CALL(ane_cuda_comm_unique_id(id));
        char tmp[4096];
        snprintf(tmp, sizeof tmp, "%s.tmp", id_file);
        FILE *f = fopen(tmp, "wb");
        if (!f || fwrite(id, 1, sizeof id, f) != sizeof id) { fprintf(stderr, "cannot write %s\n", tmp); return 3; }
        fclose(f);
        if (rename(tmp, id_file) != 0) { fprintf(stderr, "cannot publish %s\n", id_file); return 3; }
    } else {
        FILE *f = NULL;
        for (int tries = 0; tries < 3000 && !(f = fopen(id_file, "rb")); tries++) usleep(10000);     /* 30 s */
        if (!f || fread(id, 1, sizeof id, f) != sizeof id) { fprintf(stderr, "rank %d: no group id in %s\n", rank, id_file); return 3; }
        fclose(f);
    }
    CALL(ane_cuda_comm_init(nranks, rank, id, 60.0));

    const size_t q = (size_t)nranks * 256;
    const size_t n_padded = (N_PARAMS + q - 1) / q * q, slice = n_padded / nranks, lo = (size_t)rank * slice;
    float *hw = calloc(n_padded, 4), *hg = calloc(n_padded, 4);
    for (size_t i = 0; i < N_PARAMS; i++) { hw[i] = hashed((uint32_t)i, 7, 0.08f); hg[i] = hashed((uint32_t)i, 100 + rank, 0.04f); }
    ANECudaBuf *bw = ane_cuda_alloc(n_padded * 4), *bg = ane_cuda_alloc(n_padded * 4), *bm = ane_cuda_alloc(n_padded * 4),
               *bv = ane_cuda_alloc(n_padded * 4), *bn = ane_cuda_alloc(4);
    if (!bw || !bg || !bm || !bv || !bn) { fprintf(stderr, "rank %d: %s\n", rank, ane_cuda_last_error()); return 4; }
    float *w = ane_cuda_devptr(bw), *g = ane_cuda_devptr(bg), *m = ane_cuda_devptr(bm), *v = ane_cuda_devptr(bv), *nsq = ane_cuda_devptr(bn);
    CALL(ane_cuda_write(bw, 0, hw, n_padded * 4));
    CALL(ane_cuda_write(bg, 0, hg, n_padded * 4));
    CALL(ane_cuda_zero_dev(NULL, m, n_padded * 4));
    CALL(ane_cuda_zero_dev(NULL, v, n_padded * 4));
    CALL(ane_cuda_sync(NULL));
    if (peer) CALL(ane_cuda_comm_map_peers(w, g, n_padded));

    for (int t = 1; t <= steps; t++) {
        CALL(ane_cuda_sharded_adam_step(NULL, w, g, m, v, n_padded, N_DECAY, N_PARAMS, t, 3e-4f, 0.9f, 0.95f, 1e-8f, 0.1f, 0.5f, 1.0f,
                                        ANE_ADAM_DYNAMIC, nsq));
        CALL(ane_cuda_comm_wait(NULL, 60.0));
    }
    /* the loss all-reduce of a data-parallel step: every rank contributes rank + 1 */
    float loss = (float)(rank + 1), loss_sum = 0.0f;
    ANECudaBuf *bl = ane_cuda_alloc(4);
    CALL(ane_cuda_write(bl, 0, &loss, 4));
    CALL(ane_cuda_allreduce_f32(NULL, ane_cuda_devptr(bl), 1));
    CALL(ane_cuda_comm_wait(NULL, 60.0));
    CALL(ane_cuda_read(bl, 0, &loss_sum, 4));
    if (loss_sum != (float)(nranks * (nranks + 1) / 2)) { fprintf(stderr, "rank %d: all-reduce gave %g\n", rank, loss_sum); return 5; }

    float *ow = malloc(n_padded * 4), *om = malloc(slice * 4), *ov = malloc(slice * 4), onsq = 0.0f;
    CALL(ane_cuda_read(bw, 0, ow, n_padded * 4));
    CALL(ane_cuda_read(bm, lo * 4, om, slice * 4));
    CALL(ane_cuda_read(bv, lo * 4, ov, slice * 4));
    CALL(ane_cuda_read(bn, 0, &onsq, 4));
    FILE *f = fopen(out_file, "wb");
    if (!f) { fprintf(stderr, "cannot write %s\n", out_file); return 6; }
    fwrite(ow, 4, n_padded, f); fwrite(om, 4, slice, f); fwrite(ov, 4, slice, f); fwrite(&onsq, 4, 1, f);
    fclose(f);
    CALL(ane_cuda_comm_unmap_peers());
    CALL(ane_cuda_comm_destroy());
    ane_cuda_free(bw); ane_cuda_free(bg); ane_cuda_free(bm); ane_cuda_free(bv); ane_cuda_free(bn); ane_cuda_free(bl);
    ane_cuda_shutdown();
    printf("rank %d of %d done (%s form, %d steps, squared norm %.9g)\n", rank, nranks, peer ? "peer-memory" : "NCCL", steps, onsq);
    return 0;
}
