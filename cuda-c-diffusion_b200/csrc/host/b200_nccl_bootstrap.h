/* NCCL bootstrap for one process per GPU without a launcher-provided store: rank 0 writes the
 * communicator id to a file (atomically, via rename), the others poll for it with a bounded wait.
 * A peer that never shows up therefore ends in an error on the host, before anything is on a device. */
#ifndef B200_NCCL_BOOTSTRAP_H
#define B200_NCCL_BOOTSTRAP_H

#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

/* Returns 0 with *id filled, -1 on failure (message on stderr). */
static inline int b200_nccl_id_via_file(ncclUniqueId* id, int rank, const char* path, double wait_s)
{
    if (rank == 0) {
        char tmp[1024];
        if (ncclGetUniqueId(id) != ncclSuccess)
            return -1;
        snprintf(tmp, sizeof tmp, "%s.tmp", path);
        FILE* f = fopen(tmp, "wb");
        if (!f || fwrite(id, sizeof *id, 1, f) != 1) {
            fprintf(stderr, "cannot write %s\n", tmp);
            return -1;
        }
        fclose(f);
        return rename(tmp, path) == 0 ? 0 : -1;
    }
    for (int tries = 0; tries * 0.05 < wait_s; ++tries) {
        FILE* f = fopen(path, "rb");
        if (f) {
            const size_t got = fread(id, sizeof *id, 1, f);
            fclose(f);
            if (got == 1)
                return 0;
        }
        usleep(50000);
    }
    fprintf(stderr, "rank %d: rank 0 did not publish the NCCL id at %s within %.1f s\n", rank, path, wait_s);
    return -1;
}

#endif
