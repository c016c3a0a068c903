/* Partition arithmetic of the range-sharded optimizer; see include/b200_shard_plan.h. */
#include "b200_shard_plan.h"

#include <limits.h>

int b200_shard_plan(long total, int rank, int world, B200ShardPlan* out)
{
    if (world < 1 || rank < 0 || rank >= world)
        return B200_SHARD_BAD_RANK;
    if (total < 0)
        return B200_SHARD_BAD_SIZE;
    const long quads = (total + 3) / 4;
    const long per = (quads + world - 1) / world;
    out->total = total;
    out->shard = per * 4;
    out->padded = out->shard * world;
    out->lo = out->shard * rank;
    out->hi = out->lo + out->shard;
    out->rank = rank;
    out->world = world;
    return B200_SHARD_OK;
}

int b200_shard_layout(const int* sizes, int count, long* offsets, long* total)
{
    long at = 0;
    for (int i = 0; i < count; ++i) {
        if (sizes[i] < 0)
            return B200_SHARD_BAD_SIZE;
        offsets[i] = at;
        at += ((long)sizes[i] + 3) / 4 * 4;
    }
    *total = at;
    return B200_SHARD_OK;
}

int b200_shard_overlap(long off, int size, long lo, long hi, long* t_begin, long* t_end)
{
    const long a = off > lo ? off : lo;
    const long b = off + size < hi ? off + size : hi;
    if (b <= a) {
        *t_begin = *t_end = 0;
        return 0;
    }
    *t_begin = a - off;
    *t_end = b - off;
    return 1;
}

int b200_shard_check_peers(const long* reported, int world, const B200ShardPlan* mine, int* bad_rank)
{
    for (int r = 0; r < world; ++r) {
        const long* t = reported + 3 * r;
        if (t[0] != mine->total || t[1] != mine->shard || t[2] != (long)mine->world) {
            if (bad_rank)
                *bad_rank = r;
            return B200_SHARD_PEER_MISMATCH;
        }
    }
    return B200_SHARD_OK;
}
