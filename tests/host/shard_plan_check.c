/* Host-only check of the range-sharded optimizer's partition arithmetic (include/b200_shard_plan.h).
 * No GPU, no CUDA headers: built with gcc alone and run by the CPU test suite.
 * Failure forms covered: a rank outside the world, an empty world, negative sizes, and a peer that
 * reports another model size, shard length or world size. */
#include "b200_shard_plan.h"

#include <stdio.h>
#include <stdlib.h>

static int fails = 0;
#define EXPECT(cond)                                                  \
    do {                                                              \
        if (!(cond)) {                                                \
            printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond);     \
            ++fails;                                                  \
        }                                                             \
    } while (0)

int main(void)
{
    B200ShardPlan p;
    /* ranges tile the padded vector exactly, cuts on multiples of 4, for awkward sizes and worlds */
    const long totals[] = { 0, 1, 3, 4, 5, 1000, 4099, 1561857, 67108864 };
    for (unsigned ti = 0; ti < sizeof totals / sizeof totals[0]; ++ti)
        for (int world = 1; world <= 16; ++world) {
            long next = 0;
            for (int r = 0; r < world; ++r) {
                EXPECT(b200_shard_plan(totals[ti], r, world, &p) == B200_SHARD_OK);
                EXPECT(p.lo == next && p.hi == p.lo + p.shard && p.shard % 4 == 0 && p.lo % 4 == 0);
                EXPECT(p.total == totals[ti] && p.world == world && p.rank == r);
                next = p.hi;
            }
            EXPECT(next == p.padded && p.padded >= totals[ti] && p.padded - totals[ti] < 4L * world + 4);
        }
    /* failure forms */
    p.shard = -77;
    EXPECT(b200_shard_plan(100, 4, 4, &p) == B200_SHARD_BAD_RANK && p.shard == -77);
    EXPECT(b200_shard_plan(100, -1, 4, &p) == B200_SHARD_BAD_RANK);
    EXPECT(b200_shard_plan(100, 0, 0, &p) == B200_SHARD_BAD_RANK);
    EXPECT(b200_shard_plan(-5, 0, 2, &p) == B200_SHARD_BAD_SIZE);

    /* tensor layout: the EDM UNet's pattern of matrices and single-float gains */
    const int sizes[] = { 576, 1, 36864, 1, 8192, 1, 7, 0, 73728 };
    const int count = (int)(sizeof sizes / sizeof sizes[0]);
    long off[16], total = 0;
    EXPECT(b200_shard_layout(sizes, count, off, &total) == B200_SHARD_OK);
    long expect = 0;
    for (int i = 0; i < count; ++i) {
        EXPECT(off[i] == expect && off[i] % 4 == 0);
        expect += (sizes[i] + 3L) / 4 * 4;
    }
    EXPECT(total == expect);
    const int bad_sizes[] = { 4, -1 };
    EXPECT(b200_shard_layout(bad_sizes, 2, off, &total) == B200_SHARD_BAD_SIZE);

    /* every element of every tensor belongs to exactly one rank's range */
    EXPECT(b200_shard_layout(sizes, count, off, &total) == B200_SHARD_OK);
    for (int world = 1; world <= 8; ++world) {
        long covered = 0;
        for (int r = 0; r < world; ++r) {
            EXPECT(b200_shard_plan(total, r, world, &p) == B200_SHARD_OK);
            for (int i = 0; i < count; ++i) {
                long b, e;
                if (b200_shard_overlap(off[i], sizes[i], p.lo, p.hi, &b, &e)) {
                    EXPECT(0 <= b && b < e && e <= sizes[i]);
                    EXPECT(off[i] + b >= p.lo && off[i] + e <= p.hi);
                    covered += e - b;
                }
            }
        }
        long sum = 0;
        for (int i = 0; i < count; ++i)
            sum += sizes[i];
        EXPECT(covered == sum);
    }

    /* peers: agreement, then one peer built for another model / world */
    EXPECT(b200_shard_plan(1000, 1, 4, &p) == B200_SHARD_OK);
    long rep[12];
    for (int r = 0; r < 4; ++r) {
        rep[3 * r] = 1000;
        rep[3 * r + 1] = p.shard;
        rep[3 * r + 2] = 4;
    }
    int bad = -1;
    EXPECT(b200_shard_check_peers(rep, 4, &p, &bad) == B200_SHARD_OK && bad == -1);
    rep[3 * 2] = 1004; /* rank 2 holds a different model */
    EXPECT(b200_shard_check_peers(rep, 4, &p, &bad) == B200_SHARD_PEER_MISMATCH && bad == 2);
    rep[3 * 2] = 1000;
    rep[3 * 3 + 1] = p.shard + 4; /* rank 3 cut its shard differently */
    EXPECT(b200_shard_check_peers(rep, 4, &p, &bad) == B200_SHARD_PEER_MISMATCH && bad == 3);
    rep[3 * 3 + 1] = p.shard;
    rep[2] = 8; /* rank 0 thinks the world has 8 ranks */
    EXPECT(b200_shard_check_peers(rep, 4, &p, &bad) == B200_SHARD_PEER_MISMATCH && bad == 0);

    printf("%d failure(s)\n", fails);
    return fails ? 1 : 0;
}
