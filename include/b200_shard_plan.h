/* Partition arithmetic of the range-sharded optimizer.  Pure C, no CUDA: the same functions serve
 * the device code path (csrc/host/b200_sharded_optimizer.c) and its host-only tests.
 *
 * A flat parameter vector of `total` floats is padded to world * shard floats, shard a multiple of
 * 4 (16 bytes, so every rank keeps 128-bit accesses and an in-place all-gather has equal pieces);
 * rank r owns [r*shard, (r+1)*shard).  Replaces the per-tensor loops of the reference's
 * optimizer.c:54-69 and ema.c:29-35, which have no notion of ranks.
 */
#ifndef B200_SHARD_PLAN_H
#define B200_SHARD_PLAN_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    long total;   /* real elements */
    long padded;  /* world * shard */
    long shard;   /* elements owned by each rank (multiple of 4) */
    long lo, hi;  /* this rank's range of the padded vector */
    int rank, world;
} B200ShardPlan;

enum {
    B200_SHARD_OK = 0,
    B200_SHARD_BAD_RANK = -1,     /* rank outside [0, world) or world < 1 */
    B200_SHARD_BAD_SIZE = -2,     /* negative element count, or a count beyond int range per tensor */
    B200_SHARD_PEER_MISMATCH = -3 /* a peer reported another total / shard / world */
};

/* Fills `out` for `rank` of `world`; returns B200_SHARD_OK or a negative code (out untouched). */
int b200_shard_plan(long total, int rank, int world, B200ShardPlan* out);

/* Offsets of `count` tensors inside the flat vector: each tensor starts on a multiple of 4 floats.
   Writes offsets[count] and the flat length to *total; returns B200_SHARD_OK or B200_SHARD_BAD_SIZE. */
int b200_shard_layout(const int* sizes, int count, long* offsets, long* total);

/* The part of a tensor at [off, off+size) that falls into [lo, hi): writes the tensor-local range
   [*t_begin, *t_end); returns 1 if it is non-empty, else 0. */
int b200_shard_overlap(long off, int size, long lo, long hi, long* t_begin, long* t_end);

/* Every rank publishes (total, shard, world); `reported` holds world triples in rank order.
   Returns B200_SHARD_OK, or B200_SHARD_PEER_MISMATCH with *bad_rank set to the first rank that
   disagrees with `mine` (a rank built for another model or another world size must be caught
   before any collective runs on mismatched buffers). */
int b200_shard_check_peers(const long* reported, int world, const B200ShardPlan* mine, int* bad_rank);

#ifdef __cplusplus
}
#endif
#endif
