/* Range-sharded fused Adam+EMA for one process per GPU (NCCL over NVLink).
 *
 * The reference's optimizer_step (optimizer.c:54-69) and ema_update (ema.c:29-35) keep moments and
 * shadows for every tensor on every GPU and launch once per tensor.  Here every rank owns one
 * contiguous range of a flat parameter vector (include/b200_shard_plan.h), keeps m, v and the EMA
 * shadow ONLY for that range, updates it with one fused pass and publishes the new parameters to
 * the other ranks, either with an in-place ncclAllGather or -- B200_EXCHANGE_PEER_STORE -- from
 * inside the update kernel by plain peer stores into the other GPUs' copies of the vector
 * (launch_adam_ema_step_bcast; buffers exchanged once at creation through CUDA IPC).
 *
 * Compiled against the reference's src/nn.h (ParamList, checkpoint API); links NCCL.
 */
#ifndef B200_SHARDED_OPTIMIZER_H
#define B200_SHARDED_OPTIMIZER_H

#include "nn.h" /* the reference's header */
#include "b200_layer_kernels.h"
#include "b200_shard_plan.h"
#include <nccl.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { B200_EXCHANGE_ALLGATHER = 0, B200_EXCHANGE_PEER_STORE = 1 };

typedef struct {
    int rank, world;
    ncclComm_t comm; /* unused when world == 1 */
    float lr, beta1, beta2, eps, ema_decay;
    int exchange;     /* B200_EXCHANGE_* */
    int reduce_grads; /* 1: each rank holds partial gradient sums (data parallel): ncclReduceScatter first and
                         fold 1/world into the update; 0: the gradients are already the same on every rank */
} B200ShardedAdamConfig;

typedef struct B200ShardedAdam B200ShardedAdam;

/* Over a ParamList (tensors allocated elsewhere, e.g. by the reference's module constructors): gradients are
   packed into a flat arena before the update and parameters unpacked after it, one launch each.  Call after the
   weights hold their initial values: the EMA shadow starts as a copy of them.  Returns NULL (message on stderr)
   on a bad rank/world, a peer built for another model or world size, or a failed allocation / IPC exchange. */
B200ShardedAdam* b200_sharded_adam_create(const ParamList* pl, const B200ShardedAdamConfig* cfg, cudaStream_t s);
/* Over a flat vector of n floats that the optimizer allocates itself: fill b200_sharded_adam_params() (then call
   b200_sharded_adam_reset_shadow) and write gradients to b200_sharded_adam_grads() before every step. */
B200ShardedAdam* b200_sharded_adam_create_flat(long n, const B200ShardedAdamConfig* cfg, cudaStream_t s);
float* b200_sharded_adam_params(B200ShardedAdam* o);
float* b200_sharded_adam_grads(B200ShardedAdam* o);
const B200ShardPlan* b200_sharded_adam_plan(const B200ShardedAdam* o);
void b200_sharded_adam_reset_shadow(B200ShardedAdam* o, cudaStream_t s); /* shadow = current parameters */
void b200_sharded_adam_set_lr(B200ShardedAdam* o, float lr);
int b200_sharded_adam_timestep(const B200ShardedAdam* o);

/* One optimizer step on stream s (asynchronous).  Returns 0, or a negative value on an NCCL error.
   With B200_EXCHANGE_PEER_STORE the other ranks write into this rank's parameter vector during THEIR update
   kernels; the step ends with a one-word all-reduce so that, once it has completed on s, every peer's stores
   have landed.  A rank may start step k+1 only after every rank's readers of the step-k parameters are
   ordered before it: with reduce_grads the gradient reduce-scatter gives that order, without it the step
   opens with the same one-word all-reduce. */
int b200_sharded_adam_step(B200ShardedAdam* o, cudaStream_t s);

/* Gathers the sharded m, v and shadow and writes the reference's training checkpoint (checkpoint.c:92-114,
   per-tensor "CKTR" layout; rank 0 writes, every rank must call).  Load is the inverse: every rank reads the
   file and keeps its own range.  Both synchronise the stream.  Return 0 or the checkpoint API's negative code. */
int b200_sharded_adam_save(B200ShardedAdam* o, const char* path, int step, cudaStream_t s);
int b200_sharded_adam_load(B200ShardedAdam* o, const char* path, int* step, cudaStream_t s);
void b200_sharded_adam_free(B200ShardedAdam* o);

#ifdef __cplusplus
}
#endif
#endif
