/* Range-sharded fused Adam+EMA on a flat parameter vector: timing and self-check, one process per GPU.
 *
 *   RANK=r WORLD_SIZE=k LOCAL_RANK=d sharded_adam_bench [--params N] [--iters K] [--warmup W]
 *                                                      [--id-file PATH] [--check] [--ckpt FILE]
 *
 * Workload: N parameters ~ N(0, 0.02), gradients ~ N(0, 1e-3) (the same on every rank), Adam beta1 0.9,
 * beta2 0.999, eps 1e-8, lr 1e-4, EMA decay 0.999.  Timed, each with CUDA events on the launching stream and
 * the maximum over ranks:
 *   kernel        the fused update of this rank's range alone (36 B per owned parameter)
 *   allgather     update, then in-place ncclAllGather of the new parameters
 *   peer_store    update whose store phase also writes the other ranks' copies (launch_adam_ema_step_bcast),
 *                 then the one-word all-reduce that closes the step
 * --check: the two exchange forms and an unsharded update of the whole vector on this rank must leave
 * bit-identical parameters; --ckpt also round-trips the sharded state through the reference's
 * training checkpoint.  Prints one JSON line on rank 0.
 */
#include "b200_sharded_optimizer.h"
#include "b200_nccl_bootstrap.h"

#include <curand.h>
#include <math.h>
#include <string.h>

#define CK(call)                                                                                  \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
            exit(1);                                                                              \
        }                                                                                         \
    } while (0)
#define NK(call)                                                                                  \
    do {                                                                                          \
        ncclResult_t r_ = (call);                                                                 \
        if (r_ != ncclSuccess) {                                                                  \
            fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #call, ncclGetErrorString(r_)); \
            exit(1);                                                                              \
        }                                                                                         \
    } while (0)

static int env_int(const char* name, int dflt)
{
    const char* v = getenv(name);
    return v && v[0] ? atoi(v) : dflt;
}

static float max_over_ranks(float v, float* d_word, ncclComm_t comm, cudaStream_t s)
{
    if (!comm)
        return v;
    CK(cudaMemcpyAsync(d_word, &v, sizeof v, cudaMemcpyHostToDevice, s));
    NK(ncclAllReduce(d_word, d_word, 1, ncclFloat, ncclMax, comm, s));
    CK(cudaMemcpyAsync(&v, d_word, sizeof v, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    return v;
}

typedef struct {
    float ms;
} Timing;

/* average milliseconds of fn() over `iters` calls, events around each call, max over ranks */
#define TIME_LOOP(out, iters, comm, BODY)                           \
    do {                                                            \
        float total_ = 0.0f;                                        \
        for (int it_ = 0; it_ < (iters); ++it_) {                   \
            CK(cudaEventRecord(ev0, s));                            \
            BODY;                                                   \
            CK(cudaEventRecord(ev1, s));                            \
            CK(cudaEventSynchronize(ev1));                          \
            float ms_ = 0.0f;                                       \
            CK(cudaEventElapsedTime(&ms_, ev0, ev1));               \
            total_ += ms_;                                          \
        }                                                           \
        (out) = max_over_ranks(total_ / (iters), d_word, comm, s);  \
    } while (0)

int main(int argc, char** argv)
{
    long n = 64L << 20;
    int iters = 10, warmup = 3, check = 0;
    const char* id_file = "/tmp/sharded_adam_bench.ncclid";
    const char* ckpt = NULL;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--params") && i + 1 < argc) n = atol(argv[++i]);
        else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--id-file") && i + 1 < argc) id_file = argv[++i];
        else if (!strcmp(argv[i], "--ckpt") && i + 1 < argc) ckpt = argv[++i];
        else if (!strcmp(argv[i], "--check")) check = 1;
        else {
            fprintf(stderr, "unknown argument %s\n", argv[i]);
            return 2;
        }
    }
    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1), local = env_int("LOCAL_RANK", 0);
    CK(cudaSetDevice(local));
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    ncclComm_t comm = NULL;
    if (world > 1) {
        ncclUniqueId id;
        const char* w = getenv("B200_ID_WAIT_S");
        if (b200_nccl_id_via_file(&id, rank, id_file, w && w[0] ? atof(w) : 60.0))
            return 1;
        NK(ncclCommInitRank(&comm, world, id, rank));
    }
    float* d_word;
    CK(cudaMalloc((void**)&d_word, 256));
    cudaEvent_t ev0, ev1;
    CK(cudaEventCreate(&ev0));
    CK(cudaEventCreate(&ev1));

    B200ShardedAdamConfig cfg = { .rank = rank, .world = world, .comm = comm, .lr = 1e-4f, .beta1 = 0.9f, .beta2 = 0.999f,
        .eps = 1e-8f, .ema_decay = 0.999f, .exchange = B200_EXCHANGE_ALLGATHER, .reduce_grads = 0 };
    B200ShardedAdam* ag = b200_sharded_adam_create_flat(n, &cfg, s);
    cfg.exchange = B200_EXCHANGE_PEER_STORE;
    B200ShardedAdam* ps = b200_sharded_adam_create_flat(n, &cfg, s);
    if (!ag || !ps)
        return 1;
    const B200ShardPlan* plan = b200_sharded_adam_plan(ag);

    /* the same parameters and gradients on every rank and in both optimizers */
    curandGenerator_t gen;
    if (curandCreateGenerator(&gen, CURAND_RNG_PSEUDO_DEFAULT) != CURAND_STATUS_SUCCESS
        || curandSetPseudoRandomGeneratorSeed(gen, 7ULL) != CURAND_STATUS_SUCCESS || curandSetStream(gen, s) != CURAND_STATUS_SUCCESS)
        return 1;
    const size_t even = (size_t)(n + 1) / 2 * 2 <= (size_t)plan->padded ? (size_t)(n + 1) / 2 * 2 : (size_t)n / 2 * 2;
    curandGenerateNormal(gen, b200_sharded_adam_params(ag), even, 0.0f, 0.02f);
    curandGenerateNormal(gen, b200_sharded_adam_grads(ag), even, 0.0f, 1e-3f);
    if (plan->padded > n) { /* the padding tail stays zero */
        CK(cudaMemsetAsync(b200_sharded_adam_params(ag) + n, 0, (size_t)(plan->padded - n) * sizeof(float), s));
        CK(cudaMemsetAsync(b200_sharded_adam_grads(ag) + n, 0, (size_t)(plan->padded - n) * sizeof(float), s));
    }
    CK(cudaMemcpyAsync(b200_sharded_adam_params(ps), b200_sharded_adam_params(ag), (size_t)plan->padded * sizeof(float),
        cudaMemcpyDeviceToDevice, s));
    CK(cudaMemcpyAsync(b200_sharded_adam_grads(ps), b200_sharded_adam_grads(ag), (size_t)plan->padded * sizeof(float),
        cudaMemcpyDeviceToDevice, s));
    b200_sharded_adam_reset_shadow(ag, s);
    b200_sharded_adam_reset_shadow(ps, s);

    int failures = 0;
    double worst = 0.0;
    if (check) {
        /* reference on this rank: the whole vector in one unsharded launch per step */
        float *rp, *rm, *rv, *rs;
        const size_t bytes = (size_t)plan->padded * sizeof(float);
        CK(cudaMalloc((void**)&rp, bytes));
        CK(cudaMalloc((void**)&rm, bytes));
        CK(cudaMalloc((void**)&rv, bytes));
        CK(cudaMalloc((void**)&rs, bytes));
        CK(cudaMemcpyAsync(rp, b200_sharded_adam_params(ag), bytes, cudaMemcpyDeviceToDevice, s));
        CK(cudaMemcpyAsync(rs, rp, bytes, cudaMemcpyDeviceToDevice, s));
        CK(cudaMemsetAsync(rm, 0, bytes, s));
        CK(cudaMemsetAsync(rv, 0, bytes, s));
        for (int t = 1; t <= 3; ++t) {
            const float bc1 = 1.0f - powf(0.9f, (float)t), bc2 = 1.0f - powf(0.999f, (float)t);
            launch_adam_ema_step(rp, rm, rv, rs, b200_sharded_adam_grads(ag), 1e-4f, 0.9f, 0.999f, 1e-8f, bc1, bc2, 0.999f,
                1.0f, (long long)plan->padded, s);
            if (b200_sharded_adam_step(ag, s) || b200_sharded_adam_step(ps, s))
                return 1;
        }
        CK(cudaStreamSynchronize(s));
        float* h[3];
        const float* d[3] = { rp, b200_sharded_adam_params(ag), b200_sharded_adam_params(ps) };
        for (int k = 0; k < 3; ++k) {
            h[k] = (float*)malloc(bytes);
            CK(cudaMemcpy(h[k], d[k], bytes, cudaMemcpyDeviceToHost));
        }
        long diff_ag = 0, diff_ps = 0;
        for (long i = 0; i < plan->padded; ++i) {
            diff_ag += h[1][i] != h[0][i];
            diff_ps += h[2][i] != h[0][i];
            const double e = fabs((double)h[2][i] - h[0][i]);
            if (e > worst)
                worst = e;
        }
        if (diff_ag || diff_ps) {
            fprintf(stderr, "rank %d: %ld (all-gather) / %ld (peer store) of %ld parameters differ from the unsharded update\n",
                rank, diff_ag, diff_ps, plan->padded);
            failures++;
        }
        if (ckpt) { /* sharded state -> reference checkpoint -> sharded state */
            float* keep = (float*)malloc((size_t)plan->shard * sizeof(float));
            float* back = (float*)malloc((size_t)plan->shard * sizeof(float));
            int step = 0;
            if (b200_sharded_adam_save(ps, ckpt, 3, s) != 0)
                failures++;
            if (comm) { /* rank 0 has finished writing before anybody reads */
                NK(ncclAllReduce(d_word, d_word, 1, ncclFloat, ncclSum, comm, s));
                CK(cudaStreamSynchronize(s));
            }
            /* the optimizer keeps m/v/shadow private; compare through a second save after a load into `ag` */
            if (b200_sharded_adam_load(ag, ckpt, &step, s) != 0 || step != 3 || b200_sharded_adam_timestep(ag) != 3)
                failures++;
            /* after loading ps's state, one more identical step must give identical parameters again */
            if (b200_sharded_adam_step(ag, s) || b200_sharded_adam_step(ps, s))
                return 1;
            CK(cudaStreamSynchronize(s));
            CK(cudaMemcpy(keep, b200_sharded_adam_params(ag) + plan->lo, (size_t)plan->shard * sizeof(float), cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(back, b200_sharded_adam_params(ps) + plan->lo, (size_t)plan->shard * sizeof(float), cudaMemcpyDeviceToHost));
            long d2 = 0;
            for (long i = 0; i < plan->shard; ++i)
                d2 += keep[i] != back[i];
            if (d2) {
                fprintf(stderr, "rank %d: %ld parameters differ after the checkpoint round trip\n", rank, d2);
                failures++;
            }
            free(keep);
            free(back);
        }
        for (int k = 0; k < 3; ++k)
            free(h[k]);
        cudaFree(rp);
        cudaFree(rm);
        cudaFree(rv);
        cudaFree(rs);
        failures = (int)max_over_ranks((float)failures, d_word, comm, s);
    }

    /* ---- timing */
    float kern_ms = 0, ag_ms = 0, ps_ms = 0;
    float *km, *kv, *ksh;
    CK(cudaMalloc((void**)&km, (size_t)plan->shard * sizeof(float)));
    CK(cudaMalloc((void**)&kv, (size_t)plan->shard * sizeof(float)));
    CK(cudaMalloc((void**)&ksh, (size_t)plan->shard * sizeof(float)));
    CK(cudaMemsetAsync(km, 0, (size_t)plan->shard * sizeof(float), s));
    CK(cudaMemsetAsync(kv, 0, (size_t)plan->shard * sizeof(float), s));
    CK(cudaMemsetAsync(ksh, 0, (size_t)plan->shard * sizeof(float), s));
#define KERNEL_ONLY                                                                                                  \
    launch_adam_ema_step(b200_sharded_adam_params(ag) + plan->lo, km, kv, ksh, b200_sharded_adam_grads(ag) + plan->lo, \
        1e-4f, 0.9f, 0.999f, 1e-8f, 0.19f, 0.002f, 0.999f, 1.0f, (long long)plan->shard, s)
    for (int i = 0; i < warmup; ++i) {
        KERNEL_ONLY;
        b200_sharded_adam_step(ag, s);
        b200_sharded_adam_step(ps, s);
    }
    CK(cudaStreamSynchronize(s));
    TIME_LOOP(kern_ms, iters, comm, KERNEL_ONLY);
    TIME_LOOP(ag_ms, iters, comm, b200_sharded_adam_step(ag, s));
    TIME_LOOP(ps_ms, iters, comm, b200_sharded_adam_step(ps, s));

    if (rank == 0) {
        const double shard_b = (double)plan->shard;
        printf("{\"sharded_adam_ema\": {\"params\": %ld, \"n_gpus\": %d, \"shard\": %ld, \"kernel_ms\": %.4f, "
               "\"kernel_GBps_per_gpu\": %.1f, \"update_then_allgather_ms\": %.4f, \"update_with_peer_stores_ms\": %.4f, "
               "\"allgather_GBps_per_gpu_in\": %.1f, \"peer_store_GBps_per_gpu_in\": %.1f, \"checked\": %s, "
               "\"failures\": %d, \"host\": \"csrc/host/b200_sharded_optimizer.c (C, NCCL, CUDA IPC)\"}}\n",
            n, world, plan->shard, kern_ms, 36.0 * shard_b / (kern_ms * 1e-3) / 1e9, ag_ms, ps_ms,
            world > 1 ? (world - 1) * shard_b * 4.0 / ((ag_ms - kern_ms) * 1e-3) / 1e9 : 0.0,
            world > 1 ? (world - 1) * shard_b * 4.0 / (ps_ms * 1e-3) / 1e9 : 0.0, check ? "true" : "false", failures);
        if (world > 1)
            unlink(id_file);
    }
    b200_sharded_adam_free(ag);
    b200_sharded_adam_free(ps);
    if (comm)
        ncclCommDestroy(comm);
    return failures ? 1 : 0;
}
