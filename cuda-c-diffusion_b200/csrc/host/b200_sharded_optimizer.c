/* Range-sharded fused Adam+EMA; see include/b200_sharded_optimizer.h. */
#include "b200_sharded_optimizer.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct B200ShardedAdam {
    B200ShardedAdamConfig cfg;
    B200ShardPlan plan;
    int t;
    /* tensors of the ParamList (count == 0 in flat mode) */
    int count;
    int* sizes;
    long* offsets;
    float **tensor_param, **tensor_grad;
    B200CopyItem *pack, *unpack; /* pack: gradients AND current parameters into the arena (2*count items) */
    /* device */
    float *params, *grads;     /* [padded] */
    float *m, *v, *shadow;     /* [shard] */
    float* flag;               /* one word for the barrier all-reduce */
    float* peer_base[B200_MAX_PEERS + 1]; /* other ranks' `params`, opened through CUDA IPC (NULL for self) */
    B200PeerDests dests;
};

#define SO_FAIL(o, ...)                    \
    do {                                   \
        fprintf(stderr, "b200_sharded_adam: " __VA_ARGS__); \
        fprintf(stderr, "\n");             \
        b200_sharded_adam_free(o);         \
        return NULL;                       \
    } while (0)
#define SO_CUDA(o, call)                                                          \
    do {                                                                          \
        cudaError_t e_ = (call);                                                  \
        if (e_ != cudaSuccess)                                                    \
            SO_FAIL(o, "%s failed: %s", #call, cudaGetErrorString(e_));          \
    } while (0)
#define SO_NCCL(o, call)                                                          \
    do {                                                                          \
        ncclResult_t r_ = (call);                                                 \
        if (r_ != ncclSuccess)                                                    \
            SO_FAIL(o, "%s failed: %s", #call, ncclGetErrorString(r_));          \
    } while (0)

static B200ShardedAdam* create_common(long total, const B200ShardedAdamConfig* cfg, cudaStream_t s, B200ShardedAdam* o)
{
    o->cfg = *cfg;
    const int rc = b200_shard_plan(total, cfg->rank, cfg->world, &o->plan);
    if (rc != B200_SHARD_OK)
        SO_FAIL(o, "rank %d of %d over %ld elements is not a valid partition (code %d)", cfg->rank, cfg->world, total, rc);
    if (cfg->world - 1 > B200_MAX_PEERS)
        SO_FAIL(o, "at most %d ranks", B200_MAX_PEERS + 1);
    const B200ShardPlan* p = &o->plan;
    SO_CUDA(o, cudaMalloc((void**)&o->params, (size_t)p->padded * sizeof(float)));
    SO_CUDA(o, cudaMalloc((void**)&o->grads, (size_t)p->padded * sizeof(float)));
    SO_CUDA(o, cudaMalloc((void**)&o->m, (size_t)p->shard * sizeof(float)));
    SO_CUDA(o, cudaMalloc((void**)&o->v, (size_t)p->shard * sizeof(float)));
    SO_CUDA(o, cudaMalloc((void**)&o->shadow, (size_t)p->shard * sizeof(float)));
    SO_CUDA(o, cudaMalloc((void**)&o->flag, 256));
    SO_CUDA(o, cudaMemsetAsync(o->params, 0, (size_t)p->padded * sizeof(float), s));
    SO_CUDA(o, cudaMemsetAsync(o->grads, 0, (size_t)p->padded * sizeof(float), s));
    SO_CUDA(o, cudaMemsetAsync(o->m, 0, (size_t)p->shard * sizeof(float), s));
    SO_CUDA(o, cudaMemsetAsync(o->v, 0, (size_t)p->shard * sizeof(float), s));
    SO_CUDA(o, cudaMemsetAsync(o->shadow, 0, (size_t)p->shard * sizeof(float), s));
    SO_CUDA(o, cudaMemsetAsync(o->flag, 0, 256, s));
    if (cfg->world == 1)
        return o;

    /* every rank must describe the same partition before a collective touches the buffers */
    long mine[3] = { p->total, p->shard, (long)p->world };
    long* d_rep = NULL;
    long* h_rep = (long*)malloc((size_t)cfg->world * 3 * sizeof(long));
    SO_CUDA(o, cudaMalloc((void**)&d_rep, (size_t)cfg->world * 3 * sizeof(long)));
    SO_CUDA(o, cudaMemcpyAsync(d_rep + 3 * cfg->rank, mine, sizeof mine, cudaMemcpyHostToDevice, s));
    SO_NCCL(o, ncclAllGather(d_rep + 3 * cfg->rank, d_rep, 3, ncclInt64, cfg->comm, s));
    SO_CUDA(o, cudaMemcpyAsync(h_rep, d_rep, (size_t)cfg->world * 3 * sizeof(long), cudaMemcpyDeviceToHost, s));
    SO_CUDA(o, cudaStreamSynchronize(s));
    int bad = -1;
    const int chk = b200_shard_check_peers(h_rep, cfg->world, p, &bad);
    cudaFree(d_rep);
    if (chk != B200_SHARD_OK) {
        const long* t = h_rep + 3 * bad;
        fprintf(stderr, "b200_sharded_adam: rank %d reports %ld elements / shard %ld / world %ld, this rank %ld / %ld / %d\n",
            bad, t[0], t[1], t[2], p->total, p->shard, p->world);
        free(h_rep);
        b200_sharded_adam_free(o);
        return NULL;
    }
    free(h_rep);

    if (cfg->exchange == B200_EXCHANGE_PEER_STORE) {
        /* publish this rank's vector, open everybody else's */
        cudaIpcMemHandle_t h_mine, *h_all = (cudaIpcMemHandle_t*)malloc((size_t)cfg->world * sizeof(cudaIpcMemHandle_t));
        char* d_h = NULL;
        SO_CUDA(o, cudaIpcGetMemHandle(&h_mine, o->params));
        SO_CUDA(o, cudaMalloc((void**)&d_h, (size_t)cfg->world * sizeof(cudaIpcMemHandle_t)));
        SO_CUDA(o, cudaMemcpyAsync(d_h + (size_t)cfg->rank * sizeof h_mine, &h_mine, sizeof h_mine, cudaMemcpyHostToDevice, s));
        SO_NCCL(o, ncclAllGather(d_h + (size_t)cfg->rank * sizeof h_mine, d_h, sizeof h_mine, ncclChar, cfg->comm, s));
        SO_CUDA(o, cudaMemcpyAsync(h_all, d_h, (size_t)cfg->world * sizeof h_mine, cudaMemcpyDeviceToHost, s));
        SO_CUDA(o, cudaStreamSynchronize(s));
        cudaFree(d_h);
        o->dests.count = 0;
        for (int r = 0; r < cfg->world; ++r) {
            if (r == cfg->rank)
                continue;
            void* base = NULL;
            cudaError_t e = cudaIpcOpenMemHandle(&base, h_all[r], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                free(h_all);
                SO_FAIL(o, "cannot map rank %d's parameter vector (cudaIpcOpenMemHandle: %s)", r, cudaGetErrorString(e));
            }
            o->peer_base[r] = (float*)base;
            o->dests.dst[o->dests.count++] = (float*)base + p->lo;
        }
        free(h_all);
    }
    return o;
}

B200ShardedAdam* b200_sharded_adam_create_flat(long n, const B200ShardedAdamConfig* cfg, cudaStream_t s)
{
    B200ShardedAdam* o = (B200ShardedAdam*)calloc(1, sizeof *o);
    return create_common(n, cfg, s, o);
}

B200ShardedAdam* b200_sharded_adam_create(const ParamList* pl, const B200ShardedAdamConfig* cfg, cudaStream_t s)
{
    B200ShardedAdam* o = (B200ShardedAdam*)calloc(1, sizeof *o);
    const int n = pl->count;
    o->count = n;
    o->sizes = (int*)malloc((size_t)n * sizeof(int));
    o->offsets = (long*)malloc((size_t)n * sizeof(long));
    o->tensor_param = (float**)malloc((size_t)n * sizeof(float*));
    o->tensor_grad = (float**)malloc((size_t)n * sizeof(float*));
    o->pack = (B200CopyItem*)malloc((size_t)2 * n * sizeof(B200CopyItem));
    o->unpack = (B200CopyItem*)malloc((size_t)n * sizeof(B200CopyItem));
    for (int i = 0; i < n; ++i) {
        o->sizes[i] = pl->items[i].size;
        o->tensor_param[i] = pl->items[i].param;
        o->tensor_grad[i] = pl->items[i].grad;
    }
    long total = 0;
    if (b200_shard_layout(o->sizes, n, o->offsets, &total) != B200_SHARD_OK)
        SO_FAIL(o, "a tensor of the ParamList has a negative size");
    if (!create_common(total, cfg, s, o))
        return NULL;
    for (int i = 0; i < n; ++i) {
        o->pack[i].dst = o->grads + o->offsets[i];
        o->pack[i].src = o->tensor_grad[i];
        o->pack[i].n = o->sizes[i];
        /* the model may change its weights between steps (forced weight normalisation rewrites them in
           place in every forward, mp_linear.c:16-18, conv2d.c:28-30): the update starts from the tensors */
        o->pack[n + i].dst = o->params + o->offsets[i];
        o->pack[n + i].src = o->tensor_param[i];
        o->pack[n + i].n = o->sizes[i];
        o->unpack[i].dst = o->tensor_param[i];
        o->unpack[i].src = o->params + o->offsets[i];
        o->unpack[i].n = o->sizes[i];
    }
    /* arena <- current weights; shadow starts as a copy of them (ema.c:12-27) */
    launch_copy_multi(o->pack + n, n, s);
    b200_sharded_adam_reset_shadow(o, s);
    return o;
}

float* b200_sharded_adam_params(B200ShardedAdam* o) { return o->params; }
float* b200_sharded_adam_grads(B200ShardedAdam* o) { return o->grads; }
const B200ShardPlan* b200_sharded_adam_plan(const B200ShardedAdam* o) { return &o->plan; }
void b200_sharded_adam_set_lr(B200ShardedAdam* o, float lr) { o->cfg.lr = lr; }
int b200_sharded_adam_timestep(const B200ShardedAdam* o) { return o->t; }

void b200_sharded_adam_reset_shadow(B200ShardedAdam* o, cudaStream_t s)
{
    cudaMemcpyAsync(o->shadow, o->params + o->plan.lo, (size_t)o->plan.shard * sizeof(float), cudaMemcpyDeviceToDevice, s);
}

static int barrier_word(B200ShardedAdam* o, cudaStream_t s)
{
    return ncclAllReduce(o->flag, o->flag, 1, ncclFloat, ncclSum, o->cfg.comm, s) == ncclSuccess ? 0 : -1;
}

int b200_sharded_adam_step(B200ShardedAdam* o, cudaStream_t s)
{
    const B200ShardedAdamConfig* c = &o->cfg;
    const B200ShardPlan* p = &o->plan;
    const int multi = c->world > 1;
    const int peer = multi && c->exchange == B200_EXCHANGE_PEER_STORE;
    o->t++;
    const float bc1 = 1.0f - powf(c->beta1, (float)o->t); /* optimizer.c:62-64 */
    const float bc2 = 1.0f - powf(c->beta2, (float)o->t);
    float scale = 1.0f;
    if (o->count)
        launch_copy_multi(o->pack, 2 * o->count, s);
    if (multi && c->reduce_grads) {
        if (ncclReduceScatter(o->grads, o->grads + p->lo, (size_t)p->shard, ncclFloat, ncclSum, c->comm, s) != ncclSuccess)
            return -1;
        scale = 1.0f / (float)c->world;
    } else if (peer && barrier_word(o, s)) {
        return -1;
    }
    if (peer) {
        launch_adam_ema_step_bcast(o->params + p->lo, o->m, o->v, o->shadow, o->grads + p->lo, &o->dests, c->lr, c->beta1,
            c->beta2, c->eps, bc1, bc2, c->ema_decay, scale, (long long)p->shard, s);
        if (barrier_word(o, s))
            return -1;
    } else {
        launch_adam_ema_step(o->params + p->lo, o->m, o->v, o->shadow, o->grads + p->lo, c->lr, c->beta1, c->beta2, c->eps,
            bc1, bc2, c->ema_decay, scale, (long long)p->shard, s);
        if (multi && ncclAllGather(o->params + p->lo, o->params, (size_t)p->shard, ncclFloat, c->comm, s) != ncclSuccess)
            return -1;
    }
    if (o->count)
        launch_copy_multi(o->unpack, o->count, s);
    return 0;
}

/* Full-length copies of the three sharded states, [3][padded] floats: shadow, m, v. */
static float* gather_states(B200ShardedAdam* o, cudaStream_t s)
{
    const B200ShardPlan* p = &o->plan;
    float* full = NULL;
    if (cudaMalloc((void**)&full, (size_t)3 * p->padded * sizeof(float)) != cudaSuccess)
        return NULL;
    const float* src[3] = { o->shadow, o->m, o->v };
    for (int k = 0; k < 3; ++k) {
        float* dst = full + (size_t)k * p->padded;
        cudaMemcpyAsync(dst + p->lo, src[k], (size_t)p->shard * sizeof(float), cudaMemcpyDeviceToDevice, s);
        if (p->world > 1 && ncclAllGather(dst + p->lo, dst, (size_t)p->shard, ncclFloat, o->cfg.comm, s) != ncclSuccess) {
            cudaFree(full);
            return NULL;
        }
    }
    return full;
}

static void state_lists(B200ShardedAdam* o, float* full, ParamList* par, ParamList* sh, ParamList* m, ParamList* v)
{
    const B200ShardPlan* p = &o->plan;
    param_list_init(par);
    param_list_init(sh);
    param_list_init(m);
    param_list_init(v);
    if (o->count == 0) {
        param_list_add(par, o->params, NULL, (int)p->total);
        param_list_add(sh, full, NULL, (int)p->total);
        param_list_add(m, full + p->padded, NULL, (int)p->total);
        param_list_add(v, full + 2 * p->padded, NULL, (int)p->total);
        return;
    }
    for (int i = 0; i < o->count; ++i) {
        param_list_add(par, o->params + o->offsets[i], NULL, o->sizes[i]);
        param_list_add(sh, full + o->offsets[i], NULL, o->sizes[i]);
        param_list_add(m, full + p->padded + o->offsets[i], NULL, o->sizes[i]);
        param_list_add(v, full + 2 * p->padded + o->offsets[i], NULL, o->sizes[i]);
    }
}

int b200_sharded_adam_save(B200ShardedAdam* o, const char* path, int step, cudaStream_t s)
{
    float* full = gather_states(o, s);
    if (!full)
        return -10;
    if (cudaStreamSynchronize(s) != cudaSuccess) {
        cudaFree(full);
        return -11;
    }
    int rc = 0;
    if (o->cfg.rank == 0) {
        ParamList par, sh, m, v;
        state_lists(o, full, &par, &sh, &m, &v);
        rc = checkpoint_save_training(path, step, o->t, &par, &sh, &m, &v);
        param_list_free(&par);
        param_list_free(&sh);
        param_list_free(&m);
        param_list_free(&v);
    }
    cudaFree(full);
    return rc;
}

int b200_sharded_adam_load(B200ShardedAdam* o, const char* path, int* step, cudaStream_t s)
{
    const B200ShardPlan* p = &o->plan;
    float* full = NULL;
    if (cudaMalloc((void**)&full, (size_t)3 * p->padded * sizeof(float)) != cudaSuccess)
        return -10;
    cudaMemsetAsync(full, 0, (size_t)3 * p->padded * sizeof(float), s);
    cudaStreamSynchronize(s);
    ParamList par, sh, m, v;
    state_lists(o, full, &par, &sh, &m, &v);
    int st = 0, t = 0;
    const int rc = checkpoint_load_training(path, &st, &t, &par, &sh, &m, &v);
    param_list_free(&par);
    param_list_free(&sh);
    param_list_free(&m);
    param_list_free(&v);
    if (rc == 0) {
        float* dst[3] = { o->shadow, o->m, o->v };
        for (int k = 0; k < 3; ++k)
            cudaMemcpyAsync(dst[k], full + (size_t)k * p->padded + p->lo, (size_t)p->shard * sizeof(float),
                cudaMemcpyDeviceToDevice, s);
        if (o->count)
            launch_copy_multi(o->unpack, o->count, s);
        o->t = t;
        if (step)
            *step = st;
        cudaStreamSynchronize(s);
    }
    cudaFree(full);
    return rc;
}

void b200_sharded_adam_free(B200ShardedAdam* o)
{
    if (!o)
        return;
    for (int r = 0; r <= B200_MAX_PEERS; ++r)
        if (o->peer_base[r])
            cudaIpcCloseMemHandle(o->peer_base[r]);
    cudaFree(o->params);
    cudaFree(o->grads);
    cudaFree(o->m);
    cudaFree(o->v);
    cudaFree(o->shadow);
    cudaFree(o->flag);
    free(o->sizes);
    free(o->offsets);
    free(o->tensor_param);
    free(o->tensor_grad);
    free(o->pack);
    free(o->unpack);
    free(o);
}
