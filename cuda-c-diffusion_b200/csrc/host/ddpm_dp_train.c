/* Data-parallel DDPM training step on the reference's DDPM UNet (src/ddpm_unet.c), timestep
 * embedding, Adam and EMA objects, with this library's kernels: one process per GPU, NCCL.
 *
 *   RANK=r WORLD_SIZE=k LOCAL_RANK=d ddpm_dp_train [--batch B_local] [--steps K] [--warmup W] [--graph]
 *                [--fp32] [--sharded allgather|peer] [--id-file PATH] [--dump FILE] [--check]
 *
 * The reference's step (diffusion/ddpm.c:172-197, diffusion/train.c:40-55) launches one
 * weighted_sum per sample for the forward diffusion and another per sample for the loss weights,
 * copies the batch image by image with blocking copies and reads the loss back every step.  Here:
 *   - noisy = sqrt(ab_t) x0 + sqrt(1-ab_t) noise and the min-SNR-weighted MSE gradient are ONE
 *     launch_axpby_rows each, with per-sample coefficients uploaded in one pinned copy;
 *   - the batch goes up in one pinned copy (double-buffered); the loss is read back on logging steps;
 *   - forward + backward are captured into a CUDA graph (--graph) and replayed;
 *   - gradients: one grouped ncclAllReduce + the fused multi-tensor Adam+EMA, or (--sharded) a
 *     reduce-scatter, the range-sharded update and the parameter exchange fused into its kernel.
 * Linked with csrc/host/b200_conv_residual.c (GroupNorm+SiLU fused in the residual block) and
 * b200_conv2d.c in place of the reference's conv_residual.c / conv2d.c.
 *
 * Model: the reference's ddpm.ini (channels 32/64/128, emb 64, 4 heads, 32 groups, T = 1000,
 * beta 1e-4..0.02, min-SNR gamma 5), 28x28x1 synthetic images (pixel -1 with p = 0.8, else U(-1,1)).
 * --check (one rank): the reference's own ddpm_loss_step on the same model from the same host and
 * device random state must give the same loss and gradients as this file's step.
 * Rank 0 prints one JSON line.
 */
#include "b200_fused_modules.h"
#include "b200_sharded_optimizer.h"
#include "b200_nccl_bootstrap.h"
#include "ddpm.h" /* reference diffusion/ddpm.h: schedule; ddpm_loss_step only for --check */

#include <math.h>
#include <string.h>

#define NCCL_OK(call)                                                                      \
    do {                                                                                   \
        ncclResult_t r_ = (call);                                                          \
        if (r_ != ncclSuccess) {                                                           \
            fprintf(stderr, "NCCL error %s:%d: %s\n", __FILE__, __LINE__, ncclGetErrorString(r_)); \
            exit(1);                                                                       \
        }                                                                                  \
    } while (0)

enum { K_AB = 0, K_NOISE, K_GPOS, K_GNEG, K_T, K_ROWS }; /* rows of the per-sample coefficient table */

typedef struct {
    DDPMUNet* unet;
    Sequential* embed;
    DDPMSchedule sched;
    float* snr_weight; /* [T] min(snr, gamma) / gamma */
    int cond_slot, img_dim, batch;
    float *d_x0, *d_noise, *d_noisy, *d_pred, *d_grad, *d_sink, *d_coef, *d_loss_row;
    float *h_coef2[2], *h_x02[2]; /* pinned, double-buffered */
    float* h_w;                   /* loss weights of the current batch */
    cudaEvent_t copied[2];
    int slot;
} Model;

static float* pinned(size_t n)
{
    float* p = NULL;
    NN_CUDA_CHECK(cudaMallocHost((void**)&p, n * sizeof(float)));
    return p;
}

/* same construction order as ddpm_denoiser_create (diffusion/ddpm.c:101-131): identical weights from
   the same generator state */
static Model* model_create(Context* ctx, DDPMUNetConfig cfg, int C, int H, int W, int batch)
{
    Model* m = (Model*)calloc(1, sizeof *m);
    cfg.cond_slot = ctx_add_cond(ctx, cfg.emb_dim, batch);
    Module* emb[4] = {
        sinusoidal_create(cfg.emb_dim, 10000.0f),
        linear_create(ctx, cfg.emb_dim, cfg.emb_dim),
        activation_create(cfg.emb_dim, ACT_SILU),
        linear_create(ctx, cfg.emb_dim, cfg.emb_dim),
    };
    m->embed = sequential_create(emb, 4, batch);
    m->unet = ddpm_unet_create(ctx, &cfg, C, C, H, W, batch);
    m->cond_slot = cfg.cond_slot;
    m->img_dim = H * W * C;
    m->batch = batch;
    ddpm_schedule_init(&m->sched, 1000, 1e-4f, 0.02f);
    m->snr_weight = (float*)malloc((size_t)m->sched.T * sizeof(float));
    for (int t = 0; t < m->sched.T; ++t) { /* diffusion/ddpm.c:157-160, gamma = 5 */
        const float snr = m->sched.alpha_bar[t] / (1.0f - m->sched.alpha_bar[t]);
        m->snr_weight[t] = fminf(snr, 5.0f) / 5.0f;
    }
    const size_t n = (size_t)batch * m->img_dim;
    float** bufs[6] = { &m->d_x0, &m->d_noise, &m->d_noisy, &m->d_pred, &m->d_grad, &m->d_sink };
    for (int i = 0; i < 6; ++i)
        *bufs[i] = nn_device_alloc(n);
    m->d_coef = nn_device_alloc((size_t)K_ROWS * batch);
    m->d_loss_row = nn_device_alloc((size_t)batch);
    m->h_w = (float*)malloc((size_t)batch * sizeof(float));
    for (int i = 0; i < 2; ++i) {
        m->h_coef2[i] = pinned((size_t)K_ROWS * batch);
        m->h_x02[i] = pinned(n);
        NN_CUDA_CHECK(cudaEventCreateWithFlags(&m->copied[i], cudaEventDisableTiming));
    }
    return m;
}

static void model_parameters(Model* m, ParamList* pl)
{
    sequential_parameters(m->embed, pl);
    ddpm_unet_parameters(m->unet, pl);
}

/* timesteps from the host generator in the reference's order (diffusion/ddpm.c:178-181) and the
   coefficients that depend on them */
static void draw_levels(Model* m)
{
    const int B = m->batch;
    float* k = m->h_coef2[m->slot];
    const float norm = 2.0f / (float)(B * m->img_dim);
    for (int b = 0; b < B; ++b) {
        const int t = rand() % m->sched.T;
        const float w = m->snr_weight[t];
        m->h_w[b] = w;
        k[K_AB * B + b] = m->sched.sqrt_ab[t];
        k[K_NOISE * B + b] = m->sched.sqrt_1mab[t];
        k[K_GPOS * B + b] = norm * w; /* w * 2 (pred - x0) / (B d): loss.c:52-72 in one pass */
        k[K_GNEG * B + b] = -(norm * w);
        k[K_T * B + b] = (float)t;
    }
}

static void stage_batch(Model* m, const float* images, int n_images)
{
    float* dst = m->h_x02[m->slot];
    for (int b = 0; b < m->batch; ++b) {
        const int idx = rand() % n_images;
        memcpy(dst + (size_t)b * m->img_dim, images + (size_t)idx * m->img_dim, (size_t)m->img_dim * sizeof(float));
    }
}

static void upload_inputs(Model* m, Context* ctx)
{
    const size_t n = (size_t)m->batch * m->img_dim;
    NN_CUDA_CHECK(cudaMemcpyAsync(m->d_x0, m->h_x02[m->slot], n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    NN_CUDA_CHECK(cudaMemcpyAsync(m->d_coef, m->h_coef2[m->slot], (size_t)K_ROWS * m->batch * sizeof(float),
        cudaMemcpyHostToDevice, ctx->stream));
    NN_CUDA_CHECK(cudaEventRecord(m->copied[m->slot], ctx->stream));
    nn_fill_normal(ctx->curand, m->d_noise, n, 0.0f, 1.0f);
}

/* kernels and device-to-device copies only: capturable */
static void forward_backward(Model* m, Context* ctx)
{
    const int B = m->batch, d = m->img_dim;
    const float* k = m->d_coef;
    cudaStream_t s = ctx->stream;
    launch_axpby_rows(m->d_noisy, m->d_x0, m->d_noise, k + K_AB * B, k + K_NOISE * B, B, d, s);
    ctx_set_cond(ctx, m->cond_slot, NULL);
    sequential_forward(m->embed, k + K_T * B, B, ctx);
    ctx_set_cond(ctx, m->cond_slot, sequential_output(m->embed));
    ddpm_unet_forward(m->unet, m->d_noisy, m->d_pred, B, ctx);
    launch_axpby_rows(m->d_grad, m->d_pred, m->d_x0, k + K_GPOS * B, k + K_GNEG * B, B, d, s);
    ctx_zero_cond_grad(ctx, B);
    ddpm_unet_backward(m->unet, m->d_noisy, NULL, m->d_grad, m->d_sink, B, ctx);
    sequential_backward(m->embed, ctx->cond[m->cond_slot].grad, B, ctx);
}

static float loss_value(Model* m, Context* ctx)
{
    const int B = m->batch;
    launch_mse_fwd_bwd(m->d_sink, m->d_loss_row, m->d_pred, m->d_x0, B, m->img_dim, ctx->stream);
    float* h = (float*)malloc((size_t)B * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpyAsync(h, m->d_loss_row, (size_t)B * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    NN_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    float total = 0.0f;
    for (int b = 0; b < B; ++b)
        total += h[b] * m->h_w[b];
    free(h);
    return total / (float)B;
}

static float* make_images(int n, int dim, unsigned seed)
{
    float* img = (float*)malloc((size_t)n * dim * sizeof(float));
    unsigned long long s = 0x9E3779B97F4A7C15ull ^ seed;
    for (size_t i = 0; i < (size_t)n * dim; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const double u = (double)(s >> 11) / 9007199254740992.0;
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const double v = (double)(s >> 11) / 9007199254740992.0;
        img[i] = u < 0.8 ? -1.0f : (float)(2.0 * v - 1.0);
    }
    return img;
}

static void context_init(Context* ctx, int tf32, unsigned long long seed, int own_stream)
{
    NN_CUBLAS_CHECK(cublasCreate(&ctx->cublas));
    if (tf32)
        NN_CUBLAS_CHECK(cublasSetMathMode(ctx->cublas, CUBLAS_TF32_TENSOR_OP_MATH));
    ctx->stream = 0;
    if (own_stream) {
        NN_CUDA_CHECK(cudaStreamCreate(&ctx->stream));
        NN_CUBLAS_CHECK(cublasSetStream(ctx->cublas, ctx->stream));
    }
    NN_CURAND_CHECK(curandCreateGenerator(&ctx->curand, CURAND_RNG_PSEUDO_DEFAULT));
    NN_CURAND_CHECK(curandSetPseudoRandomGeneratorSeed(ctx->curand, seed));
    NN_CURAND_CHECK(curandSetStream(ctx->curand, ctx->stream));
    ctx->n_cond = 0;
}

/* largest |a-b| and largest |b| of two device vectors */
static void max_diff(const float* da, const float* db, int n, double* diff, double* mag)
{
    float* a = (float*)malloc((size_t)n * sizeof(float));
    float* b = (float*)malloc((size_t)n * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpy(a, da, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    NN_CUDA_CHECK(cudaMemcpy(b, db, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    *diff = 0.0;
    *mag = 0.0;
    for (int i = 0; i < n; ++i) {
        const double d = fabs((double)a[i] - b[i]);
        *diff = d > *diff ? d : *diff;
        *mag = fabs((double)b[i]) > *mag ? fabs((double)b[i]) : *mag;
    }
    free(a);
    free(b);
}

/* --check: the reference's ddpm_loss_step against this file's step, same weights, same host RNG state,
   same device RNG state.  Gradients are compared tensor by tensor. */
static int run_check(DDPMUNetConfig cfg, int C, int H, int W, int batch, const float* images, int n_images, unsigned seed)
{
    int failures = 0;
    float loss[2] = { 0, 0 };
    float** grads[2] = { NULL, NULL };
    int count = 0;
    int* sizes = NULL;
    for (int which = 0; which < 2; ++which) {
        Context ctx;
        context_init(&ctx, 0, 42ULL, 0);
        srand(seed);
        ParamList pl;
        param_list_init(&pl);
        float* d_x0 = NULL;
        if (which == 0) { /* reference step on the reference's denoiser and loss objects */
            Denoiser* den = ddpm_denoiser_create(&ctx, &cfg, C, H, W, batch);
            den->parameters(den, &pl);
            DDPMSchedule sched;
            ddpm_schedule_init(&sched, 1000, 1e-4f, 0.02f);
            DDPMLoss* l = ddpm_loss_create(&sched, 5.0f, H * W * C, batch);
            d_x0 = nn_device_alloc((size_t)batch * H * W * C);
            /* batch indices first, then (inside ddpm_loss_step) the timesteps: train.c:44 then ddpm.c:178 */
            float* h = (float*)malloc((size_t)batch * H * W * C * sizeof(float));
            for (int b = 0; b < batch; ++b)
                memcpy(h + (size_t)b * H * W * C, images + (size_t)(rand() % n_images) * H * W * C, (size_t)H * W * C * sizeof(float));
            NN_CUDA_CHECK(cudaMemcpy(d_x0, h, (size_t)batch * H * W * C * sizeof(float), cudaMemcpyHostToDevice));
            free(h);
            loss[0] = ddpm_loss_step(l, den, d_x0, batch, &ctx);
        } else {
            Model* m = model_create(&ctx, cfg, C, H, W, batch);
            model_parameters(m, &pl);
            stage_batch(m, images, n_images);
            draw_levels(m);
            upload_inputs(m, &ctx);
            forward_backward(m, &ctx);
            loss[1] = loss_value(m, &ctx);
        }
        NN_CUDA_CHECK(cudaDeviceSynchronize());
        count = pl.count;
        grads[which] = (float**)malloc((size_t)count * sizeof(float*));
        sizes = (int*)malloc((size_t)count * sizeof(int));
        for (int i = 0; i < count; ++i) { /* keep copies: the second model overwrites nothing, but be explicit */
            sizes[i] = pl.items[i].size;
            grads[which][i] = nn_device_alloc((size_t)sizes[i]);
            NN_CUDA_CHECK(cudaMemcpy(grads[which][i], pl.items[i].grad, (size_t)sizes[i] * sizeof(float), cudaMemcpyDeviceToDevice));
        }
        param_list_free(&pl);
        ctx_free_cond(&ctx);
    }
    const double dl = fabs((double)loss[0] - loss[1]) / fabs((double)loss[0]);
    printf("%s loss: reference %.6f, this step %.6f (rel %.2e)\n", dl <= 1e-5 ? "PASS" : "FAIL", loss[0], loss[1], dl);
    failures += dl > 1e-5;
    /* each tensor relative to its own largest gradient, but never below 1e-3 of the largest gradient of the
       model: convolution biases in front of a GroupNorm with one channel per group have an exactly zero
       gradient, and what both steps leave there is rounding noise */
    double* diff = (double*)malloc((size_t)count * sizeof(double));
    double* mag = (double*)malloc((size_t)count * sizeof(double));
    double top = 0.0, worst = 0.0;
    for (int i = 0; i < count; ++i) {
        max_diff(grads[1][i], grads[0][i], sizes[i], &diff[i], &mag[i]);
        top = mag[i] > top ? mag[i] : top;
    }
    for (int i = 0; i < count; ++i) {
        const double den = mag[i] > 1e-3 * top ? mag[i] : 1e-3 * top;
        worst = diff[i] / den > worst ? diff[i] / den : worst;
    }
    free(diff);
    free(mag);
    printf("%s gradients of %d parameter tensors: worst relative difference %.2e\n", worst <= 1e-4 ? "PASS" : "FAIL",
        count, worst);
    failures += worst > 1e-4;
    printf("%d failure(s)\n", failures);
    return failures;
}

static int env_int(const char* name, int dflt)
{
    const char* v = getenv(name);
    return v && v[0] ? atoi(v) : dflt;
}

int main(int argc, char** argv)
{
    int steps = 20, warmup = 5, batch = 256, tf32 = 1, use_graph = 0, sharded = -1, check = 0;
    const char* id_file = "/tmp/ddpm_dp_train.ncclid";
    const char* dump_path = NULL;
    unsigned seed = 1234u;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--steps") && i + 1 < argc) steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) batch = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--id-file") && i + 1 < argc) id_file = argv[++i];
        else if (!strcmp(argv[i], "--dump") && i + 1 < argc) dump_path = argv[++i];
        else if (!strcmp(argv[i], "--fp32")) tf32 = 0;
        else if (!strcmp(argv[i], "--graph")) use_graph = 1;
        else if (!strcmp(argv[i], "--check")) check = 1;
        else if (!strcmp(argv[i], "--sharded") && i + 1 < argc) {
            const char* how = argv[++i];
            sharded = !strcmp(how, "peer") ? B200_EXCHANGE_PEER_STORE : B200_EXCHANGE_ALLGATHER;
        } else {
            fprintf(stderr, "unknown argument %s\n", argv[i]);
            return 2;
        }
    }
    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1), local = env_int("LOCAL_RANK", 0);
    NN_CUDA_CHECK(cudaSetDevice(local));
    const int C = 1, H = 28, W = 28, n_images = 4096;
    int channels[3] = { 32, 64, 128 };
    DDPMUNetConfig ucfg = { .levels = 2, .channels = channels, .emb_dim = 64, .heads = 4, .num_groups = 32, .cond_slot = -1 };
    float* images = make_images(n_images, H * W * C, 0u);
    if (check) {
        if (world != 1) {
            fprintf(stderr, "--check runs on one rank\n");
            return 2;
        }
        return run_check(ucfg, C, H, W, batch < 16 ? batch : 16, images, n_images, seed);
    }
    if (use_graph && warmup < 2) {
        fprintf(stderr, "--graph needs at least 2 warm-up steps\n");
        return 2;
    }

    ncclComm_t comm = NULL;
    if (world > 1) {
        ncclUniqueId id;
        const char* w = getenv("B200_ID_WAIT_S");
        if (b200_nccl_id_via_file(&id, rank, id_file, w && w[0] ? atof(w) : 60.0))
            return 1;
        NCCL_OK(ncclCommInitRank(&comm, world, id, rank));
    }
    Context ctx;
    context_init(&ctx, tf32, seed, 1); /* same seed everywhere: identical initial weights */
    Model* m = model_create(&ctx, ucfg, C, H, W, batch);
    ParamList params;
    param_list_init(&params);
    model_parameters(m, &params);
    const float lr = 1e-3f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, decay = 0.999f;
    Optimizer* opt = optimizer_adam(&params, lr, b1, b2, eps);
    EMA* ema = ema_create(&params, decay);
    B200ShardedAdam* so = NULL;
    if (sharded >= 0) {
        B200ShardedAdamConfig scfg = { .rank = rank, .world = world, .comm = comm, .lr = lr, .beta1 = b1, .beta2 = b2,
            .eps = eps, .ema_decay = decay, .exchange = sharded, .reduce_grads = 1 };
        so = b200_sharded_adam_create(&params, &scfg, ctx.stream);
        if (!so)
            return 1;
    }
    /* batches and noise differ per rank */
    NN_CURAND_CHECK(curandSetGeneratorOffset(ctx.curand, (unsigned long long)(rank + 1) << 40));
    srand(seed + 7919u * (unsigned)rank);
    long n_params = 0;
    for (int i = 0; i < params.count; ++i)
        n_params += params.items[i].size;

    float* d_sync = nn_device_alloc(4);
    NN_CUDA_CHECK(cudaMemset(d_sync, 0, 4 * sizeof(float)));
    cudaEvent_t ev0, ev1;
    NN_CUDA_CHECK(cudaEventCreate(&ev0));
    NN_CUDA_CHECK(cudaEventCreate(&ev1));
    cudaGraphExec_t graph_exec = NULL;
    size_t graph_nodes = 0;
    if (use_graph) { /* cuBLAS may not allocate while a stream is being captured */
        void* ws = NULL;
        NN_CUDA_CHECK(cudaMalloc(&ws, (size_t)128 << 20));
        NN_CUBLAS_CHECK(cublasSetWorkspace(ctx.cublas, ws, (size_t)128 << 20));
    }
    float first_loss = 0.0f, last_loss = 0.0f;
    long long launches_timed = 0;

    for (int step = 1; step <= warmup + steps; ++step) {
        if (step == warmup + 1) {
            if (comm)
                NCCL_OK(ncclAllReduce(d_sync, d_sync, 1, ncclFloat, ncclSum, comm, ctx.stream));
            NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
            launches_timed = b200_launch_count();
            NN_CUDA_CHECK(cudaEventRecord(ev0, ctx.stream));
        }
        const float cur_lr = lr_inv_sqrt(lr, step, 500, 2000);
        m->slot ^= 1;
        NN_CUDA_CHECK(cudaEventSynchronize(m->copied[m->slot]));
        stage_batch(m, images, n_images);
        draw_levels(m);
        upload_inputs(m, &ctx);
        if (graph_exec) {
            NN_CUDA_CHECK(cudaGraphLaunch(graph_exec, ctx.stream));
        } else {
            const int capture = use_graph && step == warmup;
            if (capture)
                NN_CUDA_CHECK(cudaStreamBeginCapture(ctx.stream, cudaStreamCaptureModeThreadLocal));
            forward_backward(m, &ctx);
            if (capture) {
                cudaGraph_t graph = NULL;
                NN_CUDA_CHECK(cudaStreamEndCapture(ctx.stream, &graph));
                NN_CUDA_CHECK(cudaGraphGetNodes(graph, NULL, &graph_nodes));
                NN_CUDA_CHECK(cudaGraphInstantiate(&graph_exec, graph, 0));
                NN_CUDA_CHECK(cudaGraphDestroy(graph));
                NN_CUDA_CHECK(cudaGraphLaunch(graph_exec, ctx.stream));
            }
        }
        if (so) {
            b200_sharded_adam_set_lr(so, cur_lr);
            if (b200_sharded_adam_step(so, ctx.stream) != 0)
                return 1;
        } else {
            if (comm) {
                NCCL_OK(ncclGroupStart());
                for (int i = 0; i < params.count; ++i)
                    NCCL_OK(ncclAllReduce(params.items[i].grad, params.items[i].grad, (size_t)params.items[i].size, ncclFloat,
                        ncclSum, comm, ctx.stream));
                NCCL_OK(ncclGroupEnd());
            }
            optimizer_ema_step_fused(opt, ema, &params, cur_lr, b1, b2, eps, decay, 1.0f / (float)world, &ctx);
        }
        if (step == 1 || step == warmup + steps) {
            last_loss = loss_value(m, &ctx);
            if (step == 1)
                first_loss = last_loss;
        }
    }
    if (steps == 0)
        NN_CUDA_CHECK(cudaEventRecord(ev0, ctx.stream));
    NN_CUDA_CHECK(cudaEventRecord(ev1, ctx.stream));
    NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
    launches_timed = b200_launch_count() - launches_timed;
    float ms = 0.0f;
    NN_CUDA_CHECK(cudaEventElapsedTime(&ms, ev0, ev1));

    /* max over ranks of the timed region; replicas must hold the same parameters */
    float p0 = 0.0f;
    NN_CUDA_CHECK(cudaMemcpy(&p0, params.items[2].param, sizeof(float), cudaMemcpyDeviceToHost));
    float h_in[4] = { ms, p0, -p0, 0.0f }, h_out[4];
    NN_CUDA_CHECK(cudaMemcpy(d_sync, h_in, sizeof h_in, cudaMemcpyHostToDevice));
    if (comm) {
        NCCL_OK(ncclAllReduce(d_sync, d_sync, 4, ncclFloat, ncclMax, comm, ctx.stream));
        NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
    }
    NN_CUDA_CHECK(cudaMemcpy(h_out, d_sync, sizeof h_out, cudaMemcpyDeviceToHost));
    const int in_sync = h_out[1] == -h_out[2];
    if (rank == 0)
        printf("{\"ddpm_dp_train\": {\"images_per_s\": %.1f, \"ms_per_step\": %.3f, \"n_gpus\": %d, \"batch_per_gpu\": %d, "
               "\"steps\": %d, \"warmup\": %d, \"params\": %ld, \"param_tensors\": %d, \"tf32\": %d, "
               "\"library_launches_per_step\": %.1f, \"cuda_graph_nodes\": %zu, \"first_loss\": %.5f, \"last_loss\": %.5f, "
               "\"replicas_in_sync\": %s, \"optimizer\": \"%s\"}}\n",
            steps ? (double)batch * world * steps / (h_out[0] * 1e-3) : 0.0, steps ? h_out[0] / steps : 0.0, world, batch,
            steps, warmup, n_params, params.count, tf32, steps ? (double)launches_timed / steps : 0.0, graph_nodes,
            first_loss, last_loss, in_sync ? "true" : "false",
            sharded < 0 ? "replicated" : (sharded == B200_EXCHANGE_PEER_STORE ? "range-sharded, peer stores" : "range-sharded, all-gather"));
    if (dump_path && rank == 0) {
        FILE* f = fopen(dump_path, "wb");
        if (!f)
            return 1;
        fwrite(&last_loss, sizeof(float), 1, f);
        for (int i = 0; i < params.count; ++i) {
            float* h = (float*)malloc((size_t)params.items[i].size * sizeof(float));
            NN_CUDA_CHECK(cudaMemcpy(h, params.items[i].param, (size_t)params.items[i].size * sizeof(float), cudaMemcpyDeviceToHost));
            fwrite(h, sizeof(float), (size_t)params.items[i].size, f);
            free(h);
        }
        fclose(f);
    }
    if (comm)
        ncclCommDestroy(comm);
    if (rank == 0 && world > 1)
        unlink(id_file);
    free(images);
    return (in_sync && isfinite(last_loss)) ? 0 : 1;
}
