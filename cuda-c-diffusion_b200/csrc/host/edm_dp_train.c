/* Data-parallel EDM training step on top of the reference's own host modules.
 *
 * One process per GPU.  The model is the reference's: unet_create (src/unet.c) plus the
 * mp_fourier -> mp_linear -> mp_silu time embedding that diffusion/edm.c:147-153 builds, with
 * every layer kernel coming from libb200_layer_kernels.so.  What differs from the reference's
 * single-GPU loop (diffusion/train.c:40-56 + diffusion/edm.c:192-215):
 *
 *   - per-sample launch loops (edm.c:56-58, 62-64, 75-80, 205-207 and loss.c:65-70) are one
 *     launch_axpby_rows each, with the per-sample coefficients uploaded in ONE pinned H2D copy;
 *   - the batch is staged in pinned memory and uploaded in one copy (train.c:44-49 copies
 *     image by image, blocking);
 *   - the loss value is read back only on logging steps (loss.c:62 synchronises every step);
 *   - gradients are summed over ranks with one grouped ncclAllReduce between backward and the
 *     update, and 1/ranks is folded into the update's grad_scale;
 *   - Adam and the EMA update are one multi-tensor launch (optimizer_ema_step_fused).
 *
 * Usage: edm_dp_train [--steps K] [--warmup W] [--batch B_local] [--check] [--fp32] [--graph]
 *                     [--id-file PATH] [--seed S] [--log-every N] [--dump FILE]
 *   --dump FILE: rank 0 writes the last loss and all parameters (raw float32) after the run.
 *   --no-wn-batch: keep one weight-normalisation launch per weight (default: one launch for all).
 *   --save FILE / --resume FILE: the reference's training checkpoint (checkpoint.c: parameters, EMA
 *   shadows, Adam moments, step and Adam counters).  Rank 0 writes it after the last step; every rank
 *   reads it before the first (replicas hold identical state, so no gather is involved).
 *   --graph: forward + backward are captured into one CUDA graph on the last warm-up step and
 *   replayed afterwards (uploads, noise, the gradient all-reduce and the update stay outside).
 *   RANK / WORLD_SIZE / LOCAL_RANK come from the environment (torchrun sets them).
 *   --check (single rank): runs the reference's own edm_loss_step + optimizer_step + ema_update
 *   and this file's step from identical state and prints the largest relative differences.
 * Rank 0 prints one JSON line with the timing.
 */
#include "b200_fused_modules.h"
#include "edm.h" /* reference diffusion/edm.h: only used by --check */
#include "b200_sharded_optimizer.h"

#include <math.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#define NCCL_OK(call)                                                                      \
    do {                                                                                   \
        ncclResult_t r_ = (call);                                                          \
        if (r_ != ncclSuccess) {                                                           \
            fprintf(stderr, "NCCL error %s:%d: %s\n", __FILE__, __LINE__, ncclGetErrorString(r_)); \
            exit(1);                                                                       \
        }                                                                                  \
    } while (0)

/* rows of the per-sample coefficient table (each row has `batch` floats) */
enum { K_ONE = 0, K_ZERO, K_SIGMA, K_CIN, K_CSKIP, K_COUT, K_GPOS, K_GNEG, K_CNOISE, K_ROWS };

typedef struct {
    UNet* unet;
    Sequential* embed;
    int cond_slot, img_dim, batch;
    float sigma_data, p_mean, p_std, sigma_min, sigma_max;
    float *d_x0, *d_noise, *d_noisy, *d_scaled, *d_F, *d_pred, *d_gF, *d_sink, *d_coef, *d_loss_row;
    /* pinned staging, double-buffered: the host fills slot s while the copy of slot 1-s may
       still be in flight; copied[s] is recorded after the uploads of slot s */
    float *h_coef2[2], *h_x02[2];
    cudaEvent_t copied[2];
    int slot;
    float *h_coef, *h_x0; /* = the current slot */
} DpModel;

static float* pinned(size_t n_floats)
{
    float* p = NULL;
    NN_CUDA_CHECK(cudaMallocHost((void**)&p, n_floats * sizeof(float)));
    return p;
}

/* Same construction order as edm_denoiser_create (diffusion/edm.c:139-156), so that with the
   same cuRAND seed and offset both draw identical initial weights and Fourier features. */
static DpModel* dp_model_create(Context* ctx, UNetConfig cfg, int C, int H, int W, int batch, float sigma_data)
{
    DpModel* m = (DpModel*)calloc(1, sizeof(DpModel));
    cfg.cond_slot = ctx_add_cond(ctx, cfg.emb_dim, batch);
    Module* emb[3] = {
        mp_fourier_create(ctx, cfg.emb_dim, 1.0f),
        mp_linear_create(ctx, cfg.emb_dim, cfg.emb_dim, 1.0f),
        activation_create(cfg.emb_dim, ACT_MP_SILU),
    };
    m->embed = sequential_create(emb, 3, batch);
    m->unet = unet_create(ctx, &cfg, C, C, H, W, batch);
    m->cond_slot = cfg.cond_slot;
    m->img_dim = H * W * C;
    m->batch = batch;
    m->sigma_data = sigma_data;
    m->p_mean = -1.2f;
    m->p_std = 1.2f;
    m->sigma_min = 0.002f;
    m->sigma_max = 80.0f;
    const size_t n = (size_t)batch * m->img_dim;
    float** bufs[8] = { &m->d_x0, &m->d_noise, &m->d_noisy, &m->d_scaled, &m->d_F, &m->d_pred, &m->d_gF, &m->d_sink };
    for (int i = 0; i < 8; ++i)
        *bufs[i] = nn_device_alloc(n);
    m->d_coef = nn_device_alloc((size_t)K_ROWS * batch);
    m->d_loss_row = nn_device_alloc((size_t)batch);
    for (int i = 0; i < 2; ++i) {
        m->h_coef2[i] = pinned((size_t)K_ROWS * batch);
        m->h_x02[i] = pinned(n);
        NN_CUDA_CHECK(cudaEventCreateWithFlags(&m->copied[i], cudaEventDisableTiming));
    }
    m->slot = 0;
    m->h_coef = m->h_coef2[0];
    m->h_x0 = m->h_x02[0];
    return m;
}

static void dp_model_parameters(DpModel* m, ParamList* pl)
{
    sequential_parameters(m->embed, pl);
    unet_parameters(m->unet, pl);
}

/* sigma ~ exp(N(p_mean, p_std)) clamped, EDM weight and preconditioning coefficients
   (Karras et al.; same expressions and host RNG order as diffusion/edm.c:7-13, 197-203). */
static void dp_draw_levels(DpModel* m)
{
    const int B = m->batch;
    const float sd = m->sigma_data;
    float* k = m->h_coef;
    const float norm = 2.0f / (float)(B * m->img_dim);
    for (int b = 0; b < B; ++b) {
        const float u1 = ((float)rand() + 1.0f) / ((float)RAND_MAX + 2.0f);
        const float u2 = ((float)rand() + 1.0f) / ((float)RAND_MAX + 2.0f);
        const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
        float sigma = expf(m->p_mean + m->p_std * z);
        sigma = fminf(fmaxf(sigma, m->sigma_min), m->sigma_max);
        const float s2 = sigma * sigma, sd2 = sd * sd;
        const float w = (s2 + sd2) / ((sigma * sd) * (sigma * sd));
        const float cout = sigma * sd / sqrtf(s2 + sd2);
        k[K_ONE * B + b] = 1.0f;
        k[K_ZERO * B + b] = 0.0f;
        k[K_SIGMA * B + b] = sigma;
        k[K_CIN * B + b] = 1.0f / sqrtf(s2 + sd2);
        k[K_CSKIP * B + b] = sd2 / (s2 + sd2);
        k[K_COUT * B + b] = cout;
        /* dL/dF = c_out * w * 2 (pred - x0) / (B d): the loss gradient, the weight and the
           chain through D = c_skip x + c_out F folded into one pair of row coefficients */
        k[K_GPOS * B + b] = (norm * w) * cout;
        k[K_GNEG * B + b] = -((norm * w) * cout);
        k[K_CNOISE * B + b] = logf(sigma) / 4.0f;
    }
}

/* Switches to the other pinned slot and waits until its previous upload has left it. */
static void dp_next_slot(DpModel* m)
{
    m->slot ^= 1;
    m->h_coef = m->h_coef2[m->slot];
    m->h_x0 = m->h_x02[m->slot];
    NN_CUDA_CHECK(cudaEventSynchronize(m->copied[m->slot]));
}

/* Inputs of one step: uploads the staged batch and coefficient table (one copy each) and draws
   the noise.  Kept out of the captured graph: the pinned source alternates and cuRAND advances
   its offset on the host. */
static void dp_inputs(DpModel* m, Context* ctx)
{
    const size_t n = (size_t)m->batch * m->img_dim;
    cudaStream_t s = ctx->stream;
    NN_CUDA_CHECK(cudaMemcpyAsync(m->d_x0, m->h_x0, n * sizeof(float), cudaMemcpyHostToDevice, s));
    NN_CUDA_CHECK(cudaMemcpyAsync(m->d_coef, m->h_coef, (size_t)K_ROWS * m->batch * sizeof(float), cudaMemcpyHostToDevice, s));
    NN_CUDA_CHECK(cudaEventRecord(m->copied[m->slot], s));
    nn_fill_normal(ctx->curand, m->d_noise, n, 0.0f, 1.0f);
}

/* forward + backward of the batch in d_x0 / d_coef / d_noise; leaves parameter gradients in
   the ParamList's grad buffers.  Only kernels and device-to-device copies on ctx->stream, so
   the whole function can be captured into a CUDA graph. */
static void dp_forward_backward(DpModel* m, Context* ctx)
{
    const int B = m->batch, d = m->img_dim;
    cudaStream_t s = ctx->stream;
    const float* k = m->d_coef;

    launch_axpby_rows(m->d_noisy, m->d_x0, m->d_noise, k + K_ONE * B, k + K_SIGMA * B, B, d, s);
    launch_axpby_rows(m->d_scaled, m->d_noisy, m->d_noisy, k + K_CIN * B, k + K_ZERO * B, B, d, s);

    ctx_set_cond(ctx, m->cond_slot, NULL);
    sequential_forward(m->embed, k + K_CNOISE * B, B, ctx);
    ctx_set_cond(ctx, m->cond_slot, sequential_output(m->embed));

    unet_forward(m->unet, m->d_scaled, m->d_F, B, ctx);
    launch_axpby_rows(m->d_pred, m->d_noisy, m->d_F, k + K_CSKIP * B, k + K_COUT * B, B, d, s);
    launch_axpby_rows(m->d_gF, m->d_pred, m->d_x0, k + K_GPOS * B, k + K_GNEG * B, B, d, s);

    ctx_zero_cond_grad(ctx, B);
    unet_backward(m->unet, m->d_scaled, m->d_F, m->d_gF, m->d_sink, B, ctx);
    sequential_backward(m->embed, ctx->cond[m->cond_slot].grad, B, ctx);
}

/* weighted MSE of the last forward (same value as mse_weighted_forward_backward, loss.c:52-72);
   synchronises, so it is called on logging steps only */
static float dp_loss_value(DpModel* m, Context* ctx)
{
    const int B = m->batch;
    launch_mse_fwd_bwd(m->d_sink, m->d_loss_row, m->d_pred, m->d_x0, B, m->img_dim, ctx->stream);
    float* h = (float*)malloc((size_t)B * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpyAsync(h, m->d_loss_row, (size_t)B * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    NN_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    const float sd = m->sigma_data;
    float total = 0.0f;
    for (int b = 0; b < B; ++b) {
        const float sigma = m->h_coef[K_SIGMA * B + b];
        total += h[b] * ((sigma * sigma + sd * sd) / ((sigma * sd) * (sigma * sd)));
    }
    free(h);
    return total / (float)B;
}

static void stage_batch(DpModel* m, const float* images, int n_images)
{
    for (int b = 0; b < m->batch; ++b) {
        const int idx = rand() % n_images;
        memcpy(m->h_x0 + (size_t)b * m->img_dim, images + (size_t)idx * m->img_dim, (size_t)m->img_dim * sizeof(float));
    }
}

/* synthetic stand-in for the training images: pixel -1 with probability 0.8, else U(-1,1);
   then the reference's preprocessing (zero mean, std = sigma_data; edm/main_edm.c:88-100) */
static float* make_images(int n, int dim, float sigma_data, unsigned seed)
{
    float* img = (float*)malloc((size_t)n * dim * sizeof(float));
    unsigned long long s = 0x9E3779B97F4A7C15ull ^ seed;
    double sum = 0.0, sum2 = 0.0;
    const size_t total = (size_t)n * dim;
    for (size_t i = 0; i < total; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const double u = (double)(s >> 11) / 9007199254740992.0;
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        const double v = (double)(s >> 11) / 9007199254740992.0;
        img[i] = u < 0.8 ? -1.0f : (float)(2.0 * v - 1.0);
        sum += img[i];
    }
    const float mean = (float)(sum / total);
    for (size_t i = 0; i < total; ++i)
        sum2 += (double)(img[i] - mean) * (img[i] - mean);
    const float scale = sigma_data / (float)sqrt(sum2 / total);
    for (size_t i = 0; i < total; ++i)
        img[i] = (img[i] - mean) * scale;
    return img;
}

/* own_stream: a (blocking) stream of its own for the timed loop; 0 for --check, because the
   reference's loss code reads results with synchronous copies on the default stream */
static void context_init(Context* ctx, int tf32, unsigned long long seed, int own_stream)
{
    memset(ctx, 0, sizeof *ctx);
    if (own_stream)
        NN_CUDA_CHECK(cudaStreamCreate(&ctx->stream));
    NN_CUBLAS_CHECK(cublasCreate(&ctx->cublas));
    NN_CUBLAS_CHECK(cublasSetStream(ctx->cublas, ctx->stream));
    if (tf32)
        NN_CUBLAS_CHECK(cublasSetMathMode(ctx->cublas, CUBLAS_TF32_TENSOR_OP_MATH));
    NN_CURAND_CHECK(curandCreateGenerator(&ctx->curand, CURAND_RNG_PSEUDO_DEFAULT));
    NN_CURAND_CHECK(curandSetPseudoRandomGeneratorSeed(ctx->curand, seed));
    NN_CURAND_CHECK(curandSetStream(ctx->curand, ctx->stream));
}

static double max_rel_diff(const float* da, const float* db, int n)
{
    float* a = (float*)malloc((size_t)n * sizeof(float));
    float* b = (float*)malloc((size_t)n * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpy(a, da, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    NN_CUDA_CHECK(cudaMemcpy(b, db, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    double num = 0.0, den = 1e-30;
    for (int i = 0; i < n; ++i) {
        num = fmax(num, fabs((double)a[i] - b[i]));
        den = fmax(den, fabs((double)b[i]));
    }
    free(a);
    free(b);
    return num / den;
}

/* ------------------------------------------------------------------ --check (single rank) */
/* Runs the reference's step (edm_loss_step + optimizer_step + ema_update) on one model and this
   file's step on a second model built from the same cuRAND state, with the same batch, the same
   host RNG state and the same noise, and compares gradients, parameters and EMA shadows. */
static int run_check(UNetConfig ucfg, int C, int H, int W, int batch, float sigma_data, const float* images,
    int n_images, unsigned seed)
{
    const float lr = 1e-3f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, decay = 0.999f;
    Context ca, cb;
    context_init(&ca, 0, seed, 0);
    context_init(&cb, 0, seed, 0);

    Denoiser* ref = edm_denoiser_create(&ca, &ucfg, C, H, W, batch, sigma_data);
    DpModel* mine = dp_model_create(&cb, ucfg, C, H, W, batch, sigma_data);
    ParamList pa, pb;
    param_list_init(&pa);
    param_list_init(&pb);
    ref->parameters(ref, &pa);
    dp_model_parameters(mine, &pb);
    NN_CUDA_CHECK(cudaDeviceSynchronize());
    int failures = 0;
    double e0 = 0.0;
    for (int i = 0; i < pa.count; ++i)
        e0 = fmax(e0, max_rel_diff(pb.items[i].param, pa.items[i].param, pa.items[i].size));
    printf("%s initial parameters identical (%d tensors)      err %.3e\n", e0 == 0.0 ? "PASS" : "FAIL", pa.count, e0);
    failures += e0 != 0.0;

    Optimizer* oa = optimizer_adam(&pa, lr, b1, b2, eps);
    Optimizer* ob = optimizer_adam(&pb, lr, b1, b2, eps);
    EMA* ea = ema_create(&pa, decay);
    EMA* eb = ema_create(&pb, decay);
    EDMLossCfg lcfg = { mine->p_mean, mine->p_std, mine->sigma_min, mine->sigma_max, sigma_data };
    EDMLoss* eloss = edm_loss_create(mine->img_dim, batch, lcfg);

    for (int step = 1; step <= 2; ++step) {
        srand(seed + 17u * (unsigned)step);
        stage_batch(mine, images, n_images);
        NN_CUDA_CHECK(cudaMemcpy(mine->d_x0, mine->h_x0, (size_t)batch * mine->img_dim * sizeof(float), cudaMemcpyHostToDevice));

        /* both paths draw 2 host randoms per sample and one batch of device normals */
        srand(seed + 1000u + (unsigned)step);
        NN_CURAND_CHECK(curandSetGeneratorOffset(ca.curand, 1ull << (20 + step)));
        const float loss_ref = edm_loss_step(eloss, ref, mine->d_x0, batch, &ca);
        optimizer_step(oa, &pa, &ca);
        ema_update(ea, &pa, &ca);

        srand(seed + 1000u + (unsigned)step);
        NN_CURAND_CHECK(curandSetGeneratorOffset(cb.curand, 1ull << (20 + step)));
        dp_draw_levels(mine);
        dp_inputs(mine, &cb);
        dp_forward_backward(mine, &cb);
        const float loss_mine = dp_loss_value(mine, &cb);
        optimizer_ema_step_fused(ob, eb, &pb, lr, b1, b2, eps, decay, 1.0f, &cb);
        NN_CUDA_CHECK(cudaDeviceSynchronize());

        ParamList sa, sb;
        param_list_init(&sa);
        param_list_init(&sb);
        ema_shadow_list(ea, &sa);
        ema_shadow_list(eb, &sb);
        double eg = 0.0, ep = 0.0, es = 0.0;
        for (int i = 0; i < pa.count; ++i) {
            eg = fmax(eg, max_rel_diff(pb.items[i].grad, pa.items[i].grad, pa.items[i].size));
            ep = fmax(ep, max_rel_diff(pb.items[i].param, pa.items[i].param, pa.items[i].size));
            es = fmax(es, max_rel_diff(sb.items[i].param, sa.items[i].param, pa.items[i].size));
        }
        param_list_free(&sa);
        param_list_free(&sb);
        const double el = fabs((double)loss_mine - loss_ref) / fmax(fabs((double)loss_ref), 1e-30);
        printf("%s step %d loss        ref %.6f mine %.6f      err %.3e (tol 1e-5)\n", el <= 1e-5 ? "PASS" : "FAIL", step, loss_ref, loss_mine, el);
        printf("%s step %d gradients (worst tensor)              err %.3e (tol 1e-4)\n", eg <= 1e-4 ? "PASS" : "FAIL", step, eg);
        printf("%s step %d parameters after Adam                 err %.3e (tol 1e-4)\n", ep <= 1e-4 ? "PASS" : "FAIL", step, ep);
        printf("%s step %d EMA shadows                           err %.3e (tol 1e-4)\n", es <= 1e-4 ? "PASS" : "FAIL", step, es);
        failures += (el > 1e-5) + (eg > 1e-4) + (ep > 1e-4) + (es > 1e-4);
    }
    printf("%d failure(s)\n", failures);
    return failures;
}

/* ------------------------------------------------------------------ NCCL bootstrap via a file */
static void exchange_id(ncclUniqueId* id, int rank, const char* path)
{
    char tmp[600];
    if (rank == 0) {
        NCCL_OK(ncclGetUniqueId(id));
        snprintf(tmp, sizeof tmp, "%s.tmp", path);
        FILE* f = fopen(tmp, "wb");
        if (!f || fwrite(id, sizeof *id, 1, f) != 1) {
            fprintf(stderr, "cannot write %s\n", tmp);
            exit(1);
        }
        fclose(f);
        rename(tmp, path);
        return;
    }
    /* a peer that never shows up must not hang this rank: bounded wait on the host (default 60 s,
       EDM_DP_ID_WAIT_S overrides), then a clear message and a non-zero exit; nothing is on the device yet */
    const char* w = getenv("EDM_DP_ID_WAIT_S");
    const double wait_s = (w && w[0]) ? atof(w) : 60.0;
    for (int tries = 0; tries * 0.05 < wait_s; ++tries) {
        FILE* f = fopen(path, "rb");
        if (f) {
            const size_t got = fread(id, sizeof *id, 1, f);
            fclose(f);
            if (got == 1)
                return;
        }
        usleep(50000);
    }
    fprintf(stderr, "rank %d: rank 0 did not publish the NCCL id at %s within %.1f s\n", rank, path, wait_s);
    exit(1);
}

static int g_verbose = 0;
#define TRACE(...)                                  \
    do {                                            \
        if (g_verbose) {                            \
            fprintf(stderr, __VA_ARGS__);           \
            fflush(stderr);                         \
        }                                           \
    } while (0)

static int env_int(const char* name, int dflt)
{
    const char* v = getenv(name);
    return v && v[0] ? atoi(v) : dflt;
}

int main(int argc, char** argv)
{
    int steps = 20, warmup = 5, batch = 256, check = 0, tf32 = 1, log_every = 0, use_graph = 0, batch_wn = 1;
    int sharded = -1; /* -1: replicated optimizer state; else B200_EXCHANGE_* of the range-sharded optimizer */
    unsigned seed = 410293;
    const char* id_file = "/tmp/edm_dp_train.ncclid";
    const char* dump_path = NULL;
    const char *save_path = NULL, *resume_path = NULL;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--steps") && i + 1 < argc) steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--batch") && i + 1 < argc) batch = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--seed") && i + 1 < argc) seed = (unsigned)atoi(argv[++i]);
        else if (!strcmp(argv[i], "--id-file") && i + 1 < argc) id_file = argv[++i];
        else if (!strcmp(argv[i], "--log-every") && i + 1 < argc) log_every = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--dump") && i + 1 < argc) dump_path = argv[++i];
        else if (!strcmp(argv[i], "--save") && i + 1 < argc) save_path = argv[++i];
        else if (!strcmp(argv[i], "--resume") && i + 1 < argc) resume_path = argv[++i];
        else if (!strcmp(argv[i], "--check")) check = 1;
        else if (!strcmp(argv[i], "--sharded") && i + 1 < argc) {
            const char* how = argv[++i];
            if (!strcmp(how, "allgather")) sharded = B200_EXCHANGE_ALLGATHER;
            else if (!strcmp(how, "peer")) sharded = B200_EXCHANGE_PEER_STORE;
            else {
                fprintf(stderr, "--sharded takes allgather or peer\n");
                return 2;
            }
        }
        else if (!strcmp(argv[i], "--graph")) use_graph = 1;
        else if (!strcmp(argv[i], "--no-wn-batch")) batch_wn = 0;
        else if (!strcmp(argv[i], "--verbose")) g_verbose = 1;
        else if (!strcmp(argv[i], "--fp32")) tf32 = 0;
        else {
            fprintf(stderr, "unknown argument %s\n", argv[i]);
            return 2;
        }
    }
    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1), local = env_int("LOCAL_RANK", rank);
    NN_CUDA_CHECK(cudaSetDevice(local));

    const int H = 28, W = 28, C = 1, n_images = 4096;
    const float sigma_data = 0.5f;
    int channels[3] = { 64, 128, 128 };
    UNetConfig ucfg = { .levels = 2, .channels = channels, .emb_dim = 128, .heads = 1, .t = 0.3f, .cond_slot = -1 };
    float* images = make_images(n_images, H * W * C, sigma_data, 0u);

    if (check) {
        if (world != 1) {
            fprintf(stderr, "--check runs on one rank\n");
            return 2;
        }
        return run_check(ucfg, C, H, W, batch < 16 ? batch : 16, sigma_data, images, n_images, seed);
    }

    ncclComm_t comm = NULL;
    if (world > 1) {
        ncclUniqueId id;
        exchange_id(&id, rank, id_file);
        TRACE("rank %d: have the NCCL id\n", rank);
        NCCL_OK(ncclCommInitRank(&comm, world, id, rank));
        TRACE("rank %d: communicator ready\n", rank);
    }

    /* identical initial weights on every rank (same seed); noise and batches differ per rank */
    Context ctx;
    context_init(&ctx, tf32, seed, 1);
    DpModel* m = dp_model_create(&ctx, ucfg, C, H, W, batch, sigma_data);
    ParamList params;
    param_list_init(&params);
    dp_model_parameters(m, &params);
    TRACE("rank %d: model built\n", rank);
    const float lr = 1e-3f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, decay = 0.999f;
    Optimizer* opt = optimizer_adam(&params, lr, b1, b2, eps);
    EMA* ema = ema_create(&params, decay);
    ParamList shadow_l, adam_m, adam_v;
    param_list_init(&shadow_l);
    param_list_init(&adam_m);
    param_list_init(&adam_v);
    ema_shadow_list(ema, &shadow_l);
    optimizer_moment_lists(opt, &adam_m, &adam_v);
    int first_step = 1;
    /* --sharded: moments and EMA shadows exist only for this rank's range of the flat parameter vector; the
       gradient all-reduce becomes a reduce-scatter and the updated range is published to the other ranks */
    B200ShardedAdam* so = NULL;
    if (sharded >= 0) {
        B200ShardedAdamConfig scfg = { .rank = rank, .world = world, .comm = comm, .lr = lr, .beta1 = b1, .beta2 = b2,
            .eps = eps, .ema_decay = decay, .exchange = sharded, .reduce_grads = 1 };
        so = b200_sharded_adam_create(&params, &scfg, ctx.stream);
        if (!so)
            return 1;
        if (resume_path) {
            int loaded_step = 0;
            if (b200_sharded_adam_load(so, resume_path, &loaded_step, ctx.stream) != 0) {
                fprintf(stderr, "rank %d: cannot load %s\n", rank, resume_path);
                return 1;
            }
            first_step = loaded_step + 1;
        }
    } else if (resume_path) {
        int loaded_step = 0, adam_t = 0;
        if (checkpoint_load_training(resume_path, &loaded_step, &adam_t, &params, &shadow_l, &adam_m, &adam_v) != 0) {
            fprintf(stderr, "rank %d: cannot load %s\n", rank, resume_path);
            return 1;
        }
        optimizer_set_timestep(opt, adam_t);
        first_step = loaded_step + 1;
    }
    NN_CURAND_CHECK(curandSetGeneratorOffset(ctx.curand, ((unsigned long long)(rank + 1) << 40) + ((unsigned long long)first_step << 24)));
    srand(seed + 7919u * (unsigned)rank + 104729u * (unsigned)first_step);
    long n_params = 0;
    for (int i = 0; i < params.count; ++i)
        n_params += params.items[i].size;

    float* d_sync = nn_device_alloc(1);
    NN_CUDA_CHECK(cudaMemset(d_sync, 0, sizeof(float)));
    cudaEvent_t ev0, ev1;
    NN_CUDA_CHECK(cudaEventCreate(&ev0));
    NN_CUDA_CHECK(cudaEventCreate(&ev1));
    float first_loss = 0.0f, last_loss = 0.0f;
    cudaGraphExec_t graph_exec = NULL;
    size_t graph_nodes = 0;
    if (use_graph && warmup < 2) {
        fprintf(stderr, "--graph needs at least 2 warm-up steps\n");
        return 2;
    }
    /* cuBLAS may not allocate while a stream is being captured: give it its workspace up front */
    if (use_graph) {
        void* ws = NULL;
        NN_CUDA_CHECK(cudaMalloc(&ws, (size_t)128 << 20));
        NN_CUBLAS_CHECK(cublasSetWorkspace(ctx.cublas, ws, (size_t)128 << 20));
    }
    b200_launch_count_reset();
    long long launches_timed = 0;

    for (int step = 1; step <= warmup + steps; ++step) {
        if (step == warmup + 1) { /* barrier, then start the clock on every rank */
            if (comm)
                NCCL_OK(ncclAllReduce(d_sync, d_sync, 1, ncclFloat, ncclSum, comm, ctx.stream));
            NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
            launches_timed = b200_launch_count();
            NN_CUDA_CHECK(cudaEventRecord(ev0, ctx.stream));
        }
        const float cur_lr = lr_inv_sqrt(lr, first_step - 1 + step, 500, 5000);
        dp_next_slot(m);
        stage_batch(m, images, n_images);
        dp_draw_levels(m);
        dp_inputs(m, &ctx);
        /* Forced weight normalisation: the modules normalise one weight per launch (28 forward and
           28 backward launches).  Step 1 records which weights they touch; from step 2 on every
           weight is normalised by one launch here, the modules' own calls return at once, and the
           backward calls are queued and run as one launch after the backward pass. */
        if (batch_wn)
            b200_wn_batch_mode(step == 1 ? 1 : 2);
        if (graph_exec) {
            NN_CUDA_CHECK(cudaGraphLaunch(graph_exec, ctx.stream));
        } else {
            /* the last warm-up step is captured (and then launched) when --graph is given: by
               then cuBLAS has chosen its kernels and the library's scratch arenas have their size */
            const int capture = use_graph && step == warmup;
            if (capture)
                NN_CUDA_CHECK(cudaStreamBeginCapture(ctx.stream, cudaStreamCaptureModeThreadLocal));
            if (batch_wn && step > 1)
                b200_wn_forward_all(ctx.stream);
            dp_forward_backward(m, &ctx);
            if (batch_wn && step > 1)
                b200_wn_backward_flush(ctx.stream);
            if (capture) {
                cudaGraph_t graph = NULL;
                NN_CUDA_CHECK(cudaStreamEndCapture(ctx.stream, &graph));
                NN_CUDA_CHECK(cudaGraphGetNodes(graph, NULL, &graph_nodes));
                NN_CUDA_CHECK(cudaGraphInstantiate(&graph_exec, graph, 0));
                NN_CUDA_CHECK(cudaGraphDestroy(graph));
                NN_CUDA_CHECK(cudaGraphLaunch(graph_exec, ctx.stream));
            }
        }
        /* The gradient exchange stays outside the graph: with the grouped all-reduce captured,
           two ranks stopped making progress after the capture step (NCCL 2.27.3), so it is
           issued as one ordinary grouped launch per step. */
        if (so) {
            b200_sharded_adam_set_lr(so, cur_lr);
            if (b200_sharded_adam_step(so, ctx.stream) != 0) {
                fprintf(stderr, "rank %d: sharded optimizer step failed\n", rank);
                return 1;
            }
        } else {
            if (comm) {
                NCCL_OK(ncclGroupStart());
                for (int i = 0; i < params.count; ++i)
                    NCCL_OK(ncclAllReduce(params.items[i].grad, params.items[i].grad, (size_t)params.items[i].size,
                        ncclFloat, ncclSum, comm, ctx.stream));
                NCCL_OK(ncclGroupEnd());
            }
            optimizer_ema_step_fused(opt, ema, &params, cur_lr, b1, b2, eps, decay, 1.0f / (float)world, &ctx);
        }
        TRACE("rank %d: step %d enqueued\n", rank, step);
        const int logging = step == 1 || step == warmup + steps || (log_every > 0 && step % log_every == 0);
        if (logging && (step <= warmup || step == warmup + steps)) {
            /* the last step's read-back is inside the timed region on purpose: it is the
               device-to-host result of the run */
            last_loss = dp_loss_value(m, &ctx);
            if (step == 1)
                first_loss = last_loss;
            if (rank == 0 && log_every > 0)
                fprintf(stderr, "step %d loss %.6f lr %.2e\n", step, last_loss, cur_lr);
        }
    }
    if (steps == 0) /* nothing was timed (state inspection: --resume ... --dump) */
        NN_CUDA_CHECK(cudaEventRecord(ev0, ctx.stream));
    NN_CUDA_CHECK(cudaEventRecord(ev1, ctx.stream));
    NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
    b200_wn_batch_mode(0);
    TRACE("rank %d: all steps finished\n", rank);
    launches_timed = b200_launch_count() - launches_timed;
    float ms = 0.0f;
    NN_CUDA_CHECK(cudaEventElapsedTime(&ms, ev0, ev1));

    /* max over ranks of the device-timed region; parameters must agree across ranks */
    float h_stat[2] = { ms, 0.0f };
    float p0 = 0.0f;
    NN_CUDA_CHECK(cudaMemcpy(&p0, params.items[1].param, sizeof(float), cudaMemcpyDeviceToHost));
    float* d_stat = nn_device_alloc(4);
    float h_in[4] = { ms, p0, -p0, 0.0f };
    NN_CUDA_CHECK(cudaMemcpy(d_stat, h_in, sizeof h_in, cudaMemcpyHostToDevice));
    if (comm) {
        NCCL_OK(ncclAllReduce(d_stat, d_stat, 4, ncclFloat, ncclMax, comm, ctx.stream));
        NN_CUDA_CHECK(cudaStreamSynchronize(ctx.stream));
    }
    float h_out[4];
    NN_CUDA_CHECK(cudaMemcpy(h_out, d_stat, sizeof h_out, cudaMemcpyDeviceToHost));
    h_stat[0] = h_out[0];
    const int in_sync = h_out[1] == -h_out[2]; /* max(p) == min(p) over ranks */

    if (rank == 0)
        printf("{\"edm_dp_train\": {\"images_per_s\": %.1f, \"ms_per_step\": %.3f, \"n_gpus\": %d, \"batch_per_gpu\": %d, "
               "\"steps\": %d, \"warmup\": %d, \"params\": %ld, \"param_tensors\": %d, \"tf32\": %d, "
               "\"library_launches_per_step\": %.1f, \"cuda_graph_nodes\": %zu, \"first_loss\": %.5f, \"last_loss\": %.5f, "
               "\"replicas_in_sync\": %s, \"b200_device_error\": %d, \"optimizer\": \"%s\"}}\n",
            steps ? (double)batch * world * steps / (h_stat[0] * 1e-3) : 0.0, steps ? h_stat[0] / steps : 0.0, world, batch, steps, warmup, n_params,
            params.count, tf32, steps ? (double)launches_timed / steps : 0.0, graph_nodes, first_loss, last_loss, in_sync ? "true" : "false",
            b200_device_error_status(),
            sharded < 0 ? "replicated" : (sharded == B200_EXCHANGE_PEER_STORE ? "range-sharded, peer stores" : "range-sharded, all-gather"));

    if (save_path && so) { /* every rank takes part in gathering the sharded state; rank 0 writes */
        if (b200_sharded_adam_save(so, save_path, first_step - 1 + warmup + steps, ctx.stream) != 0) {
            fprintf(stderr, "cannot write %s\n", save_path);
            return 1;
        }
    } else if (save_path && rank == 0) {
        const int rc = checkpoint_save_training(save_path, first_step - 1 + warmup + steps, optimizer_timestep(opt), &params,
            &shadow_l, &adam_m, &adam_v);
        if (rc != 0) {
            fprintf(stderr, "cannot write %s (%d)\n", save_path, rc);
            return 1;
        }
    }
    if (dump_path && rank == 0) { /* last loss, then every parameter tensor, as raw float32 */
        FILE* f = fopen(dump_path, "wb");
        if (!f) {
            fprintf(stderr, "cannot write %s\n", dump_path);
            return 1;
        }
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
