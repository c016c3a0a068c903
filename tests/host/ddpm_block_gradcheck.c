/* Central-difference check of the DDPM residual block (conv_residual_create) as linked: with this
 * repository's csrc/host/b200_conv_residual.c the block runs GroupNorm+SiLU as one fused launch each
 * way and recomputes the pre-activation in backward, so its analytic gradients are checked here the
 * way the reference checks its leaf modules (tests/gradcheck.c: L = <forward(x), g>, fp32 cuBLAS,
 * central differences with a combined absolute + relative tolerance).
 *
 * Checked: the gradient with respect to the block input, to the time embedding (it arrives through
 * the conditioning slot, and the block ADDS its share to the slot's gradient), and to every parameter
 * tensor (GroupNorm scale/shift, both convolutions and their biases, the embedding projection), on a
 * sample of coordinates per tensor.  Prints one PASS/FAIL line per tensor; exit status = failures.
 */
#include "nn.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#define STEP 1e-2f
#define ABS_TOL 2e-3
#define REL_TOL 2e-2

static Context ctx;
static int failures = 0;

static float unit_rand(void) { return (float)rand() / (float)RAND_MAX * 2.0f - 1.0f; }

static float* device_filled(int n, float scale)
{
    float* h = (float*)malloc((size_t)n * sizeof(float));
    for (int i = 0; i < n; ++i)
        h[i] = scale * unit_rand();
    float* d = nn_device_alloc((size_t)n);
    NN_CUDA_CHECK(cudaMemcpy(d, h, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    free(h);
    return d;
}

typedef struct {
    Module* block;
    int batch, n, n_emb;
    float *x, *emb, *g, *y, *gx;
} Setup;

/* L = <block(x; emb, params), g>, accumulated in double on the host */
static double loss(Setup* s)
{
    ctx_set_cond(&ctx, 0, s->emb);
    s->block->forward(s->block, s->x, s->y, s->batch, &ctx);
    NN_CUDA_CHECK(cudaDeviceSynchronize());
    float* hy = (float*)malloc((size_t)s->n * sizeof(float));
    float* hg = (float*)malloc((size_t)s->n * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpy(hy, s->y, (size_t)s->n * sizeof(float), cudaMemcpyDeviceToHost));
    NN_CUDA_CHECK(cudaMemcpy(hg, s->g, (size_t)s->n * sizeof(float), cudaMemcpyDeviceToHost));
    double acc = 0.0;
    for (int i = 0; i < s->n; ++i)
        acc += (double)hy[i] * (double)hg[i];
    free(hy);
    free(hg);
    return acc;
}

/* compares analytic[i] with (L(v+h) - L(v-h)) / 2h on up to `samples` coordinates of the device vector v */
static void check_vector(Setup* s, const char* name, float* v, const float* analytic_dev, int n, int samples)
{
    float* ana = (float*)malloc((size_t)n * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpy(ana, analytic_dev, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    double worst = 0.0;
    const int stride = n > samples ? n / samples : 1;
    int checked = 0;
    for (int i = (n > samples ? stride / 2 : 0); i < n; i += stride, ++checked) {
        float v0;
        NN_CUDA_CHECK(cudaMemcpy(&v0, v + i, sizeof(float), cudaMemcpyDeviceToHost));
        const float hi = v0 + STEP, lo = v0 - STEP;
        NN_CUDA_CHECK(cudaMemcpy(v + i, &hi, sizeof(float), cudaMemcpyHostToDevice));
        const double lp = loss(s);
        NN_CUDA_CHECK(cudaMemcpy(v + i, &lo, sizeof(float), cudaMemcpyHostToDevice));
        const double lm = loss(s);
        NN_CUDA_CHECK(cudaMemcpy(v + i, &v0, sizeof(float), cudaMemcpyHostToDevice));
        const double num = (lp - lm) / (2.0 * STEP);
        const double ratio = fabs(num - ana[i]) / (ABS_TOL + REL_TOL * (fabs(num) + fabs((double)ana[i])));
        if (ratio > worst)
            worst = ratio;
    }
    const int ok = worst <= 1.0;
    printf("%s %-28s %d coordinates, worst violation ratio %.3f\n", ok ? "PASS" : "FAIL", name, checked, worst);
    if (!ok)
        ++failures;
    free(ana);
}

static void check_block(int C, int G, int H, int W, int emb_dim, int batch)
{
    printf("-- conv_residual C=%d groups=%d %dx%d emb=%d batch=%d --\n", C, G, H, W, emb_dim, batch);
    ctx.n_cond = 0;
    const int slot = ctx_add_cond(&ctx, emb_dim, batch);
    Setup s;
    s.block = conv_residual_create(&ctx, C, emb_dim, H, W, batch, G, slot);
    s.batch = batch;
    s.n = batch * H * W * C;
    s.n_emb = batch * emb_dim;
    s.x = device_filled(s.n, 1.5f);
    s.emb = device_filled(s.n_emb, 1.0f);
    s.g = device_filled(s.n, 1.0f);
    s.y = nn_device_alloc((size_t)s.n);
    s.gx = nn_device_alloc((size_t)s.n);

    /* parameters away from their initial values (scale 1, shift 0, bias 0), so that every term of the
       backward formulas is exercised */
    ParamList pl;
    param_list_init(&pl);
    s.block->parameters(s.block, &pl);
    for (int i = 0; i < pl.count; ++i) {
        float* noise = device_filled(pl.items[i].size, 0.2f);
        launch_weighted_sum(pl.items[i].param, pl.items[i].param, noise, 1.0f, 1.0f, pl.items[i].size, ctx.stream);
        NN_CUDA_CHECK(cudaDeviceSynchronize());
        cudaFree(noise);
    }

    /* analytic gradients: one forward, one backward */
    ctx_set_cond(&ctx, slot, s.emb);
    ctx_zero_cond_grad(&ctx, batch);
    s.block->forward(s.block, s.x, s.y, batch, &ctx);
    s.block->backward(s.block, s.x, s.y, s.g, s.gx, batch, &ctx);
    NN_CUDA_CHECK(cudaDeviceSynchronize());
    /* keep copies: the finite-difference forwards below overwrite nothing of these, but the parameter
       gradients live in module buffers that a later backward would overwrite */
    float* gemb = nn_device_alloc((size_t)s.n_emb);
    NN_CUDA_CHECK(cudaMemcpy(gemb, ctx.cond[slot].grad, (size_t)s.n_emb * sizeof(float), cudaMemcpyDeviceToDevice));

    check_vector(&s, "input", s.x, s.gx, s.n, 24);
    check_vector(&s, "time embedding (cond slot)", s.emb, gemb, s.n_emb, 16);
    for (int i = 0; i < pl.count; ++i) {
        char name[64];
        snprintf(name, sizeof name, "parameter tensor %d (%d)", i, pl.items[i].size);
        check_vector(&s, name, pl.items[i].param, pl.items[i].grad, pl.items[i].size, 12);
    }
    param_list_free(&pl);
    cudaFree(gemb);
    cudaFree(s.x);
    cudaFree(s.emb);
    cudaFree(s.g);
    cudaFree(s.y);
    cudaFree(s.gx);
    s.block->free(s.block);
    ctx_free_cond(&ctx);
}

int main(void)
{
    srand(4321);
    NN_CUBLAS_CHECK(cublasCreate(&ctx.cublas)); /* default math mode: full fp32, as the reference's gradcheck */
    ctx.stream = 0;
    NN_CURAND_CHECK(curandCreateGenerator(&ctx.curand, CURAND_RNG_PSEUDO_DEFAULT));
    NN_CURAND_CHECK(curandSetPseudoRandomGeneratorSeed(ctx.curand, 99ULL));
    NN_CURAND_CHECK(curandSetStream(ctx.curand, ctx.stream));
    ctx.n_cond = 0;

    check_block(8, 4, 6, 6, 12, 2);    /* the reference gradcheck's GroupNorm shape, inside the block */
    check_block(32, 32, 7, 7, 16, 3);  /* one channel per group, as the first level of the DDPM UNet */
    check_block(64, 32, 4, 4, 8, 2);

    printf("%d failure(s)\n", failures);
    curandDestroyGenerator(ctx.curand);
    cublasDestroy(ctx.cublas);
    return failures;
}
