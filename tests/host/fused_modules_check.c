/* Checks the C host modules of the fused entry points against the reference's own host code
 * (its groupnorm / activation / optimizer / EMA modules, compiled from the reference tree and
 * linked to the same kernel library) and against central differences.
 *
 *   1. groupnorm_act_create(...)      ==  spatial_groupnorm_create(...) + launch_activation_*
 *   2. pixel_norm_create(...)         :   analytic backward vs central difference of <y, g>
 *   3. optimizer_ema_step_fused(...)  ==  optimizer_step(...) + ema_update(...)
 *
 * Prints one PASS/FAIL line per check; the exit status is the number of failures.
 * Built by oracle/Makefile (target _ref/fused_modules_check); needs a GPU to run.
 */
#include "b200_fused_modules.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static Context g_ctx;
static int g_failures = 0;

static float frand(void) { return (float)rand() / (float)RAND_MAX * 2.0f - 1.0f; }

static float* dev_random(int n, float scale)
{
    float* h = (float*)malloc((size_t)n * sizeof(float));
    for (int i = 0; i < n; ++i)
        h[i] = frand() * scale;
    float* d = nn_device_alloc((size_t)n);
    NN_CUDA_CHECK(cudaMemcpy(d, h, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    free(h);
    return d;
}

static float* to_host(const float* d, int n)
{
    float* h = (float*)malloc((size_t)n * sizeof(float));
    NN_CUDA_CHECK(cudaMemcpy(h, d, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    return h;
}

/* max |a-b| / (max |b| + tiny) */
static double rel_diff(const float* da, const float* db, int n)
{
    float *a = to_host(da, n), *b = to_host(db, n);
    double num = 0.0, den = 1e-30;
    for (int i = 0; i < n; ++i) {
        double d = fabs((double)a[i] - (double)b[i]);
        if (d > num)
            num = d;
        if (fabs((double)b[i]) > den)
            den = fabs((double)b[i]);
    }
    free(a);
    free(b);
    return num / den;
}

static void report(const char* name, double err, double tol)
{
    const int ok = err <= tol;
    printf("%s %-44s err %.3e (tol %.1e)\n", ok ? "PASS" : "FAIL", name, err, tol);
    if (!ok)
        ++g_failures;
}

static void copy_params(Module* dst, Module* src)
{
    ParamList a, b;
    param_list_init(&a);
    param_list_init(&b);
    dst->parameters(dst, &a);
    src->parameters(src, &b);
    for (int i = 0; i < a.count; ++i)
        NN_CUDA_CHECK(cudaMemcpy(a.items[i].param, b.items[i].param, (size_t)a.items[i].size * sizeof(float),
            cudaMemcpyDeviceToDevice));
    param_list_free(&a);
    param_list_free(&b);
}

/* ---------------------------------------------------------------- 1. fused GroupNorm+act module */
static void check_groupnorm_act(int batch, int H, int W, int C, int G, Activation act, const char* name)
{
    const int n = batch * H * W * C;
    Module* ref = spatial_groupnorm_create(C, G, H, W, batch);
    Module* fused = groupnorm_act_create(C, G, H, W, batch, act);

    /* random affine parameters in the reference module, copied into the fused one */
    ParamList pr;
    param_list_init(&pr);
    ref->parameters(ref, &pr);
    for (int i = 0; i < pr.count; ++i) {
        float* r = dev_random(pr.items[i].size, 1.0f);
        NN_CUDA_CHECK(cudaMemcpy(pr.items[i].param, r, (size_t)pr.items[i].size * sizeof(float), cudaMemcpyDeviceToDevice));
        cudaFree(r);
    }
    copy_params(fused, ref);

    float* x = dev_random(n, 2.0f);
    float* gy = dev_random(n, 1.0f);
    float *h0 = nn_device_alloc((size_t)n), *y_ref = nn_device_alloc((size_t)n), *y = nn_device_alloc((size_t)n);
    float *gh0 = nn_device_alloc((size_t)n), *gx_ref = nn_device_alloc((size_t)n), *gx = nn_device_alloc((size_t)n);

    ref->forward(ref, x, h0, batch, &g_ctx);
    launch_activation_forward(y_ref, h0, n, act, g_ctx.stream);
    launch_activation_backward(gh0, gy, h0, n, act, g_ctx.stream);
    ref->backward(ref, x, h0, gh0, gx_ref, batch, &g_ctx);

    fused->forward(fused, x, y, batch, &g_ctx);
    fused->backward(fused, x, y, gy, gx, batch, &g_ctx);
    NN_CUDA_CHECK(cudaDeviceSynchronize());

    char label[128];
    snprintf(label, sizeof label, "%s forward", name);
    report(label, rel_diff(y, y_ref, n), 1e-5);
    snprintf(label, sizeof label, "%s grad_in", name);
    report(label, rel_diff(gx, gx_ref, n), 1e-4);
    ParamList pf;
    param_list_init(&pf);
    fused->parameters(fused, &pf);
    snprintf(label, sizeof label, "%s dgamma", name);
    report(label, rel_diff(pf.items[0].grad, pr.items[0].grad, C), 1e-4);
    snprintf(label, sizeof label, "%s dbeta", name);
    report(label, rel_diff(pf.items[1].grad, pr.items[1].grad, C), 1e-4);

    param_list_free(&pr);
    param_list_free(&pf);
    float* bufs[8] = { x, gy, h0, y_ref, y, gh0, gx_ref, gx };
    for (int i = 0; i < 8; ++i)
        cudaFree(bufs[i]);
    ref->free(ref);
    fused->free(fused);
}

/* ---------------------------------------------------------------- 2. pixel norm module */
static double loss_of(Module* m, const float* x, float* y, const float* g_host, int batch, int n)
{
    m->forward(m, x, y, batch, &g_ctx);
    float* yh = to_host(y, n);
    double s = 0.0;
    for (int i = 0; i < n; ++i)
        s += (double)yh[i] * (double)g_host[i];
    free(yh);
    return s;
}

static void check_pixel_norm(int batch, int H, int W, int C)
{
    const int n = batch * H * W * C;
    const float fd_eps = 1e-2f;
    Module* m = pixel_norm_create(C, H, W);
    float* x = dev_random(n, 1.5f);
    float* gy = dev_random(n, 1.0f);
    float *y = nn_device_alloc((size_t)n), *gx = nn_device_alloc((size_t)n);
    m->forward(m, x, y, batch, &g_ctx);
    m->backward(m, x, y, gy, gx, batch, &g_ctx);
    float *xh = to_host(x, n), *gh = to_host(gy, n), *gxh = to_host(gx, n);

    /* unit RMS over channels for every pixel */
    float* yh = to_host(y, n);
    double worst_rms = 0.0;
    for (int p = 0; p < n / C; ++p) {
        double ss = 0.0;
        for (int c = 0; c < C; ++c)
            ss += (double)yh[p * C + c] * yh[p * C + c];
        double d = fabs(sqrt(ss / C) - 1.0);
        if (d > worst_rms)
            worst_rms = d;
    }
    free(yh);
    report("pixel_norm unit rms", worst_rms, 1e-3);

    double worst = 0.0;
    for (int k = 0; k < 24; ++k) {
        const int i = rand() % n;
        const float keep = xh[i];
        float v = keep + fd_eps;
        NN_CUDA_CHECK(cudaMemcpy(x + i, &v, sizeof(float), cudaMemcpyHostToDevice));
        const double lp = loss_of(m, x, y, gh, batch, n);
        v = keep - fd_eps;
        NN_CUDA_CHECK(cudaMemcpy(x + i, &v, sizeof(float), cudaMemcpyHostToDevice));
        const double lm = loss_of(m, x, y, gh, batch, n);
        NN_CUDA_CHECK(cudaMemcpy(x + i, &keep, sizeof(float), cudaMemcpyHostToDevice));
        const double num = (lp - lm) / (2.0 * fd_eps);
        const double viol = fabs(num - (double)gxh[i]) / (1e-2 + 2e-2 * (fabs(num) + fabs((double)gxh[i])));
        if (viol > worst)
            worst = viol;
    }
    report("pixel_norm backward vs central difference", worst, 1.0);
    free(xh);
    free(gh);
    free(gxh);
    cudaFree(x);
    cudaFree(gy);
    cudaFree(y);
    cudaFree(gx);
    m->free(m);
}

/* ---------------------------------------------------------------- 3. fused optimizer + EMA step */
static void check_optimizer_ema(void)
{
    /* odd sizes on purpose: tails and misaligned starts inside the multi-tensor launch; more
       tensors than one launch table holds, so the chunking is exercised too */
    enum { NT = 70 };
    int sizes[NT];
    for (int i = 0; i < NT; ++i)
        sizes[i] = 1 + (i * 7919) % 5003;
    sizes[3] = 300001;
    const float lr = 1e-2f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, decay = 0.99f;

    ParamList pa, pb;
    param_list_init(&pa);
    param_list_init(&pb);
    for (int i = 0; i < NT; ++i) {
        float* p = dev_random(sizes[i], 1.0f);
        float* p2 = nn_device_alloc((size_t)sizes[i]);
        NN_CUDA_CHECK(cudaMemcpy(p2, p, (size_t)sizes[i] * sizeof(float), cudaMemcpyDeviceToDevice));
        param_list_add(&pa, p, nn_device_alloc((size_t)sizes[i]), sizes[i]);
        param_list_add(&pb, p2, nn_device_alloc((size_t)sizes[i]), sizes[i]);
    }
    Optimizer* oa = optimizer_adam(&pa, lr, b1, b2, eps);
    Optimizer* ob = optimizer_adam(&pb, lr, b1, b2, eps);
    EMA* ea = ema_create(&pa, decay);
    EMA* eb = ema_create(&pb, decay);

    for (int step = 0; step < 3; ++step) {
        for (int i = 0; i < NT; ++i) {
            float* g = dev_random(sizes[i], 0.5f);
            NN_CUDA_CHECK(cudaMemcpy(pa.items[i].grad, g, (size_t)sizes[i] * sizeof(float), cudaMemcpyDeviceToDevice));
            NN_CUDA_CHECK(cudaMemcpy(pb.items[i].grad, g, (size_t)sizes[i] * sizeof(float), cudaMemcpyDeviceToDevice));
            cudaFree(g);
        }
        optimizer_step(oa, &pa, &g_ctx);
        ema_update(ea, &pa, &g_ctx);
        optimizer_ema_step_fused(ob, eb, &pb, lr, b1, b2, eps, decay, 1.0f, &g_ctx);
    }
    NN_CUDA_CHECK(cudaDeviceSynchronize());

    ParamList ma, va, mb, vb, sa, sb;
    param_list_init(&ma);
    param_list_init(&va);
    param_list_init(&mb);
    param_list_init(&vb);
    param_list_init(&sa);
    param_list_init(&sb);
    optimizer_moment_lists(oa, &ma, &va);
    optimizer_moment_lists(ob, &mb, &vb);
    ema_shadow_list(ea, &sa);
    ema_shadow_list(eb, &sb);
    double ep = 0, em = 0, ev = 0, es = 0;
    for (int i = 0; i < NT; ++i) {
        ep = fmax(ep, rel_diff(pb.items[i].param, pa.items[i].param, sizes[i]));
        em = fmax(em, rel_diff(mb.items[i].param, ma.items[i].param, sizes[i]));
        ev = fmax(ev, rel_diff(vb.items[i].param, va.items[i].param, sizes[i]));
        es = fmax(es, rel_diff(sb.items[i].param, sa.items[i].param, sizes[i]));
    }
    report("optimizer_ema_step_fused params", ep, 1e-5);
    report("optimizer_ema_step_fused m", em, 1e-6);
    report("optimizer_ema_step_fused v", ev, 1e-6);
    report("optimizer_ema_step_fused shadow", es, 1e-5);
    report("optimizer_ema_step_fused timestep", fabs((double)optimizer_timestep(ob) - optimizer_timestep(oa)), 0.0);

    ParamList* lists[6] = { &ma, &va, &mb, &vb, &sa, &sb };
    for (int i = 0; i < 6; ++i)
        param_list_free(lists[i]);
    optimizer_free(oa);
    optimizer_free(ob);
    ema_free(ea);
    ema_free(eb);
    for (int i = 0; i < NT; ++i) {
        cudaFree(pa.items[i].param);
        cudaFree(pa.items[i].grad);
        cudaFree(pb.items[i].param);
        cudaFree(pb.items[i].grad);
    }
    param_list_free(&pa);
    param_list_free(&pb);
}

int main(void)
{
    srand(1234);
    memset(&g_ctx, 0, sizeof g_ctx);
    NN_CUBLAS_CHECK(cublasCreate(&g_ctx.cublas));
    g_ctx.stream = 0;

    check_groupnorm_act(4, 32, 32, 256, 32, ACT_SILU, "groupnorm_act silu [4,32,32,256]");
    check_groupnorm_act(3, 28, 28, 64, 8, ACT_SILU, "groupnorm_act silu [3,28,28,64]");
    check_groupnorm_act(2, 7, 5, 24, 4, ACT_MP_SILU, "groupnorm_act mp_silu [2,7,5,24]");
    check_groupnorm_act(2, 16, 16, 128, 32, ACT_IDENTITY, "groupnorm_act identity [2,16,16,128]");
    check_pixel_norm(2, 8, 8, 128);
    check_pixel_norm(3, 5, 3, 20);
    check_optimizer_ema();

    cublasDestroy(g_ctx.cublas);
    printf("%d failure(s)\n", g_failures);
    return g_failures;
}
