/* Host-side C modules for the fused entry points; see include/b200_fused_modules.h.
   Compiled against the reference's src/nn.h (its Module / ParamList / Optimizer / EMA API). */
#include "b200_fused_modules.h"

#include <math.h>
#include <stdlib.h>

/* ------------------------------------------------------------------ GroupNorm + activation */
typedef struct {
    int C, G, HW;
    float eps;
    Activation act;
    float *gamma, *beta, *ggamma, *gbeta, *mu, *rstd;
} GNActState;

static void gnact_forward(Module* self, const float* in, float* out, int batch, Context* ctx)
{
    GNActState* st = (GNActState*)self->state;
    launch_groupnorm_act_forward(out, st->mu, st->rstd, in, st->gamma, st->beta, batch, st->HW, st->C, st->G,
        st->eps, st->act, ctx->stream);
}

static void gnact_backward(Module* self, const float* in, const float* out, const float* grad_out,
    float* grad_in, int batch, Context* ctx)
{
    (void)out; /* the pre-activation is recomputed from in, mu, rstd: nothing is kept from forward */
    GNActState* st = (GNActState*)self->state;
    launch_groupnorm_act_backward(grad_in, st->ggamma, st->gbeta, grad_out, in, st->gamma, st->beta, st->mu,
        st->rstd, batch, st->HW, st->C, st->G, st->act, ctx->stream);
}

static void gnact_parameters(Module* self, ParamList* pl)
{
    GNActState* st = (GNActState*)self->state;
    param_list_add(pl, st->gamma, st->ggamma, st->C);
    param_list_add(pl, st->beta, st->gbeta, st->C);
}

static void gnact_free(Module* self)
{
    GNActState* st = (GNActState*)self->state;
    float* bufs[6] = { st->gamma, st->beta, st->ggamma, st->gbeta, st->mu, st->rstd };
    for (int i = 0; i < 6; ++i)
        cudaFree(bufs[i]);
    free(st);
    free(self);
}

Module* groupnorm_act_create(int C, int num_groups, int H, int W, int max_batch, Activation act)
{
    NN_ASSERT(num_groups > 0 && C % num_groups == 0, "groupnorm_act: C must be divisible by num_groups");
    Module* m = (Module*)calloc(1, sizeof(Module));
    GNActState* st = (GNActState*)calloc(1, sizeof(GNActState));
    st->C = C;
    st->G = num_groups;
    st->HW = H * W;
    st->eps = 1e-5f;
    st->act = act;
    st->gamma = nn_device_alloc((size_t)C);
    st->beta = nn_device_alloc((size_t)C);
    st->ggamma = nn_device_alloc((size_t)C);
    st->gbeta = nn_device_alloc((size_t)C);
    st->mu = nn_device_alloc((size_t)max_batch * num_groups);
    st->rstd = nn_device_alloc((size_t)max_batch * num_groups);
    float* init = (float*)malloc((size_t)C * sizeof(float));
    for (int c = 0; c < C; ++c)
        init[c] = 1.0f;
    NN_CUDA_CHECK(cudaMemcpy(st->gamma, init, (size_t)C * sizeof(float), cudaMemcpyHostToDevice));
    NN_CUDA_CHECK(cudaMemset(st->beta, 0, (size_t)C * sizeof(float)));
    free(init);
    m->name = "groupnorm_act";
    m->in_dim = m->out_dim = H * W * C;
    m->state = st;
    m->forward = gnact_forward;
    m->backward = gnact_backward;
    m->parameters = gnact_parameters;
    m->free = gnact_free;
    return m;
}

/* ------------------------------------------------------------------ pixel norm */
typedef struct {
    int C, pixels;
    float eps;
} PixelNormState;

static void pn_forward(Module* self, const float* in, float* out, int batch, Context* ctx)
{
    PixelNormState* st = (PixelNormState*)self->state;
    launch_pixel_norm_forward(out, in, batch * st->pixels, st->C, st->eps, ctx->stream);
}

static void pn_backward(Module* self, const float* in, const float* out, const float* grad_out,
    float* grad_in, int batch, Context* ctx)
{
    (void)out;
    PixelNormState* st = (PixelNormState*)self->state;
    launch_pixel_norm_backward(grad_in, grad_out, in, batch * st->pixels, st->C, st->eps, ctx->stream);
}

static void pn_free(Module* self)
{
    free(self->state);
    free(self);
}

Module* pixel_norm_create(int C, int H, int W)
{
    Module* m = (Module*)calloc(1, sizeof(Module));
    PixelNormState* st = (PixelNormState*)calloc(1, sizeof(PixelNormState));
    st->C = C;
    st->pixels = H * W;
    st->eps = 1e-4f;
    m->name = "pixel_norm";
    m->in_dim = m->out_dim = H * W * C;
    m->state = st;
    m->forward = pn_forward;
    m->backward = pn_backward;
    m->parameters = NULL;
    m->free = pn_free;
    return m;
}

/* ------------------------------------------------------------------ fused optimizer + EMA step */
void optimizer_ema_step_fused(Optimizer* o, EMA* ema, const ParamList* pl, float lr, float beta1,
    float beta2, float eps, float ema_decay, float grad_scale, Context* ctx)
{
    const int t = optimizer_timestep(o) + 1;
    optimizer_set_timestep(o, t);
    const float bc1 = 1.0f - powf(beta1, (float)t);
    const float bc2 = 1.0f - powf(beta2, (float)t);

    ParamList m, v, shadow;
    param_list_init(&m);
    param_list_init(&v);
    param_list_init(&shadow);
    optimizer_moment_lists(o, &m, &v);
    if (ema)
        ema_shadow_list(ema, &shadow);
    NN_ASSERT(m.count == pl->count && (!ema || shadow.count == pl->count),
        "optimizer_ema_step_fused: optimizer/EMA were created for a different ParamList");

    B200ParamUpdate batch[B200_MAX_MULTI];
    int n = 0;
    for (int i = 0; i < pl->count; ++i) {
        batch[n].p = pl->items[i].param;
        batch[n].g = pl->items[i].grad;
        batch[n].m = m.items[i].param;
        batch[n].v = v.items[i].param;
        batch[n].shadow = ema ? shadow.items[i].param : NULL;
        batch[n].n = pl->items[i].size;
        if (++n == B200_MAX_MULTI || i == pl->count - 1) {
            launch_adam_ema_step_multi(batch, n, lr, beta1, beta2, eps, bc1, bc2, ema_decay, grad_scale, ctx->stream);
            n = 0;
        }
    }
    param_list_free(&m);
    param_list_free(&v);
    param_list_free(&shadow);
}
