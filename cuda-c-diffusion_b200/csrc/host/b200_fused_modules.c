/* Host-side C modules for the fused entry points; see include/b200_fused_modules.h.
   Compiled against the reference's src/nn.h (its Module / ParamList / Optimizer / EMA API). */
#include "b200_fused_modules.h"

#include <math.h>
#include <stdlib.h>

/* ------------------------------------------------------------------ GroupNorm + activation */
/* One device allocation per module: [scale | shift | scale grad | shift grad | mean | rstd]; the four
   channel vectors are padded to 16-byte multiples so that the kernels' 128-bit accesses apply. */
typedef struct {
    int channels, groups, pixels;
    Activation act;
    float epsilon;
    float* block;
    float *scale, *shift, *scale_grad, *shift_grad; /* gamma, beta and their gradients */
    float *mean, *rstd;                               /* [max_batch * groups], written by forward */
} NormAct;

static void normact_forward(Module* self, const float* x, float* y, int batch, Context* ctx)
{
    NormAct* na = (NormAct*)self->state;
    launch_groupnorm_act_forward(y, na->mean, na->rstd, x, na->scale, na->shift, batch, na->pixels, na->channels,
        na->groups, na->epsilon, na->act, ctx->stream);
}

static void normact_backward(Module* self, const float* x, const float* y, const float* dy, float* dx, int batch,
    Context* ctx)
{
    (void)y; /* the pre-activation is recomputed from x, mean, rstd: nothing is kept from forward */
    NormAct* na = (NormAct*)self->state;
    launch_groupnorm_act_backward(dx, na->scale_grad, na->shift_grad, dy, x, na->scale, na->shift, na->mean, na->rstd,
        batch, na->pixels, na->channels, na->groups, na->act, ctx->stream);
}

static void normact_parameters(Module* self, ParamList* pl)
{
    NormAct* na = (NormAct*)self->state;
    param_list_add(pl, na->scale, na->scale_grad, na->channels);
    param_list_add(pl, na->shift, na->shift_grad, na->channels);
}

static void normact_free(Module* self)
{
    NormAct* na = (NormAct*)self->state;
    cudaFree(na->block);
    free(na);
    free(self);
}

Module* groupnorm_act_create(int C, int num_groups, int H, int W, int max_batch, Activation act)
{
    NN_ASSERT(num_groups > 0 && C % num_groups == 0, "groupnorm_act: C must be divisible by num_groups");
    NormAct* na = (NormAct*)calloc(1, sizeof *na);
    na->channels = C;
    na->groups = num_groups;
    na->pixels = H * W;
    na->act = act;
    na->epsilon = 1e-5f;

    const size_t cpad = ((size_t)C + 3) & ~(size_t)3, stats = (size_t)max_batch * num_groups;
    NN_CUDA_CHECK(cudaMalloc((void**)&na->block, (4 * cpad + 2 * stats) * sizeof(float)));
    NN_CUDA_CHECK(cudaMemset(na->block, 0, (4 * cpad + 2 * stats) * sizeof(float))); /* shift = 0 */
    na->scale = na->block;
    na->shift = na->scale + cpad;
    na->scale_grad = na->shift + cpad;
    na->shift_grad = na->scale_grad + cpad;
    na->mean = na->shift_grad + cpad;
    na->rstd = na->mean + stats;
    float* ones = (float*)malloc((size_t)C * sizeof(float));
    for (int c = 0; c < C; ++c)
        ones[c] = 1.0f;
    NN_CUDA_CHECK(cudaMemcpy(na->scale, ones, (size_t)C * sizeof(float), cudaMemcpyHostToDevice));
    free(ones);

    Module* m = (Module*)calloc(1, sizeof *m);
    m->name = "groupnorm_act";
    m->in_dim = m->out_dim = H * W * C;
    m->state = na;
    m->forward = normact_forward;
    m->backward = normact_backward;
    m->parameters = normact_parameters;
    m->free = normact_free;
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
