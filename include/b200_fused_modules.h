/* Host-side C modules for the additive fused entry points of libb200_layer_kernels.so.
 *
 * These are the pieces a maintainer of the reference adds to its tree to use the fusions:
 * they implement the reference's own `Module` vtable (src/nn.h:159-174)
 * and use only its public optimizer / EMA API (src/nn.h:216-254).  The file is compiled with
 * the reference's `src/` on the include path; it needs `nn.h` and is NOT self-contained.
 */
#ifndef B200_FUSED_MODULES_H
#define B200_FUSED_MODULES_H

#include "nn.h" /* the reference's header */
#include "b200_layer_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

/* GroupNorm + affine + activation as ONE module.  Drop-in for the pair
   spatial_groupnorm_create(...) + launch_activation_forward(...) of conv_residual.c:28-29;
   same parameters (gamma, beta), same eps (1e-5), no intermediate buffer. */
Module* groupnorm_act_create(int C, int num_groups, int H, int W, int max_batch, Activation act);

/* Pixel norm over C for an NHWC tensor [batch, H, W, C]; eps 1e-4 inside the root; no parameters. */
Module* pixel_norm_create(int C, int H, int W);

/* optimizer_step (optimizer.c:54-69) and ema_update (ema.c:29-35) for the whole ParamList in ONE
   kernel launch.  The optimizer's hyper-parameters are private to optimizer.c, so the caller
   passes the values it created the optimizer with; the step counter is advanced through
   optimizer_timestep / optimizer_set_timestep.  grad_scale multiplies every gradient (1/ranks
   after a summing all-reduce).  ema may be NULL (plain Adam). */
void optimizer_ema_step_fused(Optimizer* o, EMA* ema, const ParamList* pl, float lr, float beta1,
    float beta2, float eps, float ema_decay, float grad_scale, Context* ctx);

#ifdef __cplusplus
}
#endif
#endif
