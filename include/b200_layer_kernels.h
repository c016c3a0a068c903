/* C ABI of the B200 (sm_100a) layer-kernel library: libb200_layer_kernels.so
 *
 * Part 1 is the drop-in boundary: the complete launcher set that the reference
 * declares in src/nn.h:354-462 and implements in src/kernels.cu.  The symbols,
 * argument order and argument meaning are exactly the reference's, so its
 * unmodified host modules (groupnorm.c, layernorm.c, activation.c, mp_linear.c,
 * mp_fourier.c, sinusoidal.c, optimizer.c, ema.c, unet.c, ddpm_unet.c, ...)
 * link against this library instead of build/kernels.o.  Each prototype cites
 * the reference declaration (nn.h) and implementation (kernels.cu) it replaces.
 *
 * Part 2 are additive entry points for fusions that cross the reference's call
 * boundaries (GroupNorm+activation, Adam+EMA, multi-tensor forms, pixel norm).
 *
 * Conventions (same as the reference): all pointers are DEVICE pointers to
 * dense fp32 data, extents are int, spatial tensors are NHWC, every call is
 * asynchronous on the given stream, performs no host synchronisation, and
 * parameter gradients are overwritten (not accumulated) unless stated.
 * The `act` argument uses the reference's enum values (nn.h:178-183):
 *   0 identity, 1 relu, 2 gelu, 3 silu, 4 tanh, 5 mp_silu.
 * When this header is included after the reference's nn.h the enum type is
 * the reference's `Activation`; otherwise it is declared here as plain int.
 */
#ifndef B200_LAYER_KERNELS_H
#define B200_LAYER_KERNELS_H

#include <cuda_runtime.h>

#ifdef NN_H
typedef Activation b200_act_t;
#else
typedef int b200_act_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ======================= Part 1: reference launcher set ======================= */
#ifndef NN_H /* nn.h already carries identical prototypes */

/* nn.h:354, kernels.cu:95/193   Y[M,N] += b[N] */
void launch_add_bias(float* Y, const float* b, int M, int N, cudaStream_t s);
/* nn.h:356, kernels.cu:103/199  out = act(in) */
void launch_activation_forward(float* out, const float* in, int n, b200_act_t act, cudaStream_t s);
/* nn.h:358, kernels.cu:111/206  grad_in = grad_out * act'(in); `in` is the pre-activation */
void launch_activation_backward(float* grad_in, const float* grad_out, const float* in, int n,
    b200_act_t act, cudaStream_t s);
/* nn.h:362, kernels.cu:119/215  row-wise softmax cross-entropy loss and gradient */
void launch_softmax_xent(float* grad_logits, float* loss_row, const float* logits,
    const int* targets, int batch, int C, cudaStream_t s);
/* nn.h:365, kernels.cu:148/225  gb[n] = sum_rows grad_out */
void launch_bias_grad(float* gb, const float* grad_out, int batch, int N, cudaStream_t s);
/* nn.h:368, kernels.cu:163/234 */
void launch_sgd_step(float* p, const float* g, float lr, int n, cudaStream_t s);
/* nn.h:369, kernels.cu:170/241  bc1, bc2 are the host-computed bias corrections (optimizer.c:62-64) */
void launch_adam_step(float* p, float* m, float* v, const float* g, float lr, float beta1,
    float beta2, float eps, float bc1, float bc2, int n, cudaStream_t s);
/* nn.h:374, kernels.cu:255/330  W[in,out]: every column scaled to unit norm IN PLACE,
   factor rsqrt(sum_i W_ij^2 + eps) */
void launch_weight_normalize(float* W, int in, int out, float eps, cudaStream_t s);
/* nn.h:375, kernels.cu:277/337  per column: dot=<Wn,gW>; *g_gain += dot (caller zeroes it);
   gW = gain*(gW - dot*Wn) in place */
void launch_weight_normalize_backward(float* gW, const float* Wn, const float* gain,
    float* g_gain, int in, int out, cudaStream_t s);
/* nn.h:377, kernels.cu:300/346  x *= s[0] (s is a device scalar) */
void launch_scale_by_scalar(float* x, const float* s, int n, cudaStream_t st);
/* nn.h:378, kernels.cu:360      out = ((1-t)a + t b)/sqrt((1-t)^2+t^2) */
void launch_mp_sum(float* out, const float* a, const float* b, float t, int n, cudaStream_t s);
/* nn.h:380, kernels.cu:308/353  out = wa*a + wb*b; out may alias a and/or b, a may alias b */
void launch_weighted_sum(float* out, const float* a, const float* b, float wa, float wb, int n,
    cudaStream_t s);
/* nn.h:382, kernels.cu:385/416  out[b,k] = sqrt(2) cos(2 pi (x[b] f[k] + phi[k])) */
void launch_mp_fourier(float* out, const float* x, const float* freqs, const float* phases,
    int batch, int C, cudaStream_t s);
/* nn.h:384, kernels.cu:397/425  h2 = h1*(c+1) */
void launch_modulate(float* h2, const float* h1, const float* c, int n, cudaStream_t s);
/* nn.h:385, kernels.cu:405/432 */
void launch_modulate_backward(float* gh1, float* gc, const float* gh2, const float* h1,
    const float* c, int n, cudaStream_t s);
/* nn.h:387, kernels.cu:444/569  out[b,:] = [sin(t f_j), cos(t f_j)], f_j = exp(-log_max_period j/half) */
void launch_sinusoidal(float* out, const float* t, int batch, int C, float log_max_period,
    cudaStream_t s);
/* nn.h:389, kernels.cu:459/577  table lookup, index carried as float and clamped to [0,T) */
void launch_embed_gather(float* out, const float* table, const float* idx, int batch, int C, int T,
    cudaStream_t s);
/* nn.h:391, kernels.cu:474/585  scatter-ADD into grad_table */
void launch_embed_scatter(float* grad_table, const float* grad_out, const float* idx, int batch,
    int C, int T, cudaStream_t s);
/* nn.h:393, kernels.cu:491/594  per-row LayerNorm; stores mu, rstd [batch] */
void launch_layernorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int C, float eps, cudaStream_t s);
/* nn.h:396, kernels.cu:520,550/604 */
void launch_layernorm_backward(float* grad_in, float* ggamma, float* gbeta, const float* grad_out,
    const float* x, const float* gamma, const float* mu, const float* rstd, int batch, int C,
    cudaStream_t s);
/* nn.h:400, kernels.cu:622/719  NHWC GroupNorm; stores mu, rstd [batch*G] */
void launch_groupnorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int HW, int C, int G, float eps, cudaStream_t s);
/* nn.h:404, kernels.cu:659,696/731 */
void launch_groupnorm_backward(float* dx, float* ggamma, float* gbeta, const float* dy,
    const float* x, const float* gamma, const float* mu, const float* rstd, int batch, int HW,
    int C, int G, cudaStream_t s);
/* nn.h:408, kernels.cu:318/368  scaled concat of a[batch,Na], b[batch,Nb] */
void launch_mp_cat(float* out, const float* a, const float* b, float t, int batch, int Na, int Nb,
    cudaStream_t s);
/* nn.h:412, kernels.cu:750/818 */
void launch_im2col(float* col, const float* im, int batch, int H, int W, int C, int K, int stride,
    int pad, int H_out, int W_out, cudaStream_t s);
/* nn.h:414, kernels.cu:785/829  scatter-ADD into grad_im (caller zeroes it) */
void launch_col2im(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K,
    int stride, int pad, int H_out, int W_out, cudaStream_t s);
/* nn.h:418-425, kernels.cu:843-965 */
void launch_avg_pool_2x(float* out, const float* in, int batch, int H, int W, int C, cudaStream_t s);
void launch_avg_pool_2x_backward(float* grad_in, const float* grad_out, int batch, int H, int W,
    int C, cudaStream_t s);
void launch_nearest_upsample_2x(float* out, const float* in, int batch, int H, int W, int C,
    cudaStream_t s);
void launch_nearest_upsample_2x_backward(float* grad_in, const float* grad_out, int batch, int H,
    int W, int C, cudaStream_t s);
/* nn.h:428-432, kernels.cu:970-1051; softmax may run in place */
void launch_attn_softmax(float* out, const float* in, int N, int S, cudaStream_t s);
void launch_attn_softmax_backward(float* grad_in, const float* grad_out, const float* p, int N,
    int S, cudaStream_t s);
void launch_permute_0213(float* out, const float* in, int B, int d1, int d2, int d3, cudaStream_t s);
/* nn.h:435-440, kernels.cu:1056-1127  FiLM: out = in*(cond[b,c]+1) */
void launch_spatial_modulate(float* out, const float* in, const float* cond, int batch, int H,
    int W, int C, cudaStream_t s);
void launch_spatial_modulate_backward(float* grad_in, float* grad_cond, const float* grad_out,
    const float* in, const float* cond, int batch, int H, int W, int C, cudaStream_t s);
/* nn.h:443-446, kernels.cu:1132-1178 */
void launch_spatial_add(float* inout, const float* bias, int batch, int H, int W, int C,
    cudaStream_t s);
void launch_spatial_reduce_sum(float* out, const float* in, int batch, int HW, int C, cudaStream_t s);
/* nn.h:449-456, kernels.cu:1183-1278 */
void launch_channel_cat(float* out, const float* a, const float* b, int spatial, int Ca, int Cb,
    cudaStream_t s);
void launch_channel_split(float* grad_a, float* grad_b, const float* grad_out, int spatial, int Ca,
    int Cb, cudaStream_t s);
void launch_mp_channel_cat(float* out, const float* a, const float* b, float t, int spatial,
    int Ca, int Cb, cudaStream_t s);
void launch_mp_channel_split(float* grad_a, float* grad_b, const float* grad_out, float t,
    int spatial, int Ca, int Cb, cudaStream_t s);
/* nn.h:459, kernels.cu:1284/1306 */
void launch_mse_fwd_bwd(float* grad, float* loss_row, const float* pred, const float* target,
    int batch, int dim, cudaStream_t s);
/* nn.h:462, kernels.cu:1317/1324 */
void launch_clamp(float* x, float lo, float hi, int n, cudaStream_t s);

#endif /* !NN_H */

/* ===================== Part 2: additive fused entry points ===================== */

/* GroupNorm + affine + activation in one pass.  Replaces the call pair
   gn->forward + launch_activation_forward of conv_residual.c:28-29 and :35-36.
   Writes only the activated output (plus mu, rstd). */
void launch_groupnorm_act_forward(float* y, float* mu, float* rstd, const float* x,
    const float* gamma, const float* beta, int batch, int HW, int C, int G, float eps,
    b200_act_t act, cudaStream_t s);
/* Backward of the fused op; replaces launch_activation_backward + gn->backward of
   conv_residual.c:51-52 and :62-63.  The pre-activation is recomputed from
   x, mu, rstd, gamma, beta, so no extra tensor is kept between the passes. */
void launch_groupnorm_act_backward(float* dx, float* ggamma, float* gbeta, const float* dy,
    const float* x, const float* gamma, const float* beta, const float* mu, const float* rstd,
    int batch, int HW, int C, int G, b200_act_t act, cudaStream_t s);

/* Pixel norm over the channel axis: y = x * rsqrt(mean_c(x^2) + eps).
   No counterpart in the reference (it has no pixel-norm kernel or module); the
   eps-inside-the-root convention follows its weight norm (kernels.cu:269). */
void launch_pixel_norm_forward(float* y, const float* x, int rows, int C, float eps, cudaStream_t s);
void launch_pixel_norm_backward(float* dx, const float* dy, const float* x, int rows, int C,
    float eps, cudaStream_t s);

/* Backward of mp_sum: ga = wa*g, gb = wb*g with the weights of launch_mp_sum, one read of g.
   Replaces the two launch_weighted_sum calls of cond_conv_residual.c:46 and :61. */
void launch_mp_sum_backward(float* ga, float* gb, const float* g, float t, int n, cudaStream_t s);

/* Adam step followed by the EMA shadow update in one pass over the parameters
   (36 B/param instead of 28 + 12).  Replaces launch_adam_step (optimizer.c:65-68)
   + launch_weighted_sum (ema.c:32) on the same tensor.  `grad_scale` multiplies
   the gradient first (1/k when k data-parallel ranks summed their gradients).
   shadow may be NULL (plain Adam). */
void launch_adam_ema_step(float* p, float* m, float* v, float* shadow, const float* g, float lr,
    float beta1, float beta2, float eps, float bc1, float bc2, float decay, float grad_scale,
    long long n, cudaStream_t s);

/* The same update for a whole ParamList in ONE launch.  `items` is a HOST array
   (copied into the kernel arguments, at most B200_MAX_MULTI entries per call). */
typedef struct {
    float* p;
    const float* g;
    float* m;
    float* v;
    float* shadow; /* may be NULL */
    int n;
} B200ParamUpdate;
#define B200_MAX_MULTI 64
void launch_adam_ema_step_multi(const B200ParamUpdate* items, int count, float lr, float beta1,
    float beta2, float eps, float bc1, float bc2, float decay, float grad_scale, cudaStream_t s);

/* Forced weight normalisation of several matrices in one launch (the EDM UNet
   normalises ~30 weights per forward: conv2d.c:28, mp_linear.c:16, attention.c:25-27). */
typedef struct {
    float* W;
    int in, out;
} B200WeightDesc;
void launch_weight_normalize_multi(const B200WeightDesc* items, int count, float eps, cudaStream_t s);

/* launch_weight_normalize_backward (nn.h:394, kernels.cu:277-297, :337) for several weights in one launch.
   Same per-weight semantics: gW <- gain * (gW - dot_j * Wn) per column j, *g_gain += sum_j dot_j
   (the caller zeroes g_gain, as conv2d.c:50 and mp_linear.c:31 do). */
typedef struct {
    float* gW;
    const float* Wn;
    const float* gain;
    float* g_gain;
    int in, out;
} B200WeightGradDesc;
void launch_weight_normalize_backward_multi(const B200WeightGradDesc* items, int count, cudaStream_t s);

/* Batching of the per-weight calls for hosts whose modules call launch_weight_normalize /
   launch_weight_normalize_backward one weight at a time (conv2d.c, mp_linear.c, attention.c) and whose
   driver owns the training step.  Modes:
     0  off (default).
     1  record: calls execute as usual; the forward calls' (W, in, out, eps) are remembered (one entry per W).
     2  batched: launch_weight_normalize returns at once for every RECORDED weight - the driver has normalised
        those with b200_wn_forward_all since the last parameter update; a weight that was never recorded (a
        layer first used after the recording pass, another model) is normalised at once and joins the set; launch_weight_normalize_backward only
        queues its arguments, and b200_wn_backward_flush runs the queue as one launch.  Nothing between a
        module's backward and the optimizer reads gW or g_gain, so the deferral does not change results.
   The state is per process, not per stream: one training loop at a time.  b200_wn_forward_all and
   b200_wn_backward_flush return the number of weights they covered (0 when nothing is recorded/queued). */
void b200_wn_batch_mode(int mode);
int b200_wn_forward_all(cudaStream_t s);
int b200_wn_backward_flush(cudaStream_t s);

/* Fusions inside the EDM residual block (cond_conv_residual.c:24-63):
   - out = act(in * (cond[b,c] + 1)): launch_spatial_modulate + launch_activation_forward in one pass; the
     modulated tensor itself is not materialised.
   - its backward: z = in*(cond+1), g = grad_out*act'(z), grad_in = g*(cond+1), grad_cond[b,c] = sum_hw g*in
     (launch_activation_backward + launch_spatial_modulate_backward; z is recomputed, not read).
   - out = w_skip*skip + grad_out*act'(in): launch_activation_backward + the skip branch of mp_sum's backward
     (launch_weighted_sum with wb = 1). `out` may alias `grad_out`. */
void launch_film_act_forward(float* out, const float* in, const float* cond, int batch, int H, int W, int C,
    b200_act_t act, cudaStream_t s);
void launch_film_act_backward(float* grad_in, float* grad_cond, const float* grad_out, const float* in,
    const float* cond, int batch, int H, int W, int C, b200_act_t act, cudaStream_t s);
void launch_activation_backward_axpy(float* out, const float* grad_out, const float* in, const float* skip,
    float w_skip, int n, b200_act_t act, cudaStream_t s);

/* launch_col2im (nn.h, kernels.cu:800-838) that OVERWRITES grad_im instead of accumulating into it: saves the
   cudaMemsetAsync of grad_im and its read-back that conv2d.c:61-65 pays before every col2im. */
void launch_col2im_assign(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K,
    int stride, int pad, int H_out, int W_out, cudaStream_t s);

/* out[r,:] = wa[r]*a[r,:] + wb[r]*b[r,:] with per-row DEVICE coefficients: one
   launch for the per-sample launch_weighted_sum loops of diffusion/edm.c:56-64,
   :75-80, :205-207 and loss.c:65-70.  Aliasing as for launch_weighted_sum. */
void launch_axpby_rows(float* out, const float* a, const float* b, const float* wa,
    const float* wb, int rows, int dim, cudaStream_t s);

/* Fused Adam+EMA on a parameter range that ALSO writes the new parameters into up to B200_MAX_PEERS further
   buffers: the range-sharded optimizer's update and its all-gather in one kernel.  Each dst[k] is the address
   of the same range inside another GPU's copy of the parameter vector (a peer pointer obtained through CUDA
   IPC or any other peer mapping; plain 128-bit stores over NVLink, no multicast, no TMA), so the exchange
   happens in the update's store phase instead of a separate collective.  Everything else as
   launch_adam_ema_step.  p, m, v, shadow, g and every dst must be 16-byte aligned and n a multiple of 4
   (range cuts of the sharded optimizer are).  The kernel only stores to the peers: ordering against the
   peers' readers is the caller's (a collective or an event exchange after the launch). */
#define B200_MAX_PEERS 15
typedef struct {
    float* dst[B200_MAX_PEERS];
    int count;
} B200PeerDests;
void launch_adam_ema_step_bcast(float* p, float* m, float* v, float* shadow, const float* g,
    const B200PeerDests* peers, float lr, float beta1, float beta2, float eps, float bc1, float bc2, float decay,
    float grad_scale, long long n, cudaStream_t s);

/* dst_i[0:n_i] = src_i[0:n_i] for a table of up to B200_MAX_MULTI ranges per launch: packs the gradients of a
   ParamList into a flat arena (and unpacks the parameters) for the range-sharded optimizer in one launch. */
typedef struct {
    float* dst;
    const float* src;
    int n;
} B200CopyItem;
void launch_copy_multi(const B200CopyItem* items, int count, cudaStream_t s);

/* LayerNorm backward that allocates nothing.  It has no counterpart in the reference.
   For hosts that run under a fixed device-memory plan and may not enter the CUDA allocator
   after set-up (boards whose heap is sized once by the module constructors, or call sites
   where cudaMalloc is off limits, e.g. inside an allocator hook): same arguments and results
   as launch_layernorm_backward, but the per-CTA dgamma/dbeta partial rows go to a fixed
   4 MiB array that is part of the library image (every GPU that loads the library carries it
   until the process exits) instead of the on-demand scratch arena.
   - Returns 0 on success; a negative value (and an error report, see b200_set_error_mode)
     otherwise: -1 bad extents, -2 the shape needs more partial rows than the array holds, -3 the
     array's address could not be looked up, -4 a kernel launch failed (nothing after it ran).
     The size rule: for C a multiple of 128 up to
     1024 every batch fits; otherwise ceil(batch/256) * 2*C floats must be <= 1048576.
   - The first call on each device looks up the array's device address (that device must be
     current); make that first call before starting any stream capture.
   - All calls share the one array and it keeps what the previous call left there.  Nothing in
     it has to be zero beforehand (every partial row is written before it is read), but two
     calls that overlap on the GPU, from different streams or processes sharing the context,
     race on it: serialise them. */
int launch_layernorm_backward_noalloc(float* grad_in, float* ggamma, float* gbeta,
    const float* grad_out, const float* x, const float* gamma, const float* mu, const float* rstd,
    int batch, int C, cudaStream_t s);

/* ============================ library management ============================ */

/* Error handling.  Mode 0 (default) follows the reference (nn.h:13-52): print
   "file:line: message" to stderr and exit(1).  Mode 1 records the message and
   returns from the launcher without launching. */
void b200_set_error_mode(int mode);
int b200_error_count(void);
int b200_last_error(char* buf, int buflen); /* copies the last message; returns its length */
void b200_clear_error(void);
/* Error word that a kernel sets when a bounded device-side wait runs out (synchronises the device).  No kernel
   of the current library waits on another CTA, kernel or rank, so this reads 0; kept for hosts that poll it. */
int b200_device_error_status(void);

/* Number of kernels this library has launched since load (or since reset). */
long long b200_launch_count(void);
void b200_launch_count_reset(void);
/* Number of GroupNorm launches since load that took kernel family `path`: 0 one strip per CTA, 1 pipelined
   strips, 2 deep-staged strips, 3 one-barrier strips, 4 chunked strips, 5 generic; -1 for any other value.
   For tests that must know which family they exercised. */
long long b200_groupnorm_path_count(int path);
/* Which kernel family, CTA size, strip width, grid and cluster width the GroupNorm dispatcher would choose for
   a shape, written as text ("family=one-barrier threads=1024 strip_channels=32 ctas=147 cluster=4 smem=...");
   `act` as in launch_groupnorm_act_forward (0 = none), `backward` 0 or 1.  Makes no CUDA call and launches
   nothing (without a device the SM count is taken as 148), so the dispatch rules can be tested on a CPU box.
   Returns the length of the text, -1 for bad arguments.  Pointers are assumed 16-byte aligned. */
int b200_groupnorm_describe(int batch, int HW, int C, int G, int act, int backward, char* out, int out_len);

/* Pre-sizes the scratch arena used by the backward kernels on `s` so that no
   allocation happens later (call before capturing a CUDA graph). */
int b200_scratch_reserve(cudaStream_t s, long long bytes);
/* Kernel tunables for experiments, e.g. ("gn_fwd_ct", 32).  Unknown keys are stored. */
void b200_tune_set(const char* key, int value);
int b200_tune_get(const char* key, int dflt);
const char* b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_LAYER_KERNELS_H */
