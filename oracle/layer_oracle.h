/* CPU oracle for the fused layer kernels -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A plain-C, scalar restatement of the arithmetic in the reference's
 * src/kernels.cu (cited per function in layer_oracle.c).  Only the test suite,
 * the smoke check and the benchmark's CPU-baseline leg may link or load it; the
 * CUDA library never calls into it and has no CPU fallback.
 *
 * All tensors are dense fp32.  Spatial tensors are NHWC.  "act" uses the
 * reference enum order (src/nn.h:178-183):
 *   0 identity, 1 relu, 2 gelu(tanh form), 3 silu, 4 tanh, 5 mp_silu.
 *
 * Accumulation mode: reductions (sums over rows / pixels / channels) run in
 * fp32 in the reference's sequential order when oracle_set_accumulate_double(0)
 * (the "plain C port" that is timed as the CPU baseline), or in double when
 * oracle_set_accumulate_double(1) (default; the ground truth used for parity).
 */
#ifndef LAYER_ORACLE_H
#define LAYER_ORACLE_H

#ifdef __cplusplus
extern "C" {
#endif

void oracle_set_accumulate_double(int on);
void oracle_set_threads(int n); /* OpenMP threads for the outer loops; 1 = scalar */
int oracle_max_threads(void);

/* element-wise */
float oracle_act_apply(float v, int act);
float oracle_act_grad(float z, int act);
void oracle_activation_forward(float* out, const float* in, long n, int act);
void oracle_activation_backward(float* grad_in, const float* grad_out, const float* in, long n, int act);
void oracle_weighted_sum(float* out, const float* a, const float* b, float wa, float wb, long n);
void oracle_mp_sum(float* out, const float* a, const float* b, float t, long n);
void oracle_mp_sum_backward(float* ga, float* gb, const float* g, float t, long n);
void oracle_scale_by_scalar(float* x, const float* s, long n);
void oracle_mp_cat_weights(float t, int Na, int Nb, float* wa, float* wb);
void oracle_mp_cat(float* out, const float* a, const float* b, float t, long rows, int Na, int Nb);
void oracle_mp_channel_split(float* ga, float* gb, const float* g, float t, long rows, int Ca, int Cb);
void oracle_channel_cat(float* out, const float* a, const float* b, long rows, int Ca, int Cb);
void oracle_channel_split(float* ga, float* gb, const float* g, long rows, int Ca, int Cb);

/* forced weight normalisation, W is [in, out] row-major, columns normalised */
void oracle_weight_normalize(float* W, int in, int out, float eps);
void oracle_weight_normalize_backward(float* gW, const float* Wn, const float* gain, float* g_gain, int in, int out);

/* embeddings.  *_f32 follow the reference expression in fp32 with libm;
   *_f64 evaluate the same expression in double (the truth for tolerance checks). */
void oracle_mp_fourier(float* out, const float* x, const float* freqs, const float* phases, int batch, int C);
void oracle_mp_fourier_f64(double* out, const float* x, const float* freqs, const float* phases, int batch, int C);
void oracle_sinusoidal(float* out, const float* t, int batch, int C, float log_max_period);
void oracle_sinusoidal_f64(double* out, const float* t, int batch, int C, float log_max_period);

/* normalisation */
void oracle_layernorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, long rows, int C, float eps);
void oracle_layernorm_backward(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* mu, const float* rstd, long rows, int C);
void oracle_groupnorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int HW, int C, int G, float eps);
void oracle_groupnorm_backward(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* mu, const float* rstd, int batch, int HW, int C, int G);
/* composition GroupNorm -> activation, as the DDPM block calls it */
void oracle_groupnorm_act_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int HW, int C, int G, float eps, int act);
void oracle_groupnorm_act_backward(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd,
    int batch, int HW, int C, int G, int act);
/* pixel norm over C (no counterpart in the reference; defined by this repository) */
void oracle_pixel_norm_forward(float* y, const float* x, long rows, int C, float eps);
void oracle_pixel_norm_backward(float* dx, const float* dy, const float* x, long rows, int C, float eps);

/* optimiser */
void oracle_sgd_step(float* p, const float* g, float lr, long n);
void oracle_adam_step(float* p, float* m, float* v, const float* g, float lr, float b1, float b2,
    float eps, float bc1, float bc2, long n);
void oracle_adam_ema_step(float* p, float* m, float* v, float* shadow, const float* g, float lr,
    float b1, float b2, float eps, float bc1, float bc2, float decay, float grad_scale, long n);

/* remaining launchers of the C ABI (needed for the training step to link) */
void oracle_add_bias(float* Y, const float* b, int M, int N);
void oracle_bias_grad(float* gb, const float* grad_out, int batch, int N);
void oracle_softmax_xent(float* grad_logits, float* loss_row, const float* logits, const int* targets, int batch, int C);
void oracle_modulate(float* h2, const float* h1, const float* c, long n);
void oracle_modulate_backward(float* gh1, float* gc, const float* gh2, const float* h1, const float* c, long n);
void oracle_embed_gather(float* out, const float* table, const float* idx, int batch, int C, int T);
void oracle_embed_scatter(float* grad_table, const float* grad_out, const float* idx, int batch, int C, int T);
void oracle_im2col(float* col, const float* im, int batch, int H, int W, int C, int K, int stride, int pad, int Ho, int Wo);
void oracle_col2im(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K, int stride, int pad, int Ho, int Wo);
void oracle_avg_pool_2x(float* out, const float* in, int batch, int H, int W, int C);
void oracle_avg_pool_2x_backward(float* grad_in, const float* grad_out, int batch, int H, int W, int C);
void oracle_nearest_upsample_2x(float* out, const float* in, int batch, int H, int W, int C);
void oracle_nearest_upsample_2x_backward(float* grad_in, const float* grad_out, int batch, int H, int W, int C);
void oracle_attn_softmax(float* out, const float* in, int N, int S);
void oracle_attn_softmax_backward(float* grad_in, const float* grad_out, const float* p, int N, int S);
void oracle_permute_0213(float* out, const float* in, int B, int d1, int d2, int d3);
void oracle_spatial_modulate(float* out, const float* in, const float* cond, int batch, int H, int W, int C);
void oracle_spatial_modulate_backward(float* grad_in, float* grad_cond, const float* grad_out, const float* in,
    const float* cond, int batch, int H, int W, int C);
void oracle_spatial_add(float* inout, const float* bias, int batch, int H, int W, int C);
void oracle_spatial_reduce_sum(float* out, const float* in, int batch, int HW, int C);
void oracle_mse_fwd_bwd(float* grad, float* loss_row, const float* pred, const float* target, int batch, int dim);
void oracle_clamp(float* x, float lo, float hi, long n);
/* per-row coefficients: out[r,:] = wa[r]*a[r,:] + wb[r]*b[r,:]  (the per-sample
   loops of diffusion/edm.c:56-64 collapsed into one call) */
void oracle_axpby_rows(float* out, const float* a, const float* b, const float* wa, const float* wb, int rows, int dim);

#ifdef __cplusplus
}
#endif
#endif
