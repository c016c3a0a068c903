// The rest of the launcher set the reference's host modules link against:
// im2col / col2im feeding the cuBLAS convolutions, 2x pooling / upsampling,
// attention softmax and head permutes, FiLM backward, per-sample channel
// reductions, bias gradient, the MSE and softmax cross-entropy heads
// (reference: src/kernels.cu:119-161, :750-1178, :1284-1313).
//
// These sit either side of the fused layer kernels in a training step.  They
// are coalesced sm_100a kernels: channel-contiguous float4 accesses where
// C % 4 == 0, gathers instead of atomic scatters (col2im), strip reductions
// instead of one serial thread per output.  im2col / col2im, which move nine
// times the activation per 3x3 convolution, decode their coordinates once per
// (pixel, channel pack) and walk the K*K taps with all loads in flight; an
// overwriting col2im saves the caller's memset and read-back.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

namespace b200 {

static inline int flat_grid(long n, int threads = 256)
{
    long g = (n + threads - 1) / threads;
    const long cap = (long)sm_count() * 16;
    if (g > cap)
        g = cap;
    return g < 1 ? 1 : (int)g;
}

// ---------------------------------------------------------------------------
// im2col / col2im.  V = floats per access along C (4 when C % 4 == 0).
// col is [B*Ho*Wo, K*K*C] with column (kh*K + kw)*C + c.
// ---------------------------------------------------------------------------
template <int V>
__global__ void __launch_bounds__(256) im2col_kernel(float* __restrict__ col, const float* __restrict__ im, int H, int W,
    int C, int K, int stride, int pad, int Ho, int Wo, long total)
{
    pdl_prologue();
    const int Cv = C / V;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long tmp = i;
        const int cv = (int)(tmp % Cv); tmp /= Cv;
        const int kw = (int)(tmp % K); tmp /= K;
        const int kh = (int)(tmp % K); tmp /= K;
        const int ow = (int)(tmp % Wo); tmp /= Wo;
        const int oh = (int)(tmp % Ho); tmp /= Ho;
        const long b = tmp;
        const int ih = oh * stride + kh - pad, iw = ow * stride + kw - pad;
        Pack<V> v;
#pragma unroll
        for (int e = 0; e < V; ++e)
            v.v[e] = 0.0f;
        if (ih >= 0 && ih < H && iw >= 0 && iw < W)
            v = load_cached<V>(im + ((b * H + ih) * W + iw) * C + (long)cv * V);
        store_stream<V>(col + i * V, v);
    }
}

// float4 fast path: one thread per (output pixel, channel pack).  The coordinates are decoded once
// (32-bit arithmetic) and the K*K taps are then walked with all loads in flight, so the index
// arithmetic is paid once per K*K stores instead of once per store.  KT = K at compile time (0: runtime).
template <int KT>
__global__ void __launch_bounds__(256) im2col_taps_kernel(float4* __restrict__ col, const float4* __restrict__ im,
    int H, int W, int Cv, int K, int stride, int pad, int Ho, int Wo, unsigned total)
{
    pdl_prologue();
    const int Kk = KT ? KT : K;
    const unsigned row4 = (unsigned)(Kk * Kk) * (unsigned)Cv;  // float4 per col row
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned p = i / (unsigned)Cv, cv = i - p * (unsigned)Cv;
        const unsigned ow = p % (unsigned)Wo, t2 = p / (unsigned)Wo;
        const unsigned oh = t2 % (unsigned)Ho, b = t2 / (unsigned)Ho;
        const int ih0 = (int)oh * stride - pad, iw0 = (int)ow * stride - pad;
        const float4* src = im + (size_t)b * H * W * Cv + cv;
        float4* dst = col + (size_t)p * row4 + cv;
#pragma unroll
        for (int kh = 0; kh < Kk; ++kh) {
#pragma unroll
            for (int kw = 0; kw < Kk; ++kw) {
                const int ih = ih0 + kh, iw = iw0 + kw;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                    v = __ldg(src + (size_t)(ih * W + iw) * Cv);
                __stcs(dst + (kh * Kk + kw) * Cv, v);
            }
        }
    }
}

// grad_im[b,ih,iw,c] += sum over the (kh,kw) taps whose output pixel exists
template <int V>
__global__ void __launch_bounds__(256) col2im_gather_kernel(float* __restrict__ grad_im,
    const float* __restrict__ grad_col, int H, int W, int C, int K, int stride, int pad, int Ho, int Wo, long total)
{
    pdl_prologue();
    const int Cv = C / V;
    const long KKC = (long)K * K * C;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long tmp = i;
        const int cv = (int)(tmp % Cv); tmp /= Cv;
        const int iw = (int)(tmp % W); tmp /= W;
        const int ih = (int)(tmp % H); tmp /= H;
        const long b = tmp;
        Pack<V> acc;
#pragma unroll
        for (int e = 0; e < V; ++e)
            acc.v[e] = 0.0f;
        for (int kh = 0; kh < K; ++kh) {
            const int th = ih + pad - kh;
            if (th < 0 || th % stride != 0)
                continue;
            const int oh = th / stride;
            if (oh >= Ho)
                continue;
            for (int kw = 0; kw < K; ++kw) {
                const int tw = iw + pad - kw;
                if (tw < 0 || tw % stride != 0)
                    continue;
                const int ow = tw / stride;
                if (ow >= Wo)
                    continue;
                const Pack<V> g = load_stream<V>(
                    grad_col + ((b * Ho + oh) * Wo + ow) * KKC + ((long)kh * K + kw) * C + (long)cv * V);
#pragma unroll
                for (int e = 0; e < V; ++e)
                    acc.v[e] += g.v[e];
            }
        }
        float* dst = grad_im + i * V;
        Pack<V> old = load_stream<V>(dst);
#pragma unroll
        for (int e = 0; e < V; ++e)
            old.v[e] += acc.v[e];
        store_stream<V>(dst, old);
    }
}

// float4, stride-1 fast path of the gather: one thread per (input pixel, channel pack), coordinates
// decoded once in 32-bit arithmetic, the K*K candidate taps unrolled so that their loads overlap.
template <int KT, bool ASSIGN>
__global__ void __launch_bounds__(256) col2im_taps_kernel(float4* __restrict__ grad_im,
    const float4* __restrict__ grad_col, int H, int W, int Cv, int K, int pad, int Ho, int Wo, unsigned total)
{
    pdl_prologue();
    const int Kk = KT ? KT : K;
    const unsigned row4 = (unsigned)(Kk * Kk) * (unsigned)Cv;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned pix = i / (unsigned)Cv, cv = i - pix * (unsigned)Cv;
        const unsigned iw = pix % (unsigned)W, t2 = pix / (unsigned)W;
        const unsigned ih = t2 % (unsigned)H, b = t2 / (unsigned)H;
        const float4* src = grad_col + (size_t)b * Ho * Wo * row4 + cv;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int kh = 0; kh < Kk; ++kh) {
            const int oh = (int)ih + pad - kh;
#pragma unroll
            for (int kw = 0; kw < Kk; ++kw) {
                const int ow = (int)iw + pad - kw;
                if (oh >= 0 && oh < Ho && ow >= 0 && ow < Wo) {
                    const float4 g = __ldcs(src + (size_t)(oh * Wo + ow) * row4 + (kh * Kk + kw) * Cv);
                    acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
                }
            }
        }
        if (ASSIGN) {
            grad_im[i] = acc;
        } else {
            float4 old = grad_im[i];
            old.x += acc.x; old.y += acc.y; old.z += acc.z; old.w += acc.w;
            grad_im[i] = old;
        }
    }
}

// ---------------------------------------------------------------------------
// 2x average pool / nearest upsample and their backwards
// MODE 0: avg pool fwd (out [B,H/2,W/2,C])      MODE 1: avg pool bwd (writes the 4 covered inputs)
// MODE 2: upsample fwd (out [B,2H,2W,C])        MODE 3: upsample bwd (sum of the 2x2 block)
// `total` counts packs of the SMALL tensor for modes 0,1,3 and of the big one for mode 2.
// ---------------------------------------------------------------------------
template <int MODE, int V>
__global__ void __launch_bounds__(256) resample_kernel(float* __restrict__ dst, const float* __restrict__ src, int H,
    int W, int C, long total)
{
    pdl_prologue();
    const int Cv = C / V;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long tmp = i;
        const int cv = (int)(tmp % Cv); tmp /= Cv;
        if (MODE == 0 || MODE == 1) {
            const int Ho = H / 2, Wo = W / 2;
            const int ow = (int)(tmp % Wo); tmp /= Wo;
            const int oh = (int)(tmp % Ho); tmp /= Ho;
            const long b = tmp;
            const long big = ((b * H + 2 * oh) * W + 2 * ow) * C + (long)cv * V;
            const long rowstep = (long)W * C;
            if (MODE == 0) {
                const Pack<V> a = load_stream<V>(src + big), bq = load_stream<V>(src + big + C);
                const Pack<V> c = load_stream<V>(src + big + rowstep), d = load_stream<V>(src + big + rowstep + C);
                Pack<V> o;
#pragma unroll
                for (int e = 0; e < V; ++e)
                    o.v[e] = 0.25f * (a.v[e] + bq.v[e] + c.v[e] + d.v[e]);
                store_stream<V>(dst + i * V, o);
            } else {
                Pack<V> g = load_stream<V>(src + i * V);
#pragma unroll
                for (int e = 0; e < V; ++e)
                    g.v[e] *= 0.25f;
                store_stream<V>(dst + big, g);
                store_stream<V>(dst + big + C, g);
                store_stream<V>(dst + big + rowstep, g);
                store_stream<V>(dst + big + rowstep + C, g);
            }
        } else if (MODE == 2) {
            const int Ho = 2 * H, Wo = 2 * W;
            const int ow = (int)(tmp % Wo); tmp /= Wo;
            const int oh = (int)(tmp % Ho); tmp /= Ho;
            const long b = tmp;
            store_stream<V>(dst + i * V, load_cached<V>(src + ((b * H + oh / 2) * W + ow / 2) * C + (long)cv * V));
        } else {
            const int iw = (int)(tmp % W); tmp /= W;
            const int ih = (int)(tmp % H); tmp /= H;
            const long b = tmp;
            const int Wo = 2 * W;
            const long big = ((b * 2 * H + 2 * ih) * Wo + 2 * iw) * C + (long)cv * V;
            const long rowstep = (long)Wo * C;
            const Pack<V> a = load_stream<V>(src + big), bq = load_stream<V>(src + big + C);
            const Pack<V> c = load_stream<V>(src + big + rowstep), d = load_stream<V>(src + big + rowstep + C);
            Pack<V> o;
#pragma unroll
            for (int e = 0; e < V; ++e)
                o.v[e] = a.v[e] + bq.v[e] + c.v[e] + d.v[e];
            store_stream<V>(dst + i * V, o);
        }
    }
}

// [B,d1,d2,d3] -> [B,d2,d1,d3]
template <int V>
__global__ void __launch_bounds__(256) permute_0213_kernel(float* __restrict__ out, const float* __restrict__ in, int d1,
    int d2, int d3, long total)
{
    pdl_prologue();
    const int d3v = d3 / V;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        long tmp = i;
        const int j3 = (int)(tmp % d3v); tmp /= d3v;
        const int j2 = (int)(tmp % d2); tmp /= d2;
        const int j1 = (int)(tmp % d1); tmp /= d1;
        const long b = tmp;
        store_stream<V>(out + (((b * d2 + j2) * d1 + j1) * d3 + (long)j3 * V), load_stream<V>(in + i * V));
    }
}

// ---------------------------------------------------------------------------
// softmax rows (attention scores, S is small): one warp per row
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_softmax_kernel(float* out, const float* in, int N,
    int S)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5); row < N; row += (long)gridDim.x * 8) {
        const float* x = in + row * S;
        float* y = out + row * S;
        float m = -INFINITY;
        for (int j = lane; j < S; j += 32)
            m = fmaxf(m, x[j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float sum = 0.0f;
        for (int j = lane; j < S; j += 32) {
            const float e = expf(x[j] - m);
            y[j] = e;
            sum += e;
        }
        const float inv = 1.0f / warp_sum(sum);
        for (int j = lane; j < S; j += 32)
            y[j] *= inv;
    }
}

__global__ void __launch_bounds__(256) attn_softmax_backward_kernel(float* __restrict__ gi, const float* __restrict__ go,
    const float* __restrict__ p, int N, int S)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5); row < N; row += (long)gridDim.x * 8) {
        const float* g = go + row * S;
        const float* pr = p + row * S;
        float dot = 0.0f;
        for (int j = lane; j < S; j += 32)
            dot += g[j] * pr[j];
        dot = warp_sum(dot);
        for (int j = lane; j < S; j += 32)
            gi[row * S + j] = pr[j] * (g[j] - dot);
    }
}

// row-wise softmax cross-entropy: one warp per row
__global__ void __launch_bounds__(256) softmax_xent_kernel(float* __restrict__ grad, float* __restrict__ loss_row,
    const float* __restrict__ logits, const int* __restrict__ targets, int batch, int C)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5); row < batch; row += (long)gridDim.x * 8) {
        const float* z = logits + row * C;
        const int tg = targets[row];
        float m = -INFINITY;
        for (int j = lane; j < C; j += 32)
            m = fmaxf(m, z[j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float sum = 0.0f;
        for (int j = lane; j < C; j += 32)
            sum += expf(z[j] - m);
        sum = warp_sum(sum);
        if (lane == 0)
            loss_row[row] = (m + logf(sum)) - z[tg];
        const float inv = 1.0f / (float)batch;
        for (int j = lane; j < C; j += 32)
            grad[row * C + j] = (expf(z[j] - m) / sum - (j == tg ? 1.0f : 0.0f)) * inv;
    }
}

// ---------------------------------------------------------------------------
// strip reductions over the rows of a [rows, C] view, one output row per group
// of `rows_per_group` consecutive rows.  block = 32 columns x 8 row lanes,
// grid = (ceil(C/32), groups).
// MODE 0: out[g,c] = sum_r a[r,c]                       (spatial_reduce_sum, bias_grad)
// MODE 1: out[g,c] = sum_r a[r,c]*b[r,c]; also gin[r,c] = a[r,c]*(cond[g,c]+1)   (FiLM backward)
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256) strip_reduce_kernel(float* __restrict__ out, float* __restrict__ gin,
    const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ cond, int rows_per_group, int C,
    long total_rows)
{
    pdl_prologue();
    __shared__ float part[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const long r0 = (long)blockIdx.y * rows_per_group;
    if (r0 + rows_per_group > total_rows)  // ragged last group (bias_grad splits the rows evenly)
        rows_per_group = total_rows > r0 ? (int)(total_rows - r0) : 0;
    float acc = 0.0f;
    if (col < C) {
        const float mod = MODE == 1 ? cond[(size_t)blockIdx.y * C + col] + 1.0f : 0.0f;
        for (int r = threadIdx.y; r < rows_per_group; r += 8) {
            const size_t k = (size_t)(r0 + r) * C + col;
            const float av = a[k];
            if (MODE == 1) {
                acc += av * b[k];
                gin[k] = av * mod;
            } else {
                acc += av;
            }
        }
    }
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && col < C) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            s += part[k][threadIdx.x];
        out[(size_t)blockIdx.y * C + col] = s;
    }
}

// MSE head: one CTA per sample.  loss_row[b] = mean_i d^2, grad = 2 d / (batch*dim)
__global__ void __launch_bounds__(256) mse_kernel(float* __restrict__ grad, float* __restrict__ loss_row,
    const float* __restrict__ pred, const float* __restrict__ target, int batch, int dim)
{
    pdl_prologue();
    __shared__ float buf[32];
    const size_t base = (size_t)blockIdx.x * dim;
    const float inv = 2.0f / (float)(batch * dim);
    float part = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = pred[base + i] - target[base + i];
        part += d * d;
        grad[base + i] = d * inv;
    }
    const float tot = cta_sum(part, buf);
    if (threadIdx.x == 0)
        loss_row[blockIdx.x] = tot / (float)dim;
}

template <int MODE>
static void resample_launch(float* dst, const float* src, int batch, int H, int W, int C, long small_or_big_elems,
    cudaStream_t s)
{
    const bool vec = C % 4 == 0 && aligned16(dst) && aligned16(src);
    if (vec) {
        const long total = small_or_big_elems / 4;
        launch_k(resample_kernel<MODE, 4>, flat_grid(total), 256, 0, s, dst, src, H, W, C, total);
    } else {
        launch_k(resample_kernel<MODE, 1>, flat_grid(small_or_big_elems), 256, 0, s, dst, src, H, W, C, small_or_big_elems);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

}  // namespace b200

using namespace b200;

extern "C" {

void launch_im2col(float* col, const float* im, int batch, int H, int W, int C, int K, int stride, int pad,
    int H_out, int W_out, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && K > 0 && stride > 0 && H_out > 0 && W_out > 0,
        "im2col: bad extents");
    const long n = (long)batch * H_out * W_out * K * K * C;
    if (n == 0)
        return;
    const long units = (long)batch * H_out * W_out * (C / 4);  // (pixel, channel pack) pairs
    if (C % 4 == 0 && aligned16(col) && aligned16(im) && units < 4294967296L && !tune_get("im2col_flat", 0)) {
        const float4* im4 = reinterpret_cast<const float4*>(im);
        float4* col4 = reinterpret_cast<float4*>(col);
        if (K == 3)
            launch_k(im2col_taps_kernel<3>, flat_grid(units), 256, 0, s, col4, im4, H, W, C / 4, K, stride, pad, H_out, W_out,
                (unsigned)units);
        else
            launch_k(im2col_taps_kernel<0>, flat_grid(units), 256, 0, s, col4, im4, H, W, C / 4, K, stride, pad, H_out, W_out,
                (unsigned)units);
    } else if (C % 4 == 0 && aligned16(col) && aligned16(im))
        launch_k(im2col_kernel<4>, flat_grid(n / 4), 256, 0, s, col, im, H, W, C, K, stride, pad, H_out, W_out, n / 4);
    else
        launch_k(im2col_kernel<1>, flat_grid(n), 256, 0, s, col, im, H, W, C, K, stride, pad, H_out, W_out, n);
    count_launch();
    B200_CHECK_LAUNCH();
}

static bool col2im_fast(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K, int stride, int pad,
    int H_out, int W_out, bool assign, cudaStream_t s)
{
    const long n = (long)batch * H * W * C;
    if (!(C % 4 == 0 && stride == 1 && aligned16(grad_im) && aligned16(grad_col) && n / 4 < 4294967296L
            && (long)batch * H_out * W_out * K * K * (C / 4) < 4294967296L && !tune_get("col2im_flat", 0)))
        return false;
    float4* gi4 = reinterpret_cast<float4*>(grad_im);
    const float4* gc4 = reinterpret_cast<const float4*>(grad_col);
    const int grid = flat_grid(n / 4);
    const unsigned total = (unsigned)(n / 4);
    if (K == 3 && assign)
        launch_k(col2im_taps_kernel<3, true>, grid, 256, 0, s, gi4, gc4, H, W, C / 4, K, pad, H_out, W_out, total);
    else if (K == 3)
        launch_k(col2im_taps_kernel<3, false>, grid, 256, 0, s, gi4, gc4, H, W, C / 4, K, pad, H_out, W_out, total);
    else if (assign)
        launch_k(col2im_taps_kernel<0, true>, grid, 256, 0, s, gi4, gc4, H, W, C / 4, K, pad, H_out, W_out, total);
    else
        launch_k(col2im_taps_kernel<0, false>, grid, 256, 0, s, gi4, gc4, H, W, C / 4, K, pad, H_out, W_out, total);
    count_launch();
    B200_CHECK_LAUNCH();
    return true;
}

void launch_col2im(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K, int stride,
    int pad, int H_out, int W_out, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && K > 0 && stride > 0 && H_out > 0 && W_out > 0,
        "col2im: bad extents");
    const long n = (long)batch * H * W * C;
    if (n == 0)
        return;
    if (col2im_fast(grad_im, grad_col, batch, H, W, C, K, stride, pad, H_out, W_out, false, s))
        return;
    if (C % 4 == 0 && aligned16(grad_im) && aligned16(grad_col))
        launch_k(col2im_gather_kernel<4>, flat_grid(n / 4), 256, 0, s, grad_im, grad_col, H, W, C, K, stride, pad, H_out,
            W_out, n / 4);
    else
        launch_k(col2im_gather_kernel<1>, flat_grid(n), 256, 0, s, grad_im, grad_col, H, W, C, K, stride, pad, H_out, W_out,
            n);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_col2im_assign(float* grad_im, const float* grad_col, int batch, int H, int W, int C, int K, int stride,
    int pad, int H_out, int W_out, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && K > 0 && stride > 0 && H_out > 0 && W_out > 0,
        "col2im_assign: bad extents");
    const long n = (long)batch * H * W * C;
    if (n == 0)
        return;
    if (col2im_fast(grad_im, grad_col, batch, H, W, C, K, stride, pad, H_out, W_out, true, s))
        return;
    // shapes outside the fast path: clear, then accumulate as launch_col2im does
    B200_CUDA_OK(cudaMemsetAsync(grad_im, 0, (size_t)n * sizeof(float), s));
    launch_col2im(grad_im, grad_col, batch, H, W, C, K, stride, pad, H_out, W_out, s);
}

void launch_avg_pool_2x(float* out, const float* in, int batch, int H, int W, int C, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 1 && W > 1 && C > 0, "avg_pool_2x: bad extents");
    const long n = (long)batch * (H / 2) * (W / 2) * C;
    if (n > 0)
        resample_launch<0>(out, in, batch, H, W, C, n, s);
}

void launch_avg_pool_2x_backward(float* grad_in, const float* grad_out, int batch, int H, int W, int C,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 1 && W > 1 && C > 0, "avg_pool_2x_backward: bad extents");
    const long n = (long)batch * (H / 2) * (W / 2) * C;
    if (n > 0)
        resample_launch<1>(grad_in, grad_out, batch, H, W, C, n, s);
}

void launch_nearest_upsample_2x(float* out, const float* in, int batch, int H, int W, int C, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0, "nearest_upsample_2x: bad extents");
    const long n = (long)batch * 4 * H * W * C;
    if (n > 0)
        resample_launch<2>(out, in, batch, H, W, C, n, s);
}

void launch_nearest_upsample_2x_backward(float* grad_in, const float* grad_out, int batch, int H, int W, int C,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0, "nearest_upsample_2x_backward: bad extents");
    const long n = (long)batch * H * W * C;
    if (n > 0)
        resample_launch<3>(grad_in, grad_out, batch, H, W, C, n, s);
}

void launch_attn_softmax(float* out, const float* in, int N, int S, cudaStream_t s)
{
    B200_REQUIRE(N >= 0 && S > 0, "attn_softmax: N=%d S=%d", N, S);
    if (N == 0)
        return;
    launch_k(attn_softmax_kernel, flat_grid((long)N, 8), 256, 0, s, out, in, N, S);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_attn_softmax_backward(float* grad_in, const float* grad_out, const float* p, int N, int S,
    cudaStream_t s)
{
    B200_REQUIRE(N >= 0 && S > 0, "attn_softmax_backward: N=%d S=%d", N, S);
    if (N == 0)
        return;
    launch_k(attn_softmax_backward_kernel, flat_grid((long)N, 8), 256, 0, s, grad_in, grad_out, p, N, S);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_permute_0213(float* out, const float* in, int B, int d1, int d2, int d3, cudaStream_t s)
{
    B200_REQUIRE(B >= 0 && d1 > 0 && d2 > 0 && d3 > 0, "permute_0213: bad extents");
    const long n = (long)B * d1 * d2 * d3;
    if (n == 0)
        return;
    if (d3 % 4 == 0 && aligned16(out) && aligned16(in))
        launch_k(permute_0213_kernel<4>, flat_grid(n / 4), 256, 0, s, out, in, d1, d2, d3, n / 4);
    else
        launch_k(permute_0213_kernel<1>, flat_grid(n), 256, 0, s, out, in, d1, d2, d3, n);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_spatial_modulate_backward(float* grad_in, float* grad_cond, const float* grad_out, const float* in,
    const float* cond, int batch, int H, int W, int C, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && batch <= 65535 && H > 0 && W > 0 && C > 0, "spatial_modulate_backward: bad extents");
    if (batch == 0)
        return;
    launch_k(strip_reduce_kernel<1>, dim3((C + 31) / 32, batch), dim3(32, 8), 0, s, grad_cond, grad_in, grad_out, in, cond,
        H * W, C, (long)batch * H * W);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_spatial_reduce_sum(float* out, const float* in, int batch, int HW, int C, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && batch <= 65535 && HW > 0 && C > 0, "spatial_reduce_sum: bad extents");
    if (batch == 0)
        return;
    launch_k(strip_reduce_kernel<0>, dim3((C + 31) / 32, batch), dim3(32, 8), 0, s, out, nullptr, in, nullptr, nullptr, HW,
        C, (long)batch * HW);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_bias_grad(float* gb, const float* grad_out, int batch, int N, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && N > 0, "bias_grad: batch=%d N=%d", batch, N);
    // Column sums of a [batch, N] matrix (reference: one thread per column walking every row,
    // src/kernels.cu:148-161).  The rows are split over enough CTAs to fill the chip; each writes one
    // partial row and a fixed-order fold adds them, so the result does not depend on scheduling.
    const int col_ctas = (N + 31) / 32;
    long want = ((long)sm_count() * 4 + col_ctas - 1) / col_ctas;  // row groups for ~4 CTAs per SM
    const long most = ((long)batch + 63) / 64;                      // at least 64 rows per group
    if (want > most)
        want = most;
    if (want <= 1) {
        launch_k(strip_reduce_kernel<0>, dim3(col_ctas, 1), dim3(32, 8), 0, s, gb, nullptr, grad_out, nullptr, nullptr, batch,
            N, (long)batch);
        count_launch();
        B200_CHECK_LAUNCH();
        return;
    }
    const int groups = (int)want;
    const int per = (batch + groups - 1) / groups;
    Scratch sc;
    B200_REQUIRE(scratch_get(s, (size_t)groups * N, 0, &sc), "bias_grad: scratch allocation failed (the arena cannot grow during stream capture: call b200_scratch_reserve before capturing)");
    launch_k(strip_reduce_kernel<0>, dim3(col_ctas, groups), dim3(32, 8), 0, s, sc.partials, nullptr, grad_out, nullptr,
        nullptr, per, N, (long)batch);
    count_launch();
    B200_CHECK_LAUNCH();
    fold_partials(gb, gb, sc.partials, groups, N, N, s);
}

void launch_mse_fwd_bwd(float* grad, float* loss_row, const float* pred, const float* target, int batch, int dim,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && dim > 0, "mse_fwd_bwd: batch=%d dim=%d", batch, dim);
    if (batch == 0)
        return;
    launch_k(mse_kernel, batch, 256, 0, s, grad, loss_row, pred, target, batch, dim);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_softmax_xent(float* grad_logits, float* loss_row, const float* logits, const int* targets, int batch,
    int C, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0, "softmax_xent: batch=%d C=%d", batch, C);
    if (batch == 0)
        return;
    launch_k(softmax_xent_kernel, flat_grid((long)batch, 8), 256, 0, s, grad_logits, loss_row, logits, targets, batch, C);
    count_launch();
    B200_CHECK_LAUNCH();
}

}  // extern "C"
