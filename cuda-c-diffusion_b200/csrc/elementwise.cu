// Streaming element-wise kernels: activations, weighted sums (mp_sum, EMA,
// residual adds), scale, scaled channel concat / split, per-row axpby, FiLM
// forward, bias adds, clamp, SGD.
//
// All of them are HBM-bound (1-3 tensors in, 1-2 out, a handful of flops per
// element), so the whole design is about bytes in flight: 128-bit accesses,
// U independent packs per thread issued before any is consumed, streaming
// cache policy, and a grid sized as a multiple of the SM count.  Operands whose
// pointers are not 16-byte aligned take the same kernel with 32-bit accesses.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

#include <math.h>

namespace b200 {

constexpr int EW_THREADS = 256;

// Generic driver.  Op provides
//   template<int W> struct Regs;                      registers for one pack
//   template<int W> void load(long e, Regs<W>&) const  e = float offset of the pack
//   template<int W> void store(long e, const Regs<W>&) const
// The first (n/W) packs go through the W-wide path; the n%W left-over floats
// are handled with W=1 by the first threads of block 0.
template <int W, int U, class Op>
__global__ void __launch_bounds__(EW_THREADS) ew_kernel(const Op op, const long n)
{
    pdl_prologue();
    const long npack = n / W;
    const long stride = (long)gridDim.x * (EW_THREADS * U);
    for (long i = (long)blockIdx.x * (EW_THREADS * U) + threadIdx.x; i < npack; i += stride) {
        typename Op::template Regs<W> r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + (long)u * EW_THREADS;
            if (k < npack)
                op.template load<W>(k * W, r[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + (long)u * EW_THREADS;
            if (k < npack)
                op.template store<W>(k * W, r[u]);
        }
    }
    if constexpr (W > 1) {
        const long tail0 = npack * W;
        if (blockIdx.x == 0 && tail0 + threadIdx.x < n) {
            typename Op::template Regs<1> r;
            op.template load<1>(tail0 + threadIdx.x, r);
            op.template store<1>(tail0 + threadIdx.x, r);
        }
    }
}

static inline int ew_grid(long npack, int U)
{
    const long per_block = (long)EW_THREADS * U;
    long want = (npack + per_block - 1) / per_block;
    const long cap = (long)sm_count() * tune_get("ew_blocks_per_sm", 16);
    if (want > cap)
        want = cap;
    return want < 1 ? 1 : (int)want;
}

template <class Op>
static void ew_launch(const Op& op, long n, bool vec_ok, cudaStream_t s)
{
    if (n <= 0)
        return;
    const int U = tune_get("ew_unroll", 4);
    if (vec_ok) {
        const long npack = n / 4;
        if (U >= 8)
            launch_k(ew_kernel<4, 8, Op>, ew_grid(npack, 8), EW_THREADS, 0, s, op, n);
        else if (U >= 4)
            launch_k(ew_kernel<4, 4, Op>, ew_grid(npack, 4), EW_THREADS, 0, s, op, n);
        else
            launch_k(ew_kernel<4, 2, Op>, ew_grid(npack, 2), EW_THREADS, 0, s, op, n);
    } else {
        launch_k(ew_kernel<1, 4, Op>, ew_grid(n, 4), EW_THREADS, 0, s, op, n);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

// ---------------------------------------------------------------------------
// ops
// ---------------------------------------------------------------------------
template <int ACT>
struct ActFwdOp {
    float* out;
    const float* in;
    template <int W> struct Regs { Pack<W> x; };
    template <int W> __device__ void load(long e, Regs<W>& r) const { r.x = load_stream<W>(in + e); }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = act_value<ACT>(r.x.v[k]);
        store_stream<W>(out + e, y);
    }
};

template <int ACT>
struct ActBwdOp {
    float* gin;
    const float* gout;
    const float* in;
    template <int W> struct Regs { Pack<W> g, x; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.g = load_stream<W>(gout + e);
        r.x = load_stream<W>(in + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.g.v[k] * act_slope<ACT>(r.x.v[k]);
        store_stream<W>(gin + e, y);
    }
};

// out = wa*a + wb*b.  Every pack is read completely before the same pack is
// written by the same thread, so out may alias a and/or b.
struct AxpbyOp {
    float* out;
    const float* a;
    const float* b;
    float wa, wb;
    template <int W> struct Regs { Pack<W> a, b; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.a = load_stream<W>(a + e);
        r.b = load_stream<W>(b + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = wa * r.a.v[k] + wb * r.b.v[k];
        store_stream<W>(out + e, y);
    }
};

// out = wa*a + wb*a read once (a aliases b: diffusion/edm.c:57 style calls)
struct ScaleCopyOp {
    float* out;
    const float* a;
    float wa, wb;
    template <int W> struct Regs { Pack<W> a; };
    template <int W> __device__ void load(long e, Regs<W>& r) const { r.a = load_stream<W>(a + e); }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = wa * r.a.v[k] + wb * r.a.v[k];
        store_stream<W>(out + e, y);
    }
};

// ga = wa*g, gb = wb*g
struct FanOutOp {
    float* ga;
    float* gb;
    const float* g;
    float wa, wb;
    template <int W> struct Regs { Pack<W> g; };
    template <int W> __device__ void load(long e, Regs<W>& r) const { r.g = load_stream<W>(g + e); }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> ya, yb;
#pragma unroll
        for (int k = 0; k < W; ++k) {
            ya.v[k] = wa * r.g.v[k];
            yb.v[k] = wb * r.g.v[k];
        }
        store_stream<W>(ga + e, ya);
        store_stream<W>(gb + e, yb);
    }
};

// x *= s[0]
struct ScaleByDeviceScalarOp {
    float* x;
    const float* s;
    template <int W> struct Regs { Pack<W> x; float f; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.x = load_stream<W>(x + e);
        r.f = __ldg(s);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.x.v[k] * r.f;
        store_stream<W>(x + e, y);
    }
};

struct ClampOp {
    float* x;
    float lo, hi;
    template <int W> struct Regs { Pack<W> x; };
    template <int W> __device__ void load(long e, Regs<W>& r) const { r.x = load_stream<W>(x + e); }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = fminf(fmaxf(r.x.v[k], lo), hi);
        store_stream<W>(x + e, y);
    }
};

struct SgdOp {
    float* p;
    const float* g;
    float lr;
    template <int W> struct Regs { Pack<W> p, g; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.p = load_stream<W>(p + e);
        r.g = load_stream<W>(g + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.p.v[k] - lr * r.g.v[k];
        store_stream<W>(p + e, y);
    }
};

// h2 = h1*(c+1)
struct ModulateOp {
    float* h2;
    const float* h1;
    const float* c;
    template <int W> struct Regs { Pack<W> h, c; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.h = load_stream<W>(h1 + e);
        r.c = load_stream<W>(c + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.h.v[k] * (r.c.v[k] + 1.0f);
        store_stream<W>(h2 + e, y);
    }
};

// gh1 = g*(c+1), gc = g*h1
struct ModulateBwdOp {
    float* gh1;
    float* gc;
    const float* gh2;
    const float* h1;
    const float* c;
    template <int W> struct Regs { Pack<W> g, h, c; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.g = load_stream<W>(gh2 + e);
        r.h = load_stream<W>(h1 + e);
        r.c = load_stream<W>(c + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> a, b;
#pragma unroll
        for (int k = 0; k < W; ++k) {
            a.v[k] = r.g.v[k] * (r.c.v[k] + 1.0f);
            b.v[k] = r.g.v[k] * r.h.v[k];
        }
        store_stream<W>(gh1 + e, a);
        store_stream<W>(gc + e, b);
    }
};

// --- ops with a (row, channel) structure --------------------------------------
// The W=4 path is only taken when every row length involved is a multiple of 4,
// so a pack never straddles a row or the a|b seam.  Offsets fit in 32 bits
// because the C ABI carries extents as int.

// out[r, 0:Na] = wa*a[r,:], out[r, Na:Na+Nb] = wb*b[r,:]
struct CatOp {
    float* out;
    const float* a;
    const float* b;
    float wa, wb;
    unsigned Na, Nb;
    template <int W> struct Regs { Pack<W> x; float w; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        const unsigned N = Na + Nb;
        const unsigned row = (unsigned)e / N, col = (unsigned)e - row * N;
        if (col < Na) {
            r.x = load_stream<W>(a + (size_t)row * Na + col);
            r.w = wa;
        } else {
            r.x = load_stream<W>(b + (size_t)row * Nb + (col - Na));
            r.w = wb;
        }
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.w * r.x.v[k];
        store_stream<W>(out + e, y);
    }
};

// ga[r,:] = wa*g[r, 0:Ca], gb[r,:] = wb*g[r, Ca:Ca+Cb]
struct SplitOp {
    float* ga;
    float* gb;
    const float* g;
    float wa, wb;
    unsigned Ca, Cb;
    template <int W> struct Regs { Pack<W> x; };
    template <int W> __device__ void load(long e, Regs<W>& r) const { r.x = load_stream<W>(g + e); }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        const unsigned N = Ca + Cb;
        const unsigned row = (unsigned)e / N, col = (unsigned)e - row * N;
        Pack<W> y;
        const float w = col < Ca ? wa : wb;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = w * r.x.v[k];
        if (col < Ca)
            store_stream<W>(ga + (size_t)row * Ca + col, y);
        else
            store_stream<W>(gb + (size_t)row * Cb + (col - Ca), y);
    }
};

// MODE 0: x[m, n] += v[n]               (bias over rows; period = N)
// MODE 1: x[b, hw, c] += v[b, c]        (per-sample bias; inner = HW*C, C)
// MODE 2: out = in * (v[b, c] + 1)      (FiLM forward / backward-in)
template <int MODE>
struct BroadcastOp {
    float* out;
    const float* in;
    const float* v;
    unsigned C, HWC;
    template <int W> struct Regs { Pack<W> x, s; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.x = load_stream<W>(in + e);
        unsigned c = (unsigned)e % C;
        if constexpr (MODE == 0) {
            r.s = load_cached<W>(v + c);
        } else {
            unsigned b = (unsigned)e / HWC;
            r.s = load_cached<W>(v + (size_t)b * C + c);
        }
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = (MODE == 2) ? r.x.v[k] * (r.s.v[k] + 1.0f) : r.x.v[k] + r.s.v[k];
        store_stream<W>(out + e, y);
    }
};

// out = act(in * (v[b, c] + 1)): FiLM modulation followed by the activation (cond_conv_residual.c:31-33)
template <int ACT>
struct FilmActOp {
    float* out;
    const float* in;
    const float* v;
    unsigned C, HWC;
    template <int W> struct Regs { Pack<W> x, s; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.x = load_stream<W>(in + e);
        const unsigned c = (unsigned)e % C, b = (unsigned)e / HWC;
        r.s = load_cached<W>(v + (size_t)b * C + c);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = act_value<ACT>(r.x.v[k] * (r.s.v[k] + 1.0f));
        store_stream<W>(out + e, y);
    }
};

// out = w * skip + gz * act'(z): activation backward joined with the skip branch of mp_sum's backward
// (cond_conv_residual.c:54, :61)
template <int ACT>
struct ActBwdAxpyOp {
    float* out;
    const float* gz;
    const float* z;
    const float* skip;
    float w;
    template <int W> struct Regs { Pack<W> g, z, k; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        r.g = load_stream<W>(gz + e);
        r.z = load_stream<W>(z + e);
        r.k = load_stream<W>(skip + e);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = fmaf(w, r.k.v[k], r.g.v[k] * act_slope<ACT>(r.z.v[k]));
        store_stream<W>(out + e, y);
    }
};

// FiLM + activation backward.  z = in*(cond+1); g = grad_out*act'(z); grad_in = g*(cond+1);
// grad_cond[b,c] = sum_hw g*in.  block = 32 columns x 8 row lanes, grid = (ceil(C/32), batch, row splits);
// with row splits > 1 the per-split sums go to `partial[split][b][c]` and a second tiny kernel adds them.
template <int ACT>
__global__ void __launch_bounds__(256) film_act_backward_kernel(float* __restrict__ grad_in, float* __restrict__ sums,
    const float* __restrict__ grad_out, const float* __restrict__ in, const float* __restrict__ cond, int HW, int C,
    int rows_per_split)
{
    pdl_prologue();
    __shared__ float part[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int b = blockIdx.y;
    const int r_lo = blockIdx.z * rows_per_split, r_hi = min(HW, r_lo + rows_per_split);
    float acc = 0.0f;
    if (col < C) {
        const float m = cond[(size_t)b * C + col] + 1.0f;
        const size_t base = (size_t)b * HW * C + col;
        for (int r = r_lo + threadIdx.y; r < r_hi; r += 8) {
            const size_t k = base + (size_t)r * C;
            const float x = in[k];
            const float g = grad_out[k] * act_slope<ACT>(x * m);
            acc = fmaf(g, x, acc);
            grad_in[k] = g * m;
        }
    }
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && col < C) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            t += part[k][threadIdx.x];
        sums[((size_t)blockIdx.z * gridDim.y + b) * C + col] = t;
    }
}

__global__ void film_fold_splits_kernel(float* __restrict__ out, const float* __restrict__ partial, int n, int splits)
{
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float t = 0.0f;
        for (int s = 0; s < splits; ++s)
            t += partial[(size_t)s * n + i];
        out[i] = t;
    }
}

// out[r,:] = wa[r]*a[r,:] + wb[r]*b[r,:]
struct AxpbyRowsOp {
    float* out;
    const float* a;
    const float* b;
    const float* wa;
    const float* wb;
    unsigned dim;
    template <int W> struct Regs { Pack<W> a, b; float wa, wb; };
    template <int W> __device__ void load(long e, Regs<W>& r) const
    {
        const unsigned row = (unsigned)e / dim;
        r.a = load_stream<W>(a + e);
        r.b = load_stream<W>(b + e);
        r.wa = __ldg(wa + row);
        r.wb = __ldg(wb + row);
    }
    template <int W> __device__ void store(long e, const Regs<W>& r) const
    {
        Pack<W> y;
#pragma unroll
        for (int k = 0; k < W; ++k)
            y.v[k] = r.wa * r.a.v[k] + r.wb * r.b.v[k];
        store_stream<W>(out + e, y);
    }
};

template <template <int> class OpT, class... Args>
static bool dispatch_act(int act, long n, bool vec, cudaStream_t s, Args... args)
{
    switch (act) {
    case ACT_IDENTITY: ew_launch(OpT<ACT_IDENTITY>{ args... }, n, vec, s); return true;
    case ACT_RELU: ew_launch(OpT<ACT_RELU>{ args... }, n, vec, s); return true;
    case ACT_GELU: ew_launch(OpT<ACT_GELU>{ args... }, n, vec, s); return true;
    case ACT_SILU: ew_launch(OpT<ACT_SILU>{ args... }, n, vec, s); return true;
    case ACT_TANH: ew_launch(OpT<ACT_TANH>{ args... }, n, vec, s); return true;
    case ACT_MP_SILU: ew_launch(OpT<ACT_MP_SILU>{ args... }, n, vec, s); return true;
    default: return false;
    }
}

static void mp_cat_weights(float t, int Na, int Nb, float* wa, float* wb)
{
    // same expression order as the reference host code (kernels.cu:371-374)
    const float denom = (1.0f - t) * (1.0f - t) + t * t;
    const float c = sqrtf((float)(Na + Nb) / denom);
    *wa = c / sqrtf((float)Na) * (1.0f - t);
    *wb = c / sqrtf((float)Nb) * t;
}

static void cat_launch(float* out, const float* a, const float* b, float wa, float wb, long rows, int Na,
    int Nb, cudaStream_t s)
{
    B200_REQUIRE(rows >= 0 && Na > 0 && Nb > 0, "concat: bad extents rows=%ld Na=%d Nb=%d", rows, Na, Nb);
    B200_REQUIRE(rows * ((long)Na + Nb) < 2147483648L, "concat: more than 2^31-1 elements");
    const bool vec = Na % 4 == 0 && Nb % 4 == 0 && aligned16(out) && aligned16(a) && aligned16(b);
    ew_launch(CatOp{ out, a, b, wa, wb, (unsigned)Na, (unsigned)Nb }, rows * ((long)Na + Nb), vec, s);
}

static void split_launch(float* ga, float* gb, const float* g, float wa, float wb, long rows, int Ca, int Cb,
    cudaStream_t s)
{
    B200_REQUIRE(rows >= 0 && Ca > 0 && Cb > 0, "split: bad extents rows=%ld Ca=%d Cb=%d", rows, Ca, Cb);
    B200_REQUIRE(rows * ((long)Ca + Cb) < 2147483648L, "split: more than 2^31-1 elements");
    const bool vec = Ca % 4 == 0 && Cb % 4 == 0 && aligned16(ga) && aligned16(gb) && aligned16(g);
    ew_launch(SplitOp{ ga, gb, g, wa, wb, (unsigned)Ca, (unsigned)Cb }, rows * ((long)Ca + Cb), vec, s);
}

template <int ACT>
static void film_act_backward_launch(float* grad_in, float* grad_cond, const float* grad_out, const float* in,
    const float* cond, int batch, int HW, int C, cudaStream_t s)
{
    // enough CTAs to fill the GPU: split the rows of a sample when (C/32)*batch alone is too few
    const int base_ctas = ((C + 31) / 32) * batch;
    int splits = 1;
    while (splits < 16 && base_ctas * splits < 4 * sm_count() && HW / (splits * 2) >= 64)
        splits *= 2;
    const int rows_per_split = (HW + splits - 1) / splits;
    float* sums = grad_cond;
    if (splits > 1) {
        Scratch sc;
        if (!scratch_get(s, (size_t)splits * batch * C, 0, &sc)) {
            report_error(__FILE__, __LINE__, "film_act_backward: no scratch memory");
            return;
        }
        sums = sc.partials;
    }
    launch_k(film_act_backward_kernel<ACT>, dim3((C + 31) / 32, batch, splits), dim3(32, 8), 0, s, grad_in, sums, grad_out, in,
        cond, HW, C, rows_per_split);
    count_launch();
    B200_CHECK_LAUNCH();
    if (splits > 1) {
        const int n = batch * C;
        launch_k(film_fold_splits_kernel, (n + 255) / 256, 256, 0, s, grad_cond, sums, n, splits);
        count_launch();
        B200_CHECK_LAUNCH();
    }
}

}  // namespace b200

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using namespace b200;

extern "C" {

void launch_activation_forward(float* out, const float* in, int n, b200_act_t act, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "activation_forward: n=%d", n);
    const bool vec = aligned16(out) && aligned16(in);
    const bool ok = dispatch_act<ActFwdOp>((int)act, n, vec, s, out, in);
    B200_REQUIRE(ok, "activation_forward: unknown activation %d", (int)act);
}

void launch_activation_backward(float* grad_in, const float* grad_out, const float* in, int n,
    b200_act_t act, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "activation_backward: n=%d", n);
    const bool vec = aligned16(grad_in) && aligned16(grad_out) && aligned16(in);
    const bool ok = dispatch_act<ActBwdOp>((int)act, n, vec, s, grad_in, grad_out, in);
    B200_REQUIRE(ok, "activation_backward: unknown activation %d", (int)act);
}

void launch_weighted_sum(float* out, const float* a, const float* b, float wa, float wb, int n,
    cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "weighted_sum: n=%d", n);
    const bool vec = aligned16(out) && aligned16(a) && aligned16(b);
    if (a == b)
        ew_launch(ScaleCopyOp{ out, a, wa, wb }, n, vec, s);
    else
        ew_launch(AxpbyOp{ out, a, b, wa, wb }, n, vec, s);
}

void launch_mp_sum(float* out, const float* a, const float* b, float t, int n, cudaStream_t s)
{
    const float d = sqrtf((1.0f - t) * (1.0f - t) + t * t);
    launch_weighted_sum(out, a, b, (1.0f - t) / d, t / d, n, s);
}

void launch_mp_sum_backward(float* ga, float* gb, const float* g, float t, int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "mp_sum_backward: n=%d", n);
    const float d = sqrtf((1.0f - t) * (1.0f - t) + t * t);
    const bool vec = aligned16(ga) && aligned16(gb) && aligned16(g);
    ew_launch(FanOutOp{ ga, gb, g, (1.0f - t) / d, t / d }, n, vec, s);
}

void launch_scale_by_scalar(float* x, const float* sc, int n, cudaStream_t st)
{
    B200_REQUIRE(n >= 0, "scale_by_scalar: n=%d", n);
    ew_launch(ScaleByDeviceScalarOp{ x, sc }, n, aligned16(x), st);
}

void launch_clamp(float* x, float lo, float hi, int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "clamp: n=%d", n);
    ew_launch(ClampOp{ x, lo, hi }, n, aligned16(x), s);
}

void launch_sgd_step(float* p, const float* g, float lr, int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "sgd_step: n=%d", n);
    ew_launch(SgdOp{ p, g, lr }, n, aligned16(p) && aligned16(g), s);
}

void launch_modulate(float* h2, const float* h1, const float* c, int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "modulate: n=%d", n);
    ew_launch(ModulateOp{ h2, h1, c }, n, aligned16(h2) && aligned16(h1) && aligned16(c), s);
}

void launch_modulate_backward(float* gh1, float* gc, const float* gh2, const float* h1, const float* c,
    int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "modulate_backward: n=%d", n);
    const bool vec = aligned16(gh1) && aligned16(gc) && aligned16(gh2) && aligned16(h1) && aligned16(c);
    ew_launch(ModulateBwdOp{ gh1, gc, gh2, h1, c }, n, vec, s);
}

void launch_mp_cat(float* out, const float* a, const float* b, float t, int batch, int Na, int Nb,
    cudaStream_t s)
{
    float wa, wb;
    mp_cat_weights(t, Na, Nb, &wa, &wb);
    cat_launch(out, a, b, wa, wb, batch, Na, Nb, s);
}

void launch_mp_channel_cat(float* out, const float* a, const float* b, float t, int spatial, int Ca,
    int Cb, cudaStream_t s)
{
    float wa, wb;
    mp_cat_weights(t, Ca, Cb, &wa, &wb);
    cat_launch(out, a, b, wa, wb, spatial, Ca, Cb, s);
}

void launch_channel_cat(float* out, const float* a, const float* b, int spatial, int Ca, int Cb,
    cudaStream_t s)
{
    cat_launch(out, a, b, 1.0f, 1.0f, spatial, Ca, Cb, s);
}

void launch_mp_channel_split(float* grad_a, float* grad_b, const float* grad_out, float t,
    int spatial, int Ca, int Cb, cudaStream_t s)
{
    float wa, wb;
    mp_cat_weights(t, Ca, Cb, &wa, &wb);
    split_launch(grad_a, grad_b, grad_out, wa, wb, spatial, Ca, Cb, s);
}

void launch_channel_split(float* grad_a, float* grad_b, const float* grad_out, int spatial, int Ca,
    int Cb, cudaStream_t s)
{
    split_launch(grad_a, grad_b, grad_out, 1.0f, 1.0f, spatial, Ca, Cb, s);
}

void launch_add_bias(float* Y, const float* b, int M, int N, cudaStream_t s)
{
    B200_REQUIRE(M >= 0 && N > 0 && (long)M * N < 2147483648L, "add_bias: M=%d N=%d", M, N);
    const bool vec = N % 4 == 0 && aligned16(Y) && aligned16(b);
    ew_launch(BroadcastOp<0>{ Y, Y, b, (unsigned)N, (unsigned)N }, (long)M * N, vec, s);
}

void launch_spatial_add(float* inout, const float* bias, int batch, int H, int W, int C, cudaStream_t s)
{
    const long n = (long)batch * H * W * C;
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && n < 2147483648L, "spatial_add: bad extents");
    const bool vec = C % 4 == 0 && aligned16(inout) && aligned16(bias);
    ew_launch(BroadcastOp<1>{ inout, inout, bias, (unsigned)C, (unsigned)(H * W * C) }, n, vec, s);
}

void launch_spatial_modulate(float* out, const float* in, const float* cond, int batch, int H, int W,
    int C, cudaStream_t s)
{
    const long n = (long)batch * H * W * C;
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && n < 2147483648L, "spatial_modulate: bad extents");
    const bool vec = C % 4 == 0 && aligned16(out) && aligned16(in) && aligned16(cond);
    ew_launch(BroadcastOp<2>{ out, in, cond, (unsigned)C, (unsigned)(H * W * C) }, n, vec, s);
}

void launch_film_act_forward(float* out, const float* in, const float* cond, int batch, int H, int W, int C,
    b200_act_t act, cudaStream_t s)
{
    const long n = (long)batch * H * W * C;
    B200_REQUIRE(batch >= 0 && H > 0 && W > 0 && C > 0 && n < 2147483648L, "film_act_forward: bad extents");
    const bool vec = C % 4 == 0 && aligned16(out) && aligned16(in) && aligned16(cond);
    const bool ok = dispatch_act<FilmActOp>((int)act, n, vec, s, out, in, cond, (unsigned)C, (unsigned)(H * W * C));
    B200_REQUIRE(ok, "film_act_forward: unknown activation %d", (int)act);
}

void launch_film_act_backward(float* grad_in, float* grad_cond, const float* grad_out, const float* in,
    const float* cond, int batch, int H, int W, int C, b200_act_t act, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && batch <= 65535 && H > 0 && W > 0 && C > 0, "film_act_backward: bad extents");
    if (batch == 0)
        return;
    switch ((int)act) {
    case ACT_IDENTITY: film_act_backward_launch<ACT_IDENTITY>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    case ACT_RELU: film_act_backward_launch<ACT_RELU>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    case ACT_GELU: film_act_backward_launch<ACT_GELU>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    case ACT_SILU: film_act_backward_launch<ACT_SILU>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    case ACT_TANH: film_act_backward_launch<ACT_TANH>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    case ACT_MP_SILU: film_act_backward_launch<ACT_MP_SILU>(grad_in, grad_cond, grad_out, in, cond, batch, H * W, C, s); break;
    default: report_error(__FILE__, __LINE__, "film_act_backward: unknown activation %d", (int)act);
    }
}

void launch_activation_backward_axpy(float* out, const float* grad_out, const float* in, const float* skip, float w_skip,
    int n, b200_act_t act, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "activation_backward_axpy: n=%d", n);
    const bool vec = aligned16(out) && aligned16(grad_out) && aligned16(in) && aligned16(skip);
    const bool ok = dispatch_act<ActBwdAxpyOp>((int)act, n, vec, s, out, grad_out, in, skip, w_skip);
    B200_REQUIRE(ok, "activation_backward_axpy: unknown activation %d", (int)act);
}

void launch_axpby_rows(float* out, const float* a, const float* b, const float* wa, const float* wb,
    int rows, int dim, cudaStream_t s)
{
    const long n = (long)rows * dim;
    B200_REQUIRE(rows >= 0 && dim > 0 && n < 2147483648L, "axpby_rows: rows=%d dim=%d", rows, dim);
    const bool vec = dim % 4 == 0 && aligned16(out) && aligned16(a) && aligned16(b);
    ew_launch(AxpbyRowsOp{ out, a, b, wa, wb, (unsigned)dim }, n, vec, s);
}

}  // extern "C"
