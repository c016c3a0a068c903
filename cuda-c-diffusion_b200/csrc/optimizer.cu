// Adam and the fused Adam + EMA parameter update (reference: src/kernels.cu:170-183
// called once per tensor by optimizer.c:65-68, followed by ema.c:29-35 which
// re-reads every parameter through launch_weighted_sum).
//
// The fused pass reads p, m, v, g, shadow and writes p, m, v, shadow once:
// 36 B/param instead of 28 + 12.  It is HBM-bound with nine streams, so it uses
// 128-bit streaming accesses with U packs in flight per thread.  The multi-tensor
// form takes a table of tensors in the kernel arguments and maps CTAs to
// tensors by a prefix sum, so a whole ParamList (58 tensors in the EDM UNet,
// half of them single floats) is ONE launch.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

namespace b200 {

constexpr int OPT_THREADS = 256;

struct AdamHyper {
    float lr, b1, b2, eps, inv_bc1, bc2, decay, grad_scale;
    float one_minus_b1, one_minus_b2, one_minus_decay;
};

// One element.  Same operation order as the reference kernel:
//   m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;  p -= lr*(m/bc1)/(sqrt(v/bc2)+eps)
// with correctly rounded division and square root.
template <bool EMA>
__device__ __forceinline__ void adam_one(float& p, float& m, float& v, float& sh, float g, const AdamHyper& h, float bc1)
{
    g *= h.grad_scale;
    m = h.b1 * m + h.one_minus_b1 * g;
    v = h.b2 * v + h.one_minus_b2 * g * g;
    p -= h.lr * (m / bc1) / (sqrtf(v / h.bc2) + h.eps);
    if (EMA)
        sh = h.decay * sh + h.one_minus_decay * p;
}

template <int W, bool EMA>
__device__ __forceinline__ void adam_span(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
    float* __restrict__ sh, const float* __restrict__ g, long n, const AdamHyper& h, float bc1, long first_pack,
    long pack_stride)
{
    constexpr int U = (W == 4) ? 2 : 4;
    const long npack = n / W;
    for (long i = first_pack; i < npack; i += pack_stride * U) {
        Pack<W> rp[U], rm[U], rv[U], rg[U], rs[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + u * pack_stride;
            if (k < npack) {
                rp[u] = load_stream<W>(p + k * W);
                rm[u] = load_stream<W>(m + k * W);
                rv[u] = load_stream<W>(v + k * W);
                rg[u] = load_stream<W>(g + k * W);
                if (EMA)
                    rs[u] = load_stream<W>(sh + k * W);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + u * pack_stride;
            if (k < npack) {
#pragma unroll
                for (int e = 0; e < W; ++e)
                    adam_one<EMA>(rp[u].v[e], rm[u].v[e], rv[u].v[e], rs[u].v[e], rg[u].v[e], h, bc1);
                store_stream<W>(p + k * W, rp[u]);
                store_stream<W>(m + k * W, rm[u]);
                store_stream<W>(v + k * W, rv[u]);
                if (EMA)
                    store_stream<W>(sh + k * W, rs[u]);
            }
        }
    }
}

template <int W, bool EMA>
__global__ void __launch_bounds__(OPT_THREADS) adam_flat_kernel(float* p, float* m, float* v, float* sh,
    const float* g, long n, const AdamHyper h, const float bc1)
{
    pdl_prologue();
    const long first = (long)blockIdx.x * OPT_THREADS + threadIdx.x;
    const long stride = (long)gridDim.x * OPT_THREADS;
    adam_span<W, EMA>(p, m, v, sh, g, n, h, bc1, first, stride);
    if (W > 1) {
        const long tail = (n / W) * W + first;
        if (tail < n) {
            float dummy = 0.0f;
            adam_one<EMA>(p[tail], m[tail], v[tail], EMA ? sh[tail] : dummy, g[tail], h, bc1);
        }
    }
}

// Fused update of a parameter range whose new values also go to `np` peer copies of the vector.
// W = 4 only: the sharded optimizer cuts ranges on 16-byte boundaries.
struct PeerTable {
    float* dst[B200_MAX_PEERS];
    int count;
};

template <bool EMA>
__global__ void __launch_bounds__(OPT_THREADS) adam_bcast_kernel(float* __restrict__ p, float* __restrict__ m,
    float* __restrict__ v, float* __restrict__ sh, const float* __restrict__ g, const PeerTable peers, long n,
    const AdamHyper h, const float bc1)
{
    pdl_prologue();
    constexpr int U = 2;
    const long npack = n / 4;
    const long stride = (long)gridDim.x * OPT_THREADS;
    for (long i = (long)blockIdx.x * OPT_THREADS + threadIdx.x; i < npack; i += stride * U) {
        Pack<4> rp[U], rm[U], rv[U], rg[U], rs[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + u * stride;
            if (k < npack) {
                rp[u] = load_stream<4>(p + k * 4);
                rm[u] = load_stream<4>(m + k * 4);
                rv[u] = load_stream<4>(v + k * 4);
                rg[u] = load_stream<4>(g + k * 4);
                if (EMA)
                    rs[u] = load_stream<4>(sh + k * 4);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long k = i + u * stride;
            if (k < npack) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    adam_one<EMA>(rp[u].v[e], rm[u].v[e], rv[u].v[e], rs[u].v[e], rg[u].v[e], h, bc1);
                const float4 np4 = make_float4(rp[u].v[0], rp[u].v[1], rp[u].v[2], rp[u].v[3]);
                // the peers first: their stores take the longest to drain
                for (int d = 0; d < peers.count; ++d)
                    *reinterpret_cast<float4*>(peers.dst[d] + k * 4) = np4;
                store_stream<4>(p + k * 4, rp[u]);
                store_stream<4>(m + k * 4, rm[u]);
                store_stream<4>(v + k * 4, rv[u]);
                if (EMA)
                    store_stream<4>(sh + k * 4, rs[u]);
            }
        }
    }
}

struct CopyTable {
    float* dst[B200_MAX_MULTI];
    const float* src[B200_MAX_MULTI];
    int n[B200_MAX_MULTI];
    int block0[B200_MAX_MULTI + 1];
    int count;
};

__global__ void __launch_bounds__(OPT_THREADS) copy_multi_kernel(const CopyTable tb)
{
    pdl_prologue();
    int lo = 0, hi = tb.count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tb.block0[mid] <= (int)blockIdx.x)
            lo = mid;
        else
            hi = mid - 1;
    }
    float* dst = tb.dst[lo];
    const float* src = tb.src[lo];
    const int n = tb.n[lo];
    const int first = (blockIdx.x - tb.block0[lo]) * OPT_THREADS + threadIdx.x;
    const int stride = (tb.block0[lo + 1] - tb.block0[lo]) * OPT_THREADS;
    if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
        const int n4 = n / 4;
        for (int i = first; i < n4; i += stride)
            reinterpret_cast<float4*>(dst)[i] = __ldg(reinterpret_cast<const float4*>(src) + i);
        for (int i = n4 * 4 + first; i < n; i += stride)
            dst[i] = src[i];
    } else {
        for (int i = first; i < n; i += stride)
            dst[i] = src[i];
    }
}

struct AdamTable {
    float* p[B200_MAX_MULTI];
    const float* g[B200_MAX_MULTI];
    float* m[B200_MAX_MULTI];
    float* v[B200_MAX_MULTI];
    float* sh[B200_MAX_MULTI];
    int n[B200_MAX_MULTI];
    int block0[B200_MAX_MULTI + 1];  // prefix sum of CTAs per tensor
    int count;
};

constexpr int OPT_MULTI_ELEMS_PER_BLOCK = OPT_THREADS * 4 * 4;  // 4096 floats per CTA

__global__ void __launch_bounds__(OPT_THREADS) adam_multi_kernel(const AdamTable tb, const AdamHyper h, const float bc1)
{
    pdl_prologue();
    int lo = 0, hi = tb.count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tb.block0[mid] <= (int)blockIdx.x)
            lo = mid;
        else
            hi = mid - 1;
    }
    const int local_block = blockIdx.x - tb.block0[lo];
    const int nblocks = tb.block0[lo + 1] - tb.block0[lo];
    float* p = tb.p[lo];
    float* m = tb.m[lo];
    float* v = tb.v[lo];
    float* sh = tb.sh[lo];
    const float* g = tb.g[lo];
    const long n = tb.n[lo];
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)
                          | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(sh))
                         & 15u)
        == 0;
    const long first = (long)local_block * OPT_THREADS + threadIdx.x;
    const long stride = (long)nblocks * OPT_THREADS;
    if (vec) {
        if (sh)
            adam_span<4, true>(p, m, v, sh, g, n, h, bc1, first, stride);
        else
            adam_span<4, false>(p, m, v, sh, g, n, h, bc1, first, stride);
        const long tail = (n / 4) * 4 + first;
        if (tail < n) {
            float dummy = 0.0f;
            if (sh)
                adam_one<true>(p[tail], m[tail], v[tail], sh[tail], g[tail], h, bc1);
            else
                adam_one<false>(p[tail], m[tail], v[tail], dummy, g[tail], h, bc1);
        }
    } else {
        if (sh)
            adam_span<1, true>(p, m, v, sh, g, n, h, bc1, first, stride);
        else
            adam_span<1, false>(p, m, v, sh, g, n, h, bc1, first, stride);
    }
}

static AdamHyper make_hyper(float lr, float b1, float b2, float eps, float bc1, float bc2, float decay, float gs)
{
    AdamHyper h;
    h.lr = lr; h.b1 = b1; h.b2 = b2; h.eps = eps; h.inv_bc1 = 1.0f / bc1; h.bc2 = bc2;
    h.decay = decay; h.grad_scale = gs;
    h.one_minus_b1 = 1.0f - b1;
    h.one_minus_b2 = 1.0f - b2;
    h.one_minus_decay = 1.0f - decay;
    return h;
}

static void adam_flat(float* p, float* m, float* v, float* sh, const float* g, long n, const AdamHyper& h,
    float bc1, cudaStream_t s)
{
    if (n <= 0)
        return;
    const bool vec = aligned16(p) && aligned16(m) && aligned16(v) && aligned16(g) && (sh == nullptr || aligned16(sh));
    const long npack = vec ? n / 4 : n;
    const long per_block = (long)OPT_THREADS * (vec ? 2 : 4);
    long grid = (npack + per_block - 1) / per_block;
    const long cap = (long)sm_count() * tune_get("adam_blocks_per_sm", 16);
    if (grid > cap)
        grid = cap;
    if (grid < 1)
        grid = 1;
    if (vec) {
        if (sh)
            launch_k(adam_flat_kernel<4, true>, (int)grid, OPT_THREADS, 0, s, p, m, v, sh, g, n, h, bc1);
        else
            launch_k(adam_flat_kernel<4, false>, (int)grid, OPT_THREADS, 0, s, p, m, v, sh, g, n, h, bc1);
    } else {
        if (sh)
            launch_k(adam_flat_kernel<1, true>, (int)grid, OPT_THREADS, 0, s, p, m, v, sh, g, n, h, bc1);
        else
            launch_k(adam_flat_kernel<1, false>, (int)grid, OPT_THREADS, 0, s, p, m, v, sh, g, n, h, bc1);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

}  // namespace b200

using namespace b200;

extern "C" {

void launch_adam_step(float* p, float* m, float* v, const float* g, float lr, float beta1, float beta2,
    float eps, float bc1, float bc2, int n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "adam_step: n=%d", n);
    adam_flat(p, m, v, nullptr, g, n, make_hyper(lr, beta1, beta2, eps, bc1, bc2, 0.0f, 1.0f), bc1, s);
}

void launch_adam_ema_step(float* p, float* m, float* v, float* shadow, const float* g, float lr, float beta1,
    float beta2, float eps, float bc1, float bc2, float decay, float grad_scale, long long n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0, "adam_ema_step: n=%lld", n);
    adam_flat(p, m, v, shadow, g, (long)n, make_hyper(lr, beta1, beta2, eps, bc1, bc2, decay, grad_scale), bc1, s);
}

void launch_adam_ema_step_bcast(float* p, float* m, float* v, float* shadow, const float* g,
    const B200PeerDests* peers, float lr, float beta1, float beta2, float eps, float bc1, float bc2, float decay,
    float grad_scale, long long n, cudaStream_t s)
{
    B200_REQUIRE(n >= 0 && n % 4 == 0, "adam_ema_step_bcast: n=%lld must be a multiple of 4", n);
    B200_REQUIRE(peers && peers->count >= 0 && peers->count <= B200_MAX_PEERS, "adam_ema_step_bcast: bad peer table");
    bool ok = aligned16(p) && aligned16(m) && aligned16(v) && aligned16(g) && (shadow == nullptr || aligned16(shadow));
    PeerTable tb;
    tb.count = peers->count;
    for (int d = 0; d < peers->count; ++d) {
        tb.dst[d] = peers->dst[d];
        ok = ok && peers->dst[d] != nullptr && aligned16(peers->dst[d]);
    }
    B200_REQUIRE(ok, "adam_ema_step_bcast: every pointer must be 16-byte aligned (and no destination NULL)");
    if (n == 0)
        return;
    const AdamHyper h = make_hyper(lr, beta1, beta2, eps, bc1, bc2, decay, grad_scale);
    long grid = (n / 4 + OPT_THREADS * 2 - 1) / (OPT_THREADS * 2);
    const long cap = (long)sm_count() * tune_get("adam_blocks_per_sm", 16);
    if (grid > cap)
        grid = cap;
    if (shadow)
        launch_k(adam_bcast_kernel<true>, (int)grid, OPT_THREADS, 0, s, p, m, v, shadow, g, tb, (long)n, h, bc1);
    else
        launch_k(adam_bcast_kernel<false>, (int)grid, OPT_THREADS, 0, s, p, m, v, shadow, g, tb, (long)n, h, bc1);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_copy_multi(const B200CopyItem* items, int count, cudaStream_t s)
{
    B200_REQUIRE(count >= 0 && (count == 0 || items), "copy_multi: count=%d", count);
    const int per_tensor_cap = sm_count() * 4;
    int i = 0;
    while (i < count) {
        CopyTable tb;
        tb.count = 0;
        tb.block0[0] = 0;
        while (i < count && tb.count < B200_MAX_MULTI) {
            const B200CopyItem& it = items[i++];
            B200_REQUIRE(it.n >= 0, "copy_multi: item %d has n=%d", i - 1, it.n);
            if (it.n == 0)
                continue;
            const int k = tb.count++;
            tb.dst[k] = it.dst; tb.src[k] = it.src; tb.n[k] = it.n;
            int nb = (it.n + OPT_MULTI_ELEMS_PER_BLOCK - 1) / OPT_MULTI_ELEMS_PER_BLOCK;
            if (nb > per_tensor_cap)
                nb = per_tensor_cap;
            tb.block0[k + 1] = tb.block0[k] + nb;
        }
        if (tb.count == 0)
            break;
        launch_k(copy_multi_kernel, tb.block0[tb.count], OPT_THREADS, 0, s, tb);
        count_launch();
        B200_CHECK_LAUNCH();
    }
}

void launch_adam_ema_step_multi(const B200ParamUpdate* items, int count, float lr, float beta1, float beta2,
    float eps, float bc1, float bc2, float decay, float grad_scale, cudaStream_t s)
{
    B200_REQUIRE(count >= 0 && (count == 0 || items), "adam_ema_step_multi: count=%d", count);
    const AdamHyper h = make_hyper(lr, beta1, beta2, eps, bc1, bc2, decay, grad_scale);
    const int per_tensor_cap = sm_count() * 8;
    int i = 0;
    while (i < count) {
        AdamTable tb;
        tb.count = 0;
        tb.block0[0] = 0;
        while (i < count && tb.count < B200_MAX_MULTI) {
            const B200ParamUpdate& it = items[i++];
            B200_REQUIRE(it.n >= 0, "adam_ema_step_multi: item %d has n=%d", i - 1, it.n);
            if (it.n == 0)
                continue;
            const int k = tb.count++;
            tb.p[k] = it.p; tb.g[k] = it.g; tb.m[k] = it.m; tb.v[k] = it.v; tb.sh[k] = it.shadow;
            tb.n[k] = it.n;
            int nb = (it.n + OPT_MULTI_ELEMS_PER_BLOCK - 1) / OPT_MULTI_ELEMS_PER_BLOCK;
            if (nb > per_tensor_cap)
                nb = per_tensor_cap;
            tb.block0[k + 1] = tb.block0[k] + nb;
        }
        if (tb.count == 0)
            break;
        launch_k(adam_multi_kernel, tb.block0[tb.count], OPT_THREADS, 0, s, tb, h, bc1);
        count_launch();
        B200_CHECK_LAUNCH();
    }
}

}  // extern "C"
