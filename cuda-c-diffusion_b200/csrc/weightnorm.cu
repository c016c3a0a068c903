// Forced weight normalisation of W[in, out] (row-major): every output column is
// scaled to unit L2 norm in place, and the matching backward
// (reference: src/kernels.cu:255-297, launchers :330-344).
//
// The matrices are small (<= ~600 KB), so the op is latency-bound: what counts is
// how few dependent memory round trips a launch needs and how many matrices one
// launch covers.  Cluster kernel: a cluster of CS CTAs splits the `in` rows of a
// 32-column strip; each thread keeps its <= 12 float4 of the strip in registers
// (single read of W), column sums of squares are folded in shared memory and
// then across the cluster through distributed shared memory, and the scaled
// values are written straight from registers.  A table of matrices lets one
// launch normalise every MP weight of a model, forward and backward; hosts whose
// modules call the per-weight launchers can have those calls recorded once and
// then batched (b200_wn_batch_mode).
// Shapes outside the cluster kernel's limits (out % 4 != 0, in > 3072,
// misaligned) use the strip kernel (two sweeps, any shape).
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

#include <cooperative_groups.h>
#include <mutex>
#include <vector>

namespace cg = cooperative_groups;

namespace b200 {

constexpr int WN_THREADS = 256;
constexpr int WN_COLS = 32;       // columns per strip
constexpr int WN_VMAX = 12;       // float4 per thread -> at most 384 rows per CTA
constexpr int WN_MAX_ROWS = 3072; // 8 CTAs x 384 rows (3x3 convolutions of 256 input channels: 2304)

struct WnTable {
    float* W[B200_MAX_MULTI];
    int in[B200_MAX_MULTI];
    int out[B200_MAX_MULTI];
    int strip0[B200_MAX_MULTI + 1];  // prefix sum of strips per matrix
    int count;
};

__device__ __forceinline__ int wn_find(const WnTable& tb, int strip)
{
    int lo = 0, hi = tb.count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tb.strip0[mid] <= strip)
            lo = mid;
        else
            hi = mid - 1;
    }
    return lo;
}

// Folds a float4 per thread over the 32 row lanes; returns for threads t < 32 the
// total of column t of the strip (other threads get garbage).
__device__ __forceinline__ float wn_fold_lanes(float (*fold)[WN_COLS + 1], int qc, int rl, float4 v)
{
    fold[rl][4 * qc + 0] = v.x;
    fold[rl][4 * qc + 1] = v.y;
    fold[rl][4 * qc + 2] = v.z;
    fold[rl][4 * qc + 3] = v.w;
    __syncthreads();
    float s = 0.0f;
    if (threadIdx.x < WN_COLS) {
#pragma unroll 8
        for (int r = 0; r < 32; ++r)
            s += fold[r][threadIdx.x];
    }
    __syncthreads();
    return s;
}

// grid = (CS, total strips), cluster = (CS,1,1), block = 256 = 8 float4 columns x 32 row lanes
__global__ void __launch_bounds__(WN_THREADS) wn_forward_cluster(const WnTable tb, const float eps)
{
    pdl_prologue();
    __shared__ float fold[32][WN_COLS + 1];
    __shared__ float colsum[WN_COLS];  // read by cluster peers
    __shared__ float colinv[WN_COLS];
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = gridDim.x, rank = blockIdx.x;
    const int m = wn_find(tb, blockIdx.y);
    const int in = tb.in[m], out = tb.out[m];
    float* W = tb.W[m];
    const int col0 = (blockIdx.y - tb.strip0[m]) * WN_COLS;
    const int qc = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int col = col0 + 4 * qc;
    const int rows_per = (in + CS - 1) / CS;
    const int r0 = rank * rows_per;
    const int r1 = min(in, r0 + rows_per);
    const bool col_ok = col < out;

    float4 w[WN_VMAX];
    float4 ss = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        const int r = r0 + rl + 32 * j;
        w[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col_ok && r < r1)
            w[j] = *reinterpret_cast<const float4*>(W + (size_t)r * out + col);
    }
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        ss.x += w[j].x * w[j].x;
        ss.y += w[j].y * w[j].y;
        ss.z += w[j].z * w[j].z;
        ss.w += w[j].w * w[j].w;
    }
    const float mine = wn_fold_lanes(fold, qc, rl, ss);
    if (threadIdx.x < WN_COLS)
        colsum[threadIdx.x] = mine;
    cluster.sync();
    if (threadIdx.x < WN_COLS) {
        float tot = 0.0f;
        for (int k = 0; k < CS; ++k)
            tot += cluster.map_shared_rank(colsum, k)[threadIdx.x];
        colinv[threadIdx.x] = rsqrtf(tot + eps);
    }
    __syncthreads();
    const float i0 = colinv[4 * qc], i1 = colinv[4 * qc + 1], i2 = colinv[4 * qc + 2], i3 = colinv[4 * qc + 3];
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        const int r = r0 + rl + 32 * j;
        if (col_ok && r < r1)
            *reinterpret_cast<float4*>(W + (size_t)r * out + col)
                = make_float4(w[j].x * i0, w[j].y * i1, w[j].z * i2, w[j].w * i3);
    }
    cluster.sync();
}

struct WnGradTable {
    float* gW[B200_MAX_MULTI];
    const float* Wn[B200_MAX_MULTI];
    const float* gain[B200_MAX_MULTI];
    float* g_gain[B200_MAX_MULTI];
    int in[B200_MAX_MULTI];
    int out[B200_MAX_MULTI];
    int strip0[B200_MAX_MULTI + 1];
    int count;
};

__device__ __forceinline__ int wn_find_grad(const WnGradTable& tb, int strip)
{
    int lo = 0, hi = tb.count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tb.strip0[mid] <= strip)
            lo = mid;
        else
            hi = mid - 1;
    }
    return lo;
}

// table of matrices; per matrix: gW <- gain * (gW - dot_j * Wn), *g_gain += sum_j dot_j
// grid = (CS, total strips), cluster = (CS,1,1)
__global__ void __launch_bounds__(WN_THREADS) wn_backward_cluster(const WnGradTable tb)
{
    pdl_prologue();
    __shared__ float fold[32][WN_COLS + 1];
    __shared__ float colsum[WN_COLS];
    __shared__ float coldot[WN_COLS];
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = gridDim.x, rank = blockIdx.x;
    const int m = wn_find_grad(tb, blockIdx.y);
    const int in = tb.in[m], out = tb.out[m];
    float* __restrict__ gW = tb.gW[m];
    const float* __restrict__ Wn = tb.Wn[m];
    const int col0 = (blockIdx.y - tb.strip0[m]) * WN_COLS;
    const int qc = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int col = col0 + 4 * qc;
    const int rows_per = (in + CS - 1) / CS;
    const int r0 = rank * rows_per;
    const int r1 = min(in, r0 + rows_per);
    const bool col_ok = col < out;

    float4 w[WN_VMAX], gw[WN_VMAX];
    float4 dot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        const int r = r0 + rl + 32 * j;
        w[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        gw[j] = w[j];
        if (col_ok && r < r1) {
            w[j] = *reinterpret_cast<const float4*>(Wn + (size_t)r * out + col);
            gw[j] = *reinterpret_cast<const float4*>(gW + (size_t)r * out + col);
        }
    }
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        dot.x += w[j].x * gw[j].x;
        dot.y += w[j].y * gw[j].y;
        dot.z += w[j].z * gw[j].z;
        dot.w += w[j].w * gw[j].w;
    }
    const float mine = wn_fold_lanes(fold, qc, rl, dot);
    if (threadIdx.x < WN_COLS)
        colsum[threadIdx.x] = mine;
    cluster.sync();
    if (threadIdx.x < WN_COLS) {
        float tot = 0.0f;
        for (int k = 0; k < CS; ++k)
            tot += cluster.map_shared_rank(colsum, k)[threadIdx.x];
        coldot[threadIdx.x] = tot;
        // one atomic per strip: rank 0 adds the strip's 32 column dots
        if (rank == 0) {
            const float strip = warp_sum((col0 + (int)threadIdx.x < out) ? tot : 0.0f);
            if (threadIdx.x == 0)
                atomicAdd(tb.g_gain[m], strip);
        }
    }
    __syncthreads();
    const float gn = __ldg(tb.gain[m]);
    const float d0 = coldot[4 * qc], d1 = coldot[4 * qc + 1], d2 = coldot[4 * qc + 2], d3 = coldot[4 * qc + 3];
#pragma unroll
    for (int j = 0; j < WN_VMAX; ++j) {
        const int r = r0 + rl + 32 * j;
        if (col_ok && r < r1)
            *reinterpret_cast<float4*>(gW + (size_t)r * out + col) = make_float4(gn * (gw[j].x - d0 * w[j].x),
                gn * (gw[j].y - d1 * w[j].y), gn * (gw[j].z - d2 * w[j].z), gn * (gw[j].w - d3 * w[j].w));
    }
    cluster.sync();
}

// Narrow matrices (a handful of output columns, e.g. the last convolution of a UNet with one image channel):
// one CTA per column, its 256 threads stride over the rows.  The strip kernel below would leave 8 threads of one
// CTA walking the whole column twice (24 us for [576, 1]).
// MODE 0: forward.  MODE 1: backward.
template <int MODE>
__global__ void __launch_bounds__(256) wn_column(float* __restrict__ A, const float* __restrict__ Wn,
    const float* __restrict__ gain, float* __restrict__ g_gain, int in, int out, float eps)
{
    pdl_prologue();
    __shared__ float buf[32];
    const int col = blockIdx.x;
    float acc = 0.0f;
    for (int r = threadIdx.x; r < in; r += 256) {
        const float a = A[(size_t)r * out + col];
        acc += MODE == 0 ? a * a : a * Wn[(size_t)r * out + col];
    }
    const float tot = cta_sum(acc, buf);
    if (MODE == 1 && threadIdx.x == 0)
        atomicAdd(g_gain, tot);
    const float cv = MODE == 0 ? rsqrtf(tot + eps) : tot;
    const float gn = MODE == 1 ? gain[0] : 0.0f;
    for (int r = threadIdx.x; r < in; r += 256) {
        const size_t k = (size_t)r * out + col;
        A[k] = MODE == 0 ? A[k] * cv : gn * (A[k] - cv * Wn[k]);
    }
}

// Strip kernel for any shape: block = 32 columns x 8 row lanes, two sweeps.
// MODE 0: forward.  MODE 1: backward.
template <int MODE>
__global__ void __launch_bounds__(256) wn_strip(float* __restrict__ A, const float* __restrict__ Wn,
    const float* __restrict__ gain, float* __restrict__ g_gain, int in, int out, float eps)
{
    pdl_prologue();
    __shared__ float part[8][33];
    __shared__ float colv[32];
    const int col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.0f;
    if (col < out)
        for (int r = threadIdx.y; r < in; r += 8) {
            const float a = A[(size_t)r * out + col];
            acc += MODE == 0 ? a * a : a * Wn[(size_t)r * out + col];
        }
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            s += part[k][threadIdx.x];
        if (MODE == 0) {
            colv[threadIdx.x] = rsqrtf(s + eps);
        } else {
            colv[threadIdx.x] = s;
            const float strip = warp_sum(col < out ? s : 0.0f);
            if (threadIdx.x == 0)
                atomicAdd(g_gain, strip);
        }
    }
    __syncthreads();
    if (col < out) {
        const float cv = colv[threadIdx.x];
        const float gn = MODE == 1 ? gain[0] : 0.0f;
        for (int r = threadIdx.y; r < in; r += 8) {
            const size_t k = (size_t)r * out + col;
            A[k] = MODE == 0 ? A[k] * cv : gn * (A[k] - cv * Wn[k]);
        }
    }
}

static int wn_cluster_size(int in)
{
    int cs = 1;
    while (cs < 8 && cs * 64 < in)
        cs *= 2;
    while (cs < 8 && (in + cs - 1) / cs > 32 * WN_VMAX)
        cs *= 2;
    return cs;
}

static bool wn_cluster_ok(const void* p, int in, int out)
{
    return out % 4 == 0 && in <= WN_MAX_ROWS && aligned16(p);
}

static void wn_launch_cluster_fwd(const WnTable& tb, int cs, float eps, cudaStream_t s)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    cfg.gridDim = dim3((unsigned)cs, (unsigned)tb.strip0[tb.count], 1);
    cfg.blockDim = dim3(WN_THREADS, 1, 1);
    cfg.stream = s;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    unsigned nat = 1;
    pdl_attribute(attr, &nat, (long)cs * tb.strip0[tb.count] * WN_THREADS);
    cfg.attrs = attr;
    cfg.numAttrs = nat;
    cudaError_t e = cudaLaunchKernelEx(&cfg, wn_forward_cluster, tb, eps);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "weight_normalize launch failed: %s", cudaGetErrorString(e));
        return;
    }
    count_launch();
}

static void wn_launch_cluster_bwd(const WnGradTable& tb, int cs, cudaStream_t s)
{
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    cfg.gridDim = dim3((unsigned)cs, (unsigned)tb.strip0[tb.count], 1);
    cfg.blockDim = dim3(WN_THREADS, 1, 1);
    cfg.stream = s;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    unsigned nat = 1;
    pdl_attribute(attr, &nat, (long)cs * tb.strip0[tb.count] * WN_THREADS);
    cfg.attrs = attr;
    cfg.numAttrs = nat;
    cudaError_t e = cudaLaunchKernelEx(&cfg, wn_backward_cluster, tb);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "weight_normalize_backward launch failed: %s", cudaGetErrorString(e));
        return;
    }
    count_launch();
}

// --- batching session (b200_wn_batch_mode) -----------------------------------
struct WnSession {
    std::mutex mu;
    int mode = 0;
    float eps = 0.0f;
    std::vector<B200WeightDesc> fwd;       // recorded in mode 1, one entry per W
    std::vector<B200WeightGradDesc> bwd;   // queued in mode 2
};
static WnSession g_wn;

}  // namespace b200

using namespace b200;

extern "C" {

static void weight_normalize_now(float* W, int in, int out, float eps, cudaStream_t s);

void launch_weight_normalize(float* W, int in, int out, float eps, cudaStream_t s)
{
    B200_REQUIRE(in > 0 && out > 0, "weight_normalize: in=%d out=%d", in, out);
    {
        std::lock_guard<std::mutex> lk(g_wn.mu);
        if (g_wn.mode != 0) {
            bool seen = false;
            for (const B200WeightDesc& d : g_wn.fwd)
                seen = seen || d.W == W;
            // mode 2: the driver has normalised every RECORDED weight itself (b200_wn_forward_all).  A weight
            // that was never recorded (a layer first used after the recording pass, a second model in the
            // process) is normalised here and now, and joins the set for the following passes.
            if (seen && g_wn.mode == 2)
                return;
            if (!seen)
                g_wn.fwd.push_back(B200WeightDesc{ W, in, out });
            g_wn.eps = eps;
        }
    }
    weight_normalize_now(W, in, out, eps, s);
}

static void weight_normalize_now(float* W, int in, int out, float eps, cudaStream_t s)
{
    if (wn_cluster_ok(W, in, out) && !tune_get("wn_force_strip", 0)) {
        WnTable tb;
        tb.count = 1;
        tb.W[0] = W;
        tb.in[0] = in;
        tb.out[0] = out;
        tb.strip0[0] = 0;
        tb.strip0[1] = (out + WN_COLS - 1) / WN_COLS;
        wn_launch_cluster_fwd(tb, wn_cluster_size(in), eps, s);
        return;
    }
    if (out <= 8)
        launch_k(wn_column<0>, out, 256, 0, s, W, nullptr, nullptr, nullptr, in, out, eps);
    else
        launch_k(wn_strip<0>, (out + 31) / 32, dim3(32, 8), 0, s, W, nullptr, nullptr, nullptr, in, out, eps);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_weight_normalize_multi(const B200WeightDesc* items, int count, float eps, cudaStream_t s)
{
    B200_REQUIRE(count >= 0 && (count == 0 || items), "weight_normalize_multi: count=%d", count);
    WnTable tb;
    tb.count = 0;
    tb.strip0[0] = 0;
    for (int i = 0; i < count; ++i) {
        B200_REQUIRE(items[i].in > 0 && items[i].out > 0, "weight_normalize_multi: item %d in=%d out=%d", i,
            items[i].in, items[i].out);
        if (!wn_cluster_ok(items[i].W, items[i].in, items[i].out)) {
            weight_normalize_now(items[i].W, items[i].in, items[i].out, eps, s);
            continue;
        }
        const int k = tb.count++;
        tb.W[k] = items[i].W;
        tb.in[k] = items[i].in;
        tb.out[k] = items[i].out;
        tb.strip0[k + 1] = tb.strip0[k] + (items[i].out + WN_COLS - 1) / WN_COLS;
        if (tb.count == B200_MAX_MULTI) {
            wn_launch_cluster_fwd(tb, 8, eps, s);
            tb.count = 0;
        }
    }
    if (tb.count > 0)
        wn_launch_cluster_fwd(tb, 8, eps, s);
}

static void weight_normalize_backward_now(float* gW, const float* Wn, const float* gain, float* g_gain, int in, int out,
    cudaStream_t s)
{
    if (wn_cluster_ok(gW, in, out) && aligned16(Wn) && !tune_get("wn_force_strip", 0)) {
        WnGradTable tb;
        tb.count = 1;
        tb.gW[0] = gW;
        tb.Wn[0] = Wn;
        tb.gain[0] = gain;
        tb.g_gain[0] = g_gain;
        tb.in[0] = in;
        tb.out[0] = out;
        tb.strip0[0] = 0;
        tb.strip0[1] = (out + WN_COLS - 1) / WN_COLS;
        wn_launch_cluster_bwd(tb, wn_cluster_size(in), s);
        return;
    }
    if (out <= 8)
        launch_k(wn_column<1>, out, 256, 0, s, gW, Wn, gain, g_gain, in, out, 0.0f);
    else
        launch_k(wn_strip<1>, (out + 31) / 32, dim3(32, 8), 0, s, gW, Wn, gain, g_gain, in, out, 0.0f);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_weight_normalize_backward(float* gW, const float* Wn, const float* gain, float* g_gain, int in,
    int out, cudaStream_t s)
{
    B200_REQUIRE(in > 0 && out > 0, "weight_normalize_backward: in=%d out=%d", in, out);
    {
        std::lock_guard<std::mutex> lk(g_wn.mu);
        if (g_wn.mode == 2) {
            g_wn.bwd.push_back(B200WeightGradDesc{ gW, Wn, gain, g_gain, in, out });
            return;
        }
    }
    weight_normalize_backward_now(gW, Wn, gain, g_gain, in, out, s);
}

void launch_weight_normalize_backward_multi(const B200WeightGradDesc* items, int count, cudaStream_t s)
{
    B200_REQUIRE(count >= 0 && (count == 0 || items), "weight_normalize_backward_multi: count=%d", count);
    WnGradTable tb;
    tb.count = 0;
    tb.strip0[0] = 0;
    for (int i = 0; i < count; ++i) {
        const B200WeightGradDesc& d = items[i];
        B200_REQUIRE(d.in > 0 && d.out > 0, "weight_normalize_backward_multi: item %d in=%d out=%d", i, d.in, d.out);
        if (!(wn_cluster_ok(d.gW, d.in, d.out) && aligned16(d.Wn)) || tune_get("wn_force_strip", 0)) {
            weight_normalize_backward_now(d.gW, d.Wn, d.gain, d.g_gain, d.in, d.out, s);
            continue;
        }
        const int k = tb.count++;
        tb.gW[k] = d.gW;
        tb.Wn[k] = d.Wn;
        tb.gain[k] = d.gain;
        tb.g_gain[k] = d.g_gain;
        tb.in[k] = d.in;
        tb.out[k] = d.out;
        tb.strip0[k + 1] = tb.strip0[k] + (d.out + WN_COLS - 1) / WN_COLS;
        if (tb.count == B200_MAX_MULTI) {
            wn_launch_cluster_bwd(tb, 8, s);
            tb.count = 0;
        }
    }
    if (tb.count > 0)
        wn_launch_cluster_bwd(tb, 8, s);
}

void b200_wn_batch_mode(int mode)
{
    std::lock_guard<std::mutex> lk(g_wn.mu);
    if (mode == 1 && g_wn.mode != 1)
        g_wn.fwd.clear();
    if (mode != 2)
        g_wn.bwd.clear();
    g_wn.mode = mode < 0 || mode > 2 ? 0 : mode;
}

int b200_wn_forward_all(cudaStream_t s)
{
    std::vector<B200WeightDesc> items;
    float eps;
    {
        std::lock_guard<std::mutex> lk(g_wn.mu);
        items = g_wn.fwd;
        eps = g_wn.eps;
    }
    if (!items.empty())
        launch_weight_normalize_multi(items.data(), (int)items.size(), eps, s);
    return (int)items.size();
}

int b200_wn_backward_flush(cudaStream_t s)
{
    std::vector<B200WeightGradDesc> items;
    {
        std::lock_guard<std::mutex> lk(g_wn.mu);
        items.swap(g_wn.bwd);
    }
    if (!items.empty())
        launch_weight_normalize_backward_multi(items.data(), (int)items.size(), s);
    return (int)items.size();
}

}  // extern "C"
