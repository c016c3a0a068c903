// Row-wise normalisations over a contiguous channel axis: LayerNorm forward /
// backward (reference: src/kernels.cu:491-616) and pixel norm (no reference
// counterpart).
//
// Fast path (C a multiple of 128, C <= 1024, 16-byte aligned): one warp owns a
// whole row in registers -- C/128 float4 per lane -- so x (and dy) are read
// from HBM exactly once, the row statistics are pure warp shuffles, and a warp
// keeps R rows in flight.  In backward every lane also accumulates dgamma/dbeta
// for its own columns across all rows it visits; the CTA folds its warps
// together in shared memory and writes ONE partial row, and a small second
// kernel sums the partial rows in a fixed order (deterministic, overwrite
// semantics like the reference).
// Any other shape takes the generic kernels (one warp per row, strided loops).
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

namespace b200 {

constexpr int RN_THREADS = 256;
constexpr int RN_WARPS = RN_THREADS / 32;

// ---------------------------------------------------------------------------
// fast path
// ---------------------------------------------------------------------------
template <int VPT>
struct RowRegs {
    float4 v[VPT];
};

template <int VPT>
__device__ __forceinline__ void row_load(RowRegs<VPT>& r, const float* base, int lane)
{
#pragma unroll
    for (int j = 0; j < VPT; ++j)
        r.v[j] = __ldcs(reinterpret_cast<const float4*>(base) + lane + 32 * j);
}

template <int VPT>
__device__ __forceinline__ void row_store(float* base, const RowRegs<VPT>& r, int lane)
{
#pragma unroll
    for (int j = 0; j < VPT; ++j)
        __stcs(reinterpret_cast<float4*>(base) + lane + 32 * j, r.v[j]);
}

template <int VPT>
__device__ __forceinline__ void row_load_param(RowRegs<VPT>& r, const float* base, int lane)
{
#pragma unroll
    for (int j = 0; j < VPT; ++j)
        r.v[j] = __ldg(reinterpret_cast<const float4*>(base) + lane + 32 * j);
}

#define FOR_EACH_LANE_ELEM(j, VPT) _Pragma("unroll") for (int j = 0; j < VPT; ++j)

template <int VPT, int R>
__global__ void __launch_bounds__(RN_THREADS) layernorm_fwd_rows(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, long rows, float eps)
{
    pdl_prologue();
    constexpr int C = VPT * 128;
    const int lane = threadIdx.x & 31;
    const long warp0 = ((long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5)) * R;
    const long wstride = (long)gridDim.x * RN_WARPS * R;
    RowRegs<VPT> g, b;
    row_load_param<VPT>(g, gamma, lane);
    row_load_param<VPT>(b, beta, lane);
    const float invC = 1.0f / (float)C;

    for (long row = warp0; row < rows; row += wstride) {
        RowRegs<VPT> xr[R];
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (row + k < rows)
                row_load<VPT>(xr[k], x + (row + k) * C, lane);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (row + k >= rows)
                break;
            float s = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT) s += (xr[k].v[j].x + xr[k].v[j].y) + (xr[k].v[j].z + xr[k].v[j].w);
            const float m = warp_sum(s) * invC;
            float vs = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                const float d0 = xr[k].v[j].x - m, d1 = xr[k].v[j].y - m, d2 = xr[k].v[j].z - m, d3 = xr[k].v[j].w - m;
                vs += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
            }
            const float rs = rsqrtf(warp_sum(vs) * invC + eps);
            if (lane == 0) {
                mu[row + k] = m;
                rstd[row + k] = rs;
            }
            RowRegs<VPT> o;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                o.v[j].x = g.v[j].x * ((xr[k].v[j].x - m) * rs) + b.v[j].x;
                o.v[j].y = g.v[j].y * ((xr[k].v[j].y - m) * rs) + b.v[j].y;
                o.v[j].z = g.v[j].z * ((xr[k].v[j].z - m) * rs) + b.v[j].z;
                o.v[j].w = g.v[j].w * ((xr[k].v[j].w - m) * rs) + b.v[j].w;
            }
            row_store<VPT>(y + (row + k) * C, o, lane);
        }
    }
}

// dx per row; per-CTA partial sums of dgamma/dbeta go to partials[blockIdx][2*C]
// (first C: dgamma, next C: dbeta).
template <int VPT, int R>
__global__ void __launch_bounds__(RN_THREADS) layernorm_bwd_rows(float* __restrict__ dx, float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ mu, const float* __restrict__ rstd, long rows)
{
    pdl_prologue();
    constexpr int C = VPT * 128;
    __shared__ float fold[2 * C];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long warp0 = ((long)blockIdx.x * RN_WARPS + warp) * R;
    const long wstride = (long)gridDim.x * RN_WARPS * R;
    RowRegs<VPT> g, dg, db;
    row_load_param<VPT>(g, gamma, lane);
    FOR_EACH_LANE_ELEM(j, VPT)
    {
        dg.v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        db.v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float invC = 1.0f / (float)C;

    for (long row = warp0; row < rows; row += wstride) {
        RowRegs<VPT> xr[R], gr[R];
        float m[R], rs[R];
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (row + k < rows) {
                row_load<VPT>(xr[k], x + (row + k) * C, lane);
                row_load<VPT>(gr[k], dy + (row + k) * C, lane);
                m[k] = __ldg(mu + row + k);
                rs[k] = __ldg(rstd + row + k);
            }
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (row + k >= rows)
                break;
            float pg = 0.0f, pgx = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                // x-hat replaces x in registers, g*gamma is recomputed below
                float4& xv = xr[k].v[j];
                const float4 dv = gr[k].v[j];
                xv.x = (xv.x - m[k]) * rs[k];
                xv.y = (xv.y - m[k]) * rs[k];
                xv.z = (xv.z - m[k]) * rs[k];
                xv.w = (xv.w - m[k]) * rs[k];
                const float g0 = dv.x * g.v[j].x, g1 = dv.y * g.v[j].y, g2 = dv.z * g.v[j].z, g3 = dv.w * g.v[j].w;
                pg += (g0 + g1) + (g2 + g3);
                pgx += (g0 * xv.x + g1 * xv.y) + (g2 * xv.z + g3 * xv.w);
                dg.v[j].x += dv.x * xv.x;
                dg.v[j].y += dv.y * xv.y;
                dg.v[j].z += dv.z * xv.z;
                dg.v[j].w += dv.w * xv.w;
                db.v[j].x += dv.x;
                db.v[j].y += dv.y;
                db.v[j].z += dv.z;
                db.v[j].w += dv.w;
            }
            const float sg = warp_sum(pg) * invC, sgx = warp_sum(pgx) * invC;
            RowRegs<VPT> o;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                const float4 xv = xr[k].v[j], dv = gr[k].v[j];
                o.v[j].x = rs[k] * (dv.x * g.v[j].x - sg - xv.x * sgx);
                o.v[j].y = rs[k] * (dv.y * g.v[j].y - sg - xv.y * sgx);
                o.v[j].z = rs[k] * (dv.z * g.v[j].z - sg - xv.z * sgx);
                o.v[j].w = rs[k] * (dv.w * g.v[j].w - sg - xv.w * sgx);
            }
            row_store<VPT>(dx + (row + k) * C, o, lane);
        }
    }

    // fold the warps of this CTA in a fixed order (warp 0 first)
    for (int w = 0; w < RN_WARPS; ++w) {
        if (warp == w) {
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                float4* pg4 = reinterpret_cast<float4*>(fold) + lane + 32 * j;
                float4* pb4 = reinterpret_cast<float4*>(fold + C) + lane + 32 * j;
                if (w == 0) {
                    *pg4 = dg.v[j];
                    *pb4 = db.v[j];
                } else {
                    float4 a = *pg4, b = *pb4;
                    a.x += dg.v[j].x; a.y += dg.v[j].y; a.z += dg.v[j].z; a.w += dg.v[j].w;
                    b.x += db.v[j].x; b.y += db.v[j].y; b.z += db.v[j].z; b.w += db.v[j].w;
                    *pg4 = a;
                    *pb4 = b;
                }
            }
        }
        __syncthreads();
    }
    float* dst = partials + (size_t)blockIdx.x * (2 * C);
    for (int i = threadIdx.x; i < 2 * C; i += RN_THREADS)
        dst[i] = fold[i];
}

// out[c] = sum_p partials[p][c] for c in [0, width); fixed summation order.
// grid = ceil(width/32), block = 32 x 32: threadIdx.x -> column, threadIdx.y -> row lane.
__global__ void __launch_bounds__(1024) fold_partials_kernel(float* __restrict__ out_a, float* __restrict__ out_b,
    const float* __restrict__ partials, int nparts, int width, int split)
{
    pdl_prologue();
    __shared__ float tile[32][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.0f;
    if (col < width)
        for (int p = threadIdx.y; p < nparts; p += 32)
            acc += __ldcg(partials + (size_t)p * width + col);
    tile[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && col < width) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 32; ++r)
            s += tile[r][threadIdx.x];
        if (col < split)
            out_a[col] = s;
        else
            out_b[col - split] = s;
    }
}

template <int VPT, int R>
__global__ void __launch_bounds__(RN_THREADS) pixelnorm_fwd_rows(float* __restrict__ y, const float* __restrict__ x,
    long rows, float eps)
{
    pdl_prologue();
    constexpr int C = VPT * 128;
    const int lane = threadIdx.x & 31;
    const long warp0 = ((long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5)) * R;
    const long wstride = (long)gridDim.x * RN_WARPS * R;
    const float invC = 1.0f / (float)C;
    for (long row = warp0; row < rows; row += wstride) {
        RowRegs<VPT> xr[R];
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (row + k < rows)
                row_load<VPT>(xr[k], x + (row + k) * C, lane);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (row + k >= rows)
                break;
            float ss = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                const float4 v = xr[k].v[j];
                ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            }
            const float rn = rsqrtf(warp_sum(ss) * invC + eps);
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                xr[k].v[j].x *= rn;
                xr[k].v[j].y *= rn;
                xr[k].v[j].z *= rn;
                xr[k].v[j].w *= rn;
            }
            row_store<VPT>(y + (row + k) * C, xr[k], lane);
        }
    }
}

template <int VPT, int R>
__global__ void __launch_bounds__(RN_THREADS) pixelnorm_bwd_rows(float* __restrict__ dx, const float* __restrict__ dy,
    const float* __restrict__ x, long rows, float eps)
{
    pdl_prologue();
    constexpr int C = VPT * 128;
    const int lane = threadIdx.x & 31;
    const long warp0 = ((long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5)) * R;
    const long wstride = (long)gridDim.x * RN_WARPS * R;
    const float invC = 1.0f / (float)C;
    for (long row = warp0; row < rows; row += wstride) {
        RowRegs<VPT> xr[R], gr[R];
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (row + k < rows) {
                row_load<VPT>(xr[k], x + (row + k) * C, lane);
                row_load<VPT>(gr[k], dy + (row + k) * C, lane);
            }
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (row + k >= rows)
                break;
            float ss = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                const float4 v = xr[k].v[j];
                ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            }
            const float rn = rsqrtf(warp_sum(ss) * invC + eps);
            float dot = 0.0f;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                float4& v = xr[k].v[j];
                const float4 d = gr[k].v[j];
                v.x *= rn; v.y *= rn; v.z *= rn; v.w *= rn;
                dot += (d.x * v.x + d.y * v.y) + (d.z * v.z + d.w * v.w);
            }
            const float md = warp_sum(dot) * invC;
            RowRegs<VPT> o;
            FOR_EACH_LANE_ELEM(j, VPT)
            {
                const float4 v = xr[k].v[j], d = gr[k].v[j];
                o.v[j].x = rn * (d.x - v.x * md);
                o.v[j].y = rn * (d.y - v.y * md);
                o.v[j].z = rn * (d.z - v.z * md);
                o.v[j].w = rn * (d.w - v.w * md);
            }
            row_store<VPT>(dx + (row + k) * C, o, lane);
        }
    }
}

// ---------------------------------------------------------------------------
// generic path: any C, any alignment; one warp per row, strided scalar loops
// (the row is re-read from L1/L2 for the second and third sweep)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(RN_THREADS) layernorm_fwd_generic(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, long rows, int C, float eps)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long wstride = (long)gridDim.x * RN_WARPS;
    for (long row = (long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5); row < rows; row += wstride) {
        const float* xr = x + row * C;
        float s = 0.0f;
        for (int c = lane; c < C; c += 32)
            s += xr[c];
        const float m = warp_sum(s) / (float)C;
        float vs = 0.0f;
        for (int c = lane; c < C; c += 32) {
            const float d = xr[c] - m;
            vs += d * d;
        }
        const float rs = rsqrtf(warp_sum(vs) / (float)C + eps);
        if (lane == 0) {
            mu[row] = m;
            rstd[row] = rs;
        }
        for (int c = lane; c < C; c += 32)
            y[row * C + c] = gamma[c] * ((xr[c] - m) * rs) + beta[c];
    }
}

__global__ void __launch_bounds__(RN_THREADS) layernorm_bwd_dx_generic(float* __restrict__ dx,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ mu, const float* __restrict__ rstd, long rows, int C)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long wstride = (long)gridDim.x * RN_WARPS;
    const float invC = 1.0f / (float)C;
    for (long row = (long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5); row < rows; row += wstride) {
        const float* xr = x + row * C;
        const float* gr = dy + row * C;
        const float m = mu[row], rs = rstd[row];
        float pg = 0.0f, pgx = 0.0f;
        for (int c = lane; c < C; c += 32) {
            const float xh = (xr[c] - m) * rs, gv = gr[c] * gamma[c];
            pg += gv;
            pgx += gv * xh;
        }
        const float sg = warp_sum(pg) * invC, sgx = warp_sum(pgx) * invC;
        for (int c = lane; c < C; c += 32) {
            const float xh = (xr[c] - m) * rs, gv = gr[c] * gamma[c];
            dx[row * C + c] = rs * (gv - sg - xh * sgx);
        }
    }
}

// Column sums of dy*xhat and dy over a chunk of rows.
// grid = (ceil(C/32), nchunks), block = 32 x 8; partials[chunk][2*C].
__global__ void __launch_bounds__(256) layernorm_bwd_param_generic(float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ mu,
    const float* __restrict__ rstd, long rows, int C, int chunk_rows)
{
    pdl_prologue();
    __shared__ float sg[8][33], sb[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const long r0 = (long)blockIdx.y * chunk_rows;
    const long r1 = min(rows, r0 + (long)chunk_rows);
    float gg = 0.0f, gb = 0.0f;
    if (col < C)
        for (long r = r0 + threadIdx.y; r < r1; r += 8) {
            const float go = dy[r * C + col];
            gg += go * ((x[r * C + col] - mu[r]) * rstd[r]);
            gb += go;
        }
    sg[threadIdx.y][threadIdx.x] = gg;
    sb[threadIdx.y][threadIdx.x] = gb;
    __syncthreads();
    if (threadIdx.y == 0 && col < C) {
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            a += sg[k][threadIdx.x];
            b += sb[k][threadIdx.x];
        }
        partials[(size_t)blockIdx.y * (2 * C) + col] = a;
        partials[(size_t)blockIdx.y * (2 * C) + C + col] = b;
    }
}

__global__ void __launch_bounds__(RN_THREADS) pixelnorm_generic(float* __restrict__ out, const float* __restrict__ dy,
    const float* __restrict__ x, long rows, int C, float eps, int backward)
{
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const long wstride = (long)gridDim.x * RN_WARPS;
    for (long row = (long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5); row < rows; row += wstride) {
        const float* xr = x + row * C;
        float ss = 0.0f;
        for (int c = lane; c < C; c += 32)
            ss += xr[c] * xr[c];
        const float rn = rsqrtf(warp_sum(ss) / (float)C + eps);
        if (!backward) {
            for (int c = lane; c < C; c += 32)
                out[row * C + c] = xr[c] * rn;
        } else {
            const float* gr = dy + row * C;
            float dot = 0.0f;
            for (int c = lane; c < C; c += 32)
                dot += gr[c] * (xr[c] * rn);
            const float md = warp_sum(dot) / (float)C;
            for (int c = lane; c < C; c += 32)
                out[row * C + c] = rn * (gr[c] - (xr[c] * rn) * md);
        }
    }
}

// ---------------------------------------------------------------------------
// host dispatch
// ---------------------------------------------------------------------------
// (the key varies per caller, so this site uses the uncached lookup)
static inline int rows_grid(long rows, int rows_per_block, const char* key, int dflt)
{
    long want = (rows + rows_per_block - 1) / rows_per_block;
    const long cap = (long)sm_count() * tune_lookup(key, dflt);
    if (want > cap)
        want = cap;
    return want < 1 ? 1 : (int)want;
}

static inline bool fast_rows_ok(int C) { return C % 128 == 0 && C >= 128 && C <= 1024; }

void fold_partials(float* out_a, float* out_b, const float* partials, int nparts, int width, int split,
    cudaStream_t s)
{
    if (planning_only())
        return;
    launch_k(fold_partials_kernel, (width + 31) / 32, dim3(32, 32), 0, s, out_a, out_b, partials, nparts, width, split);
    count_launch();
    B200_CHECK_LAUNCH();
}

#define RN_DISPATCH_VPT(C, CALL)         \
    switch ((C) / 128) {                 \
    case 1: { constexpr int VPT = 1, R = 4; CALL; } break; \
    case 2: { constexpr int VPT = 2, R = 2; CALL; } break; \
    case 3: { constexpr int VPT = 3, R = 1; CALL; } break; \
    case 4: { constexpr int VPT = 4, R = 1; CALL; } break; \
    case 5: { constexpr int VPT = 5, R = 1; CALL; } break; \
    case 6: { constexpr int VPT = 6, R = 1; CALL; } break; \
    case 7: { constexpr int VPT = 7, R = 1; CALL; } break; \
    default: { constexpr int VPT = 8, R = 1; CALL; } break; \
    }

}  // namespace b200

using namespace b200;

extern "C" {

void launch_layernorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int C, float eps, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0, "layernorm_forward: batch=%d C=%d", batch, C);
    if (batch == 0)
        return;
    const long rows = batch;
    if (fast_rows_ok(C) && aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta)) {
        RN_DISPATCH_VPT(C, (launch_k(layernorm_fwd_rows<VPT, R>, rows_grid(rows, RN_WARPS * R, "ln_blocks_per_sm", 64),
                                RN_THREADS, 0, s, y, mu, rstd, x, gamma, beta, rows, eps)));
    } else {
        launch_k(layernorm_fwd_generic, rows_grid(rows, RN_WARPS, "ln_blocks_per_sm", 64), RN_THREADS, 0, s,
            y, mu, rstd, x, gamma, beta, rows, C, eps);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_layernorm_backward(float* grad_in, float* ggamma, float* gbeta, const float* grad_out,
    const float* x, const float* gamma, const float* mu, const float* rstd, int batch, int C,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0, "layernorm_backward: batch=%d C=%d", batch, C);
    const long rows = batch;
    Scratch sc;
    if (fast_rows_ok(C) && rows > 0 && aligned16(grad_in) && aligned16(grad_out) && aligned16(x) && aligned16(gamma)) {
        const int R = (C / 128 == 1) ? 4 : (C / 128 == 2 ? 2 : 1);
        const int grid = rows_grid(rows, RN_WARPS * R, "ln_bwd_blocks_per_sm", 2);
        B200_REQUIRE(scratch_get(s, (size_t)grid * 2 * C, 0, &sc), "layernorm_backward: scratch allocation failed (the arena cannot grow during stream capture: call b200_scratch_reserve before capturing)");
        RN_DISPATCH_VPT(C, (launch_k(layernorm_bwd_rows<VPT, R>, grid, RN_THREADS, 0, s, grad_in, sc.partials, grad_out, x,
                                gamma, mu, rstd, rows)));
        count_launch();
        B200_CHECK_LAUNCH();
        fold_partials(ggamma, gbeta, sc.partials, grid, 2 * C, C, s);
        return;
    }
    if (rows > 0) {
        launch_k(layernorm_bwd_dx_generic, rows_grid(rows, RN_WARPS, "ln_blocks_per_sm", 64), RN_THREADS, 0, s,
            grad_in, grad_out, x, gamma, mu, rstd, rows, C);
        count_launch();
        B200_CHECK_LAUNCH();
    }
    const int chunk_rows = 256;
    const int nchunks = rows > 0 ? (int)((rows + chunk_rows - 1) / chunk_rows) : 1;
    B200_REQUIRE(nchunks <= 65535, "layernorm_backward: too many rows for the generic path");
    B200_REQUIRE(scratch_get(s, (size_t)nchunks * 2 * C, 0, &sc), "layernorm_backward: scratch allocation failed (the arena cannot grow during stream capture: call b200_scratch_reserve before capturing)");
    launch_k(layernorm_bwd_param_generic, dim3((C + 31) / 32, nchunks), dim3(32, 8), 0, s, sc.partials, grad_out, x, mu,
        rstd, rows, C, chunk_rows);
    count_launch();
    B200_CHECK_LAUNCH();
    fold_partials(ggamma, gbeta, sc.partials, nchunks, 2 * C, C, s);
}

void launch_pixel_norm_forward(float* y, const float* x, int rows_i, int C, float eps, cudaStream_t s)
{
    B200_REQUIRE(rows_i >= 0 && C > 0, "pixel_norm_forward: rows=%d C=%d", rows_i, C);
    if (rows_i == 0)
        return;
    const long rows = rows_i;
    if (fast_rows_ok(C) && aligned16(y) && aligned16(x)) {
        RN_DISPATCH_VPT(C, (launch_k(pixelnorm_fwd_rows<VPT, R>, rows_grid(rows, RN_WARPS * R, "pn_blocks_per_sm", 64),
                                RN_THREADS, 0, s, y, x, rows, eps)));
    } else {
        launch_k(pixelnorm_generic, rows_grid(rows, RN_WARPS, "pn_blocks_per_sm", 64), RN_THREADS, 0, s, y, nullptr, x,
            rows, C, eps, 0);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_pixel_norm_backward(float* dx, const float* dy, const float* x, int rows_i, int C, float eps,
    cudaStream_t s)
{
    B200_REQUIRE(rows_i >= 0 && C > 0, "pixel_norm_backward: rows=%d C=%d", rows_i, C);
    if (rows_i == 0)
        return;
    const long rows = rows_i;
    if (fast_rows_ok(C) && aligned16(dx) && aligned16(dy) && aligned16(x)) {
        RN_DISPATCH_VPT(C, (launch_k(pixelnorm_bwd_rows<VPT, R>, rows_grid(rows, RN_WARPS * R, "pn_blocks_per_sm", 64),
                                RN_THREADS, 0, s, dx, dy, x, rows, eps)));
    } else {
        launch_k(pixelnorm_generic, rows_grid(rows, RN_WARPS, "pn_blocks_per_sm", 64), RN_THREADS, 0, s, dx, dy, x, rows,
            C, eps, 1);
    }
    count_launch();
    B200_CHECK_LAUNCH();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// LayerNorm backward for callers that may not allocate device memory
// ---------------------------------------------------------------------------
// Some hosts of these kernels run under a fixed device-memory plan: every buffer is created
// once by the module constructors and the training loop must not enter the CUDA allocator
// again (small shared-memory boards where the heap is sized up front, or code that calls the
// backward pass from a place where cudaMalloc is off limits, such as inside an allocator hook
// or a section that holds the allocator's lock).  launch_layernorm_backward keeps its
// per-CTA dgamma/dbeta partial rows in a scratch arena that it allocates on first use, which
// such a caller cannot accept.  This variant keeps the partial rows in a fixed array that is
// part of the library image instead.
//
// The array lives in this translation unit.  Its name is only a host-side handle here; the
// device address is looked up once per device with cudaGetSymbolAddress and handed to the
// kernels as an ordinary pointer.
namespace b200 {

constexpr size_t LN_NOALLOC_MAX_FLOATS = (size_t)1 << 20;  // 4 MiB of partial rows
static __device__ __align__(256) float g_ln_noalloc_scratch[LN_NOALLOC_MAX_FLOATS];

// Device address of the fixed scratch array on the current device (looked up once per device,
// with that device current).  Returns nullptr and reports when the lookup fails.
static float* ln_noalloc_scratch_address()
{
    static float* cached[64] = { nullptr };
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        report_error(__FILE__, __LINE__, "layernorm_backward_noalloc: cannot identify the current device (%s)",
            cudaGetErrorString(e));
        return nullptr;
    }
    if (!cached[dev]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_ln_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            report_error(__FILE__, __LINE__, "layernorm_backward_noalloc: cudaGetSymbolAddress failed (%s)",
                cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev] = ptr;
    }
    return cached[dev];
}

}  // namespace b200

extern "C" int launch_layernorm_backward_noalloc(float* grad_in, float* ggamma, float* gbeta,
    const float* grad_out, const float* x, const float* gamma, const float* mu, const float* rstd, int batch,
    int C, cudaStream_t s)
{
    using namespace b200;
    if (batch < 0 || C <= 0) {
        report_error(__FILE__, __LINE__, "layernorm_backward_noalloc: batch=%d C=%d", batch, C);
        return -1;
    }
    const long rows = batch;
    const bool fast = fast_rows_ok(C) && rows > 0 && aligned16(grad_in) && aligned16(grad_out) && aligned16(x)
        && aligned16(gamma);
    // partial rows this call needs: one per CTA (fast path) or one per 256-row chunk (generic path)
    const int R = (C / 128 == 1) ? 4 : (C / 128 == 2 ? 2 : 1);
    const int chunk_rows = 256;
    long nparts;
    if (fast) {
        nparts = rows_grid(rows, RN_WARPS * R, "ln_bwd_blocks_per_sm", 2);
        const long fit = (long)(LN_NOALLOC_MAX_FLOATS / (2 * (size_t)C));
        if (nparts > fit)
            nparts = fit;  // fewer, longer-running CTAs: the grid-stride loop covers all rows
    } else {
        nparts = rows > 0 ? (rows + chunk_rows - 1) / chunk_rows : 1;
    }
    if (nparts < 1 || (size_t)nparts * 2 * (size_t)C > LN_NOALLOC_MAX_FLOATS || nparts > 65535) {
        report_error(__FILE__, __LINE__,
            "layernorm_backward_noalloc: batch=%d C=%d needs %ld partial rows of %d floats, more than the fixed "
            "scratch of %zu floats (use launch_layernorm_backward, which allocates)",
            batch, C, nparts, 2 * C, (size_t)LN_NOALLOC_MAX_FLOATS);
        return -2;
    }
    float* scratch = ln_noalloc_scratch_address();
    if (!scratch)
        return -3;
    // a launch that fails is reported (b200_set_error_mode) AND ends the call with -4: nothing later in
    // the sequence runs on results that were never produced
#define NOALLOC_LAUNCHED()                                        \
    do {                                                          \
        count_launch();                                           \
        const cudaError_t le_ = cudaPeekAtLastError();            \
        B200_CHECK_LAUNCH();                                      \
        if (le_ != cudaSuccess)                                   \
            return -4;                                            \
    } while (0)
    if (fast) {
        const int grid = (int)nparts;
        RN_DISPATCH_VPT(C, (launch_k(layernorm_bwd_rows<VPT, R>, grid, RN_THREADS, 0, s, grad_in, scratch, grad_out, x, gamma,
                                mu, rstd, rows)));
        NOALLOC_LAUNCHED();
        fold_partials(ggamma, gbeta, scratch, grid, 2 * C, C, s);
        return cudaPeekAtLastError() == cudaSuccess ? 0 : -4;
    }
    if (rows > 0) {
        launch_k(layernorm_bwd_dx_generic, rows_grid(rows, RN_WARPS, "ln_blocks_per_sm", 64), RN_THREADS, 0, s, grad_in,
            grad_out, x, gamma, mu, rstd, rows, C);
        NOALLOC_LAUNCHED();
    }
    launch_k(layernorm_bwd_param_generic, dim3((C + 31) / 32, (unsigned)nparts), dim3(32, 8), 0, s, scratch, grad_out, x, mu,
        rstd, rows, C, chunk_rows);
    NOALLOC_LAUNCHED();
#undef NOALLOC_LAUNCHED
    fold_partials(ggamma, gbeta, scratch, (int)nparts, 2 * C, C, s);
    return cudaPeekAtLastError() == cudaSuccess ? 0 : -4;
}
