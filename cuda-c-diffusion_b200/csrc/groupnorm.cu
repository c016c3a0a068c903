// NHWC GroupNorm forward / backward, optionally fused with an activation
// (reference: src/kernels.cu:622-745, composed with :103-117 by conv_residual.c).
//
// x is viewed as a matrix [B*HW, C]; a work item is (sample b, Ct channels covering whole groups).
// Three kernel families, tried in this order by gn_forward / gn_backward:
//
//   1. register-resident strips (groupnorm_strip.cuh, groupnorm_dstrip.cuh, groupnorm_ostrip.cuh): the
//      default.  A CTA keeps all HW rows of an item in registers, statistics and output come from
//      registers, the next item is staged with cp.async while the current one is processed.  x (and dy)
//      cross HBM exactly once.  Launches with many strips per CTA take the one-barrier kernels of
//      groupnorm_ostrip.cuh (forward in clusters of 4 CTAs whose staging bursts are kept in step).
//   2. chunked strips (groupnorm_cstrip.cuh): samples too tall for the register file; the strip is
//      walked twice in chunks, the second read coming from L2 while the strips in flight fit there.
//   3. generic kernels (this file): any shape, any alignment (C % 4 != 0, misaligned pointers) and the
//      activations the strips do not instantiate.
//
// Two more families were built, measured and removed.  Persistent thread-block clusters on 2-D TMA
// tiles with a DSMEM combine: 0.44-0.48 of the copy peak against 0.8 for the strips on every shape (the
// cluster barrier and the DSMEM round trip sit on each item's critical path).  Two passes of fully
// contiguous streaming kernels per 16-80 MB chunk of samples, the second pass reading from L2: correct,
// but [256,32,32,256] took 174-290 us forward and 340-690 us backward against 100 / 155 us for the
// strips: a chunk small enough to stay in L2 is too small a launch to reach the HBM rate, and only about
// half of the second pass's reads hit L2.  And for small launches, where a strip's latency chain rather
// than bandwidth sets the time, the rows of a strip split over a cluster of 2 or 4 CTAs with one DSMEM
// exchange of the partial sums: [128,28,28,64] took 15.7-37 us forward and 28-41 us backward against
// 12.2 / 18.0 us for the plain strips -- two cluster barriers cost more than half a strip's latency.  The
// same split for samples too tall for one CTA (one-barrier kernels, every warp pushing its group sums into
// the shared memory of all CTAs of the cluster, ONE cluster barrier per strip, x read once): [32,64,64,256]
// 76 us forward / 101-120 us backward against 62 / 102 us for the chunked strips, which read x twice but the
// second time from L2 -- the barrier between the two phases waits for the slowest of 4-8 CTAs with nothing
// else resident on the SM (with remote LOADS after the barrier instead of remote stores before it: 131 us).
//
// Backward in every family reuses the per-channel sums of g and g*xhat (g = dy * act'(z)) for BOTH
// the group sums that dx needs and the per-sample dgamma/dbeta partials, which a fixed-order fold
// adds up: parameter gradients are overwritten and bit-reproducible.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

#include <atomic>
#include <mutex>

namespace b200 {

constexpr int GN_GENERIC_THREADS = 256;

// launches per kernel family, for tests that must know which family they exercised (b200_groupnorm_path_count)
enum : int { GN_PATH_STRIP = 0, GN_PATH_PIPELINED, GN_PATH_DEEP, GN_PATH_ONE_BARRIER, GN_PATH_CHUNKED, GN_PATH_GENERIC, GN_PATHS };
static std::atomic<long long> g_gn_path[GN_PATHS];
static inline bool gn_path(int path, bool launched)
{
    if (launched)
        g_gn_path[path].fetch_add(1, std::memory_order_relaxed);
    return launched;
}

}  // namespace b200

#include "tma_desc.cuh"
#include "groupnorm_strip.cuh"
#include "groupnorm_dstrip.cuh"
#include "groupnorm_ostrip.cuh"
#include "groupnorm_cstrip.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// generic kernels: one CTA per (sample, group), any C / HW / alignment.
// The group is re-read from L2 for the second and third sweep.
// ---------------------------------------------------------------------------
template <int ACT>
__global__ void __launch_bounds__(GN_GENERIC_THREADS) gn_fwd_generic(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, int HW, int C, int G, float eps)
{
    pdl_prologue();
    __shared__ float buf[32];
    const int b = blockIdx.x / G, grp = blockIdx.x % G;
    const int cpg = C / G, n = HW * cpg, cbase = grp * cpg;
    const float* xb = x + (size_t)b * HW * C;
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_GENERIC_THREADS)
        s += xb[(size_t)(i / cpg) * C + cbase + i % cpg];
    const float mean = cta_sum(s, buf) / (float)n;
    float vs = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_GENERIC_THREADS) {
        const float d = xb[(size_t)(i / cpg) * C + cbase + i % cpg] - mean;
        vs += d * d;
    }
    const float rs = rsqrtf(cta_sum(vs, buf) / (float)n + eps);
    if (threadIdx.x == 0) {
        mu[blockIdx.x] = mean;
        rstd[blockIdx.x] = rs;
    }
    float* yb = y + (size_t)b * HW * C;
    for (int i = threadIdx.x; i < n; i += GN_GENERIC_THREADS) {
        const int cl = i % cpg;
        const size_t off = (size_t)(i / cpg) * C + cbase + cl;
        yb[off] = act_value<ACT>(gamma[cbase + cl] * ((xb[off] - mean) * rs) + beta[cbase + cl]);
    }
}

template <int ACT>
__device__ __forceinline__ float gn_effective_grad(float dyv, float xhat, float gm, float bt)
{
    if (ACT == ACT_IDENTITY)
        return dyv;
    return dyv * act_slope<ACT>(gm * xhat + bt);
}

template <int ACT>
__global__ void __launch_bounds__(GN_GENERIC_THREADS) gn_bwd_dx_generic(float* __restrict__ dx, const float* __restrict__ dy,
    const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    const float* __restrict__ mu, const float* __restrict__ rstd, int HW, int C, int G)
{
    pdl_prologue();
    __shared__ float buf[32];
    const int b = blockIdx.x / G, grp = blockIdx.x % G;
    const int cpg = C / G, n = HW * cpg, cbase = grp * cpg;
    const size_t sample = (size_t)b * HW * C;
    const float mean = mu[blockIdx.x], rs = rstd[blockIdx.x];
    float pg = 0.0f, pgx = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_GENERIC_THREADS) {
        const int cl = i % cpg;
        const size_t off = sample + (size_t)(i / cpg) * C + cbase + cl;
        const float xh = (x[off] - mean) * rs;
        const float bt = ACT == ACT_IDENTITY ? 0.0f : beta[cbase + cl];
        const float gv = gn_effective_grad<ACT>(dy[off], xh, gamma[cbase + cl], bt) * gamma[cbase + cl];
        pg += gv;
        pgx += gv * xh;
    }
    const float inv_n = 1.0f / (float)n;
    const float sg = cta_sum(pg, buf) * inv_n;
    const float sgx = cta_sum(pgx, buf) * inv_n;
    for (int i = threadIdx.x; i < n; i += GN_GENERIC_THREADS) {
        const int cl = i % cpg;
        const size_t off = sample + (size_t)(i / cpg) * C + cbase + cl;
        const float xh = (x[off] - mean) * rs;
        const float bt = ACT == ACT_IDENTITY ? 0.0f : beta[cbase + cl];
        const float gv = gn_effective_grad<ACT>(dy[off], xh, gamma[cbase + cl], bt) * gamma[cbase + cl];
        dx[off] = rs * (gv - sg - xh * sgx);
    }
}

// Per-sample column sums.  grid = (ceil(C/32), B), block = 32 x 8; partials[b][2*C].
template <int ACT>
__global__ void __launch_bounds__(256) gn_bwd_param_generic(float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mu, const float* __restrict__ rstd, int HW, int C, int G)
{
    pdl_prologue();
    __shared__ float sg[8][33], sb[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int b = blockIdx.y;
    float gg = 0.0f, gb = 0.0f;
    if (col < C) {
        const int grp = col / (C / G);
        const float mean = mu[b * G + grp], rs = rstd[b * G + grp];
        const float gm = gamma[col], bt = ACT == ACT_IDENTITY ? 0.0f : beta[col];
        for (int hw = threadIdx.y; hw < HW; hw += 8) {
            const size_t off = ((size_t)b * HW + hw) * C + col;
            const float xh = (x[off] - mean) * rs;
            const float go = gn_effective_grad<ACT>(dy[off], xh, gm, bt);
            gg += go * xh;
            gb += go;
        }
    }
    sg[threadIdx.y][threadIdx.x] = gg;
    sb[threadIdx.y][threadIdx.x] = gb;
    __syncthreads();
    if (threadIdx.y == 0 && col < C) {
        float a = 0.0f, c = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            a += sg[k][threadIdx.x];
            c += sb[k][threadIdx.x];
        }
        partials[(size_t)b * (2 * C) + col] = a;
        partials[(size_t)b * (2 * C) + C + col] = c;
    }
}

// ---------------------------------------------------------------------------
// strip (register-resident) dispatch
// ---------------------------------------------------------------------------
struct StripPlan {
    int NT, VPT;
    StripGeom g;
    size_t smem;
};

// Chooses CTA size and strip width Ct such that all HW rows of a strip fit the CTA's
// registers: HW <= (NT / (Ct/4)) * VPT.  Wider strips mean longer contiguous runs in memory.
// (Splitting the rows of a wider strip over a cluster was measured and is slower than
// narrower strips without one: the cluster barrier lengthens every CTA's critical path.)
static bool strip_plan(StripPlan* out, int B, int HW, int C, int G, int max_vpt, int force_ct, int force_nt,
    int ctas_per_sm_hint)
{
    if (C % 4 != 0 || C % G != 0)
        return false;
    const int cpg = C / G;
    long best = -1;
    const int nts[3] = { 512, 1024, 256 };
    for (int ni = 0; ni < 3; ++ni) {
        const int NT = nts[ni];
        if (force_nt > 0 ? NT != force_nt : NT == 256)
            continue;  // 256-thread CTAs only on request
        for (int Ct = 4; Ct <= C && Ct <= 1024; Ct += 4) {
            if (C % Ct != 0 || Ct % cpg != 0)
                continue;
            if (force_ct > 0 && Ct != force_ct)
                continue;
            const int Q = Ct / 4;
            if (Q > NT || NT % Q != 0)
                continue;
            const int rstep = NT / Q;
            const int need = (HW + rstep - 1) / rstep;
            int vpt = 2;
            while (vpt < need)
                vpt *= 2;
            if (vpt > max_vpt)
                continue;
            // backward (two tensors per thread): 8 rows per tensor only fit 512-thread CTAs
            if (ctas_per_sm_hint == 1 && vpt == 8 && NT != 512)
                continue;
            long score = 0;
            if (Ct * 4 >= 64)
                score += 1000000;
            score += (long)Ct * 100;
            score += (long)(100.0 * HW / ((double)rstep * vpt));  // register utilisation
            if (NT == 512)
                score += 5000;  // two CTAs per SM overlap each other's phases
            // forward only: a 1024-thread CTA with 128-byte runs whose rows fill every register slot
            // measured 2 % faster than two 512-thread CTAs with 64-byte runs; any ragged fill is slower
            if (ctas_per_sm_hint == 0 && NT == 1024 && vpt == 8 && rstep * vpt == HW && Ct * 4 >= 128)
                score += 4000;
            if (score > best) {
                best = score;
                out->NT = NT;
                out->VPT = vpt;
                StripGeom g;
                g.HW = HW; g.C = C; g.G = G; g.cpg = cpg; g.Ct = Ct; g.Q = Q; g.RSTEP = rstep;
                g.Gt = Ct / cpg; g.nct = C / Ct;
                g.paced = 0; g.hint = tune_get("gn_strip_l2_hint", 0);
                out->g = g;
                const int red = (Q <= 32 && 32 % Q == 0) ? 2 * (NT / 32) * Ct : 2 * NT * 4;
                out->smem = (size_t)(red + 2 * Ct + 2 * g.Gt) * sizeof(float);
            }
        }
    }
    if (best < 0)
        return false;
    return true;
}

// What the dispatcher decided, recorded in planning-only mode (b200_groupnorm_describe).
struct PlannedLaunch {
    int path, nt, ct, rows_per_cta, cluster;
    long grid;
    size_t smem;
};
static thread_local PlannedLaunch t_planned;

template <class T>
static inline void note_geometry(const T&) {}
static inline void note_geometry(const StripGeom& g)
{
    t_planned.ct = g.Ct;
    t_planned.rows_per_cta = g.RSTEP;  // rows per register slot; the kernel's slot count is part of its name
}

// Cluster width for the next strip launch of this thread (1 = no cluster); with a width above 1 the grid is
// cut to the clusters the device can hold at once (the kernels are persistent: fewer CTAs walk more strips).
static thread_local int t_gn_cluster = 1;
struct ClusterScope {
    explicit ClusterScope(int w)
    {
        t_gn_cluster = w;
        t_planned.cluster = w;
    }
    ~ClusterScope() { t_gn_cluster = 1; }
};

template <class... KArgs, class... Args>
static bool strip_launch(int path, void (*kernel)(KArgs...), long grid, int NT, size_t smem, cudaStream_t s, Args... args)
{
    if (planning_only()) {
        t_planned.path = path;
        t_planned.nt = NT;
        t_planned.grid = grid;
        t_planned.smem = smem;
        (note_geometry(args), ...);
        return true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    unsigned nat = 0;
    pdl_attribute(at, &nat, grid * NT);
    if (t_gn_cluster > 1) {
        const int w = t_gn_cluster;
        at[nat].id = cudaLaunchAttributeClusterDimension;
        at[nat].val.clusterDim.x = (unsigned)w;
        at[nat].val.clusterDim.y = 1;
        at[nat].val.clusterDim.z = 1;
        ++nat;
        cfg.attrs = at;
        cfg.numAttrs = nat;
        cfg.gridDim.x = (unsigned)((grid + w - 1) / w * w);
        // resident clusters of this kernel at this size: asked of the driver once per (kernel, device, size)
        struct Known {
            const void* fn;
            int dev, w, nt, clusters;
            size_t smem;
        };
        static Known known[32];
        static int nknown = 0;
        static std::mutex mu;
        int dev = 0, nclusters = 0;
        (void)cudaGetDevice(&dev);
        {
            std::lock_guard<std::mutex> lock(mu);
            for (int i = 0; i < nknown; ++i)
                if (known[i].fn == (const void*)kernel && known[i].dev == dev && known[i].w == w && known[i].nt == NT
                    && known[i].smem == smem)
                    nclusters = known[i].clusters;
            if (nclusters == 0) {
                if (cudaOccupancyMaxActiveClusters(&nclusters, kernel, &cfg) != cudaSuccess || nclusters < 1) {
                    (void)cudaGetLastError();
                    nclusters = -1;  // no cluster of this shape fits this device (or partition)
                }
                if (nknown < 32)
                    known[nknown++] = Known{ (const void*)kernel, dev, w, NT, nclusters, smem };
            }
        }
        if (nclusters < 1) {
            // plain CTAs instead: the kernels find a cluster of one and skip the cluster barrier
            --nat;
            cfg.gridDim.x = (unsigned)grid;
        } else if ((long)nclusters * w < (long)cfg.gridDim.x) {
            cfg.gridDim.x = (unsigned)(nclusters * w);
        }
    }
    cfg.attrs = at;
    cfg.numAttrs = nat;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "groupnorm strip launch failed: %s", cudaGetErrorString(e));
        return false;
    }
    count_launch();
    return gn_path(path, true);
}

template <class... KArgs, class... Args>
static bool pstrip_launch(int path, void (*kernel)(KArgs...), bool* attr_done, long grid, int NT, size_t smem, cudaStream_t s,
    Args... args)
{
    if (planning_only())
        return strip_launch(path, kernel, grid, NT, smem, s, args...);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return false;
    if (!attr_done[dev]) {
        // the opt-in limit (227 KB per CTA) covers static and dynamic shared memory together
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess
            || cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                   227 * 1024 - (int)fa.sharedSizeBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        attr_done[dev] = true;
    }
    return strip_launch(path, kernel, grid, NT, smem, s, args...);
}

#define PSTRIP_FWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv && per_sm == MBv) {                                              \
        static bool done[64] = { false };                                                                   \
        if (full) {                                                                                         \
            static bool donef[64] = { false };                                                              \
            return pstrip_launch(GN_PATH_PIPELINED, gn_fwd_pstrip<NTv, VPTv, ACT, MBv, true>, donef, pgrid, NTv, psmem, s, y, mu, rstd, x, \
                gamma, beta, plan.g, eps, (int)grid);                                                       \
        }                                                                                                   \
        return pstrip_launch(GN_PATH_PIPELINED, gn_fwd_pstrip<NTv, VPTv, ACT, MBv, false>, done, pgrid, NTv, psmem, s, y, mu, rstd, x, \
            gamma, beta, plan.g, eps, (int)grid);                                                           \
    }
#define PSTRIP_BWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv) {                                                               \
        static bool done[64] = { false };                                                                   \
        return pstrip_launch(GN_PATH_PIPELINED, gn_bwd_pstrip<NTv, VPTv, ACT, MBv>, done, pgrid, NTv, psmem, s, dx, sc.partials,       \
                   dy, x, gamma, beta, mu, rstd, plan.g, (int)grid)                                   \
            && (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true);            \
    }

// deep-staged variants (groupnorm_dstrip.cuh)
#define DSTRIP_BWD_CASE(NTv, VPTv)                                                                          \
    if (plan.NT == NTv && plan.VPT == VPTv) {                                                               \
        static bool done[64] = { false };                                                                   \
        static bool donef[64] = { false };                                                                  \
        const bool ok = full                                                                                \
            ? pstrip_launch(GN_PATH_DEEP, gn_bwd_dstrip<NTv, VPTv, ACT, true>, donef, pgrid, NTv, dsmem, s, dx, sc.partials, dy, x,  \
                  gamma, beta, mu, rstd, plan.g, (int)grid)                                           \
            : pstrip_launch(GN_PATH_DEEP, gn_bwd_dstrip<NTv, VPTv, ACT, false>, done, pgrid, NTv, dsmem, s, dx, sc.partials, dy, x,  \
                  gamma, beta, mu, rstd, plan.g, (int)grid);                                          \
        return ok && (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true);      \
    }

// one-barrier strips (groupnorm_ostrip.cuh): groups per float4 column the kernels are built for, 0 = not eligible
static int ostrip_gpt(const StripGeom& g)
{
    if (g.Q > 32 || (g.Q & (g.Q - 1)) != 0 || g.C > 2048)
        return 0;
    if (g.cpg == 2)
        return 2;
    if (g.cpg % 4 == 0 && ((g.cpg / 4) & (g.cpg / 4 - 1)) == 0)
        return 1;
    return 0;
}

template <int NT, int VPT, int ACT, int MB, class... Args>
static bool ostrip_fwd_launch(bool full, int gpt, long pgrid, size_t smem, cudaStream_t s, Args... args)
{
    static bool done[4][64] = {};
    if (full)
        return gpt == 1
            ? pstrip_launch(GN_PATH_ONE_BARRIER, gn_fwd_ostrip<NT, VPT, ACT, MB, true, 1>, done[0], pgrid, NT, smem, s, args...)
            : pstrip_launch(GN_PATH_ONE_BARRIER, gn_fwd_ostrip<NT, VPT, ACT, MB, true, 2>, done[1], pgrid, NT, smem, s, args...);
    return gpt == 1
        ? pstrip_launch(GN_PATH_ONE_BARRIER, gn_fwd_ostrip<NT, VPT, ACT, MB, false, 1>, done[2], pgrid, NT, smem, s, args...)
        : pstrip_launch(GN_PATH_ONE_BARRIER, gn_fwd_ostrip<NT, VPT, ACT, MB, false, 2>, done[3], pgrid, NT, smem, s, args...);
}

// Backward one-barrier strips.  On request (tunable "gn_bwd_tma") whole strips are staged by TMA: one box per
// warp, tensor and strip out of a tensor map over the [B * HW, C] view of x and of dy, encoded here per launch.
template <int NT, int VPT, int ACT>
static bool ostrip_bwd_launch(bool full, int gpt, long pgrid, size_t smem, cudaStream_t s, float* dx, float* partials,
    const float* dy, const float* x, const float* gamma, const float* beta, const float* mu, const float* rstd,
    const StripGeom& g, int nitems, int B)
{
    static bool done[6][64] = {};
    CUtensorMap mx, md;
    memset(&mx, 0, sizeof(mx));
    memset(&md, 0, sizeof(md));
    int* err = nullptr;
    // "gn_bwd_tma": 0 (default) = cp.async staging; 1 = TMA for 512 x 8 strips with an activation; 2 = TMA wherever
    // strips are whole (the measurements that keep it off by default are at gn_bwd_ostrip).
    const int tma_mode = tune_get("gn_bwd_tma", 0);
    if (full && (tma_mode == 2 || (tma_mode == 1 && ACT != ACT_IDENTITY && NT == 512 && VPT == 8))) {
        const uint32_t box_rows = (uint32_t)(VPT * 32 / g.Q);
        const int l2p = tune_get("gn_bwd_tma_l2", 0);
        bool ok = planning_only();
        if (!ok)
            ok = make_tensor_map_2d(&mx, x, (uint64_t)B * g.HW, (uint64_t)g.C, box_rows, (uint32_t)g.Ct, l2p)
                && make_tensor_map_2d(&md, dy, (uint64_t)B * g.HW, (uint64_t)g.C, box_rows, (uint32_t)g.Ct, l2p)
                && (err = device_error_word()) != nullptr;
        if (ok)
            return gpt == 1 ? pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, true, 1, true>, done[4], pgrid, NT, smem, s,
                                  dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md)
                            : pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, true, 2, true>, done[5], pgrid, NT, smem, s,
                                  dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md);
        err = nullptr;
    }
    if (full)
        return gpt == 1 ? pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, true, 1, false>, done[0], pgrid, NT, smem, s,
                              dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md)
                        : pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, true, 2, false>, done[1], pgrid, NT, smem, s,
                              dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md);
    return gpt == 1 ? pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, false, 1, false>, done[2], pgrid, NT, smem, s,
                          dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md)
                    : pstrip_launch(GN_PATH_ONE_BARRIER, gn_bwd_ostrip<NT, VPT, ACT, false, 2, false>, done[3], pgrid, NT, smem, s,
                          dx, partials, dy, x, gamma, beta, mu, rstd, g, nitems, err, mx, md);
}

#define OSTRIP_FWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv && per_sm == MBv)                                                \
        return plan.g.hint = tune_get("gn_fwd_l2_hint", fwd_hint_default), ostrip_fwd_launch<NTv, VPTv, ACT, MBv>(full, gpt, pgrid, osmem, s, y, mu, rstd, x, gamma, beta, plan.g, \
            eps, (int)grid);
#define OSTRIP_BWD_CASE(NTv, VPTv)                                                                          \
    if (plan.NT == NTv && plan.VPT == VPTv)                                                                 \
        return plan.g.hint = tune_get("gn_bwd_l2_hint", 0), ostrip_bwd_launch<NTv, VPTv, ACT>(full, gpt, pgrid, osmem, s, dx, sc.partials, dy, x, gamma, beta, mu,  \
                   rstd, plan.g, (int)grid, B)                                                              \
            && (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true);

#define STRIP_FWD_CASE(NTv, VPTv)                                                                          \
    if (plan.NT == NTv && plan.VPT == VPTv)                                                                \
        return strip_launch(GN_PATH_STRIP, gn_fwd_strip<NTv, VPTv, ACT>, grid, NTv, plan.smem, s, y, mu, rstd, x, gamma, \
            beta, plan.g, eps);
#define STRIP_BWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv)                                                                \
        return strip_launch(GN_PATH_STRIP, gn_bwd_strip<NTv, VPTv, ACT, MBv>, grid, NTv, plan.smem, s, dx, sc.partials,      \
                   dy, x, gamma, beta, mu, rstd, plan.g, B)                                          \
            && (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true);

static bool cstrip_plan(StripPlan* out, int HW, int C, int G);

// A register-resident plan whose runs are shorter than 64 bytes only exists because the sample is tall;
// the chunked strips keep 64-byte runs for such samples and are preferred when they apply.
static bool strip_too_narrow(const StripPlan& plan, int HW, int C, int G)
{
    if (plan.g.Ct * 4 >= 64 || tune_get("gn_no_cstrip", 0))
        return false;
    StripPlan wide;
    return cstrip_plan(&wide, HW, C, G) && wide.g.Ct > plan.g.Ct;
}

// Exact-fill plans for the one-barrier kernels: CTAs of 7 * 64 or 7 * 128 threads whose 7 register slots per thread
// hold exactly HW rows (HW = 7 * NT / Q; 28 x 28 and 14 x 14 samples), so that the predicate-free FULL kernels apply
// where the power-of-two CTAs would leave a quarter of their slots empty.
static bool exact7_plan(StripPlan* out, int HW, int C, int G, int NT)
{
    if (C % 4 != 0 || C % G != 0 || HW % 7 != 0)
        return false;
    const int cpg = C / G;
    for (int Q = 32; Q >= 1; Q >>= 1) {  // widest strip first
        const int Ct = 4 * Q;
        if (NT % Q != 0 || (NT / Q) * 7 != HW || C % Ct != 0 || Ct % cpg != 0 || Ct * 4 < 64)
            continue;
        StripGeom g;
        g.HW = HW; g.C = C; g.G = G; g.cpg = cpg; g.Ct = Ct; g.Q = Q; g.RSTEP = NT / Q;
        g.Gt = Ct / cpg; g.nct = C / Ct;
        g.paced = 0; g.hint = tune_get("gn_strip_l2_hint", 0);
        out->NT = NT;
        out->VPT = 7;
        out->g = g;
        out->smem = 0;
        return ostrip_gpt(g) != 0;
    }
    return false;
}

template <int ACT>
static bool gn_forward_exact7(float* y, float* mu, float* rstd, const float* x, const float* gamma, const float* beta,
    int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    if (!tune_get("gn_exact7", 1) || !tune_get("gn_one_barrier", 1))
        return false;
    // one 896-thread CTA per SM (wider strips) when that leaves every CTA at least 6 strips, else two of 448 threads
    StripPlan plan;
    int per_sm = 1;
    long grid = 0, resident = 0, per_cta = 0;
    const int forced = tune_get("gn_exact7_fwd_nt", 0);
    for (int pass = 0; pass < 2; ++pass) {
        const int NT = pass == 0 ? 896 : 448;
        per_cta = 0;
        if ((forced && forced != NT) || !exact7_plan(&plan, HW, C, G, NT))
            continue;
        per_sm = NT == 896 ? 1 : 2;
        grid = (long)B * plan.g.nct;
        resident = (long)sm_count() * per_sm;
        if (grid <= resident || grid > 2147483647L)
            continue;
        per_cta = (grid + resident - 1) / resident;
        if (per_cta >= (NT == 896 ? 6 : tune_get("gn_exact7_min_fwd", 2)))
            break;
        per_cta = 0;
    }
    if (per_cta == 0)
        return false;
    const long pgrid = (grid + per_cta - 1) / per_cta;
    const int gpt = ostrip_gpt(plan.g);
    const size_t osmem = (size_t)plan.VPT * plan.NT * 16
        + (size_t)(gpt * plan.NT + 2 * C + 2 * plan.g.Gt * ostrip_row_floats(plan.NT / 32)) * sizeof(float);
    if (osmem * per_sm > 226 * 1024)
        return false;
    const bool full = true;
    plan.g.paced = per_cta >= 8;  // paced stores in the kernels without activation
    // (clusters of 4 as for the 1024-thread strips: [256,28,28,256] 0.83 -> 0.80, so none here)
    // staged loads marked evict_last: [256,28,28,256] forward 76.4 -> 66.7 us (0.82 -> 0.94), [256,28,28,128] 35.8 -> 34.6 us
    // (0.88 -> 0.91), [128,28,28,64] 11.4 -> 11.3 us
    const int fwd_hint_default = 1;
    OSTRIP_FWD_CASE(896, 7, 1) OSTRIP_FWD_CASE(448, 7, 2)
    return false;
}

template <int ACT>
static bool gn_backward_exact7(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    if (!tune_get("gn_exact7", 1) || !tune_get("gn_one_barrier", 1))
        return false;
    StripPlan plan;
    if (!exact7_plan(&plan, HW, C, G, 448))
        return false;
    const long grid = (long)B * plan.g.nct, resident = sm_count();
    if (grid <= resident || grid > 2147483647L)
        return false;
    const long per_cta = (grid + resident - 1) / resident;
    const long pgrid = (grid + per_cta - 1) / per_cta;
    if (per_cta < tune_get("gn_exact7_min_bwd", 6)) {
        // few strips per CTA: the three-barrier pipeline on the same exact-fill geometry, where there is an activation
        // to pay for ([128,28,28,64]: 21.9 -> 20.4 us with SiLU, but 18.0 -> 18.6 us without)
        if (ACT == ACT_IDENTITY || !tune_get("gn_exact7_pstrip", 1))
            return false;
        const int red = 2 * (plan.NT / 32) * plan.g.Ct;
        const size_t psmem = (size_t)2 * plan.VPT * plan.NT * 16 + (size_t)(red + 2 * plan.g.Ct + 2 * plan.g.Gt) * sizeof(float);
        Scratch sc;
        if (psmem > 220 * 1024 || !scratch_get(s, (size_t)2 * B * C, 0, &sc))
            return false;
        PSTRIP_BWD_CASE(448, 7, 1)
        return false;
    }
    const int gpt = ostrip_gpt(plan.g), nw = plan.NT / 32;
    const size_t osmem = (size_t)3 * plan.VPT * plan.NT * 16
        + (size_t)(2 * C + 2 * plan.g.Gt * ostrip_row_floats(nw)) * sizeof(float) + (size_t)2 * nw * 2 * plan.g.Q * 16 + (plan.g.Q == 4 ? (size_t)nw * 1024 : 0) + 128;
    if (osmem > 226 * 1024)
        return false;
    Scratch sc;
    if (!scratch_get(s, (size_t)2 * B * C, 0, &sc))
        return false;
    const bool full = true;
    OSTRIP_BWD_CASE(448, 7)
    return false;
}

template <int ACT>
static bool gn_forward_strip(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    if constexpr (ACT != ACT_IDENTITY && ACT != ACT_SILU && ACT != ACT_MP_SILU) {
        return false;
    } else {
        if (tune_get("gn_force_generic", 0) || tune_get("gn_no_strip", 0))
            return false;
        if (!(aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta)) || (long)B * HW * C >= 2147483648L)
            return false;
        if (gn_forward_exact7<ACT>(y, mu, rstd, x, gamma, beta, B, HW, C, G, eps, s))
            return true;
        StripPlan plan;
        if (!strip_plan(&plan, B, HW, C, G, 8, tune_get("gn_fwd_strip_ct", 0), tune_get("gn_fwd_strip_nt", 0), 0))
            return false;
        if (!tune_get("gn_fwd_strip_ct", 0) && strip_too_narrow(plan, HW, C, G))
            return false;
        const long grid = (long)B * plan.g.nct;
        if (grid > 2147483647L)
            return false;
        {
            // CTAs per SM: two 512-thread CTAs at 64 registers, or one at 128 registers (no spills)
            int per_sm = plan.NT <= 256 ? 4 : (plan.NT <= 512 ? tune_get("gn_fwd_pstrip_ctas", 2) : 1);
            const long resident = (long)sm_count() * per_sm;
            const size_t psmem = (size_t)plan.VPT * plan.NT * 16 + plan.smem;
            if (!tune_get("gn_no_pipeline", 0) && grid > resident && psmem * per_sm <= 220 * 1024) {
                // even share: every CTA gets (almost) the same number of strips
                const long per_cta = (grid + resident - 1) / resident;
                const long pgrid = (grid + per_cta - 1) / per_cta;
                const bool full = plan.g.RSTEP * plan.VPT == HW;
                // one barrier per strip
                const int gpt = tune_get("gn_one_barrier", 1) ? ostrip_gpt(plan.g) : 0;
                const size_t osmem = (size_t)plan.VPT * plan.NT * 16
                    + (size_t)(gpt * plan.NT + 2 * C + 2 * plan.g.Gt * ostrip_row_floats(plan.NT / 32)) * sizeof(float);
                // (with few strips per CTA the longer set-up of these kernels costs more than the barriers save)
                if (gpt && osmem * per_sm <= 226 * 1024 && per_cta >= tune_get("gn_one_barrier_min_fwd", 3)) {
                    // clusters of 4 neighbouring strips, staged in step (see gn_fwd_ostrip)
                    const int cw = tune_get("gn_fwd_cluster", 4);
                    // (ragged strips, 28 x 28 in 1024 slots, lose from it: 0.66 -> 0.58)
                    const bool clustered = cw > 1 && per_sm == 1 && full && plan.g.nct % cw == 0 && per_cta >= 8;
                    ClusterScope cluster(clustered ? cw : 1);
                    plan.g.paced = per_cta >= 8;  // paced stores in the kernels without activation
                    // staged loads marked evict_last: [256,32,32,128] 50.7 -> 46.5 us (0.81 -> 0.88); [256,32,32,256] (in
                    // clusters) and [256,16,16,256] within 1 % either way.  (In the backward and in the pipelined and
                    // chunked kernels -- tunables "gn_bwd_l2_hint", "gn_strip_l2_hint" -- nothing moved by more than 1 %.)
                    const int fwd_hint_default = 1;
                    OSTRIP_FWD_CASE(1024, 4, 1) OSTRIP_FWD_CASE(1024, 8, 1)
                    OSTRIP_FWD_CASE(512, 4, 2) OSTRIP_FWD_CASE(512, 8, 2)
                }
                PSTRIP_FWD_CASE(1024, 4, 1) PSTRIP_FWD_CASE(1024, 8, 1)
                PSTRIP_FWD_CASE(512, 4, 2) PSTRIP_FWD_CASE(512, 8, 2) PSTRIP_FWD_CASE(512, 8, 1)
                PSTRIP_FWD_CASE(256, 4, 4) PSTRIP_FWD_CASE(256, 8, 4)
            }
        }
        STRIP_FWD_CASE(1024, 2) STRIP_FWD_CASE(1024, 4) STRIP_FWD_CASE(1024, 8)
        STRIP_FWD_CASE(512, 2) STRIP_FWD_CASE(512, 4) STRIP_FWD_CASE(512, 8)
        STRIP_FWD_CASE(256, 2) STRIP_FWD_CASE(256, 4) STRIP_FWD_CASE(256, 8)
        return false;
    }
}

template <int ACT>
static bool gn_backward_strip(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    if constexpr (ACT != ACT_IDENTITY && ACT != ACT_SILU && ACT != ACT_MP_SILU) {
        return false;
    } else {
        if (tune_get("gn_force_generic", 0) || tune_get("gn_no_strip", 0))
            return false;
        if (!(aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(gamma)) || (long)B * HW * C >= 2147483648L)
            return false;
        if (ACT != ACT_IDENTITY && !aligned16(beta))
            return false;
        if (gn_backward_exact7<ACT>(dx, dgamma, dbeta, dy, x, gamma, beta, mu, rstd, B, HW, C, G, s))
            return true;
        StripPlan plan;
        const int force_nt = tune_get("gn_bwd_strip_nt", 0);
        // 512-thread CTAs may hold 8 rows per tensor (one CTA per SM, 128 registers per thread)
        const int max_vpt = tune_get("gn_bwd_strip_vpt", 8);
        if (!strip_plan(&plan, B, HW, C, G, max_vpt, tune_get("gn_bwd_strip_ct", 0), force_nt, max_vpt == 8 ? 1 : 0))
            return false;
        if (plan.VPT == 8 && plan.NT != 512)
            return false;
        if (!tune_get("gn_bwd_strip_ct", 0) && strip_too_narrow(plan, HW, C, G))
            return false;
        const long grid = (long)B * plan.g.nct;
        if (grid > 2147483647L)
            return false;
        Scratch sc;
        if (!scratch_get(s, (size_t)2 * B * C, 0, &sc))
            return false;
        {
            const int per_sm = (plan.VPT == 8 || plan.NT == 1024) ? 1 : (plan.NT <= 256 ? 2 : 1);
            const long resident = (long)sm_count() * per_sm;
            const size_t psmem = (size_t)2 * plan.VPT * plan.NT * 16 + plan.smem;
            if (tune_get("gn_bwd_pipeline", 1) && grid > resident && psmem * per_sm <= 220 * 1024) {
                // even share: every CTA gets (almost) the same number of strips
                const long per_cta = (grid + resident - 1) / resident;
                const long pgrid = (grid + per_cta - 1) / per_cta;
                const bool full = plan.g.RSTEP * plan.VPT == HW;
                const size_t dsmem = (size_t)3 * plan.VPT * plan.NT * 16 + plan.smem;
                // (2 % faster than the plain pipeline when every CTA walks many strips; with only a few strips per
                // CTA the longer prologue costs more than the deeper staging gains)
                const int gpt = tune_get("gn_one_barrier", 1) ? ostrip_gpt(plan.g) : 0;
                const int nw = plan.NT / 32;
                const size_t osmem = (size_t)3 * plan.VPT * plan.NT * 16
                    + (size_t)(2 * C + 2 * plan.g.Gt * ostrip_row_floats(nw)) * sizeof(float)
                    + (size_t)2 * nw * 2 * plan.g.Q * 16 + (plan.g.Q == 4 ? (size_t)nw * 1024 : 0) + 128;
                // (a cluster barrier per strip, as in the forward kernel, was measured here too: 0.89 -> 0.78 with
                // pairs, worse with wider clusters -- the backward has no idle time to absorb the lock step)
                if (gpt && per_sm == 1 && osmem <= 226 * 1024 && per_cta >= tune_get("gn_one_barrier_min", 6)) {
                    OSTRIP_BWD_CASE(1024, 4) OSTRIP_BWD_CASE(512, 4) OSTRIP_BWD_CASE(512, 8)
                }
                if (tune_get("gn_deep", 1) && per_sm == 1 && dsmem <= 226 * 1024 && grid >= 8 * pgrid) {
                    DSTRIP_BWD_CASE(1024, 4) DSTRIP_BWD_CASE(512, 4) DSTRIP_BWD_CASE(512, 8)
                }
                PSTRIP_BWD_CASE(1024, 4, 1) PSTRIP_BWD_CASE(512, 4, 1) PSTRIP_BWD_CASE(512, 8, 1)
                PSTRIP_BWD_CASE(256, 4, 2)
            }
        }
        STRIP_BWD_CASE(1024, 2, 1) STRIP_BWD_CASE(1024, 4, 1)
        STRIP_BWD_CASE(512, 2, 2) STRIP_BWD_CASE(512, 4, 2) STRIP_BWD_CASE(512, 8, 1)
        STRIP_BWD_CASE(256, 2, 4) STRIP_BWD_CASE(256, 4, 4)
        return false;
    }
}

// Chunked strips for samples too tall for the register-resident strips: 512 threads, strip width Ct =
// the narrowest whole-group width with runs of at least 64 bytes (more strips, smaller L2 footprint).
static bool cstrip_plan(StripPlan* out, int HW, int C, int G)
{
    if (C % 4 != 0 || C % G != 0)
        return false;
    const int NT = 512, cpg = C / G;
    int best = 0;
    for (int Ct = 4; Ct <= C && Ct <= 512; Ct += 4) {
        if (C % Ct != 0 || Ct % cpg != 0 || NT % (Ct / 4) != 0)
            continue;
        if (best == 0 || (best * 4 < 64 && Ct > best))
            best = Ct;
    }
    if (best == 0)
        return false;
    StripGeom g;
    g.HW = HW; g.C = C; g.G = G; g.cpg = cpg; g.Ct = best; g.Q = best / 4; g.RSTEP = NT / g.Q;
    g.Gt = best / cpg; g.nct = C / best;
    g.paced = 0; g.hint = tune_get("gn_strip_l2_hint", 0);
    out->NT = NT;
    out->VPT = 0;
    out->g = g;
    const int red = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * (NT / 32) * best : 2 * NT * 4;
    out->smem = (size_t)(red + 2 * best + 2 * g.Gt) * sizeof(float);
    return true;
}

template <int ACT>
static bool gn_forward_cstrip(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    if constexpr (ACT != ACT_IDENTITY && ACT != ACT_SILU && ACT != ACT_MP_SILU) {
        return false;
    } else {
        if (tune_get("gn_force_generic", 0) || tune_get("gn_no_cstrip", 0))
            return false;
        if (!(aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta)) || (long)B * HW * C >= 2147483648L)
            return false;
        StripPlan plan;
        if (!cstrip_plan(&plan, HW, C, G))
            return false;
        // 4 rows per thread keep the kernel inside 64 registers (two CTAs per SM, no spills); 8 rows double the
        // bytes each CTA has in flight at the price of a few spilled registers
        const int VPT = tune_get("gn_fwd_cstrip_vpt", 4) == 8 ? 8 : 4;
        constexpr int MB = 2;
        const long items = (long)B * plan.g.nct;
        const long resident = (long)sm_count() * MB;
        const long per_cta = (items + resident - 1) / resident;
        const long pgrid = (items + per_cta - 1) / per_cta;
        const int nchunks = (HW + plan.g.RSTEP * VPT - 1) / (plan.g.RSTEP * VPT);
        const size_t psmem = (size_t)VPT * plan.NT * 16 + plan.smem;
        static bool done4[64] = { false }, done8[64] = { false };
        if (VPT == 8)
            return pstrip_launch(GN_PATH_CHUNKED, gn_fwd_cstrip<512, 8, ACT, MB>, done8, pgrid, 512, psmem, s, y, mu, rstd, x, gamma, beta,
                plan.g, eps, (int)items, nchunks);
        return pstrip_launch(GN_PATH_CHUNKED, gn_fwd_cstrip<512, 4, ACT, MB>, done4, pgrid, 512, psmem, s, y, mu, rstd, x, gamma, beta,
            plan.g, eps, (int)items, nchunks);
    }
}

template <int ACT>
static bool gn_backward_cstrip(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    if constexpr (ACT != ACT_IDENTITY && ACT != ACT_SILU && ACT != ACT_MP_SILU) {
        return false;
    } else {
        if (tune_get("gn_force_generic", 0) || tune_get("gn_no_cstrip", 0))
            return false;
        if (!(aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(gamma)) || (long)B * HW * C >= 2147483648L)
            return false;
        if (ACT != ACT_IDENTITY && !aligned16(beta))
            return false;
        StripPlan plan;
        if (!cstrip_plan(&plan, HW, C, G))
            return false;
        Scratch sc;
        if (!scratch_get(s, (size_t)2 * B * C, 0, &sc))
            return false;
        // 8 rows per tensor and thread at one CTA per SM (128 registers), or 4 rows at two CTAs per SM (64
        // registers, some spills in the SiLU variants)
        const int VPT = tune_get("gn_bwd_cstrip_vpt", 8) == 4 ? 4 : 8, MB = VPT == 4 ? 2 : 1;
        const long items = (long)B * plan.g.nct;
        const long resident = (long)sm_count() * MB;
        const long per_cta = (items + resident - 1) / resident;
        const long pgrid = (items + per_cta - 1) / per_cta;
        const int nchunks = (HW + plan.g.RSTEP * VPT - 1) / (plan.g.RSTEP * VPT);
        const size_t psmem = (size_t)2 * VPT * plan.NT * 16 + plan.smem;
        static bool done4[64] = { false }, done8[64] = { false };
        const bool ok = VPT == 4
            ? pstrip_launch(GN_PATH_CHUNKED, gn_bwd_cstrip<512, 4, ACT, 2>, done4, pgrid, 512, psmem, s, dx, sc.partials, dy, x, gamma, beta,
                  mu, rstd, plan.g, (int)items, nchunks)
            : pstrip_launch(GN_PATH_CHUNKED, gn_bwd_cstrip<512, 8, ACT, 1>, done8, pgrid, 512, psmem, s, dx, sc.partials, dy, x, gamma, beta,
                  mu, rstd, plan.g, (int)items, nchunks);
        return ok && (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true);
    }
}

template <int ACT>
static void gn_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma, const float* beta,
    int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    if (gn_forward_strip<ACT>(y, mu, rstd, x, gamma, beta, B, HW, C, G, eps, s))
        return;
    if (gn_forward_cstrip<ACT>(y, mu, rstd, x, gamma, beta, B, HW, C, G, eps, s))
        return;
    if (planning_only()) {
        t_planned.path = GN_PATH_GENERIC;
        t_planned.nt = GN_GENERIC_THREADS;
        t_planned.grid = (long)B * G;
        return;
    }
    gn_path(GN_PATH_GENERIC, true);
    launch_k(gn_fwd_generic<ACT>, B * G, GN_GENERIC_THREADS, 0, s, y, mu, rstd, x, gamma, beta, HW, C, G, eps);
    count_launch();
    B200_CHECK_LAUNCH();
}

template <int ACT>
static void gn_backward(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    if (gn_backward_strip<ACT>(dx, dgamma, dbeta, dy, x, gamma, beta, mu, rstd, B, HW, C, G, s))
        return;
    if (gn_backward_cstrip<ACT>(dx, dgamma, dbeta, dy, x, gamma, beta, mu, rstd, B, HW, C, G, s))
        return;
    Scratch sc;
    B200_REQUIRE(scratch_get(s, (size_t)2 * B * C, 0, &sc), "groupnorm_backward: scratch allocation failed (the arena cannot grow during stream capture: call b200_scratch_reserve before capturing)");
    B200_REQUIRE(B <= 65535, "groupnorm_backward: batch %d too large for the generic path", B);
    if (planning_only()) {
        t_planned.path = GN_PATH_GENERIC;
        t_planned.nt = GN_GENERIC_THREADS;
        t_planned.grid = (long)B * G;
        return;
    }
    gn_path(GN_PATH_GENERIC, true);
    launch_k(gn_bwd_dx_generic<ACT>, B * G, GN_GENERIC_THREADS, 0, s, dx, dy, x, gamma, beta, mu, rstd, HW, C, G);
    count_launch();
    B200_CHECK_LAUNCH();
    launch_k(gn_bwd_param_generic<ACT>, dim3((C + 31) / 32, B), dim3(32, 8), 0, s, sc.partials, dy, x, gamma, beta, mu,
        rstd, HW, C, G);
    count_launch();
    B200_CHECK_LAUNCH();
    fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s);
}

#define GN_DISPATCH_ACT(act, CALL)                                       \
    switch (act) {                                                       \
    case ACT_IDENTITY: { constexpr int A = ACT_IDENTITY; CALL; } break;  \
    case ACT_RELU: { constexpr int A = ACT_RELU; CALL; } break;          \
    case ACT_GELU: { constexpr int A = ACT_GELU; CALL; } break;          \
    case ACT_SILU: { constexpr int A = ACT_SILU; CALL; } break;          \
    case ACT_TANH: { constexpr int A = ACT_TANH; CALL; } break;          \
    case ACT_MP_SILU: { constexpr int A = ACT_MP_SILU; CALL; } break;    \
    default: report_error(__FILE__, __LINE__, "groupnorm: unknown activation %d", (int)(act)); break; \
    }

static bool gn_args_ok(const char* who, int batch, int HW, int C, int G)
{
    if (batch < 0 || HW <= 0 || C <= 0 || G <= 0 || C % G != 0) {
        report_error(__FILE__, __LINE__, "%s: bad extents batch=%d HW=%d C=%d G=%d (C must be divisible by G)", who,
            batch, HW, C, G);
        return false;
    }
    if ((long)batch * HW * C >= 2147483648L) {
        report_error(__FILE__, __LINE__, "%s: more than 2^31-1 elements", who);
        return false;
    }
    return true;
}

}  // namespace b200

using namespace b200;

extern "C" {

void launch_groupnorm_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int HW, int C, int G, float eps, cudaStream_t s)
{
    if (!gn_args_ok("groupnorm_forward", batch, HW, C, G) || batch == 0)
        return;
    gn_forward<ACT_IDENTITY>(y, mu, rstd, x, gamma, beta, batch, HW, C, G, eps, s);
}

void launch_groupnorm_backward(float* dx, float* ggamma, float* gbeta, const float* dy, const float* x,
    const float* gamma, const float* mu, const float* rstd, int batch, int HW, int C, int G, cudaStream_t s)
{
    if (!gn_args_ok("groupnorm_backward", batch, HW, C, G) || batch == 0)
        return;
    gn_backward<ACT_IDENTITY>(dx, ggamma, gbeta, dy, x, gamma, nullptr, mu, rstd, batch, HW, C, G, s);
}

void launch_groupnorm_act_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int batch, int HW, int C, int G, float eps, b200_act_t act, cudaStream_t s)
{
    if (!gn_args_ok("groupnorm_act_forward", batch, HW, C, G) || batch == 0)
        return;
    GN_DISPATCH_ACT((int)act, (gn_forward<A>(y, mu, rstd, x, gamma, beta, batch, HW, C, G, eps, s)));
}

void launch_groupnorm_act_backward(float* dx, float* ggamma, float* gbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int batch, int HW, int C,
    int G, b200_act_t act, cudaStream_t s)
{
    if (!gn_args_ok("groupnorm_act_backward", batch, HW, C, G) || batch == 0)
        return;
    GN_DISPATCH_ACT((int)act, (gn_backward<A>(dx, ggamma, gbeta, dy, x, gamma, beta, mu, rstd, batch, HW, C, G, s)));
}

int b200_groupnorm_describe(int batch, int HW, int C, int G, int act, int backward, char* out, int out_len)
{
    if (!out || out_len <= 0 || batch <= 0 || HW <= 0 || C <= 0 || G <= 0 || C % G != 0)
        return -1;
    static const char* const names[] = { "strip", "pipelined", "deep-staged", "one-barrier", "chunked", "generic" };
    b200::t_planned = b200::PlannedLaunch();
    b200::t_planned.path = -1;
    b200::t_planned.cluster = 1;
    b200::planning_only_set(true);
    float* none = nullptr;
    if (backward) {
        GN_DISPATCH_ACT(act, (gn_backward<A>(none, none, none, none, none, none, none, none, none, batch, HW, C, G, nullptr)));
    } else {
        GN_DISPATCH_ACT(act, (gn_forward<A>(none, none, none, none, none, none, batch, HW, C, G, 1e-5f, nullptr)));
    }
    b200::planning_only_set(false);
    const b200::PlannedLaunch& p = b200::t_planned;
    if (p.path < 0 || p.path >= b200::GN_PATHS)
        return -1;
    return snprintf(out, (size_t)out_len, "family=%s threads=%d strip_channels=%d ctas=%ld cluster=%d smem=%zu", names[p.path],
        p.nt, p.ct, p.grid, p.cluster, p.smem);
}

long long b200_groupnorm_path_count(int path)
{
    return path >= 0 && path < b200::GN_PATHS ? b200::g_gn_path[path].load(std::memory_order_relaxed) : -1;
}

}  // extern "C"
