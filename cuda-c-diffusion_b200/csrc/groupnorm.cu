// NHWC GroupNorm forward / backward, optionally fused with an activation
// (reference: src/kernels.cu:622-745, composed with :103-117 by conv_residual.c).
//
// x is viewed as a matrix [B*HW, C]; a work item is (sample b, Ct channels covering whole groups).
// Four kernel families, tried in this order by gn_forward / gn_backward:
//
//   1. register-resident strips (groupnorm_strip.cuh): the default.  A CTA keeps all HW rows of an
//      item in registers, statistics and output come from registers, the next item is staged with
//      cp.async while the current one is processed.  x (and dy) cross HBM exactly once.
//   2. chunked strips (groupnorm_cstrip.cuh): samples too tall for the register file; the strip is
//      walked twice in chunks, the second read coming from L2 while the strips in flight fit there.
//   3. tile kernels (this file), kept selectable (tunables gn_no_strip / gn_no_cstrip): a thread-block
//      cluster of CS CTAs splits the rows of an item and holds it in shared memory; 2-D bulk tensor
//      copies (TMA) with mbarrier completion bring tiles in and take results out, clusters are
//      persistent and double-buffered, per-channel partial statistics are folded with warp shuffles
//      and across the cluster through distributed shared memory, and the last item of a channel tile
//      (atomic ticket) adds the per-sample dgamma/dbeta partials in a fixed order.  Every wait on an
//      mbarrier is bounded and reports through the device error word.  Slower than 1 and 2 on every
//      shape measured (the cluster barrier and the DSMEM round trip sit on each item's critical path).
//   4. generic kernels (this file): any shape, any alignment (C % 4 != 0, misaligned pointers).
//
// Backward in every family reuses the per-channel sums of g and g*xhat (g = dy * act'(z)) for BOTH
// the group sums that dx needs and the per-sample dgamma/dbeta partials, which a fixed-order fold
// adds up: parameter gradients are overwritten and bit-reproducible.
#include "dev_common.cuh"
#include "tma_desc.cuh"
#include "../../include/b200_layer_kernels.h"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace b200 {

constexpr int GN_THREADS = 512;
constexpr int GN_WARPS = GN_THREADS / 32;
constexpr int GN_NBUF = 2;         // tile buffers per CTA (double buffering)
constexpr int GN_MAX_CHUNKS = 8;   // TMA boxes per tile
constexpr int GN_GENERIC_THREADS = 256;

struct GnGeom {
    int HW, C, G, cpg;
    int Ct;        // channels per tile (multiple of cpg and of 4)
    int Q;         // Ct / 4 float4 columns
    int RSTEP;     // row lanes = GN_THREADS / Q
    int CS;        // cluster size: CTAs that split the HW rows of an item
    int R;         // rows per CTA = HW / CS
    int RB;        // rows per TMA box
    int nchunk;    // R / RB
    int Gt;        // groups per tile = Ct / cpg
    int nct;       // channel tiles per sample = C / Ct
    int items;     // B * nct
    int nclusters; // clusters in the grid (each loops over items)
    int shuffle;   // 1: Q divides 32, row lanes of a warp are folded with shuffles
    int red_floats;
    int ntensors;  // 1 forward (x), 2 backward (x, dy)
};

// tile footprint in shared memory, padded so that the next tile stays 128-byte aligned
__host__ __device__ static inline size_t gn_tile_bytes(const GnGeom& g)
{
    return ((size_t)g.R * g.Ct * sizeof(float) + 127) & ~(size_t)127;
}

static inline size_t gn_smem_bytes(const GnGeom& g)
{
    // tiles | fold buffer | per-channel pairs (one per buffer) | per-group pair | barriers
    return (size_t)GN_NBUF * g.ntensors * gn_tile_bytes(g) + (size_t)g.red_floats * sizeof(float)
        + (size_t)GN_NBUF * 2 * g.Ct * sizeof(float) + 2 * g.Gt * sizeof(float)
        + GN_NBUF * GN_MAX_CHUNKS * sizeof(uint64_t) + 128 + 16;
}

static int largest_divisor_leq(int n, int cap)
{
    for (int d = cap < n ? cap : n; d >= 1; --d)
        if (n % d == 0)
            return d;
    return 1;
}

// Picks (Ct, CS) and the persistent grid.
// Preference: the double-buffered tile set within `budget` bytes (so that
// `ctas_per_sm` CTAs share an SM), rows of at least 128 bytes, the smallest
// cluster, then the widest tile.
static bool gn_pick_geometry(GnGeom* out, int B, int HW, int C, int G, int ntensors, int force_ct, int force_cs,
    size_t budget, int ctas_per_sm)
{
    if (C % 4 != 0 || G <= 0 || C % G != 0)
        return false;
    const int cpg = C / G;
    const size_t hard_cap = 200 * 1024;
    bool found = false;
    long best_score = -1;
    for (int Ct = 4; Ct <= C && Ct <= 256; Ct += 4) {
        if (C % Ct != 0 || Ct % cpg != 0)
            continue;
        if (force_ct > 0 && Ct != force_ct)
            continue;
        const int Q = Ct / 4;
        if (Q > GN_THREADS)
            continue;
        for (int CS = 1; CS <= 8; CS *= 2) {
            if (HW % CS != 0)
                continue;
            if (force_cs > 0 && CS != force_cs)
                continue;
            GnGeom g = {};
            g.HW = HW; g.C = C; g.G = G; g.cpg = cpg;
            g.Ct = Ct; g.Q = Q; g.RSTEP = GN_THREADS / Q; g.CS = CS;
            g.R = HW / CS;
            g.RB = largest_divisor_leq(g.R, 256);
            g.nchunk = g.R / g.RB;
            g.Gt = Ct / cpg;
            g.nct = C / Ct;
            g.items = B * g.nct;
            g.ntensors = ntensors;
            g.shuffle = (Q <= 32 && 32 % Q == 0) ? 1 : 0;
            g.red_floats = g.shuffle ? 2 * GN_WARPS * Ct : 2 * GN_THREADS * 4;
            if (g.nchunk > GN_MAX_CHUNKS || (g.RB < 8 && g.R >= 8) || g.R < 2)
                continue;
            // every chunk must start on a 128-byte boundary of shared memory
            if (g.nchunk > 1 && (g.RB * Ct) % 32 != 0)
                continue;
            const size_t bytes = (size_t)GN_NBUF * ntensors * gn_tile_bytes(g);
            if (bytes > hard_cap)
                continue;
            long score = 0;
            if (bytes <= budget)
                score += 1000000;
            if (Ct * 4 >= 128)
                score += 100000;
            score += (8 - CS) * 10000;
            score += Ct;
            if (bytes > budget)
                score -= (long)(bytes / 1024);
            if (score > best_score) {
                best_score = score;
                *out = g;
                found = true;
            }
        }
    }
    if (!found)
        return false;
    // persistent grid: as many clusters as fit, then evened out so that every
    // cluster gets (almost) the same number of items
    GnGeom& g = *out;
    const size_t smem = gn_smem_bytes(g);
    int fit = (int)((size_t)227 * 1024 / (smem + 1024));
    if (fit < 1)
        fit = 1;
    if (fit > ctas_per_sm)
        fit = ctas_per_sm;
    if (fit * GN_THREADS > 2048)
        fit = 2048 / GN_THREADS;
    int max_clusters = sm_count() * fit / g.CS;
    if (max_clusters < 1)
        max_clusters = 1;
    if (g.items <= max_clusters) {
        g.nclusters = g.items;
    } else {
        const int per = (g.items + max_clusters - 1) / max_clusters;
        g.nclusters = (g.items + per - 1) / per;
    }
    return true;
}

// ---------------------------------------------------------------------------
// shared pieces of the tile kernels
// ---------------------------------------------------------------------------
struct GnSmem {
    float* tiles;   // [GN_NBUF][ntensors] tiles
    float* red;     // red_floats
    float* chan;    // [GN_NBUF][2*Ct], read by cluster peers
    float* gstat;   // 2*Gt
    uint64_t* bars; // [GN_NBUF][GN_MAX_CHUNKS]
    size_t tile_floats;
};

__device__ __forceinline__ GnSmem gn_carve(unsigned char* raw, const GnGeom& g)
{
    GnSmem s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(raw) + 127) & ~uintptr_t(127);
    s.tiles = reinterpret_cast<float*>(p);
    s.tile_floats = gn_tile_bytes(g) / sizeof(float);
    p += (size_t)GN_NBUF * g.ntensors * gn_tile_bytes(g);
    s.red = reinterpret_cast<float*>(p);
    p += (size_t)g.red_floats * sizeof(float);
    s.chan = reinterpret_cast<float*>(p);
    p += (size_t)GN_NBUF * 2 * g.Ct * sizeof(float);
    s.gstat = reinterpret_cast<float*>(p);
    p += 2 * g.Gt * sizeof(float);
    p = (p + 7) & ~uintptr_t(7);
    s.bars = reinterpret_cast<uint64_t*>(p);
    return s;
}

__device__ __forceinline__ float* gn_tile(const GnSmem& s, const GnGeom& g, int buf, int tensor)
{
    return s.tiles + (size_t)(buf * g.ntensors + tensor) * s.tile_floats;
}

__device__ __forceinline__ float4 shfl_xor4(float4 v, int off)
{
    v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
    v.z += __shfl_xor_sync(0xffffffffu, v.z, off);
    v.w += __shfl_xor_sync(0xffffffffu, v.w, off);
    return v;
}

// Sums the per-thread float4 pairs (a, b) over all row lanes of the CTA and
// stores, for every channel c of the tile, the totals into dst[c] and
// dst[Ct + c].  The caller synchronises before reading dst and before the next
// use of `red`.
__device__ __forceinline__ void gn_fold_rows(float* red, float* dst, const GnGeom& g, int q, int rr, bool active,
    float4 a, float4 b)
{
    const int t = threadIdx.x;
    if (g.shuffle) {
        for (int off = g.Q; off < 32; off <<= 1) {
            a = shfl_xor4(a, off);
            b = shfl_xor4(b, off);
        }
        const int lane = t & 31, warp = t >> 5;
        if (lane < g.Q) {
            reinterpret_cast<float4*>(red)[warp * g.Q + lane] = a;
            reinterpret_cast<float4*>(red + GN_WARPS * g.Ct)[warp * g.Q + lane] = b;
        }
        __syncthreads();
        if (t < g.Ct) {
            float sa = 0.0f, sb = 0.0f;
#pragma unroll
            for (int w = 0; w < GN_WARPS; ++w) {
                sa += red[w * g.Ct + t];
                sb += red[GN_WARPS * g.Ct + w * g.Ct + t];
            }
            dst[t] = sa;
            dst[g.Ct + t] = sb;
        }
    } else {
        float4* ra = reinterpret_cast<float4*>(red);
        float4* rb = reinterpret_cast<float4*>(red + GN_THREADS * 4);
        if (active) {
            ra[rr * g.Q + q] = a;
            rb[rr * g.Q + q] = b;
        }
        __syncthreads();
        if (t < g.Ct) {
            float sa = 0.0f, sb = 0.0f;
            for (int r = 0; r < g.RSTEP; ++r) {
                sa += red[r * g.Ct + t];
                sb += red[GN_THREADS * 4 + r * g.Ct + t];
            }
            dst[t] = sa;
            dst[g.Ct + t] = sb;
        }
    }
}

// thread 0: (re)arm the barriers of buffer `buf` and start the loads of `item`
__device__ __forceinline__ void gn_issue_loads(const GnSmem& sm, const GnGeom& g, int buf, int item, int rank,
    const CUtensorMap* map0, const CUtensorMap* map1)
{
    const int ctile = item % g.nct, b = item / g.nct;
    const int c0 = ctile * g.Ct;
    const int row0 = b * g.HW + rank * g.R;
    const unsigned chunk_bytes = (unsigned)(g.RB * g.Ct * sizeof(float));
    for (int c = 0; c < g.nchunk; ++c) {
        uint64_t* bar = &sm.bars[buf * GN_MAX_CHUNKS + c];
        mbar_expect_tx(bar, chunk_bytes * g.ntensors);
        tma_load_2d(gn_tile(sm, g, buf, 0) + (size_t)c * g.RB * g.Ct, map0, c0, row0 + c * g.RB, bar);
        if (g.ntensors == 2)
            tma_load_2d(gn_tile(sm, g, buf, 1) + (size_t)c * g.RB * g.Ct, map1, c0, row0 + c * g.RB, bar);
    }
}

// Warp-parallel combine of the per-channel (mean, centred sum of squares) pairs of
// all CTAs of the cluster into group statistics (Chan et al. pairwise update with
// equal counts).  Warp w handles groups w, w+GN_WARPS, ...
__device__ __forceinline__ void gn_group_stats(cg::cluster_group& cluster, const GnSmem& sm, const GnGeom& g,
    float* chan, int rank, int group0, float eps, float* __restrict__ mu, float* __restrict__ rstd, int b)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nparts = g.CS * g.cpg;
    for (int grp = warp; grp < g.Gt; grp += GN_WARPS) {
        float msum = 0.0f;
        for (int e = lane; e < nparts; e += 32) {
            const float* peer = cluster.map_shared_rank(chan, e / g.cpg);
            msum += peer[grp * g.cpg + e % g.cpg];
        }
        const float mean = warp_sum(msum) / (float)nparts;
        float m2 = 0.0f;
        for (int e = lane; e < nparts; e += 32) {
            const float* peer = cluster.map_shared_rank(chan, e / g.cpg);
            const int ch = grp * g.cpg + e % g.cpg;
            const float d = peer[ch] - mean;
            m2 += peer[g.Ct + ch] + (float)g.R * d * d;
        }
        m2 = warp_sum(m2);
        const float rs = rsqrtf(m2 / ((float)g.R * (float)nparts) + eps);
        if (lane == 0) {
            sm.gstat[grp] = mean;
            sm.gstat[g.Gt + grp] = rs;
            if (rank == 0) {
                mu[b * g.G + group0 + grp] = mean;
                rstd[b * g.G + group0 + grp] = rs;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <int ACT>
__global__ void __launch_bounds__(GN_THREADS, 2) gn_fwd_tile(const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_y, float* __restrict__ mu, float* __restrict__ rstd,
    const float* __restrict__ gamma, const float* __restrict__ beta, const GnGeom g, const float eps, int* err)
{
    extern __shared__ unsigned char gn_smem_raw[];
    cg::cluster_group cluster = cg::this_cluster();
    const GnSmem sm = gn_carve(gn_smem_raw, g);
    const int t = threadIdx.x;
    const int rank = (int)cluster.block_rank();
    const int cluster_id = blockIdx.x / g.CS;
    const int q = t % g.Q, rr = t / g.Q;
    const bool active = rr < g.RSTEP;

    if (t == 0) {
        for (int i = 0; i < GN_NBUF * GN_MAX_CHUNKS; ++i)
            mbar_init(&sm.bars[i], 1);
        mbar_init_fence();
        gn_issue_loads(sm, g, 0, cluster_id, rank, &map_x, nullptr);
    }
    __syncthreads();

    int it = 0;
    for (int item = cluster_id; item < g.items; item += g.nclusters, ++it) {
        const int buf = it & 1;
        const unsigned parity = (unsigned)(it >> 1) & 1u;
        const int ctile = item % g.nct, b = item / g.nct;
        const int c0 = ctile * g.Ct;
        const int row0 = b * g.HW + rank * g.R;
        // prefetch the next item into the other buffer once its stores have drained
        if (t == 0 && item + g.nclusters < g.items) {
            tma_store_wait_read();
            gn_issue_loads(sm, g, buf ^ 1, item + g.nclusters, rank, &map_x, nullptr);
        }
        float* tile = gn_tile(sm, g, buf, 0);
        float* chan = sm.chan + (size_t)buf * 2 * g.Ct;

        // ---- statistics, shifted by row 0 of the tile (K) so that the one-pass
        //      sums of (x-K) and (x-K)^2 do not cancel
        const float4* tile4 = reinterpret_cast<const float4*>(tile);
        float4 K = make_float4(0.f, 0.f, 0.f, 0.f), s1 = K, s2 = K;
        for (int c = 0; c < g.nchunk; ++c) {
            mbar_wait(&sm.bars[buf * GN_MAX_CHUNKS + c], parity, err);
            if (active) {
                if (c == 0)
                    K = tile4[q];
                for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                    const float4 v = tile4[(size_t)(c * g.RB + lr) * g.Q + q];
                    const float d0 = v.x - K.x, d1 = v.y - K.y, d2 = v.z - K.z, d3 = v.w - K.w;
                    s1.x += d0; s1.y += d1; s1.z += d2; s1.w += d3;
                    s2.x += d0 * d0; s2.y += d1 * d1; s2.z += d2 * d2; s2.w += d3 * d3;
                }
            }
        }
        gn_fold_rows(sm.red, chan, g, q, rr, active, s1, s2);
        if (t < g.Ct) {
            const float invR = 1.0f / (float)g.R;
            const float S1 = chan[t], S2 = chan[g.Ct + t];
            chan[t] = tile[t] + S1 * invR;          // channel mean over this CTA's rows
            chan[g.Ct + t] = S2 - S1 * S1 * invR;   // centred sum of squares
        }
        if (g.CS > 1)
            cluster.sync();
        else
            __syncthreads();
        gn_group_stats(cluster, sm, g, chan, rank, c0 / g.cpg, eps, mu, rstd, b);
        __syncthreads();

        // ---- y = act(x*a + b') with a = gamma*rstd, b' = beta - mean*a; in place, then TMA store
        float4 sc = make_float4(0.f, 0.f, 0.f, 0.f), sh = sc;
        if (active) {
            const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
            const float4 be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
            const int cb = 4 * q;
            const int g0 = (cb + 0) / g.cpg, g1 = (cb + 1) / g.cpg, g2 = (cb + 2) / g.cpg, g3 = (cb + 3) / g.cpg;
            sc.x = ga.x * sm.gstat[g.Gt + g0]; sh.x = be.x - sm.gstat[g0] * sc.x;
            sc.y = ga.y * sm.gstat[g.Gt + g1]; sh.y = be.y - sm.gstat[g1] * sc.y;
            sc.z = ga.z * sm.gstat[g.Gt + g2]; sh.z = be.z - sm.gstat[g2] * sc.z;
            sc.w = ga.w * sm.gstat[g.Gt + g3]; sh.w = be.w - sm.gstat[g3] * sc.w;
        }
        float4* wtile4 = reinterpret_cast<float4*>(tile);
        for (int c = 0; c < g.nchunk; ++c) {
            if (active) {
                for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                    float4* p = wtile4 + (size_t)(c * g.RB + lr) * g.Q + q;
                    float4 v = *p;
                    v.x = act_value<ACT>(fmaf(v.x, sc.x, sh.x));
                    v.y = act_value<ACT>(fmaf(v.y, sc.y, sh.y));
                    v.z = act_value<ACT>(fmaf(v.z, sc.z, sh.z));
                    v.w = act_value<ACT>(fmaf(v.w, sc.w, sh.w));
                    *p = v;
                }
            }
            fence_async_smem();
            __syncthreads();
            if (t == 0) {
                tma_store_2d(&map_y, tile + (size_t)c * g.RB * g.Ct, c0, row0 + c * g.RB);
                tma_store_commit();
            }
        }
    }
    if (t == 0)
        tma_store_wait_read();
    cluster.sync();  // peers may still be reading this CTA's per-channel pairs
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// partials layout: [C/Ct tiles][B samples][2*Ct]  (first Ct: dgamma, next Ct: dbeta)
template <int ACT>
__global__ void __launch_bounds__(GN_THREADS, 2) gn_bwd_tile(const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_dx,
    float* __restrict__ partials, unsigned int* __restrict__ tickets, float* __restrict__ dgamma,
    float* __restrict__ dbeta, const float* __restrict__ gamma, const float* __restrict__ beta,
    const float* __restrict__ mu, const float* __restrict__ rstd, const GnGeom g, const int B, int* err)
{
    extern __shared__ unsigned char gn_smem_raw[];
    __shared__ int s_is_last;
    cg::cluster_group cluster = cg::this_cluster();
    const GnSmem sm = gn_carve(gn_smem_raw, g);
    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    const int rank = (int)cluster.block_rank();
    const int cluster_id = blockIdx.x / g.CS;
    const int q = t % g.Q, rr = t / g.Q;
    const bool active = rr < g.RSTEP;
    const int cb = 4 * q;
    const int gl0 = (cb + 0) / g.cpg, gl1 = (cb + 1) / g.cpg, gl2 = (cb + 2) / g.cpg, gl3 = (cb + 3) / g.cpg;

    if (t == 0) {
        for (int i = 0; i < GN_NBUF * GN_MAX_CHUNKS; ++i)
            mbar_init(&sm.bars[i], 1);
        mbar_init_fence();
        gn_issue_loads(sm, g, 0, cluster_id, rank, &map_x, &map_dy);
    }
    __syncthreads();

    int it = 0;
    for (int item = cluster_id; item < g.items; item += g.nclusters, ++it) {
        const int buf = it & 1;
        const unsigned parity = (unsigned)(it >> 1) & 1u;
        const int ctile = item % g.nct, b = item / g.nct;
        const int c0 = ctile * g.Ct;
        const int row0 = b * g.HW + rank * g.R;
        if (t == 0 && item + g.nclusters < g.items) {
            tma_store_wait_read();
            gn_issue_loads(sm, g, buf ^ 1, item + g.nclusters, rank, &map_x, &map_dy);
        }
        float* chan = sm.chan + (size_t)buf * 2 * g.Ct;
        float4* xt4 = reinterpret_cast<float4*>(gn_tile(sm, g, buf, 0));
        float4* gt4 = reinterpret_cast<float4*>(gn_tile(sm, g, buf, 1));

        float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), be = ga, rs4 = ga, nm4 = ga;
        if (active) {
            ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
            if (ACT != ACT_IDENTITY)
                be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
            const int gbase = b * g.G + c0 / g.cpg;
            rs4.x = __ldg(rstd + gbase + gl0); nm4.x = -__ldg(mu + gbase + gl0) * rs4.x;
            rs4.y = __ldg(rstd + gbase + gl1); nm4.y = -__ldg(mu + gbase + gl1) * rs4.y;
            rs4.z = __ldg(rstd + gbase + gl2); nm4.z = -__ldg(mu + gbase + gl2) * rs4.z;
            rs4.w = __ldg(rstd + gbase + gl3); nm4.w = -__ldg(mu + gbase + gl3) * rs4.w;
        }

        // ---- pass 1: xhat and the effective upstream gradient replace x and dy in
        //      shared memory; per-channel sums of dy and dy*xhat
        float4 sA = make_float4(0.f, 0.f, 0.f, 0.f), sB = sA;
        for (int c = 0; c < g.nchunk; ++c) {
            mbar_wait(&sm.bars[buf * GN_MAX_CHUNKS + c], parity, err);
            if (active) {
                for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                    const size_t idx = (size_t)(c * g.RB + lr) * g.Q + q;
                    float4 xv = xt4[idx], dv = gt4[idx];
                    xv.x = fmaf(xv.x, rs4.x, nm4.x);
                    xv.y = fmaf(xv.y, rs4.y, nm4.y);
                    xv.z = fmaf(xv.z, rs4.z, nm4.z);
                    xv.w = fmaf(xv.w, rs4.w, nm4.w);
                    if (ACT != ACT_IDENTITY) {
                        dv.x *= act_slope<ACT>(fmaf(ga.x, xv.x, be.x));
                        dv.y *= act_slope<ACT>(fmaf(ga.y, xv.y, be.y));
                        dv.z *= act_slope<ACT>(fmaf(ga.z, xv.z, be.z));
                        dv.w *= act_slope<ACT>(fmaf(ga.w, xv.w, be.w));
                        gt4[idx] = dv;
                    }
                    xt4[idx] = xv;
                    sA.x += dv.x; sA.y += dv.y; sA.z += dv.z; sA.w += dv.w;
                    sB.x = fmaf(dv.x, xv.x, sB.x); sB.y = fmaf(dv.y, xv.y, sB.y);
                    sB.z = fmaf(dv.z, xv.z, sB.z); sB.w = fmaf(dv.w, xv.w, sB.w);
                }
            }
        }
        // chan[c] = sum_rows dy (-> dbeta), chan[Ct+c] = sum_rows dy*xhat (-> dgamma)
        gn_fold_rows(sm.red, chan, g, q, rr, active, sA, sB);
        if (g.CS > 1)
            cluster.sync();
        else
            __syncthreads();

        // ---- group sums over the cluster (one warp per group); sample partials
        {
            const int nparts = g.CS * g.cpg;
            const float inv_n = 1.0f / ((float)g.HW * (float)g.cpg);
            for (int grp = warp; grp < g.Gt; grp += GN_WARPS) {
                float sg = 0.0f, sgx = 0.0f;
                for (int e = lane; e < nparts; e += 32) {
                    const float* peer = cluster.map_shared_rank(chan, e / g.cpg);
                    const int ch = grp * g.cpg + e % g.cpg;
                    const float gm = __ldg(gamma + c0 + ch);
                    sg = fmaf(gm, peer[ch], sg);
                    sgx = fmaf(gm, peer[g.Ct + ch], sgx);
                }
                sg = warp_sum(sg);
                sgx = warp_sum(sgx);
                if (lane == 0) {
                    sm.gstat[grp] = sg * inv_n;
                    sm.gstat[g.Gt + grp] = sgx * inv_n;
                }
            }
            if (rank == 0 && t < g.Ct) {
                float a = 0.0f, bsum = 0.0f;
                for (int k = 0; k < g.CS; ++k) {
                    const float* peer = cluster.map_shared_rank(chan, k);
                    a += peer[t];
                    bsum += peer[g.Ct + t];
                }
                float* dst = partials + ((size_t)ctile * B + b) * (2 * g.Ct);
                dst[t] = bsum;
                dst[g.Ct + t] = a;
            }
        }
        __syncthreads();

        // ---- pass 2: dx = rstd * (gamma*dy - mean(gamma*dy) - xhat * mean(gamma*dy*xhat))
        float4 mg = make_float4(0.f, 0.f, 0.f, 0.f), mgx = mg;
        if (active) {
            mg.x = sm.gstat[gl0]; mgx.x = sm.gstat[g.Gt + gl0];
            mg.y = sm.gstat[gl1]; mgx.y = sm.gstat[g.Gt + gl1];
            mg.z = sm.gstat[gl2]; mgx.z = sm.gstat[g.Gt + gl2];
            mg.w = sm.gstat[gl3]; mgx.w = sm.gstat[g.Gt + gl3];
        }
        for (int c = 0; c < g.nchunk; ++c) {
            if (active) {
                for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                    const size_t idx = (size_t)(c * g.RB + lr) * g.Q + q;
                    const float4 xv = xt4[idx];
                    float4 dv = gt4[idx];
                    dv.x = rs4.x * (fmaf(dv.x, ga.x, -mg.x) - xv.x * mgx.x);
                    dv.y = rs4.y * (fmaf(dv.y, ga.y, -mg.y) - xv.y * mgx.y);
                    dv.z = rs4.z * (fmaf(dv.z, ga.z, -mg.z) - xv.z * mgx.z);
                    dv.w = rs4.w * (fmaf(dv.w, ga.w, -mg.w) - xv.w * mgx.w);
                    gt4[idx] = dv;
                }
            }
            fence_async_smem();
            __syncthreads();
            if (t == 0) {
                tma_store_2d(&map_dx, gn_tile(sm, g, buf, 1) + (size_t)c * g.RB * g.Ct, c0, row0 + c * g.RB);
                tma_store_commit();
            }
        }

        // ---- the last sample to finish a channel tile adds the B partial rows
        if (rank == 0) {
            __threadfence();
            __syncthreads();
            if (t == 0) {
                const unsigned old = atomicAdd(&tickets[ctile], 1u);
                s_is_last = (old == (unsigned)B - 1u);
            }
            __syncthreads();
            if (s_is_last) {
                __threadfence();
                const int width = 2 * g.Ct;
                const int nq = width / 4;                 // float4 columns of a partial row
                const int blanes = GN_THREADS / nq;       // samples summed concurrently
                const int qi = t % nq, bl = t / nq;
                const float* src = partials + (size_t)ctile * B * width;
                // sm.red may be too small for blanes*width floats: reuse the x tile of this buffer
                float* fold = gn_tile(sm, g, buf, 0);
                const int cap = (int)(sm.tile_floats / width);
                const int lanes = blanes < cap ? blanes : cap;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                if (bl < lanes) {
                    for (int bb = bl; bb < B; bb += lanes) {
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)bb * width) + qi);
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    reinterpret_cast<float4*>(fold)[bl * nq + qi] = acc;
                }
                __syncthreads();
                for (int j = t; j < width; j += GN_THREADS) {
                    float s = 0.0f;
                    for (int r = 0; r < lanes; ++r)
                        s += fold[r * width + j];
                    if (j < g.Ct)
                        dgamma[c0 + j] = s;
                    else
                        dbeta[c0 + j - g.Ct] = s;
                }
                if (t == 0)
                    tickets[ctile] = 0;  // ready for the next launch
                __syncthreads();
            }
        }
    }
    if (t == 0)
        tma_store_wait_read();
    cluster.sync();
}

}  // namespace b200

#include "groupnorm_strip.cuh"
#include "groupnorm_dstrip.cuh"
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

void fold_partials(float* out_a, float* out_b, const float* partials, int nparts, int width, int split,
    cudaStream_t s);  // rownorm.cu

// ---------------------------------------------------------------------------
// host dispatch
// ---------------------------------------------------------------------------
constexpr int GN_MAX_DYN_SMEM = 216 * 1024;

template <class K>
static bool gn_allow_big_smem(K kernel, bool* done_for_device)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return false;
    if (!done_for_device[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GN_MAX_DYN_SMEM) != cudaSuccess)
            return false;
        done_for_device[dev] = true;
    }
    return true;
}

static void gn_fill_launch(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, const GnGeom& g, int B, size_t smem,
    cudaStream_t s)
{
    (void)B;
    cfg->gridDim = dim3((unsigned)(g.CS * g.nclusters), 1, 1);
    cfg->blockDim = dim3(GN_THREADS, 1, 1);
    cfg->dynamicSmemBytes = smem;
    cfg->stream = s;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

static bool gn_tile_shape_ok(int B, int HW, int C)
{
    return B > 0 && (long)B * HW < 2147483647L && (long)B * HW * C < 2147483648L && C % 4 == 0;
}

// returns true if the tile kernel was launched
template <int ACT>
static bool gn_forward_tile(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    static bool smem_ok[64] = { false };
    if (tune_get("gn_force_generic", 0) || tune_get("gn_no_tile", 0) || !gn_tile_shape_ok(B, HW, C))
        return false;
    if (!(aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta)))
        return false;
    GnGeom g;
    const size_t budget = (size_t)tune_get("gn_fwd_budget_kb", 96) * 1024;
    if (!gn_pick_geometry(&g, B, HW, C, G, 1, tune_get("gn_fwd_ct", 0), tune_get("gn_fwd_cs", 0), budget,
            tune_get("gn_ctas_per_sm", 2)))
        return false;
    const size_t smem = gn_smem_bytes(g);
    if (smem > (size_t)GN_MAX_DYN_SMEM || !gn_allow_big_smem(gn_fwd_tile<ACT>, smem_ok))
        return false;
    CUtensorMap map_x, map_y;
    if (!make_tensor_map_2d(&map_x, x, (uint64_t)B * HW, (uint64_t)C, (uint32_t)g.RB, (uint32_t)g.Ct)
        || !make_tensor_map_2d(&map_y, y, (uint64_t)B * HW, (uint64_t)C, (uint32_t)g.RB, (uint32_t)g.Ct))
        return false;
    int* err = device_error_word();
    if (!err)
        return false;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    gn_fill_launch(&cfg, attr, g, B, smem, s);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gn_fwd_tile<ACT>, map_x, map_y, mu, rstd, gamma, beta, g, eps, err);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "groupnorm forward tile launch failed: %s", cudaGetErrorString(e));
        return true;
    }
    count_launch();
    return true;
}


// ---------------------------------------------------------------------------
// strip (register-resident) dispatch
// ---------------------------------------------------------------------------
void fold_partials(float* out_a, float* out_b, const float* partials, int nparts, int width, int split,
    cudaStream_t s);  // rownorm.cu

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
                g.stagger_lo = g.stagger_hi = g.stagger_ns = 0;
                out->g = g;
                const int red = (Q <= 32 && 32 % Q == 0) ? 2 * (NT / 32) * Ct : 2 * NT * 4;
                out->smem = (size_t)(red + 2 * Ct + 2 * g.Gt) * sizeof(float);
            }
        }
    }
    if (best < 0)
        return false;
    // Start the second CTA of every SM half a strip period later (only the first wave needs it:
    // later CTAs inherit the phase of the slot they replace).
    const long grid = (long)B * out->g.nct;
    const int per_sm = ctas_per_sm_hint > 0 ? ctas_per_sm_hint : (out->NT <= 256 ? 4 : (out->NT <= 512 ? 2 : 1));
    const int ns = tune_get("gn_stagger_ns", 0);  // measured: no effect on B200, so off unless requested
    if (per_sm >= 2 && grid > (long)sm_count() * per_sm && ns > 0) {
        out->g.stagger_lo = sm_count();
        out->g.stagger_hi = sm_count() * 2;
        out->g.stagger_ns = ns;
    }
    return true;
}

template <class... KArgs, class... Args>
static bool strip_launch(void (*kernel)(KArgs...), long grid, int NT, size_t smem, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)NT, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "groupnorm strip launch failed: %s", cudaGetErrorString(e));
        return false;
    }
    count_launch();
    return true;
}

template <class... KArgs, class... Args>
static bool pstrip_launch(void (*kernel)(KArgs...), bool* attr_done, long grid, int NT, size_t smem, cudaStream_t s,
    Args... args)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return false;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        attr_done[dev] = true;
    }
    return strip_launch(kernel, grid, NT, smem, s, args...);
}

#define PSTRIP_FWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv && per_sm == MBv) {                                              \
        static bool done[64] = { false };                                                                   \
        if (full) {                                                                                         \
            static bool donef[64] = { false };                                                              \
            return pstrip_launch(gn_fwd_pstrip<NTv, VPTv, ACT, MBv, true>, donef, pgrid, NTv, psmem, s, y, mu, rstd, x, \
                gamma, beta, plan.g, eps, (int)grid);                                                       \
        }                                                                                                   \
        return pstrip_launch(gn_fwd_pstrip<NTv, VPTv, ACT, MBv, false>, done, pgrid, NTv, psmem, s, y, mu, rstd, x, \
            gamma, beta, plan.g, eps, (int)grid);                                                           \
    }
#define PSTRIP_BWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv) {                                                               \
        static bool done[64] = { false };                                                                   \
        return pstrip_launch(gn_bwd_pstrip<NTv, VPTv, ACT, MBv>, done, pgrid, NTv, psmem, s, dx, sc.partials,       \
                   dy, x, gamma, beta, mu, rstd, plan.g, (int)grid, fold)                                   \
            && (fold.rows || (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true));            \
    }

// deep-staged variants (groupnorm_dstrip.cuh)
#define DSTRIP_FWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv && per_sm == MBv) {                                              \
        static bool done[64] = { false };                                                                   \
        if (full) {                                                                                         \
            static bool donef[64] = { false };                                                              \
            return pstrip_launch(gn_fwd_dstrip<NTv, VPTv, ACT, MBv, true>, donef, pgrid, NTv, dsmem, s, y, mu, rstd, x, \
                gamma, beta, plan.g, eps, (int)grid);                                                       \
        }                                                                                                   \
        return pstrip_launch(gn_fwd_dstrip<NTv, VPTv, ACT, MBv, false>, done, pgrid, NTv, dsmem, s, y, mu, rstd, x, \
            gamma, beta, plan.g, eps, (int)grid);                                                           \
    }
#define DSTRIP_BWD_CASE(NTv, VPTv)                                                                          \
    if (plan.NT == NTv && plan.VPT == VPTv) {                                                               \
        static bool done[64] = { false };                                                                   \
        static bool donef[64] = { false };                                                                  \
        const bool ok = full                                                                                \
            ? pstrip_launch(gn_bwd_dstrip<NTv, VPTv, ACT, true>, donef, pgrid, NTv, dsmem, s, dx, sc.partials, dy, x,  \
                  gamma, beta, mu, rstd, plan.g, (int)grid, fold)                                           \
            : pstrip_launch(gn_bwd_dstrip<NTv, VPTv, ACT, false>, done, pgrid, NTv, dsmem, s, dx, sc.partials, dy, x,  \
                  gamma, beta, mu, rstd, plan.g, (int)grid, fold);                                          \
        return ok && (fold.rows || (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true));      \
    }

#define STRIP_FWD_CASE(NTv, VPTv)                                                                          \
    if (plan.NT == NTv && plan.VPT == VPTv)                                                                \
        return strip_launch(gn_fwd_strip<NTv, VPTv, ACT>, grid, NTv, plan.smem, s, y, mu, rstd, x, gamma, \
            beta, plan.g, eps);
#define STRIP_BWD_CASE(NTv, VPTv, MBv)                                                                     \
    if (plan.NT == NTv && plan.VPT == VPTv)                                                                \
        return strip_launch(gn_bwd_strip<NTv, VPTv, ACT, MBv>, grid, NTv, ssmem, s, dx, sc.partials,      \
                   dy, x, gamma, beta, mu, rstd, plan.g, B, fold)                                          \
            && (fold.rows || (fold_partials(dgamma, dbeta, sc.partials, B, 2 * C, C, s), true));

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
                // deep staging: half a strip more in flight, in the shared memory the plain pipeline leaves unused
                const size_t dsmem = (size_t)(plan.VPT + plan.VPT / 2) * plan.NT * 16 + plan.smem;
                // (measured on [256,32,32,256]: 2 % slower than the plain pipeline in forward, so off unless asked for)
                if (tune_get("gn_deep_fwd", 0) && dsmem * per_sm <= 226 * 1024 && grid >= 3 * pgrid) {
                    DSTRIP_FWD_CASE(1024, 4, 1) DSTRIP_FWD_CASE(1024, 8, 1)
                    DSTRIP_FWD_CASE(512, 4, 2) DSTRIP_FWD_CASE(512, 8, 2) DSTRIP_FWD_CASE(512, 8, 1)
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
        if (!scratch_get(s, (size_t)2 * B * C, 1, &sc))
            return false;
        // small tables of partial rows are added by the last CTA of the same launch (one ticket per launch)
        StripFold fold;
        fold.ticket = sc.tickets;
        fold.dgamma = dgamma;
        fold.dbeta = dbeta;
        fold.rows = ((long)B * 2 * C <= (long)tune_get("gn_inline_fold_floats", 65536) && 2 * C <= 4096) ? B : 0;
        // the in-kernel fold borrows NT floats of shared memory once the strips are done
        const size_t ssmem = plan.smem < (size_t)plan.NT * 4 ? (size_t)plan.NT * 4 : plan.smem;
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
    g.stagger_lo = g.stagger_hi = g.stagger_ns = 0;
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
            return pstrip_launch(gn_fwd_cstrip<512, 8, ACT, MB>, done8, pgrid, 512, psmem, s, y, mu, rstd, x, gamma, beta,
                plan.g, eps, (int)items, nchunks);
        return pstrip_launch(gn_fwd_cstrip<512, 4, ACT, MB>, done4, pgrid, 512, psmem, s, y, mu, rstd, x, gamma, beta,
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
            ? pstrip_launch(gn_bwd_cstrip<512, 4, ACT, 2>, done4, pgrid, 512, psmem, s, dx, sc.partials, dy, x, gamma, beta,
                  mu, rstd, plan.g, (int)items, nchunks)
            : pstrip_launch(gn_bwd_cstrip<512, 8, ACT, 1>, done8, pgrid, 512, psmem, s, dx, sc.partials, dy, x, gamma, beta,
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
    if (gn_forward_tile<ACT>(y, mu, rstd, x, gamma, beta, B, HW, C, G, eps, s))
        return;
    gn_fwd_generic<ACT><<<B * G, GN_GENERIC_THREADS, 0, s>>>(y, mu, rstd, x, gamma, beta, HW, C, G, eps);
    count_launch();
    B200_CHECK_LAUNCH();
}

template <int ACT>
static bool gn_backward_tile(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    static bool smem_ok[64] = { false };
    if (tune_get("gn_force_generic", 0) || tune_get("gn_no_tile", 0) || !gn_tile_shape_ok(B, HW, C))
        return false;
    if (!(aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(gamma)))
        return false;
    if (ACT != ACT_IDENTITY && !aligned16(beta))
        return false;
    GnGeom g;
    const size_t budget = (size_t)tune_get("gn_bwd_budget_kb", 96) * 1024;
    if (!gn_pick_geometry(&g, B, HW, C, G, 2, tune_get("gn_bwd_ct", 0), tune_get("gn_bwd_cs", 0), budget,
            tune_get("gn_ctas_per_sm", 2)))
        return false;
    const size_t smem = gn_smem_bytes(g);
    if (smem > (size_t)GN_MAX_DYN_SMEM || !gn_allow_big_smem(gn_bwd_tile<ACT>, smem_ok))
        return false;
    CUtensorMap map_x, map_dy, map_dx;
    const uint64_t rows = (uint64_t)B * HW;
    if (!make_tensor_map_2d(&map_x, x, rows, (uint64_t)C, (uint32_t)g.RB, (uint32_t)g.Ct)
        || !make_tensor_map_2d(&map_dy, dy, rows, (uint64_t)C, (uint32_t)g.RB, (uint32_t)g.Ct)
        || !make_tensor_map_2d(&map_dx, dx, rows, (uint64_t)C, (uint32_t)g.RB, (uint32_t)g.Ct))
        return false;
    Scratch sc;
    if (!scratch_get(s, (size_t)2 * B * C, (size_t)(C / g.Ct), &sc))
        return false;
    int* err = device_error_word();
    if (!err)
        return false;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    gn_fill_launch(&cfg, attr, g, B, smem, s);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gn_bwd_tile<ACT>, map_x, map_dy, map_dx, sc.partials, sc.tickets,
        dgamma, dbeta, gamma, beta, mu, rstd, g, B, err);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        report_error(__FILE__, __LINE__, "groupnorm backward tile launch failed: %s", cudaGetErrorString(e));
        return true;
    }
    count_launch();
    return true;
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
    if (gn_backward_tile<ACT>(dx, dgamma, dbeta, dy, x, gamma, beta, mu, rstd, B, HW, C, G, s))
        return;
    Scratch sc;
    B200_REQUIRE(scratch_get(s, (size_t)2 * B * C, 0, &sc), "groupnorm_backward: scratch allocation failed (the arena cannot grow during stream capture: call b200_scratch_reserve before capturing)");
    B200_REQUIRE(B <= 65535, "groupnorm_backward: batch %d too large for the generic path", B);
    gn_bwd_dx_generic<ACT><<<B * G, GN_GENERIC_THREADS, 0, s>>>(dx, dy, x, gamma, beta, mu, rstd, HW, C, G);
    count_launch();
    B200_CHECK_LAUNCH();
    gn_bwd_param_generic<ACT><<<dim3((C + 31) / 32, B), dim3(32, 8), 0, s>>>(sc.partials, dy, x, gamma, beta, mu,
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

}  // extern "C"
