// NHWC GroupNorm forward / backward, optionally fused with an activation
// (reference: src/kernels.cu:622-745, composed with :103-117 by conv_residual.c).
//
// Tile kernels (the fast path).  x is viewed as a matrix [B*HW, C].  One CTA owns
// the tile  [R rows of one sample] x [Ct channels]  where Ct covers whole groups;
// a thread-block cluster of CS CTAs splits the HW rows of one sample, so the
// cluster together holds every element of Ct/cpg groups of that sample in
// shared memory.  Consequences:
//   * x (and dy) cross HBM exactly once: bulk tensor copies (TMA) bring the
//     tile in chunk by chunk, statistics and the normalised output are both
//     produced from shared memory, and the result leaves through TMA stores;
//   * statistics are accumulated while later chunks are still in flight;
//   * group statistics are combined across the cluster through distributed
//     shared memory (no global round trip, no atomics);
//   * backward reuses the per-channel sums of dy and dy*xhat for BOTH the group
//     sums that dx needs and the per-sample dgamma/dbeta partials; the last CTA
//     of a channel tile (atomic ticket) adds the partials in a fixed order.
// Shapes the tile path cannot take (C % 4 != 0, no usable row chunking, a
// sample tile larger than a cluster's shared memory, misaligned pointers) use
// the generic kernels at the end of this file.
#include "dev_common.cuh"
#include "tma_desc.cuh"
#include "../../include/b200_layer_kernels.h"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace b200 {

constexpr int GN_THREADS = 256;
constexpr int GN_MAX_CHUNKS = 32;
constexpr int GN_RED_FLOATS = 2 * GN_THREADS * 4;  // two float4 per thread

struct GnGeom {
    int HW, C, G, cpg;
    int Ct;      // channels per tile (multiple of cpg and of 4)
    int Q;       // Ct / 4 float4 columns
    int RSTEP;   // row lanes = GN_THREADS / Q
    int CS;      // cluster size: CTAs that split the HW rows of a sample
    int R;       // rows per CTA = HW / CS
    int RB;      // rows per TMA box
    int nchunk;  // R / RB
    int Gt;      // groups per tile = Ct / cpg
};

// tile footprint in shared memory, padded so that a second tile stays 128-byte aligned
__host__ __device__ static inline size_t gn_tile_bytes(const GnGeom& g)
{
    return ((size_t)g.R * g.Ct * sizeof(float) + 127) & ~(size_t)127;
}

static inline size_t gn_smem_bytes(const GnGeom& g, int ntiles)
{
    // tiles | reduction buffer | per-channel pair | per-group pair | barriers
    return ntiles * gn_tile_bytes(g) + GN_RED_FLOATS * sizeof(float) + 2 * g.Ct * sizeof(float)
        + 2 * g.Gt * sizeof(float) + GN_MAX_CHUNKS * sizeof(uint64_t) + 128;
}

static int largest_divisor_leq(int n, int cap)
{
    for (int d = cap < n ? cap : n; d >= 1; --d)
        if (n % d == 0)
            return d;
    return 1;
}

// Picks (Ct, CS).  ntiles = 1 (forward) or 2 (backward keeps x and dy).
// Preference: tile set within `budget` bytes (so that several CTAs share an SM
// and loads of one overlap stores of another), then rows of at least 128 bytes,
// then the smallest cluster, then the widest tile.
static bool gn_pick_geometry(GnGeom* out, int HW, int C, int G, int ntiles, int force_ct, int force_cs, size_t budget)
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
            GnGeom g;
            g.HW = HW; g.C = C; g.G = G; g.cpg = cpg;
            g.Ct = Ct; g.Q = Q; g.RSTEP = GN_THREADS / Q; g.CS = CS;
            g.R = HW / CS;
            g.RB = largest_divisor_leq(g.R, 256);
            g.nchunk = g.R / g.RB;
            g.Gt = Ct / cpg;
            if (g.nchunk > GN_MAX_CHUNKS || (g.RB < 8 && g.R >= 8))
                continue;
            // every chunk must start on a 128-byte boundary of shared memory
            if (g.nchunk > 1 && (g.RB * Ct) % 32 != 0)
                continue;
            const size_t bytes = ntiles * gn_tile_bytes(g);
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
    return found;
}

// ---------------------------------------------------------------------------
// shared pieces of the tile kernels
// ---------------------------------------------------------------------------
struct GnSmem {
    float* tile0;
    float* tile1;
    float* red;     // GN_RED_FLOATS
    float* chan;    // 2*Ct, read by cluster peers
    float* gstat;   // 2*Gt
    uint64_t* bars; // GN_MAX_CHUNKS
};

__device__ __forceinline__ GnSmem gn_carve(unsigned char* raw, const GnGeom& g, int ntiles)
{
    GnSmem s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(raw) + 127) & ~uintptr_t(127);
    s.tile0 = reinterpret_cast<float*>(p);
    p += gn_tile_bytes(g);
    s.tile1 = reinterpret_cast<float*>(p);
    if (ntiles == 2)
        p += gn_tile_bytes(g);
    s.red = reinterpret_cast<float*>(p);
    p += GN_RED_FLOATS * sizeof(float);
    s.chan = reinterpret_cast<float*>(p);
    p += 2 * g.Ct * sizeof(float);
    s.gstat = reinterpret_cast<float*>(p);
    p += 2 * g.Gt * sizeof(float);
    p = (p + 7) & ~uintptr_t(7);
    s.bars = reinterpret_cast<uint64_t*>(p);
    return s;
}

// Sums the per-thread float4 pairs (a, b) over the row lanes: afterwards
// red[c] and red[Ct + c] hold the CTA totals of channel c for a and b.
// Threads with rr >= RSTEP (idle lanes when Q does not divide the CTA) pass zeros.
__device__ __forceinline__ void gn_fold_rows(float* red, const GnGeom& g, int q, int rr, bool active, float4 a, float4 b)
{
    float4* ra = reinterpret_cast<float4*>(red);
    float4* rb = reinterpret_cast<float4*>(red + GN_THREADS * 4);
    if (active) {
        ra[rr * g.Q + q] = a;
        rb[rr * g.Q + q] = b;
    }
    __syncthreads();
    float sa = 0.0f, sb = 0.0f;
    const int c = threadIdx.x;
    if (c < g.Ct) {
        for (int r = 0; r < g.RSTEP; ++r) {
            sa += red[r * g.Ct + c];
            sb += red[GN_THREADS * 4 + r * g.Ct + c];
        }
    }
    __syncthreads();
    if (c < g.Ct) {
        red[c] = sa;
        red[g.Ct + c] = sb;
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <int ACT>
__global__ void __launch_bounds__(GN_THREADS) gn_fwd_tile(const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_y, float* __restrict__ mu, float* __restrict__ rstd,
    const float* __restrict__ gamma, const float* __restrict__ beta, const GnGeom g, const float eps, int* err)
{
    extern __shared__ unsigned char gn_smem_raw[];
    cg::cluster_group cluster = cg::this_cluster();
    const GnSmem sm = gn_carve(gn_smem_raw, g, 1);
    const int t = threadIdx.x;
    const int rank = blockIdx.x;  // cluster spans gridDim.x
    const int c0 = blockIdx.y * g.Ct;
    const int b = blockIdx.z;
    const int row0 = b * g.HW + rank * g.R;
    const int q = t % g.Q, rr = t / g.Q;
    const bool active = rr < g.RSTEP;
    const unsigned chunk_bytes = (unsigned)(g.RB * g.Ct * sizeof(float));

    if (t == 0) {
        for (int c = 0; c < g.nchunk; ++c)
            mbar_init(&sm.bars[c], 1);
        mbar_init_fence();
        for (int c = 0; c < g.nchunk; ++c) {
            mbar_expect_tx(&sm.bars[c], chunk_bytes);
            tma_load_2d(sm.tile0 + (size_t)c * g.RB * g.Ct, &map_x, c0, row0 + c * g.RB, &sm.bars[c]);
        }
    }
    __syncthreads();

    // ---- statistics, shifted by row 0 of the tile (K) so that the one-pass
    //      sums of (x-K) and (x-K)^2 do not cancel
    const float4* tile4 = reinterpret_cast<const float4*>(sm.tile0);
    float4 K = make_float4(0.f, 0.f, 0.f, 0.f), s1 = K, s2 = K;
    for (int c = 0; c < g.nchunk; ++c) {
        mbar_wait(&sm.bars[c], 0, err);
        if (c == 0 && active)
            K = tile4[q];
        if (active) {
            for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                const float4 v = tile4[(size_t)(c * g.RB + lr) * g.Q + q];
                const float d0 = v.x - K.x, d1 = v.y - K.y, d2 = v.z - K.z, d3 = v.w - K.w;
                s1.x += d0; s1.y += d1; s1.z += d2; s1.w += d3;
                s2.x += d0 * d0; s2.y += d1 * d1; s2.z += d2 * d2; s2.w += d3 * d3;
            }
        }
    }
    gn_fold_rows(sm.red, g, q, rr, active, s1, s2);
    if (t < g.Ct) {
        const float invR = 1.0f / (float)g.R;
        const float S1 = sm.red[t], S2 = sm.red[g.Ct + t];
        sm.chan[t] = sm.tile0[t] + S1 * invR;          // channel mean over this CTA's rows
        sm.chan[g.Ct + t] = S2 - S1 * S1 * invR;       // centred sum of squares
    }
    cluster.sync();

    // ---- combine channels of a group and the CTAs of the cluster (Chan et al.)
    if (t < g.Gt) {
        const int nparts = g.CS * g.cpg;
        float msum = 0.0f;
        for (int k = 0; k < g.CS; ++k) {
            const float* peer = cluster.map_shared_rank(sm.chan, k);
            for (int cl = 0; cl < g.cpg; ++cl)
                msum += peer[t * g.cpg + cl];
        }
        const float mean = msum / (float)nparts;
        float m2 = 0.0f;
        for (int k = 0; k < g.CS; ++k) {
            const float* peer = cluster.map_shared_rank(sm.chan, k);
            for (int cl = 0; cl < g.cpg; ++cl) {
                const float d = peer[t * g.cpg + cl] - mean;
                m2 += peer[g.Ct + t * g.cpg + cl] + (float)g.R * d * d;
            }
        }
        const float var = m2 / ((float)g.R * (float)nparts);
        const float rs = rsqrtf(var + eps);
        sm.gstat[t] = mean;
        sm.gstat[g.Gt + t] = rs;
        if (rank == 0) {
            mu[b * g.G + c0 / g.cpg + t] = mean;
            rstd[b * g.G + c0 / g.cpg + t] = rs;
        }
    }
    __syncthreads();

    // ---- normalise + affine (+ activation) in place, store chunk by chunk
    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), be = ga, mean4 = ga, rs4 = ga;
    if (active) {
        ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        const int cb = 4 * q;
        mean4.x = sm.gstat[(cb + 0) / g.cpg]; rs4.x = sm.gstat[g.Gt + (cb + 0) / g.cpg];
        mean4.y = sm.gstat[(cb + 1) / g.cpg]; rs4.y = sm.gstat[g.Gt + (cb + 1) / g.cpg];
        mean4.z = sm.gstat[(cb + 2) / g.cpg]; rs4.z = sm.gstat[g.Gt + (cb + 2) / g.cpg];
        mean4.w = sm.gstat[(cb + 3) / g.cpg]; rs4.w = sm.gstat[g.Gt + (cb + 3) / g.cpg];
    }
    float4* wtile4 = reinterpret_cast<float4*>(sm.tile0);
    for (int c = 0; c < g.nchunk; ++c) {
        if (active) {
            for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                float4* p = wtile4 + (size_t)(c * g.RB + lr) * g.Q + q;
                float4 v = *p;
                v.x = act_value<ACT>(ga.x * ((v.x - mean4.x) * rs4.x) + be.x);
                v.y = act_value<ACT>(ga.y * ((v.y - mean4.y) * rs4.y) + be.y);
                v.z = act_value<ACT>(ga.z * ((v.z - mean4.z) * rs4.z) + be.z);
                v.w = act_value<ACT>(ga.w * ((v.w - mean4.w) * rs4.w) + be.w);
                *p = v;
            }
        }
        fence_async_smem();
        __syncthreads();
        if (t == 0) {
            tma_store_2d(&map_y, sm.tile0 + (size_t)c * g.RB * g.Ct, c0, row0 + c * g.RB);
            tma_store_commit();
        }
    }
    if (t == 0)
        tma_store_wait_read();
    cluster.sync();  // peers may still be reading this CTA's per-channel pair
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// partials layout: [C/Ct tiles][B samples][2*Ct]  (first Ct: dgamma, next Ct: dbeta)
template <int ACT>
__global__ void __launch_bounds__(GN_THREADS) gn_bwd_tile(const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_dx,
    float* __restrict__ partials, unsigned int* __restrict__ tickets, float* __restrict__ dgamma,
    float* __restrict__ dbeta, const float* __restrict__ gamma, const float* __restrict__ beta,
    const float* __restrict__ mu, const float* __restrict__ rstd, const GnGeom g, const int B, int* err)
{
    extern __shared__ unsigned char gn_smem_raw[];
    __shared__ int s_is_last;
    cg::cluster_group cluster = cg::this_cluster();
    const GnSmem sm = gn_carve(gn_smem_raw, g, 2);
    const int t = threadIdx.x;
    const int rank = blockIdx.x;
    const int c0 = blockIdx.y * g.Ct;
    const int b = blockIdx.z;
    const int row0 = b * g.HW + rank * g.R;
    const int q = t % g.Q, rr = t / g.Q;
    const bool active = rr < g.RSTEP;
    const unsigned chunk_bytes = (unsigned)(g.RB * g.Ct * sizeof(float));

    if (t == 0) {
        for (int c = 0; c < g.nchunk; ++c)
            mbar_init(&sm.bars[c], 1);
        mbar_init_fence();
        for (int c = 0; c < g.nchunk; ++c) {
            mbar_expect_tx(&sm.bars[c], 2 * chunk_bytes);
            tma_load_2d(sm.tile0 + (size_t)c * g.RB * g.Ct, &map_x, c0, row0 + c * g.RB, &sm.bars[c]);
            tma_load_2d(sm.tile1 + (size_t)c * g.RB * g.Ct, &map_dy, c0, row0 + c * g.RB, &sm.bars[c]);
        }
    }

    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), be = ga, mean4 = ga, rs4 = ga;
    int gl0 = 0, gl1 = 0, gl2 = 0, gl3 = 0;  // tile-local group of each of the 4 lanes
    if (active) {
        ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        if (ACT != ACT_IDENTITY)
            be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        const int cb = 4 * q;
        gl0 = (cb + 0) / g.cpg; gl1 = (cb + 1) / g.cpg; gl2 = (cb + 2) / g.cpg; gl3 = (cb + 3) / g.cpg;
        const int gbase = b * g.G + c0 / g.cpg;
        mean4.x = __ldg(mu + gbase + gl0); rs4.x = __ldg(rstd + gbase + gl0);
        mean4.y = __ldg(mu + gbase + gl1); rs4.y = __ldg(rstd + gbase + gl1);
        mean4.z = __ldg(mu + gbase + gl2); rs4.z = __ldg(rstd + gbase + gl2);
        mean4.w = __ldg(mu + gbase + gl3); rs4.w = __ldg(rstd + gbase + gl3);
    }
    __syncthreads();

    // ---- pass 1: xhat and the effective upstream gradient replace x and dy in
    //      shared memory; per-channel sums of dy and dy*xhat
    float4* xt4 = reinterpret_cast<float4*>(sm.tile0);
    float4* gt4 = reinterpret_cast<float4*>(sm.tile1);
    float4 sA = make_float4(0.f, 0.f, 0.f, 0.f), sB = sA;
    for (int c = 0; c < g.nchunk; ++c) {
        mbar_wait(&sm.bars[c], 0, err);
        if (active) {
            for (int lr = rr; lr < g.RB; lr += g.RSTEP) {
                const size_t idx = (size_t)(c * g.RB + lr) * g.Q + q;
                float4 xv = xt4[idx], dv = gt4[idx];
                xv.x = (xv.x - mean4.x) * rs4.x;
                xv.y = (xv.y - mean4.y) * rs4.y;
                xv.z = (xv.z - mean4.z) * rs4.z;
                xv.w = (xv.w - mean4.w) * rs4.w;
                if (ACT != ACT_IDENTITY) {
                    dv.x *= act_slope<ACT>(ga.x * xv.x + be.x);
                    dv.y *= act_slope<ACT>(ga.y * xv.y + be.y);
                    dv.z *= act_slope<ACT>(ga.z * xv.z + be.z);
                    dv.w *= act_slope<ACT>(ga.w * xv.w + be.w);
                    gt4[idx] = dv;
                }
                xt4[idx] = xv;
                sA.x += dv.x; sA.y += dv.y; sA.z += dv.z; sA.w += dv.w;
                sB.x += dv.x * xv.x; sB.y += dv.y * xv.y; sB.z += dv.z * xv.z; sB.w += dv.w * xv.w;
            }
        }
    }
    gn_fold_rows(sm.red, g, q, rr, active, sA, sB);
    if (t < g.Ct) {
        sm.chan[t] = sm.red[t];                // sum_rows dy          (-> dbeta)
        sm.chan[g.Ct + t] = sm.red[g.Ct + t];  // sum_rows dy * xhat   (-> dgamma)
    }
    cluster.sync();

    // ---- group sums over the cluster; sample partials for dgamma/dbeta
    if (t < g.Gt) {
        float sg = 0.0f, sgx = 0.0f;
        for (int k = 0; k < g.CS; ++k) {
            const float* peer = cluster.map_shared_rank(sm.chan, k);
            for (int cl = 0; cl < g.cpg; ++cl) {
                const int ch = t * g.cpg + cl;
                const float gm = __ldg(gamma + c0 + ch);
                sg += gm * peer[ch];
                sgx += gm * peer[g.Ct + ch];
            }
        }
        const float inv_n = 1.0f / ((float)g.HW * (float)g.cpg);
        sm.gstat[t] = sg * inv_n;
        sm.gstat[g.Gt + t] = sgx * inv_n;
    }
    if (rank == 0 && t < g.Ct) {
        float a = 0.0f, bsum = 0.0f;
        for (int k = 0; k < g.CS; ++k) {
            const float* peer = cluster.map_shared_rank(sm.chan, k);
            a += peer[t];
            bsum += peer[g.Ct + t];
        }
        float* dst = partials + ((size_t)blockIdx.y * B + b) * (2 * g.Ct);
        dst[t] = bsum;
        dst[g.Ct + t] = a;
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
                dv.x = rs4.x * (dv.x * ga.x - mg.x - xv.x * mgx.x);
                dv.y = rs4.y * (dv.y * ga.y - mg.y - xv.y * mgx.y);
                dv.z = rs4.z * (dv.z * ga.z - mg.z - xv.z * mgx.z);
                dv.w = rs4.w * (dv.w * ga.w - mg.w - xv.w * mgx.w);
                gt4[idx] = dv;
            }
        }
        fence_async_smem();
        __syncthreads();
        if (t == 0) {
            tma_store_2d(&map_dx, sm.tile1 + (size_t)c * g.RB * g.Ct, c0, row0 + c * g.RB);
            tma_store_commit();
        }
    }

    // ---- the last sample to finish a channel tile adds the B partial rows
    if (rank == 0) {
        __threadfence();
        __syncthreads();
        if (t == 0) {
            const unsigned old = atomicAdd(&tickets[blockIdx.y], 1u);
            s_is_last = (old == (unsigned)B - 1u);
        }
        __syncthreads();
        if (s_is_last) {
            __threadfence();
            const int width = 2 * g.Ct;
            const int nq = width / 4;                 // float4 columns of a partial row
            const int blanes = GN_THREADS / nq;       // samples summed concurrently
            const int qi = t % nq, bl = t / nq;
            const float* src = partials + (size_t)blockIdx.y * B * width;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (bl < blanes) {
                for (int bb = bl; bb < B; bb += blanes) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)bb * width) + qi);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                reinterpret_cast<float4*>(sm.red)[bl * nq + qi] = acc;
            }
            __syncthreads();
            for (int j = t; j < width; j += GN_THREADS) {
                float s = 0.0f;
                for (int r = 0; r < blanes; ++r)
                    s += sm.red[r * width + j];
                if (j < g.Ct)
                    dgamma[c0 + j] = s;
                else
                    dbeta[c0 + j - g.Ct] = s;
            }
            if (t == 0)
                tickets[blockIdx.y] = 0;  // ready for the next launch
        }
    }
    if (t == 0)
        tma_store_wait_read();
    cluster.sync();
}

// ---------------------------------------------------------------------------
// generic kernels: one CTA per (sample, group), any C / HW / alignment.
// The group is re-read from L2 for the second and third sweep.
// ---------------------------------------------------------------------------
template <int ACT>
__global__ void __launch_bounds__(GN_THREADS) gn_fwd_generic(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, int HW, int C, int G, float eps)
{
    __shared__ float buf[32];
    const int b = blockIdx.x / G, grp = blockIdx.x % G;
    const int cpg = C / G, n = HW * cpg, cbase = grp * cpg;
    const float* xb = x + (size_t)b * HW * C;
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_THREADS)
        s += xb[(size_t)(i / cpg) * C + cbase + i % cpg];
    const float mean = cta_sum(s, buf) / (float)n;
    float vs = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_THREADS) {
        const float d = xb[(size_t)(i / cpg) * C + cbase + i % cpg] - mean;
        vs += d * d;
    }
    const float rs = rsqrtf(cta_sum(vs, buf) / (float)n + eps);
    if (threadIdx.x == 0) {
        mu[blockIdx.x] = mean;
        rstd[blockIdx.x] = rs;
    }
    float* yb = y + (size_t)b * HW * C;
    for (int i = threadIdx.x; i < n; i += GN_THREADS) {
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
__global__ void __launch_bounds__(GN_THREADS) gn_bwd_dx_generic(float* __restrict__ dx, const float* __restrict__ dy,
    const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    const float* __restrict__ mu, const float* __restrict__ rstd, int HW, int C, int G)
{
    __shared__ float buf[32];
    const int b = blockIdx.x / G, grp = blockIdx.x % G;
    const int cpg = C / G, n = HW * cpg, cbase = grp * cpg;
    const size_t sample = (size_t)b * HW * C;
    const float mean = mu[blockIdx.x], rs = rstd[blockIdx.x];
    float pg = 0.0f, pgx = 0.0f;
    for (int i = threadIdx.x; i < n; i += GN_THREADS) {
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
    for (int i = threadIdx.x; i < n; i += GN_THREADS) {
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
    cfg->gridDim = dim3((unsigned)g.CS, (unsigned)(g.C / g.Ct), (unsigned)B);
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
    return B > 0 && B <= 65535 && (long)B * HW < 2147483647L && (long)B * HW * C < 2147483648L && C % 4 == 0;
}

// returns true if the tile kernel was launched
template <int ACT>
static bool gn_forward_tile(float* y, float* mu, float* rstd, const float* x, const float* gamma,
    const float* beta, int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    static bool smem_ok[64] = { false };
    if (tune_get("gn_force_generic", 0) || !gn_tile_shape_ok(B, HW, C))
        return false;
    if (!(aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta)))
        return false;
    GnGeom g;
    const size_t budget = (size_t)tune_get("gn_fwd_budget_kb", 64) * 1024;
    if (!gn_pick_geometry(&g, HW, C, G, 1, tune_get("gn_fwd_ct", 0), tune_get("gn_fwd_cs", 0), budget))
        return false;
    const size_t smem = gn_smem_bytes(g, 1);
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

template <int ACT>
static void gn_forward(float* y, float* mu, float* rstd, const float* x, const float* gamma, const float* beta,
    int B, int HW, int C, int G, float eps, cudaStream_t s)
{
    if (gn_forward_tile<ACT>(y, mu, rstd, x, gamma, beta, B, HW, C, G, eps, s))
        return;
    gn_fwd_generic<ACT><<<B * G, GN_THREADS, 0, s>>>(y, mu, rstd, x, gamma, beta, HW, C, G, eps);
    count_launch();
    B200_CHECK_LAUNCH();
}

template <int ACT>
static bool gn_backward_tile(float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
    const float* gamma, const float* beta, const float* mu, const float* rstd, int B, int HW, int C, int G,
    cudaStream_t s)
{
    static bool smem_ok[64] = { false };
    if (tune_get("gn_force_generic", 0) || !gn_tile_shape_ok(B, HW, C))
        return false;
    if (!(aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(gamma)))
        return false;
    if (ACT != ACT_IDENTITY && !aligned16(beta))
        return false;
    GnGeom g;
    const size_t budget = (size_t)tune_get("gn_bwd_budget_kb", 64) * 1024;
    if (!gn_pick_geometry(&g, HW, C, G, 2, tune_get("gn_bwd_ct", 0), tune_get("gn_bwd_cs", 0), budget))
        return false;
    const size_t smem = gn_smem_bytes(g, 2);
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
    if (gn_backward_tile<ACT>(dx, dgamma, dbeta, dy, x, gamma, beta, mu, rstd, B, HW, C, G, s))
        return;
    Scratch sc;
    B200_REQUIRE(scratch_get(s, (size_t)2 * B * C, 0, &sc), "groupnorm_backward: scratch allocation failed");
    B200_REQUIRE(B <= 65535, "groupnorm_backward: batch %d too large for the generic path", B);
    gn_bwd_dx_generic<ACT><<<B * G, GN_THREADS, 0, s>>>(dx, dy, x, gamma, beta, mu, rstd, HW, C, G);
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
