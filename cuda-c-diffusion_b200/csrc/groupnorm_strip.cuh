// Register-resident GroupNorm "strip" kernels (included by groupnorm.cu).
//
// One CTA owns the strip [all HW rows of one sample] x [Ct channels covering
// whole groups] and keeps it entirely in REGISTERS: thread t holds the float4
// column q = t % Q (Q = Ct/4) of rows rl, rl+RSTEP, ... (RSTEP = NT/Q), VPT rows
// in all.  Statistics, the normalised output (or dx) and the parameter-gradient
// partials are all computed from registers, so x (and dy) cross HBM exactly once.
//
// Two generations live here:
//   gn_fwd_strip / gn_bwd_strip    one strip per CTA; every load of the strip is
//                                  issued before the first is consumed.
//   gn_fwd_pstrip / gn_bwd_pstrip  persistent and pipelined (the default): a CTA
//                                  walks strips blockIdx.x, +gridDim.x, ... and,
//                                  while it computes strip i from registers, its
//                                  threads stage their own float4 slots of strip
//                                  i+1 in shared memory with cp.async (each thread
//                                  reads back only what it staged, so staging needs
//                                  no barrier).  The HBM pipe therefore stays busy
//                                  during the arithmetic and the stores.
// The backward kernels write one dgamma/dbeta partial row per sample; a separate
// fixed-order fold kernel (rownorm.cu: fold_partials) sums them, which keeps the
// result deterministic and keeps fences and atomics off each strip's critical path.
//
// The strip must fit the register file: HW <= RSTEP * VPT with VPT <= 8 per
// tensor.  Taller samples take the chunked strips of groupnorm_cstrip.cuh.
#pragma once

namespace b200 {

template <int NT>
struct StripSmem {
    static constexpr int NW = NT / 32;
};

// Folds per-thread float4 pairs over all row lanes of the CTA; afterwards
// chan[c] / chan[Ct + c] hold the totals of channel c.  `red` has 2*NW*Ct floats
// when Q divides 32 (shuffle path), else 2*NT*4 floats.
template <int NT>
__device__ __forceinline__ void strip_fold(float* red, float* chan, int Q, int Ct, int q, int rl, float4 a, float4 b)
{
    constexpr int NW = NT / 32;
    const int t = threadIdx.x;
    if (Q <= 32 && 32 % Q == 0) {
        for (int off = Q; off < 32; off <<= 1) {
            a = shfl_xor4(a, off);
            b = shfl_xor4(b, off);
        }
        const int lane = t & 31, warp = t >> 5;
        if (lane < Q) {
            reinterpret_cast<float4*>(red)[warp * Q + lane] = a;
            reinterpret_cast<float4*>(red + NW * Ct)[warp * Q + lane] = b;
        }
        __syncthreads();
        if (t < Ct) {
            float sa = 0.0f, sb = 0.0f;
#pragma unroll 8
            for (int w = 0; w < NW; ++w) {
                sa += red[w * Ct + t];
                sb += red[NW * Ct + w * Ct + t];
            }
            chan[t] = sa;
            chan[Ct + t] = sb;
        }
    } else {
        const int rstep = NT / Q;
        reinterpret_cast<float4*>(red)[rl * Q + q] = a;
        reinterpret_cast<float4*>(red + NT * 4)[rl * Q + q] = b;
        __syncthreads();
        if (t < Ct) {
            float sa = 0.0f, sb = 0.0f;
            for (int r = 0; r < rstep; ++r) {
                sa += red[r * Ct + t];
                sb += red[NT * 4 + r * Ct + t];
            }
            chan[t] = sa;
            chan[Ct + t] = sb;
        }
    }
    __syncthreads();
}

struct StripGeom {
    int HW, C, G, cpg, Ct, Q, RSTEP, Gt, nct;
    int paced;  // one-barrier forward without activation: release stores as the next strip's loads land
    int hint;   // pipelined and one-barrier kernels: L2 priority of the staged loads (0 normal, 1 evict_last, 2 evict_first)
    // (Starting the second CTA of every SM half a strip period late, so that the two run out of phase, was
    // measured: no effect.)
};

// ---------------------------------------------------------------------------
// forward: grid = B * nct, block = NT
// ---------------------------------------------------------------------------
template <int NT, int VPT, int ACT>
__global__ void __launch_bounds__(NT, (NT <= 256 ? 4 : (NT <= 512 ? 2 : 1))) gn_fwd_strip(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const StripGeom g, const float eps)
{
    pdl_prologue();
    extern __shared__ float strip_smem[];
    float* red = strip_smem;
    const int red_floats = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * (NT / 32) * g.Ct : 2 * NT * 4;
    float* chan = red + red_floats;      // 2*Ct
    float* gstat = chan + 2 * g.Ct;      // 2*Gt
    const int t = threadIdx.x;
    const int ctile = blockIdx.x % g.nct, b = blockIdx.x / g.nct;
    const int c0 = ctile * g.Ct;
    const int q = t % g.Q, rl = t / g.Q;
    const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;

    // per-channel shift K = row 0 of the sample (same for every thread of a column)
    const float4 K = __ldg(reinterpret_cast<const float4*>(x + base));
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        v[j] = K;  // rows past the end contribute zero to the shifted sums
        if (r < g.HW)
            v[j] = __ldcs(reinterpret_cast<const float4*>(x + base + (size_t)r * g.C));
    }
    float4 s1 = make_float4(0.f, 0.f, 0.f, 0.f), s2 = s1;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const float d0 = v[j].x - K.x, d1 = v[j].y - K.y, d2 = v[j].z - K.z, d3 = v[j].w - K.w;
        s1.x += d0; s1.y += d1; s1.z += d2; s1.w += d3;
        s2.x = fmaf(d0, d0, s2.x); s2.y = fmaf(d1, d1, s2.y); s2.z = fmaf(d2, d2, s2.z); s2.w = fmaf(d3, d3, s2.w);
    }
    strip_fold<NT>(red, chan, g.Q, g.Ct, q, rl, s1, s2);

    // group statistics: thread grp < Gt combines its cpg channels
    if (t < g.Gt) {
        const float n = (float)g.HW * (float)g.cpg;
        const float* xrow0 = x + (size_t)b * g.HW * g.C + c0 + t * g.cpg;
        // mean = (sum_c HW*K_c + S1_c) / n ;  centred second moment via the shift identity
        float msum = 0.0f;
        for (int cl = 0; cl < g.cpg; ++cl)
            msum += chan[t * g.cpg + cl] + (float)g.HW * __ldg(xrow0 + cl);
        const float mean = msum / n;
        float m2 = 0.0f;
        for (int cl = 0; cl < g.cpg; ++cl) {
            const int ch = t * g.cpg + cl;
            const float dk = __ldg(xrow0 + cl) - mean;
            m2 += chan[g.Ct + ch] + 2.0f * dk * chan[ch] + (float)g.HW * dk * dk;
        }
        const float rs = rsqrtf(m2 / n + eps);
        gstat[t] = mean;
        gstat[g.Gt + t] = rs;
        mu[b * g.G + c0 / g.cpg + t] = mean;
        rstd[b * g.G + c0 / g.cpg + t] = rs;
    }
    __syncthreads();

    const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
    const float4 be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
    const int cb = 4 * q;
    const int g0 = (cb + 0) / g.cpg, g1 = (cb + 1) / g.cpg, g2 = (cb + 2) / g.cpg, g3 = (cb + 3) / g.cpg;
    float4 sc, sh;
    sc.x = ga.x * gstat[g.Gt + g0]; sh.x = be.x - gstat[g0] * sc.x;
    sc.y = ga.y * gstat[g.Gt + g1]; sh.y = be.y - gstat[g1] * sc.y;
    sc.z = ga.z * gstat[g.Gt + g2]; sh.z = be.z - gstat[g2] * sc.z;
    sc.w = ga.w * gstat[g.Gt + g3]; sh.w = be.w - gstat[g3] * sc.w;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        if (r < g.HW) {
            float4 o;
            o.x = act_value<ACT>(fmaf(v[j].x, sc.x, sh.x));
            o.y = act_value<ACT>(fmaf(v[j].y, sc.y, sh.y));
            o.z = act_value<ACT>(fmaf(v[j].z, sc.z, sh.z));
            o.w = act_value<ACT>(fmaf(v[j].w, sc.w, sh.w));
            __stcs(reinterpret_cast<float4*>(y + base + (size_t)r * g.C), o);
        }
    }
}

// ---------------------------------------------------------------------------
// backward: grid = B * nct, block = NT
// Per-sample partial rows of the parameter gradients go to partials[b][2*C] (first C: dgamma,
// next C: dbeta); a small fold kernel launched right after adds the B rows in a fixed order.
// (A last-CTA ticket inside this kernel was measured twice.  Per strip: its fence + atomic round
// trip sits on every strip's critical path and costs far more than the extra launch.  Per launch,
// with the last CTA adding the rows itself: one CTA walking a 128 x 128 table is a chain of L2
// round trips, [128,28,28,64] went from 19 us to 30 us, and the extra code slowed the strip loop
// of the large shapes by 10 %.  The separate fold kernel, spread over 4-16 CTAs, stays.)
// ---------------------------------------------------------------------------
template <int NT, int VPT, int ACT, int MB>
__global__ void __launch_bounds__(NT, MB) gn_bwd_strip(float* __restrict__ dx,
    float* __restrict__ partials, const float* __restrict__ dy, const float* __restrict__ x,
    const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mu,
    const float* __restrict__ rstd, const StripGeom g, const int B)
{
    pdl_prologue();
    extern __shared__ float strip_smem[];
    constexpr int NW = NT / 32;
    float* red = strip_smem;
    const int red_floats = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * NW * g.Ct : 2 * NT * 4;
    float* chan = red + red_floats;
    float* gstat = chan + 2 * g.Ct;
    const int t = threadIdx.x;
    const int ctile = blockIdx.x % g.nct, b = blockIdx.x / g.nct;
    const int c0 = ctile * g.Ct;
    const int q = t % g.Q, rl = t / g.Q;
    const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;
    const int cb = 4 * q;
    const int gl0 = (cb + 0) / g.cpg, gl1 = (cb + 1) / g.cpg, gl2 = (cb + 2) / g.cpg, gl3 = (cb + 3) / g.cpg;

    float4 xv[VPT], dv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        dv[j] = xv[j];
        if (r < g.HW) {
            xv[j] = __ldcs(reinterpret_cast<const float4*>(x + base + (size_t)r * g.C));
            dv[j] = __ldcs(reinterpret_cast<const float4*>(dy + base + (size_t)r * g.C));
        }
    }
    const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
    float4 be = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ACT != ACT_IDENTITY)
        be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
    const int gbase = b * g.G + c0 / g.cpg;
    float4 rs4, nm4;
    rs4.x = __ldg(rstd + gbase + gl0); nm4.x = -__ldg(mu + gbase + gl0) * rs4.x;
    rs4.y = __ldg(rstd + gbase + gl1); nm4.y = -__ldg(mu + gbase + gl1) * rs4.y;
    rs4.z = __ldg(rstd + gbase + gl2); nm4.z = -__ldg(mu + gbase + gl2) * rs4.z;
    rs4.w = __ldg(rstd + gbase + gl3); nm4.w = -__ldg(mu + gbase + gl3) * rs4.w;

    float4 sA = make_float4(0.f, 0.f, 0.f, 0.f), sB = sA;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        if (r < g.HW) {
            xv[j].x = fmaf(xv[j].x, rs4.x, nm4.x);
            xv[j].y = fmaf(xv[j].y, rs4.y, nm4.y);
            xv[j].z = fmaf(xv[j].z, rs4.z, nm4.z);
            xv[j].w = fmaf(xv[j].w, rs4.w, nm4.w);
            if (ACT != ACT_IDENTITY) {
                dv[j].x *= act_slope<ACT>(fmaf(ga.x, xv[j].x, be.x));
                dv[j].y *= act_slope<ACT>(fmaf(ga.y, xv[j].y, be.y));
                dv[j].z *= act_slope<ACT>(fmaf(ga.z, xv[j].z, be.z));
                dv[j].w *= act_slope<ACT>(fmaf(ga.w, xv[j].w, be.w));
            }
            sA.x += dv[j].x; sA.y += dv[j].y; sA.z += dv[j].z; sA.w += dv[j].w;
            sB.x = fmaf(dv[j].x, xv[j].x, sB.x); sB.y = fmaf(dv[j].y, xv[j].y, sB.y);
            sB.z = fmaf(dv[j].z, xv[j].z, sB.z); sB.w = fmaf(dv[j].w, xv[j].w, sB.w);
        }
    }
    // chan[c] = sum_rows dy (-> dbeta), chan[Ct+c] = sum_rows dy*xhat (-> dgamma)
    strip_fold<NT>(red, chan, g.Q, g.Ct, q, rl, sA, sB);

    if (t < g.Gt) {
        float sg = 0.0f, sgx = 0.0f;
        for (int cl = 0; cl < g.cpg; ++cl) {
            const int ch = t * g.cpg + cl;
            const float gm = __ldg(gamma + c0 + ch);
            sg = fmaf(gm, chan[ch], sg);
            sgx = fmaf(gm, chan[g.Ct + ch], sgx);
        }
        const float inv_n = 1.0f / ((float)g.HW * (float)g.cpg);
        gstat[t] = sg * inv_n;
        gstat[g.Gt + t] = sgx * inv_n;
    }
    if (t < g.Ct) {  // one partial row per sample: [b][0:C] dgamma, [b][C:2C] dbeta
        float* dst = partials + (size_t)b * (2 * g.C) + c0 + t;
        dst[0] = chan[g.Ct + t];
        dst[g.C] = chan[t];
    }
    __syncthreads();

    float4 mg, mgx;
    mg.x = gstat[gl0]; mgx.x = gstat[g.Gt + gl0];
    mg.y = gstat[gl1]; mgx.y = gstat[g.Gt + gl1];
    mg.z = gstat[gl2]; mgx.z = gstat[g.Gt + gl2];
    mg.w = gstat[gl3]; mgx.w = gstat[g.Gt + gl3];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        if (r < g.HW) {
            float4 o;
            o.x = rs4.x * (fmaf(dv[j].x, ga.x, -mg.x) - xv[j].x * mgx.x);
            o.y = rs4.y * (fmaf(dv[j].y, ga.y, -mg.y) - xv[j].y * mgx.y);
            o.z = rs4.z * (fmaf(dv[j].z, ga.z, -mg.z) - xv[j].z * mgx.z);
            o.w = rs4.w * (fmaf(dv[j].w, ga.w, -mg.w) - xv[j].w * mgx.w);
            __stcs(reinterpret_cast<float4*>(dx + base + (size_t)r * g.C), o);
        }
    }
}

// ===========================================================================
// Pipelined strips: persistent CTAs that prefetch the NEXT strip with cp.async
// ===========================================================================
// Same register-resident processing as above, but a CTA loops over strips and, while it reduces,
// normalises and stores strip i from registers, the 16-byte asynchronous copies of strip i+1 are
// already in flight into shared memory.  Every thread stages exactly the float4 slots it will later
// read itself (slot j of thread t lives at stage[j*NT + t]), so the staging needs no barrier at all:
// a thread waits for its own copy group, moves its slots to registers and immediately re-arms them
// with the copies of the following strip.  Each SM therefore always has a full strip (64-128 KB) of
// loads outstanding, also during the barrier- and arithmetic-heavy phases.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}
// L2 priority of the staged loads (StripGeom::hint).  A strip's row pieces are 64 or 128 bytes of rows whose
// neighbouring pieces are read by the neighbouring CTAs a little earlier or later, so how long a fetched line
// (and what DRAM delivered with it) survives in L2 decides how much of DRAM's work is shared between neighbours.
__device__ __forceinline__ uint64_t l2_policy(int hint)
{
    uint64_t p;
    if (hint == 1)
        asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    else if (hint == 2)
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    else
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void cp_async16_hint(void* smem_dst, const void* gmem_src, uint64_t policy)
{
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int NT, int VPT, int NTENS>
__device__ __forceinline__ void strip_prefetch(float4* stage, const StripGeom& g, int item, int q, int rl,
    const float* __restrict__ t0, const float* __restrict__ t1)
{
    const int ctile = item % g.nct, b = item / g.nct;
    const size_t base = (size_t)b * g.HW * g.C + (size_t)ctile * g.Ct + 4 * q;
    const uint64_t pol = l2_policy(g.hint);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = rl + j * g.RSTEP;
        if (r < g.HW) {
            cp_async16_hint(&stage[j * NT + threadIdx.x], t0 + base + (size_t)r * g.C, pol);
            if (NTENS == 2)
                cp_async16_hint(&stage[(VPT + j) * NT + threadIdx.x], t1 + base + (size_t)r * g.C, pol);
        }
    }
    cp_async_commit();
}

// grid = min(items, resident CTAs), block = NT; dynamic smem = stage | red | chan | gstat
// FULL: HW == RSTEP * VPT, i.e. every register slot holds a real row and no row test is needed.
//
// Measured dead ends, kept out on purpose (same-GPU A/B, [256,32,32,256], SiLU):
//  - fetching the next strip's shift K one strip ahead, or serving the group-statistics threads
//    from shared memory instead of global loads: the extra live registers spill at the 64-register
//    limit, forward 4-6 % slower;
//  - 32-bit float4 indexing with no division in the strip loop and a FULL backward: a quarter
//    fewer instructions, forward unchanged, backward 4 % slower.  With the packed arithmetic these
//    kernels are no longer bound by instruction issue but by the latency of one strip's dependent
//    phases (16-32 resident warps per SM is all the register-resident strip allows).
template <int NT, int VPT, int ACT, int MB, bool FULL>
__global__ void __launch_bounds__(NT, MB) gn_fwd_pstrip(float* __restrict__ y,
    float* __restrict__ mu, float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const StripGeom g, const float eps, const int nitems)
{
    pdl_prologue();
    extern __shared__ float4 strip_stage[];
    float4* stage = strip_stage;
    float* red = reinterpret_cast<float*>(stage + VPT * NT);
    const int red_floats = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * (NT / 32) * g.Ct : 2 * NT * 4;
    float* chan = red + red_floats;
    float* gstat = chan + 2 * g.Ct;
    const int t = threadIdx.x;
    const int q = t % g.Q, rl = t / g.Q;
    const int cb = 4 * q;
    const int g0 = (cb + 0) / g.cpg, g1 = (cb + 1) / g.cpg, g2 = (cb + 2) / g.cpg, g3 = (cb + 3) / g.cpg;

    int item = blockIdx.x;
    if (item < nitems)
        strip_prefetch<NT, VPT, 1>(stage, g, item, q, rl, x, nullptr);
    // (ctile, b) of the current item, advanced incrementally (no division in the loop)
    int ctile = item % g.nct, b = item / g.nct;
    const int step_ct = (int)gridDim.x % g.nct, step_b = (int)gridDim.x / g.nct;
    for (; item < nitems; item += gridDim.x) {
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;
        const float4 K = __ldg(reinterpret_cast<const float4*>(x + base));
        cp_async_wait_all();
        float4 v[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            v[j] = stage[j * NT + t];
            if (!FULL && rl + j * g.RSTEP >= g.HW)
                v[j] = K;
        }
        if (item + (int)gridDim.x < nitems)
            strip_prefetch<NT, VPT, 1>(stage, g, item + gridDim.x, q, rl, x, nullptr);

        float4 s1, s2;
        {
            const f32x2 nk01 = pk(-K.x, -K.y), nk23 = pk(-K.z, -K.w);
            f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;  // packed zeros
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const f32x2 d01 = pk_add(pk(v[j].x, v[j].y), nk01), d23 = pk_add(pk(v[j].z, v[j].w), nk23);
                a1 = pk_add(a1, d01);
                b1 = pk_add(b1, d23);
                a2 = pk_fma(d01, d01, a2);
                b2 = pk_fma(d23, d23, b2);
            }
            unpk(a1, s1.x, s1.y);
            unpk(b1, s1.z, s1.w);
            unpk(a2, s2.x, s2.y);
            unpk(b2, s2.z, s2.w);
        }
        strip_fold<NT>(red, chan, g.Q, g.Ct, q, rl, s1, s2);
        if (t < g.Gt) {
            const float n = (float)g.HW * (float)g.cpg;
            const float* xrow0 = x + (size_t)b * g.HW * g.C + c0 + t * g.cpg;
            float msum = 0.0f;
            for (int cl = 0; cl < g.cpg; ++cl)
                msum += chan[t * g.cpg + cl] + (float)g.HW * __ldg(xrow0 + cl);
            const float mean = msum / n;
            float m2 = 0.0f;
            for (int cl = 0; cl < g.cpg; ++cl) {
                const int ch = t * g.cpg + cl;
                const float dk = __ldg(xrow0 + cl) - mean;
                m2 += chan[g.Ct + ch] + 2.0f * dk * chan[ch] + (float)g.HW * dk * dk;
            }
            const float rs = rsqrtf(m2 / n + eps);
            gstat[t] = mean;
            gstat[g.Gt + t] = rs;
            mu[b * g.G + c0 / g.cpg + t] = mean;
            rstd[b * g.G + c0 / g.cpg + t] = rs;
        }
        __syncthreads();
        // (loading gamma/beta before the wait was measured: the 8 extra live registers spill and cost
        // more than the L2 round trip they would hide)
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        const float4 be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        float4 sc, sh;
        sc.x = ga.x * gstat[g.Gt + g0]; sh.x = be.x - gstat[g0] * sc.x;
        sc.y = ga.y * gstat[g.Gt + g1]; sh.y = be.y - gstat[g1] * sc.y;
        sc.z = ga.z * gstat[g.Gt + g2]; sh.z = be.z - gstat[g2] * sc.z;
        sc.w = ga.w * gstat[g.Gt + g3]; sh.w = be.w - gstat[g3] * sc.w;
        const f32x2 sc01 = pk(sc.x, sc.y), sc23 = pk(sc.z, sc.w), sh01 = pk(sh.x, sh.y), sh23 = pk(sh.z, sh.w);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int r = rl + j * g.RSTEP;
            if (FULL || r < g.HW) {
                float4 o;
                unpk(act_value_x2<ACT>(pk_fma(pk(v[j].x, v[j].y), sc01, sh01)), o.x, o.y);
                unpk(act_value_x2<ACT>(pk_fma(pk(v[j].z, v[j].w), sc23, sh23)), o.z, o.w);
                __stcs(reinterpret_cast<float4*>(y + base + (size_t)r * g.C), o);
            }
        }
        ctile += step_ct;
        b += step_b;
        if (ctile >= g.nct) {
            ctile -= g.nct;
            ++b;
        }
    }
}

// backward: stage holds x (slots 0..VPT-1) and dy (slots VPT..2*VPT-1)
// (mu / rstd of the next strip through the staging pipeline, as in gn_bwd_ostrip, was measured here too:
// [128,28,28,64] 18.0 -> 19.1 us with the option compiled in but off, 19.8 us with it on -- this kernel sits at
// its register limit and pays for every live value.)
template <int NT, int VPT, int ACT, int MB>
__global__ void __launch_bounds__(NT, MB) gn_bwd_pstrip(float* __restrict__ dx, float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mu, const float* __restrict__ rstd, const StripGeom g,
    const int nitems)
{
    pdl_prologue();
    extern __shared__ float4 strip_stage[];
    constexpr int NW = NT / 32;
    float4* stage = strip_stage;
    float* red = reinterpret_cast<float*>(stage + 2 * VPT * NT);
    const int red_floats = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * NW * g.Ct : 2 * NT * 4;
    float* chan = red + red_floats;
    float* gstat = chan + 2 * g.Ct;
    const int t = threadIdx.x;
    const int q = t % g.Q, rl = t / g.Q;
    const int cb = 4 * q;
    const int gl0 = (cb + 0) / g.cpg, gl1 = (cb + 1) / g.cpg, gl2 = (cb + 2) / g.cpg, gl3 = (cb + 3) / g.cpg;

    int item = blockIdx.x;
    if (item < nitems)
        strip_prefetch<NT, VPT, 2>(stage, g, item, q, rl, x, dy);
    int ctile = item % g.nct, b = item / g.nct;
    const int step_ct = (int)gridDim.x % g.nct, step_b = (int)gridDim.x / g.nct;
    for (; item < nitems; item += gridDim.x) {
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        float4 be = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ACT != ACT_IDENTITY)
            be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        const int gbase = b * g.G + c0 / g.cpg;
        float4 rs4, nm4;
        rs4.x = __ldg(rstd + gbase + gl0); nm4.x = -__ldg(mu + gbase + gl0) * rs4.x;
        rs4.y = __ldg(rstd + gbase + gl1); nm4.y = -__ldg(mu + gbase + gl1) * rs4.y;
        rs4.z = __ldg(rstd + gbase + gl2); nm4.z = -__ldg(mu + gbase + gl2) * rs4.z;
        rs4.w = __ldg(rstd + gbase + gl3); nm4.w = -__ldg(mu + gbase + gl3) * rs4.w;

        cp_async_wait_all();
        float4 xv[VPT], dv[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            xv[j] = stage[j * NT + t];
            dv[j] = stage[(VPT + j) * NT + t];
        }
        if (item + (int)gridDim.x < nitems)
            strip_prefetch<NT, VPT, 2>(stage, g, item + gridDim.x, q, rl, x, dy);

        // xv becomes xhat, dv becomes dy * act'(z), both kept as packed pairs for the second phase
        const f32x2 rs01 = pk(rs4.x, rs4.y), rs23 = pk(rs4.z, rs4.w), nm01 = pk(nm4.x, nm4.y), nm23 = pk(nm4.z, nm4.w);
        const f32x2 ga01 = pk(ga.x, ga.y), ga23 = pk(ga.z, ga.w), be01 = pk(be.x, be.y), be23 = pk(be.z, be.w);
        f32x2 xa[VPT], xb[VPT], da[VPT], db[VPT];
        float4 sA, sB;
        {
            f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;  // packed zeros
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                xa[j] = pk_fma(pk(xv[j].x, xv[j].y), rs01, nm01);
                xb[j] = pk_fma(pk(xv[j].z, xv[j].w), rs23, nm23);
                da[j] = pk(dv[j].x, dv[j].y);
                db[j] = pk(dv[j].z, dv[j].w);
                if (ACT != ACT_IDENTITY) {
                    da[j] = pk_mul(da[j], act_slope_x2<ACT>(pk_fma(ga01, xa[j], be01)));
                    db[j] = pk_mul(db[j], act_slope_x2<ACT>(pk_fma(ga23, xb[j], be23)));
                }
                if (rl + j * g.RSTEP < g.HW) {
                    a1 = pk_add(a1, da[j]);
                    b1 = pk_add(b1, db[j]);
                    a2 = pk_fma(da[j], xa[j], a2);
                    b2 = pk_fma(db[j], xb[j], b2);
                }
            }
            unpk(a1, sA.x, sA.y);
            unpk(b1, sA.z, sA.w);
            unpk(a2, sB.x, sB.y);
            unpk(b2, sB.z, sB.w);
        }
        strip_fold<NT>(red, chan, g.Q, g.Ct, q, rl, sA, sB);
        if (t < g.Gt) {
            float sg = 0.0f, sgx = 0.0f;
            for (int cl = 0; cl < g.cpg; ++cl) {
                const int ch = t * g.cpg + cl;
                const float gm = __ldg(gamma + c0 + ch);
                sg = fmaf(gm, chan[ch], sg);
                sgx = fmaf(gm, chan[g.Ct + ch], sgx);
            }
            const float inv_n = 1.0f / ((float)g.HW * (float)g.cpg);
            gstat[t] = sg * inv_n;
            gstat[g.Gt + t] = sgx * inv_n;
        }
        if (t < g.Ct) {  // one partial row per sample: [b][0:C] dgamma, [b][C:2C] dbeta
            float* dst = partials + (size_t)b * (2 * g.C) + c0 + t;
            dst[0] = chan[g.Ct + t];
            dst[g.C] = chan[t];
        }
        __syncthreads();
        float4 mg, mgx;
        mg.x = gstat[gl0]; mgx.x = gstat[g.Gt + gl0];
        mg.y = gstat[gl1]; mgx.y = gstat[g.Gt + gl1];
        mg.z = gstat[gl2]; mgx.z = gstat[g.Gt + gl2];
        mg.w = gstat[gl3]; mgx.w = gstat[g.Gt + gl3];
        // dx = rstd * (g*gamma - mg - xhat*mgx), as in the reference (kernels.cu:692)
        const f32x2 nmg01 = pk(-mg.x, -mg.y), nmg23 = pk(-mg.z, -mg.w), nmx01 = pk(-mgx.x, -mgx.y), nmx23 = pk(-mgx.z, -mgx.w);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int r = rl + j * g.RSTEP;
            if (r < g.HW) {
                float4 o;
                unpk(pk_mul(rs01, pk_fma(xa[j], nmx01, pk_fma(da[j], ga01, nmg01))), o.x, o.y);
                unpk(pk_mul(rs23, pk_fma(xb[j], nmx23, pk_fma(db[j], ga23, nmg23))), o.z, o.w);
                __stcs(reinterpret_cast<float4*>(dx + base + (size_t)r * g.C), o);
            }
        }
        ctile += step_ct;
        b += step_b;
        if (ctile >= g.nct) {
            ctile -= g.nct;
            ++b;
        }
    }
}

}  // namespace b200
