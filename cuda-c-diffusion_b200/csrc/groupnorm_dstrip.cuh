// Deep-staged GroupNorm backward strips (included by groupnorm.cu after groupnorm_strip.cuh).
//
// Same register-resident strips as gn_bwd_pstrip, with one change to the staging:
// the pipelined kernels hold exactly ONE strip of asynchronous copies in flight per CTA, so from the
// moment a strip has landed until its slots have been moved to registers and re-armed, the SM has no
// load outstanding at all -- a dead window of ~0.7 us in every ~5 us strip period when one CTA owns an
// SM.  Here part of each strip (the "head": all of x) is double-buffered in the shared memory the
// pipelined kernel leaves unused, so the head of
// strip i+2 is already in flight while strip i+1 is being consumed: 1.5 strips of loads per CTA
// instead of 1, never zero.  Every slot is re-armed immediately after it has been read (the copy for a
// slot is issued right behind the shared-memory load that frees it), not after the whole strip.
//
// cp.async groups, oldest first, when an iteration starts: head(i), tail(i), head(i+1); waiting for
// all but the newest group gives strip i.  The iteration then commits tail(i+1) and head(i+2).
// A thread only ever reads the slots it staged itself, so no barrier guards the staging buffers.
// (The forward counterpart, half of each strip double-buffered, was 2-3 % slower than the plain
// pipeline in every variant and is gone.)
#pragma once

namespace b200 {

__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// Offset (in floats) of this thread's first slot of work item `item`.
__device__ __forceinline__ size_t dstrip_item_offset(const StripGeom& g, int item, size_t rowoff)
{
    const int ctile = item % g.nct, b = item / g.nct;
    return (size_t)b * g.HW * g.C + (size_t)ctile * g.Ct + rowoff;
}

// ---------------------------------------------------------------------------
// backward.  x is the head (double-buffered: xs[2][VPT][NT]), dy the tail (ds[VPT][NT]).
// dynamic smem = 3 * VPT * NT * 16 bytes | red | chan | gstat
// ---------------------------------------------------------------------------
template <int NT, int VPT, int ACT, bool FULL>
__global__ void __launch_bounds__(NT, 1) gn_bwd_dstrip(float* __restrict__ dx, float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mu, const float* __restrict__ rstd, const StripGeom g,
    const int nitems)
{
    pdl_prologue();
    extern __shared__ float4 strip_stage[];
    constexpr int NW = NT / 32;
    float4* xs = strip_stage;              // [2][VPT][NT]
    float4* ds = xs + 2 * VPT * NT;        // [VPT][NT]
    float* red = reinterpret_cast<float*>(ds + VPT * NT);
    const int red_floats = (g.Q <= 32 && 32 % g.Q == 0) ? 2 * NW * g.Ct : 2 * NT * 4;
    float* chan = red + red_floats;
    float* gstat = chan + 2 * g.Ct;
    const int t = threadIdx.x;
    const int q = t % g.Q, rl = t / g.Q;
    const int cb = 4 * q;
    const int gl0 = (cb + 0) / g.cpg, gl1 = (cb + 1) / g.cpg, gl2 = (cb + 2) / g.cpg, gl3 = (cb + 3) / g.cpg;
    const size_t rowoff = (size_t)rl * g.C + cb;
    const size_t jstride = (size_t)g.RSTEP * g.C;
    const int G = gridDim.x;

    int item = blockIdx.x;
    {   // prologue: x(0), dy(0), x(1)
        const size_t o0 = dstrip_item_offset(g, item < nitems ? item : 0, rowoff);
        if (item < nitems) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16(&xs[j * NT + t], x + o0 + j * jstride);
        }
        cp_async_commit();
        if (item < nitems) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16(&ds[j * NT + t], dy + o0 + j * jstride);
        }
        cp_async_commit();
        if (item + G < nitems) {
            const size_t o1 = dstrip_item_offset(g, item + G, rowoff);
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16(&xs[(VPT + j) * NT + t], x + o1 + j * jstride);
        }
        cp_async_commit();
    }
    int par = 0;
    for (; item < nitems; item += G, par ^= 1) {
        const int ctile = item % g.nct, b = item / g.nct;
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0 + cb;
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
        const bool more1 = item + G < nitems, more2 = item + 2 * G < nitems;
        const float* n1 = dy + dstrip_item_offset(g, more1 ? item + G : item, rowoff);
        const float* n2 = x + dstrip_item_offset(g, more2 ? item + 2 * G : item, rowoff);
        float4* xc = xs + par * VPT * NT;

        cp_async_wait_but_one();
        float4 xv[VPT], dv[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {  // dy slots: read, then re-arm with strip i+1
            const bool live = FULL || rl + j * g.RSTEP < g.HW;
            dv[j] = live ? ds[j * NT + t] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (more1 && live)
                cp_async16(&ds[j * NT + t], n1 + j * jstride);
        }
        cp_async_commit();
#pragma unroll
        for (int j = 0; j < VPT; ++j) {  // x slots of this parity: read, then re-arm with strip i+2
            const bool live = FULL || rl + j * g.RSTEP < g.HW;
            xv[j] = live ? xc[j * NT + t] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (more2 && live)
                cp_async16(&xc[j * NT + t], n2 + j * jstride);
        }
        cp_async_commit();

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
                // rows past the end carry dy = 0, so they add nothing to either sum
                a1 = pk_add(a1, da[j]);
                b1 = pk_add(b1, db[j]);
                a2 = pk_fma(da[j], xa[j], a2);
                b2 = pk_fma(db[j], xb[j], b2);
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
        float* orow = dx + base + (size_t)rl * g.C;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (FULL || rl + j * g.RSTEP < g.HW) {
                float4 o;
                unpk(pk_mul(rs01, pk_fma(xa[j], nmx01, pk_fma(da[j], ga01, nmg01))), o.x, o.y);
                unpk(pk_mul(rs23, pk_fma(xb[j], nmx23, pk_fma(db[j], ga23, nmg23))), o.z, o.w);
                __stcs(reinterpret_cast<float4*>(orow + j * jstride), o);
            }
        }
    }
    cp_async_wait_all();
}

}  // namespace b200
