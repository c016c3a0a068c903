// Chunked GroupNorm strips (included by groupnorm.cu after groupnorm_strip.cuh): samples whose
// [HW x Ct] strip does not fit the register file (64x64 images and larger).
//
// A CTA still owns whole strips (all HW rows of one sample x Ct channels covering whole groups),
// but walks each strip twice in chunks of RSTEP*VPT rows:
//   pass 1  accumulates the shifted sums (forward) or the two group sums and the dgamma/dbeta
//           partials (backward) chunk by chunk in registers;
//   pass 2  reads the same chunks again, normalises (or forms dx) and stores.
// Both passes use the cp.async pipeline of the register-resident strips: while a chunk is processed
// from registers, the next chunk (of the same pass, of the other pass, or of the next strip) is
// already in flight into shared memory, each thread staging only the slots it reads back itself.
// The second read of a strip comes from L2 as long as the strips in flight fit there
// (resident CTAs x HW x Ct x 4 bytes per tensor against 126 MB), so DRAM still sees every input
// byte once; beyond that the strip is read from DRAM twice, which is still fewer bytes and far
// fewer barriers than the tile kernels need.
// (A two-deep ring of chunk buffers over a flattened (strip, pass, chunk) sequence was measured:
// 10 % faster on 128x128 samples, 8-12 % slower on 64x64 ones with an activation; not kept.
// So was the cluster barrier in front of every staging burst that helps the register-resident forward
// (groupnorm_ostrip.cuh): here, with two barriers per chunk, [32,64,64,256] went from 0.67 to 0.57-0.59
// of the copy rate and [16,128,128,128] from 0.51 to 0.37-0.42.)
#pragma once

namespace b200 {

template <int NT, int VPT, int NTENS>
__device__ __forceinline__ void cstrip_prefetch(float4* stage, const StripGeom& g, size_t base, int row0, int rl,
    const float* __restrict__ t0, const float* __restrict__ t1)
{
    const uint64_t pol = l2_policy(g.hint);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int r = row0 + rl + j * g.RSTEP;
        if (r < g.HW) {
            cp_async16_hint(&stage[j * NT + threadIdx.x], t0 + base + (size_t)r * g.C, pol);
            if (NTENS == 2)
                cp_async16_hint(&stage[(VPT + j) * NT + threadIdx.x], t1 + base + (size_t)r * g.C, pol);
        }
    }
    cp_async_commit();
}

// grid = min(items, resident CTAs), block = NT; dynamic smem = stage[VPT*NT float4] | red | chan | gstat
template <int NT, int VPT, int ACT, int MB>
__global__ void __launch_bounds__(NT, MB) gn_fwd_cstrip(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const StripGeom g, const float eps, const int nitems, const int nchunks)
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
    const int R = g.RSTEP * VPT;  // rows per chunk

    int item = blockIdx.x;
    int ctile = item % g.nct, b = item / g.nct;
    const int step_ct = (int)gridDim.x % g.nct, step_b = (int)gridDim.x / g.nct;
    if (item < nitems)
        cstrip_prefetch<NT, VPT, 1>(stage, g, (size_t)b * g.HW * g.C + ctile * g.Ct + 4 * q, 0, rl, x, nullptr);
    for (; item < nitems; item += gridDim.x) {
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;
        const float4 K = __ldg(reinterpret_cast<const float4*>(x + base));  // shift: row 0 of the sample
        int nctile = ctile + step_ct, nb = b + step_b;
        if (nctile >= g.nct) {
            nctile -= g.nct;
            ++nb;
        }
        const f32x2 nk01 = pk(-K.x, -K.y), nk23 = pk(-K.z, -K.w);
        f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;  // packed zeros

        // ---- pass 1: shifted sums over all chunks
        for (int k = 0; k < nchunks; ++k) {
            cp_async_wait_all();
            float4 v[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                v[j] = stage[j * NT + t];
                if (k * R + rl + j * g.RSTEP >= g.HW)
                    v[j] = K;  // rows past the end contribute zero
            }
            // next: the following chunk, or chunk 0 again for the second pass
            cstrip_prefetch<NT, VPT, 1>(stage, g, base, (k + 1 < nchunks) ? (k + 1) * R : 0, rl, x, nullptr);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const f32x2 d01 = pk_add(pk(v[j].x, v[j].y), nk01), d23 = pk_add(pk(v[j].z, v[j].w), nk23);
                a1 = pk_add(a1, d01);
                b1 = pk_add(b1, d23);
                a2 = pk_fma(d01, d01, a2);
                b2 = pk_fma(d23, d23, b2);
            }
        }
        float4 s1, s2;
        unpk(a1, s1.x, s1.y);
        unpk(b1, s1.z, s1.w);
        unpk(a2, s2.x, s2.y);
        unpk(b2, s2.z, s2.w);
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
            mu[b * g.G + ctile * g.Gt + t] = mean;
            rstd[b * g.G + ctile * g.Gt + t] = rs;
        }
        __syncthreads();
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        const float4 be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        float4 sc, sh;
        sc.x = ga.x * gstat[g.Gt + g0]; sh.x = be.x - gstat[g0] * sc.x;
        sc.y = ga.y * gstat[g.Gt + g1]; sh.y = be.y - gstat[g1] * sc.y;
        sc.z = ga.z * gstat[g.Gt + g2]; sh.z = be.z - gstat[g2] * sc.z;
        sc.w = ga.w * gstat[g.Gt + g3]; sh.w = be.w - gstat[g3] * sc.w;
        const f32x2 sc01 = pk(sc.x, sc.y), sc23 = pk(sc.z, sc.w), sh01 = pk(sh.x, sh.y), sh23 = pk(sh.z, sh.w);

        // ---- pass 2: normalise, activate, store
        for (int k = 0; k < nchunks; ++k) {
            cp_async_wait_all();
            float4 v[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                v[j] = stage[j * NT + t];
            if (k + 1 < nchunks)
                cstrip_prefetch<NT, VPT, 1>(stage, g, base, (k + 1) * R, rl, x, nullptr);
            else if (item + (int)gridDim.x < nitems)
                cstrip_prefetch<NT, VPT, 1>(stage, g, (size_t)nb * g.HW * g.C + nctile * g.Ct + 4 * q, 0, rl, x, nullptr);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int r = k * R + rl + j * g.RSTEP;
                if (r < g.HW) {
                    float4 o;
                    unpk(act_value_x2<ACT>(pk_fma(pk(v[j].x, v[j].y), sc01, sh01)), o.x, o.y);
                    unpk(act_value_x2<ACT>(pk_fma(pk(v[j].z, v[j].w), sc23, sh23)), o.z, o.w);
                    __stcs(reinterpret_cast<float4*>(y + base + (size_t)r * g.C), o);
                }
            }
        }
        // gstat / chan are rewritten only after the next strip's fold barriers
        ctile = nctile;
        b = nb;
    }
}

// backward: stage holds x (slots 0..VPT-1) and dy (slots VPT..2*VPT-1) of one chunk
template <int NT, int VPT, int ACT, int MB>
__global__ void __launch_bounds__(NT, MB) gn_bwd_cstrip(float* __restrict__ dx, float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mu, const float* __restrict__ rstd, const StripGeom g,
    const int nitems, const int nchunks)
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
    const int R = g.RSTEP * VPT;

    int item = blockIdx.x;
    int ctile = item % g.nct, b = item / g.nct;
    const int step_ct = (int)gridDim.x % g.nct, step_b = (int)gridDim.x / g.nct;
    if (item < nitems)
        cstrip_prefetch<NT, VPT, 2>(stage, g, (size_t)b * g.HW * g.C + ctile * g.Ct + 4 * q, 0, rl, x, dy);
    for (; item < nitems; item += gridDim.x) {
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0 + 4 * q;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + c0) + q);
        float4 be = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ACT != ACT_IDENTITY)
            be = __ldg(reinterpret_cast<const float4*>(beta + c0) + q);
        const int gbase = b * g.G + ctile * g.Gt;
        float4 rs4, nm4;
        rs4.x = __ldg(rstd + gbase + gl0); nm4.x = -__ldg(mu + gbase + gl0) * rs4.x;
        rs4.y = __ldg(rstd + gbase + gl1); nm4.y = -__ldg(mu + gbase + gl1) * rs4.y;
        rs4.z = __ldg(rstd + gbase + gl2); nm4.z = -__ldg(mu + gbase + gl2) * rs4.z;
        rs4.w = __ldg(rstd + gbase + gl3); nm4.w = -__ldg(mu + gbase + gl3) * rs4.w;
        int nctile = ctile + step_ct, nb = b + step_b;
        if (nctile >= g.nct) {
            nctile -= g.nct;
            ++nb;
        }
        const f32x2 rs01 = pk(rs4.x, rs4.y), rs23 = pk(rs4.z, rs4.w), nm01 = pk(nm4.x, nm4.y), nm23 = pk(nm4.z, nm4.w);
        const f32x2 ga01 = pk(ga.x, ga.y), ga23 = pk(ga.z, ga.w), be01 = pk(be.x, be.y), be23 = pk(be.z, be.w);

        // ---- pass 1: sum g and sum g*xhat per channel, g = dy * act'(z)
        f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;
        for (int k = 0; k < nchunks; ++k) {
            cp_async_wait_all();
            float4 xv[VPT], dv[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                xv[j] = stage[j * NT + t];
                dv[j] = stage[(VPT + j) * NT + t];
            }
            cstrip_prefetch<NT, VPT, 2>(stage, g, base, (k + 1 < nchunks) ? (k + 1) * R : 0, rl, x, dy);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const f32x2 xa = pk_fma(pk(xv[j].x, xv[j].y), rs01, nm01), xb = pk_fma(pk(xv[j].z, xv[j].w), rs23, nm23);
                f32x2 da = pk(dv[j].x, dv[j].y), db = pk(dv[j].z, dv[j].w);
                if (ACT != ACT_IDENTITY) {
                    da = pk_mul(da, act_slope_x2<ACT>(pk_fma(ga01, xa, be01)));
                    db = pk_mul(db, act_slope_x2<ACT>(pk_fma(ga23, xb, be23)));
                }
                if (k * R + rl + j * g.RSTEP < g.HW) {  // slots past the last row hold stale shared memory
                    a1 = pk_add(a1, da);
                    b1 = pk_add(b1, db);
                    a2 = pk_fma(da, xa, a2);
                    b2 = pk_fma(db, xb, b2);
                }
            }
        }
        float4 sA, sB;
        unpk(a1, sA.x, sA.y);
        unpk(b1, sA.z, sA.w);
        unpk(a2, sB.x, sB.y);
        unpk(b2, sB.z, sB.w);
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
        const f32x2 nmg01 = pk(-mg.x, -mg.y), nmg23 = pk(-mg.z, -mg.w), nmx01 = pk(-mgx.x, -mgx.y), nmx23 = pk(-mgx.z, -mgx.w);

        // ---- pass 2: dx = rstd * (g*gamma - mg - xhat*mgx)
        for (int k = 0; k < nchunks; ++k) {
            cp_async_wait_all();
            float4 xv[VPT], dv[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                xv[j] = stage[j * NT + t];
                dv[j] = stage[(VPT + j) * NT + t];
            }
            if (k + 1 < nchunks)
                cstrip_prefetch<NT, VPT, 2>(stage, g, base, (k + 1) * R, rl, x, dy);
            else if (item + (int)gridDim.x < nitems)
                cstrip_prefetch<NT, VPT, 2>(stage, g, (size_t)nb * g.HW * g.C + nctile * g.Ct + 4 * q, 0, rl, x, dy);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int r = k * R + rl + j * g.RSTEP;
                if (r < g.HW) {
                    const f32x2 xa = pk_fma(pk(xv[j].x, xv[j].y), rs01, nm01), xb = pk_fma(pk(xv[j].z, xv[j].w), rs23, nm23);
                    f32x2 da = pk(dv[j].x, dv[j].y), db = pk(dv[j].z, dv[j].w);
                    if (ACT != ACT_IDENTITY) {
                        da = pk_mul(da, act_slope_x2<ACT>(pk_fma(ga01, xa, be01)));
                        db = pk_mul(db, act_slope_x2<ACT>(pk_fma(ga23, xb, be23)));
                    }
                    float4 o;
                    unpk(pk_mul(rs01, pk_fma(xa, nmx01, pk_fma(da, ga01, nmg01))), o.x, o.y);
                    unpk(pk_mul(rs23, pk_fma(xb, nmx23, pk_fma(db, ga23, nmg23))), o.z, o.w);
                    __stcs(reinterpret_cast<float4*>(dx + base + (size_t)r * g.C), o);
                }
            }
        }
        ctile = nctile;
        b = nb;
    }
}

}  // namespace b200
