// One-barrier GroupNorm strip kernels (included by groupnorm.cu after groupnorm_dstrip.cuh).
//
// The pipelined strips of groupnorm_strip.cuh / groupnorm_dstrip.cuh cross three CTA barriers per
// strip, and between them a handful of threads works while the rest of the SM waits: Ct threads add
// the per-warp channel sums, then Gt threads turn channel sums into group statistics (with global
// loads of gamma, of the shift row or of mu/rstd on that path).  With one 512- or 1024-thread CTA per
// SM nothing else can run during those sections, so they are pure latency on every strip.
//
// Here a strip crosses ONE barrier:
//   * the sums that the second phase needs are reduced to GROUP level inside each warp (xor shuffles
//     over the lanes that share a group), one float2 per (warp, group) goes to shared memory, and after
//     the barrier every warp forms the totals of its own groups: the lanes that share a group split the NW
//     per-warp values between them and combine with the same shuffles -- no elected threads, no second
//     and third barrier, a fixed order of additions (results are bit-reproducible);
//   * the reduction buffers alternate with the strip parity, which is what makes the single barrier
//     sufficient (a buffer is rewritten two strips later, after every thread has passed the barrier
//     in between);
//   * everything a strip needs from global memory besides the strip itself is fetched a strip ahead by
//     the thread that uses it: the shift of the forward pass (row 0 of the group's first channel) through
//     the staging pipeline, mu/rstd of the backward pass (which come from DRAM, a microsecond away) into
//     registers; gamma and beta of all C channels are copied to shared memory once per CTA;
//   * the backward's per-channel sums (dgamma/dbeta partial rows) are still written per warp, but they
//     are added up by Ct threads AFTER those threads have issued their dx stores: off the critical path.
//
// Measured on [256,32,32,256] with SiLU, each kernel alone in a loop (fraction of the copy rate): backward
// 0.83 -> 0.88 (0.86 -> 0.97 without activation); forward 0.86 -> 0.78 as plain CTAs, 0.90 in clusters of
// 4 (see gn_fwd_ostrip).  With only a few strips per CTA the longer set-up loses, so the dispatcher keeps
// the three-barrier kernels for such launches.
//
// Forward statistics use one shift per GROUP (the group's first channel in row 0) instead of one per
// channel: mean = K + S1/n, var = S2/n - (S1/n)^2 with S1, S2 the sums of (x - K) and (x - K)^2.  S1 can be
// as large as n * |K - mean|, so its cross-warp total is carried as an unevaluated pair of floats and the
// division keeps the remainder: the mean loses nothing to the size of the shift.
//
// Applies when a thread's float4 lies in one group (cpg a multiple of 4, cpg/4 a power of two: GPT = 1)
// or in exactly two (cpg = 2: GPT = 2), Q = Ct/4 is a power of two <= 32 and C <= 2048.
#pragma once

namespace b200 {

// Floats per group row of the per-warp partial sums: NW float2 plus padding such that the rows of different
// groups never start on the same bank (a stride of exactly 32 floats, NW = 14, cost the backward of
// [256,28,28,128] 10 %: four groups per warp read their rows at once).
__host__ __device__ constexpr int ostrip_row_floats(int nw) { return (2 * nw + 4) | 4; }

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

// 128-bit shared-memory load that stays ONE instruction (left to the compiler, the backward's staging reads
// came out as four 32-bit loads each: 74 instead of 23 shared loads per thread and strip)
__device__ __forceinline__ float4 lds128(const float4* p)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_addr(p)) : "memory");
    return v;
}

// cp.async.wait_group with a run-time count in 0..7 (folds to one instruction where the count is known after unrolling)
__device__ __forceinline__ void cp_async_wait_pending(int n)
{
    switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

// --- TMA staging of the backward strips (tensor maps: tma_desc.cuh) -----------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// One arrival that also announces `bytes` of asynchronous copies.  `after` is a value loaded from the buffer that
// the copies will overwrite: naming it as an operand keeps the issue behind the return of that load (shared-memory
// loads of a warp return in order, so behind all earlier ones too).
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes, float after)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes), "f"(after) : "memory");
}
// Box of the 2-D tensor map at (cx, cy) -> dense rows at dst; completion counts on bar.  One CTA's own load.
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, int cx, int cy, uint64_t* bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(cx), "r"(cy), "r"(smem_addr(bar)), "l"(policy) : "memory");
}
// Waits for the phase of the given parity, for at most about a second; after that the error word is set and
// false returned (the caller stops waiting on anything and runs to its end).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* err)
{
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
        if (ok)
            return true;
        if (clock64() - t0 > 2000000000LL) {
            if (err)
                atomicExch(err, 0x6e01);
            return false;
        }
    }
}

// Lanes of a warp that share a group: Lg of them, this lane being number li (the same numbering in every
// warp, so every warp derives bit-identical totals from the same partials).
struct OStripLanes {
    int li, Lg;
};
template <int GPT>
__device__ __forceinline__ OStripLanes ostrip_lanes(int lane, int q, int Q, int M)
{
    OStripLanes r;
    if (GPT == 1) {
        r.Lg = M * (32 / Q);
        r.li = (q & (M - 1)) + M * (lane / Q);
    } else {
        r.Lg = 32 / Q;
        r.li = lane / Q;
    }
    return r;
}

// a + b as an unevaluated pair (sum, rounding error): Knuth's two-sum, symmetric in its arguments.
__device__ __forceinline__ void two_sum(float a, float b, float& s, float& e)
{
    s = a + b;
    const float bb = s - a;
    e = (a - (s - bb)) + (b - bb);
}

// Total over the NW per-warp float2 partials of one group after the barrier: each of the group's Lg lanes adds
// the partials li, li + Lg, ..., then the lanes combine over the same xor offsets that formed the partials.
// The first component is carried as (hi, lo): in the forward pass it is a sum of n shifted values whose
// magnitude n * |shift - mean| would otherwise cost the mean its last digits.
template <int NW, bool PAIR>
__device__ __forceinline__ void ostrip_group_total(const float* rg, const OStripLanes ln, int Q, int M, float& hi, float& lo,
    float& second)
{
    float h = 0.0f, l = 0.0f, b = 0.0f;
    for (int i = ln.li; i < NW; i += ln.Lg) {
        const float2 p = *reinterpret_cast<const float2*>(rg + 2 * i);
        if (PAIR) {
            float e;
            two_sum(h, p.x, h, e);
            l += e;
        } else {
            h += p.x;
        }
        b += p.y;
    }
    auto step = [&](int off) {
        const float h2 = __shfl_xor_sync(0xffffffffu, h, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
        if (PAIR) {
            const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
            float e;
            two_sum(h, h2, h, e);
            l = (l + l2) + e;
        } else {
            h += h2;
        }
    };
    for (int off = 1; off < M; off <<= 1)
        step(off);
    for (int off = Q; off < 32; off <<= 1)
        step(off);
    hi = h;
    lo = l;
    second = b;
}

// The same total with no shuffles: every lane reads all NW per-warp partials of its group (broadcast 128-bit loads)
// and adds them in a fixed order.  For the backward kernels (16 warps, shared-memory and shuffle queue already the
// busiest unit): fewer queue entries than the lane-split form.
template <int NW>
__device__ __forceinline__ void ostrip_group_total_direct(const float* rg, float& first, float& second)
{
    float2 a0 = make_float2(0.f, 0.f), a1 = a0;
#pragma unroll
    for (int w = 0; w < NW; w += 2) {
        const float4 p = *reinterpret_cast<const float4*>(rg + 2 * w);
        a0.x += p.x; a0.y += p.y;
        a1.x += p.z; a1.y += p.w;
    }
    first = a0.x + a1.x;
    second = a0.y + a1.y;
}

// ---------------------------------------------------------------------------
// forward: one strip staged ahead (staging half of a second strip as well, the way the backward double-buffers x,
// measured 3 % slower with and without clusters).
// dynamic smem = stage[VPT][NT] float4 | kst[GPT][NT] | gamma[C] | beta[C] | redg[2][Gt][ostrip_row_floats(NW)]
//
// Launched as clusters of 4 CTAs where that applies (1024-thread CTAs, many strips each, strips per sample a
// multiple of 4): consecutive CTAs walk consecutive strips, i.e. neighbouring 128-byte column tiles of the SAME
// rows, and a cluster barrier in front of every staging burst makes the four bursts (and later the four store
// phases) coincide, so that DRAM sees 512 contiguous bytes per row at once instead of four isolated 128-byte
// accesses at different times.  Measured on [256,32,32,256]: 0.78 -> 0.90 of the copy rate, although only 132
// of the 148 SMs can hold a cluster of 4 at one CTA per SM; widths 2 (0.85) and 8 (0.83, 120 SMs) lose.
// ---------------------------------------------------------------------------
template <int NT, int VPT, int ACT, int MB, bool FULL, int GPT>
__global__ void __launch_bounds__(NT, MB) gn_fwd_ostrip(float* __restrict__ y, float* __restrict__ mu,
    float* __restrict__ rstd, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const StripGeom g, const float eps, const int nitems)
{
    pdl_prologue();
    const uint64_t pol = l2_policy(g.hint);
    constexpr int NW = NT / 32;
    constexpr int RG = ostrip_row_floats(NW);
    extern __shared__ float4 strip_stage[];
    float4* stage = strip_stage;
    float* kst = reinterpret_cast<float*>(stage + VPT * NT);  // slot [k][t]: shift of this thread's group k
    float* gsm = kst + GPT * NT;
    float* bsm = gsm + g.C;
    float* redg = bsm + g.C;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int q = t % g.Q, rl = t / g.Q;
    const int cb = 4 * q;
    const int M = GPT == 1 ? (g.cpg >> 2) : 1;       // lanes (float4 columns) per group
    const int gl = GPT == 1 ? q / M : 2 * q;          // this thread's (first) group within the strip
    const int koff = gl * g.cpg;                      // first channel of that group: row 0 of it is the shift
    const OStripLanes ln = ostrip_lanes<GPT>(lane, q, g.Q, M);
    const float nf = (float)g.HW * (float)g.cpg;
    const bool writer = lane < g.Q && (GPT == 2 || (lane & (M - 1)) == 0);
    const float inv_n = 1.0f / nf;
    const size_t rowoff = (size_t)rl * g.C + cb;
    const size_t jstride = (size_t)g.RSTEP * g.C;
    const int G = gridDim.x;
    // Without an activation the second phase is a few instructions per element, and 128 KB of stores would leave
    // in one burst; measured, stores spread over the strip period serve DRAM better (0.84 -> 0.89 of the copy rate on
    // [256,32,32,256]; a fixed 250 ns between row blocks: 0.91).  So there each row block's store waits until one
    // more row block of the NEXT strip has landed: stores leave at the rate at which loads arrive.  With SiLU the
    // arithmetic already paces the stores and the same scheme costs 5 %.
    // Only for launches with many strips per CTA (the host sets g.paced): with 2-4 strips the waits cost more.
    const bool paced = ACT == ACT_IDENTITY && VPT <= 8 && g.paced != 0;

    for (int i = t; i < g.C / 4; i += NT) {
        reinterpret_cast<float4*>(gsm)[i] = __ldg(reinterpret_cast<const float4*>(gamma) + i);
        reinterpret_cast<float4*>(bsm)[i] = __ldg(reinterpret_cast<const float4*>(beta) + i);
    }
    // asynchronous copies of work item `it` into the staging slots of this thread (and its shift slots)
    auto stage_item = [&](int it) {
        const size_t sb = dstrip_item_offset(g, it, 0);
#pragma unroll
        for (int k = 0; k < GPT; ++k)
            cp_async4(&kst[k * NT + t], x + sb + koff + k * g.cpg);
        const float* src = x + sb + rowoff;  // advanced row block by row block: one 64-bit add per copy
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (FULL || rl + j * g.RSTEP < g.HW)
                cp_async16_hint(&stage[j * NT + t], src, pol);
            src += jstride;
            if (paced && j + 1 < VPT)
                cp_async_commit();  // one group per slot (the caller commits the last)
        }
    };
    int item = blockIdx.x;
    if (item < nitems)
        stage_item(item);
    cp_async_commit();
    __syncthreads();  // gamma / beta staged
    // CTAs of a cluster walk neighbouring strips of the same rows; a cluster barrier before each staging burst
    // keeps their requests for one DRAM page together.  Only when every CTA of a cluster runs the same number of
    // iterations (grid and item count multiples of the cluster width), else no CTA touches the barrier.
    unsigned csize;
    asm("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(csize));
    const bool csync = csize > 1 && G % (int)csize == 0 && nitems % (int)csize == 0;

    int par = 0;
    for (; item < nitems; item += G, par ^= 1) {
        const int ctile = item % g.nct, b = item / g.nct;
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0;
        cp_async_wait_all();
        if (csync)  // arrive now, wait after the shared-memory reads: the barrier's latency hides behind them
            asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        const float k0 = kst[t], k1 = kst[(GPT - 1) * NT + t];
        float4 v[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            v[j] = stage[j * NT + t];
            if (!FULL && rl + j * g.RSTEP >= g.HW)
                v[j] = make_float4(k0, k0, k1, k1);  // contributes zero to the shifted sums
        }
        if (csync)
            asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        if (item + G < nitems)
            stage_item(item + G);
        else if (paced) {
#pragma unroll
            for (int j = 0; j + 1 < VPT; ++j)
                cp_async_commit();  // empty groups keep the count per strip the same
        }
        cp_async_commit();

        float S1[GPT], S2[GPT];
        {
            const f32x2 nk01 = pk1(-k0), nk23 = pk1(-k1);
            f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;  // packed zeros
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const f32x2 d01 = pk_add(pk(v[j].x, v[j].y), nk01), d23 = pk_add(pk(v[j].z, v[j].w), nk23);
                a1 = pk_add(a1, d01);
                b1 = pk_add(b1, d23);
                a2 = pk_fma(d01, d01, a2);
                b2 = pk_fma(d23, d23, b2);
            }
            float a1l, a1h, b1l, b1h, a2l, a2h, b2l, b2h;
            unpk(a1, a1l, a1h);
            unpk(b1, b1l, b1h);
            unpk(a2, a2l, a2h);
            unpk(b2, b2l, b2h);
            if constexpr (GPT == 1) {
                S1[0] = (a1l + a1h) + (b1l + b1h);
                S2[0] = (a2l + a2h) + (b2l + b2h);
            } else {
                S1[0] = a1l + a1h; S1[1] = b1l + b1h;
                S2[0] = a2l + a2h; S2[1] = b2l + b2h;
            }
        }
        // lanes of one group within the warp: the row lanes (offsets Q .. 16) and, for GPT = 1, the M
        // neighbouring float4 columns (offsets 1 .. M/2)
        for (int off = g.Q; off < 32; off <<= 1) {
#pragma unroll
            for (int k = 0; k < GPT; ++k) {
                S1[k] += __shfl_xor_sync(0xffffffffu, S1[k], off);
                S2[k] += __shfl_xor_sync(0xffffffffu, S2[k], off);
            }
        }
        if constexpr (GPT == 1) {
            for (int off = 1; off < M; off <<= 1) {
                S1[0] += __shfl_xor_sync(0xffffffffu, S1[0], off);
                S2[0] += __shfl_xor_sync(0xffffffffu, S2[0], off);
            }
        }
        float* rg = redg + par * g.Gt * RG;
        if (writer) {
#pragma unroll
            for (int k = 0; k < GPT; ++k)
                *reinterpret_cast<float2*>(rg + (gl + k) * RG + 2 * warp) = make_float2(S1[k], S2[k]);
        }
        __syncthreads();

        float mean[GPT], rs[GPT];
#pragma unroll
        for (int k = 0; k < GPT; ++k) {
            float hi, lo, s2;
            ostrip_group_total<NW, true>(rg + (gl + k) * RG, ln, g.Q, M, hi, lo, s2);
            // S1 / n to full precision: quotient of the leading part, exact remainder, then the tail
            const float qh = hi * inv_n;
            const float rem = (fmaf(-qh, nf, hi) + lo) * inv_n;
            const float m1 = qh + rem;
            const float var = fmaxf(fmaf(-m1, m1, s2 * inv_n), 0.0f);
            rs[k] = rsqrtf(var + eps);
            mean[k] = ((k == 0 ? k0 : k1) + qh) + rem;
        }
        if (warp == 0 && writer) {
            const int gi = b * g.G + c0 / g.cpg + gl;
#pragma unroll
            for (int k = 0; k < GPT; ++k) {
                mu[gi + k] = mean[k];
                rstd[gi + k] = rs[k];
            }
        }
        const float4 ga = *reinterpret_cast<const float4*>(gsm + c0 + cb);
        const float4 be = *reinterpret_cast<const float4*>(bsm + c0 + cb);
        const float rs0 = rs[0], rs1 = rs[GPT - 1], mean0 = mean[0], mean1 = mean[GPT - 1];
        float4 sc, sh;
        sc.x = ga.x * rs0; sh.x = be.x - mean0 * sc.x;
        sc.y = ga.y * rs0; sh.y = be.y - mean0 * sc.y;
        sc.z = ga.z * rs1; sh.z = be.z - mean1 * sc.z;
        sc.w = ga.w * rs1; sh.w = be.w - mean1 * sc.w;
        const f32x2 sc01 = pk(sc.x, sc.y), sc23 = pk(sc.z, sc.w), sh01 = pk(sh.x, sh.y), sh23 = pk(sh.z, sh.w);
        float* yrow = y + base + rowoff;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (FULL || rl + j * g.RSTEP < g.HW) {
                float4 o;
                unpk(act_value_x2<ACT>(pk_fma(pk(v[j].x, v[j].y), sc01, sh01)), o.x, o.y);
                unpk(act_value_x2<ACT>(pk_fma(pk(v[j].z, v[j].w), sc23, sh23)), o.z, o.w);
                __stcs(reinterpret_cast<float4*>(yrow), o);
            }
            yrow += jstride;
            if (paced)
                cp_async_wait_pending(VPT - 1 - j);
        }
    }
    cp_async_wait_all();
}

// ---------------------------------------------------------------------------
// backward (deep-staged: x double-buffered, dy single-buffered, as in gn_bwd_dstrip).
// dynamic smem = [pad to 128 B] xs[2][VPT][NT] float4 | ds[VPT][NT] float4 | gamma[C] | beta[C]
//              | redg[2][Gt][ostrip_row_floats(NW)] | redc[2][NW][2][Q] float4 | wsum[NW][32][8] (Q == 4 only)
//
// mu and rstd of the next strip are fetched into registers one strip ahead (two or four plain loads per thread
// and strip; staged through shared memory they cost a copy and a load each on the busiest queue).
//
// TMA = true (whole strips only): the strip's rows are dealt to the warps in contiguous blocks of VPT * 32 / Q
// rows instead of interleaved, so that everything one warp reads of a tensor is ONE box of the 2-D tensor map
// [B * HW rows, C] -- [VPT * 32 / Q rows, Ct channels], dense in shared memory in the warp's slot order.  Lane 0
// of each warp issues the warp's three boxes (x twice, dy once) and every warp waits on its own mbarriers:
// staging stays private to the warp as it is private to the thread without TMA, no CTA barrier is added, and
// 16 of the about 70 shared-memory-queue entries per thread and strip disappear.
// Measured on [256,32,32,256] with SiLU: alone in a loop 133 -> 126 us (0.92 -> 0.98 of the copy rate), after a
// GroupNorm forward 152 -> 142 us, but after a LayerNorm forward 145 -> 169 us, and the benchmark step as a whole
// 438 -> 472 us when it is the first thing a process times (460 -> 452 us at the end of the same process).
// Without activation 125 -> 165 us alone; the 448 x 7 strips of [256,28,28,128] 55.6 -> 56.5 us.  So the
// dispatcher uses it only on request.  Also measured: the interleaved row order kept and one box of 32 / Q rows
// per row block (VPT boxes per warp and tensor): 141 us alone; the row blocks with cp.async: 132-135 us, as before.
// What the boxes' lines do in L2 decides the rest (StripGeom::hint, tensor-map L2 promotion): evict_first 161 us
// alone; promotion to 128 or 256 bytes 123.4 us alone (1.00 of the copy rate) but 469-472 us for the step;
// evict_last 123.3-126 us alone and, for the step, 429 us on one GPU and 451-459 us on another of the same
// pool, where the cp.async form gives 438-441 us on every one.
// ---------------------------------------------------------------------------
template <int NT, int VPT, int ACT, bool FULL, int GPT, bool TMA>
__global__ void __launch_bounds__(NT, 1) gn_bwd_ostrip(float* __restrict__ dx, float* __restrict__ partials,
    const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mu, const float* __restrict__ rstd, const StripGeom g,
    const int nitems, int* __restrict__ err, const __grid_constant__ CUtensorMap mapx,
    const __grid_constant__ CUtensorMap mapdy)
{
    static_assert(!TMA || FULL, "boxes cover whole strips");
    pdl_prologue();
    const uint64_t pol = l2_policy(g.hint);
    constexpr int NW = NT / 32;
    constexpr int RG = ostrip_row_floats(NW);
    constexpr uint32_t BOX_BYTES = VPT * 32 * 16;  // one box per warp, tensor and strip
    extern __shared__ float4 strip_stage[];
    __shared__ uint64_t mbar[TMA ? 3 * NW : 1];  // per warp: x parity 0, x parity 1, dy
    float4* xs = strip_stage + ((128u - (smem_addr(strip_stage) & 127u)) & 127u) / 16u;
    float4* ds = xs + 2 * VPT * NT;
    float* gsm = reinterpret_cast<float*>(ds + VPT * NT);
    float* bsm = gsm + g.C;
    float* redg = bsm + g.C;
    float4* redc = reinterpret_cast<float4*>(redg + 2 * g.Gt * RG);
    float* wsum = reinterpret_cast<float*>(redc + 2 * NW * 2 * g.Q);  // [NW][32][8], used when Q == 4
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int q = t % g.Q;
    const int RW = 32 / g.Q;  // rows of one warp-wide access
    const int wrow0 = warp * RW * VPT;  // TMA: first row of this warp's block
    const int rl = TMA ? wrow0 + lane / g.Q : t / g.Q;
    const int slot0 = TMA ? warp * VPT * 32 + lane : t;  // slot of row block j: slot0 + j * SSTEP
    constexpr int SSTEP = TMA ? 32 : NT;
    const int brow = wrow0, bslot = warp * VPT * 32;  // the warp's box: first row in the sample, first slot in a buffer
    const int cb = 4 * q;
    const int M = GPT == 1 ? (g.cpg >> 2) : 1;
    const int gl = GPT == 1 ? q / M : 2 * q;
    const bool writer = lane < g.Q && (GPT == 2 || (lane & (M - 1)) == 0);
    const OStripLanes ln = ostrip_lanes<GPT>(lane, q, g.Q, M);
    const float inv_n = 1.0f / ((float)g.HW * (float)g.cpg);
    const size_t rowoff = (size_t)rl * g.C + cb;
    const size_t jstride = (size_t)(TMA ? RW : g.RSTEP) * g.C;
    const int G = gridDim.x;
    uint64_t* const wbar = mbar + (TMA ? 3 * warp : 0);
    bool alive = true;  // false once a bounded wait ran out: no more waits, the kernel runs to its end

    for (int i = t; i < g.C / 4; i += NT) {
        reinterpret_cast<float4*>(gsm)[i] = __ldg(reinterpret_cast<const float4*>(gamma) + i);
        if (ACT != ACT_IDENTITY)
            reinterpret_cast<float4*>(bsm)[i] = __ldg(reinterpret_cast<const float4*>(beta) + i);
    }
    int item = blockIdx.x;
    float pmu[GPT], prs[GPT];  // statistics of the strip about to be processed
#pragma unroll
    for (int k = 0; k < GPT; ++k)
        pmu[k] = prs[k] = 0.0f;
    if (item < nitems) {
        const int gi = (item / g.nct) * g.G + (item % g.nct) * g.Gt + gl;
#pragma unroll
        for (int k = 0; k < GPT; ++k) {
            pmu[k] = __ldg(mu + gi + k);
            prs[k] = __ldg(rstd + gi + k);
        }
    }
    if constexpr (TMA) {  // prologue: x(0), dy(0), x(1)
        if (lane == 0) {
            mbar_init(wbar + 0, 1);
            mbar_init(wbar + 1, 1);
            mbar_init(wbar + 2, 1);
            fence_mbar_init();
            fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) {
            if (item < nitems) {
                const int cx = (item % g.nct) * g.Ct, cy = (item / g.nct) * g.HW + brow;
                mbar_expect_tx(wbar + 0, BOX_BYTES, 0.0f);
                tma_load_box(xs + bslot, &mapx, cx, cy, wbar + 0, pol);
                mbar_expect_tx(wbar + 2, BOX_BYTES, 0.0f);
                tma_load_box(ds + bslot, &mapdy, cx, cy, wbar + 2, pol);
            }
            if (item + G < nitems) {
                const int it = item + G;
                mbar_expect_tx(wbar + 1, BOX_BYTES, 0.0f);
                tma_load_box(xs + VPT * NT + bslot, &mapx, (it % g.nct) * g.Ct, (it / g.nct) * g.HW + brow, wbar + 1, pol);
            }
        }
        __syncwarp();
    } else {  // prologue: x(0) | dy(0) | x(1)
        const size_t o0 = dstrip_item_offset(g, item < nitems ? item : 0, rowoff);
        if (item < nitems) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16_hint(&xs[slot0 + j * SSTEP], x + o0 + j * jstride, pol);
        }
        cp_async_commit();
        if (item < nitems) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16_hint(&ds[slot0 + j * SSTEP], dy + o0 + j * jstride, pol);
        }
        cp_async_commit();
        if (item + G < nitems) {
            const size_t o1 = dstrip_item_offset(g, item + G, rowoff);
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (FULL || rl + j * g.RSTEP < g.HW)
                    cp_async16_hint(&xs[VPT * NT + slot0 + j * SSTEP], x + o1 + j * jstride, pol);
        }
        cp_async_commit();
    }
    __syncthreads();  // gamma / beta staged

    int par = 0;
    uint32_t nstrip = 0;  // strips done by this CTA: the dy barrier is in phase nstrip & 1, x[par] in (nstrip >> 1) & 1
    for (; item < nitems; item += G, par ^= 1, ++nstrip) {
        const int ctile = item % g.nct, b = item / g.nct;
        const int c0 = ctile * g.Ct;
        const size_t base = (size_t)b * g.HW * g.C + c0;
        const float4 ga = *reinterpret_cast<const float4*>(gsm + c0 + cb);
        float4 be = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ACT != ACT_IDENTITY)
            be = *reinterpret_cast<const float4*>(bsm + c0 + cb);
        const bool more1 = item + G < nitems, more2 = item + 2 * G < nitems;
        const int it1 = more1 ? item + G : item;
        const int it2 = more2 ? item + 2 * G : item;
        const float* n1 = dy + dstrip_item_offset(g, it1, rowoff);
        const float* n2 = x + dstrip_item_offset(g, it2, rowoff);
        float4* xc = xs + par * VPT * NT;

        float rsg[GPT], nmg[GPT];
#pragma unroll
        for (int k = 0; k < GPT; ++k) {
            rsg[k] = prs[k];
            nmg[k] = -pmu[k] * rsg[k];
        }
        if (more1) {
            const int gi = (it1 / g.nct) * g.G + (it1 % g.nct) * g.Gt + gl;
#pragma unroll
            for (int k = 0; k < GPT; ++k) {
                pmu[k] = __ldg(mu + gi + k);
                prs[k] = __ldg(rstd + gi + k);
            }
        }
        if constexpr (TMA) {
            if (alive)
                alive = mbar_wait_bounded(wbar + 2, nstrip & 1u, err);
        } else {
            cp_async_wait_but_one();
        }
        float4 dv[VPT];
        const float* s1 = n1;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {  // dy slots: read, then (cp.async form) re-arm with strip i+1
            const bool live = FULL || rl + j * g.RSTEP < g.HW;
            dv[j] = live ? lds128(&ds[slot0 + j * SSTEP]) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (!TMA && more1 && live)
                cp_async16_hint(&ds[slot0 + j * SSTEP], s1, pol);
            s1 += jstride;
        }
        if constexpr (TMA) {
            if (alive)
                alive = mbar_wait_bounded(wbar + par, (nstrip >> 1) & 1u, err);
        } else {
            cp_async_commit();
        }
        // xv becomes xhat, dv becomes dy * act'(z), both kept as packed pairs for the second phase.  The x slots of
        // this parity are read one row block at a time, each (cp.async form) re-armed with strip i+2 right behind
        // its read and followed by its arithmetic, so that shared-memory traffic and arithmetic overlap within the warp.
        const f32x2 rs01 = pk1(rsg[0]), rs23 = pk1(rsg[GPT - 1]), nm01 = pk1(nmg[0]), nm23 = pk1(nmg[GPT - 1]);
        const f32x2 ga01 = pk(ga.x, ga.y), ga23 = pk(ga.z, ga.w), be01 = pk(be.x, be.y), be23 = pk(be.z, be.w);
        f32x2 xa[VPT], xb[VPT], da[VPT], db[VPT];
        float4 sA, sB;
        {
            f32x2 a1 = 0ull, b1 = 0ull, a2 = 0ull, b2 = 0ull;  // packed zeros
            const float* s2 = n2;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const bool live = FULL || rl + j * g.RSTEP < g.HW;
                const float4 xv = live ? lds128(&xc[slot0 + j * SSTEP]) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (!TMA && more2 && live)
                    cp_async16_hint(&xc[slot0 + j * SSTEP], s2, pol);
                s2 += jstride;
                if (TMA && j == (VPT > 1 ? 1 : 0)) {
                    // every dy slot of the warp has been read (the last one is an operand below): the box of strip i+1
                    __syncwarp();
                    if (lane == 0 && more1) {
                        fence_proxy_async();
                        mbar_expect_tx(wbar + 2, BOX_BYTES, dv[VPT - 1].w);
                        tma_load_box(ds + bslot, &mapdy, (it1 % g.nct) * g.Ct, (it1 / g.nct) * g.HW + brow, wbar + 2, pol);
                    }
                }
                xa[j] = pk_fma(pk(xv.x, xv.y), rs01, nm01);
                xb[j] = pk_fma(pk(xv.z, xv.w), rs23, nm23);
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
            if constexpr (TMA) {
                // the sums depend on every x slot of this parity: the box of strip i+2 goes behind them
                __syncwarp();
                if (lane == 0 && more2) {
                    fence_proxy_async();
                    mbar_expect_tx(wbar + par, BOX_BYTES, sB.w);
                    tma_load_box(xc + bslot, &mapx, (it2 % g.nct) * g.Ct, (it2 / g.nct) * g.HW + brow, wbar + par, pol);
                }
            } else {
                cp_async_commit();
            }
        }
        float* rg = redg + par * g.Gt * RG;
        float4* rc = redc + (size_t)par * NW * 2 * g.Q;
        if (g.Q == 4) {
            // The strip is 4 float4 columns wide, so a warp holds 8 row lanes of each column.  Instead of three
            // rounds of eight shuffles, the warp transposes through shared memory: every lane stores its 8 partial
            // sums, then lane (col, comp) adds the 8 row lanes of ONE of the 32 (column, component) sums with
            // conflict-free 32-bit loads.  The shuffle / shared-memory queue is this kernel's busiest unit
            // (28 entries per thread and strip become 15).
            float* W = wsum + warp * 256;
            *reinterpret_cast<float4*>(W + lane * 8) = sA;
            *reinterpret_cast<float4*>(W + lane * 8 + 4) = sB;
            __syncwarp();
            const int col = lane >> 3, comp = lane & 7;
            float v = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; ++r)
                v += W[(r * 4 + col) * 8 + comp];
            float* rcf = reinterpret_cast<float*>(rc);
            rcf[(warp * 2 + (comp >> 2)) * g.Ct + col * 4 + (comp & 3)] = v;  // comp < 4: sums of g, else of g * xhat
            float gv = v * gsm[c0 + col * 4 + (comp & 3)];
            gv += __shfl_xor_sync(0xffffffffu, gv, 1);
            if constexpr (GPT == 1) {
                gv += __shfl_xor_sync(0xffffffffu, gv, 2);
                for (int off = 8; off < 8 * M; off <<= 1)
                    gv += __shfl_xor_sync(0xffffffffu, gv, off);
                if ((comp & 3) == 0 && (col & (M - 1)) == 0)
                    rg[(col / M) * RG + 2 * warp + (comp >> 2)] = gv;
            } else {
                if ((comp & 1) == 0)
                    rg[(col * 2 + ((comp >> 1) & 1)) * RG + 2 * warp + (comp >> 2)] = gv;
            }
        } else {
            // per-warp channel sums (all lanes of a float4 column end up with them) ...
            for (int off = g.Q; off < 32; off <<= 1) {
                sA = shfl_xor4(sA, off);
                sB = shfl_xor4(sB, off);
            }
            // ... and from them the gamma-weighted per-warp group sums
            float sg[GPT], sgx[GPT];
            if constexpr (GPT == 1) {
                sg[0] = fmaf(ga.x, sA.x, ga.y * sA.y) + fmaf(ga.z, sA.z, ga.w * sA.w);
                sgx[0] = fmaf(ga.x, sB.x, ga.y * sB.y) + fmaf(ga.z, sB.z, ga.w * sB.w);
                for (int off = 1; off < M; off <<= 1) {
                    sg[0] += __shfl_xor_sync(0xffffffffu, sg[0], off);
                    sgx[0] += __shfl_xor_sync(0xffffffffu, sgx[0], off);
                }
            } else {
                sg[0] = fmaf(ga.x, sA.x, ga.y * sA.y);
                sg[GPT - 1] = fmaf(ga.z, sA.z, ga.w * sA.w);
                sgx[0] = fmaf(ga.x, sB.x, ga.y * sB.y);
                sgx[GPT - 1] = fmaf(ga.z, sB.z, ga.w * sB.w);
            }
            if (lane < g.Q) {
                rc[(warp * 2 + 0) * g.Q + q] = sA;
                rc[(warp * 2 + 1) * g.Q + q] = sB;
                if (writer) {
#pragma unroll
                    for (int k = 0; k < GPT; ++k)
                        *reinterpret_cast<float2*>(rg + (gl + k) * RG + 2 * warp) = make_float2(sg[k], sgx[k]);
                }
            }
        }
        __syncthreads();

        float mgv[GPT], mgxv[GPT];
#pragma unroll
        for (int k = 0; k < GPT; ++k) {
            float hi, lo = 0.0f, second;
            if constexpr (NW % 2 == 0 && NW <= 16)
                ostrip_group_total_direct<NW>(rg + (gl + k) * RG, hi, second);
            else
                ostrip_group_total<NW, false>(rg + (gl + k) * RG, ln, g.Q, M, hi, lo, second);
            (void)lo;
            mgv[k] = hi * inv_n;
            mgxv[k] = second * inv_n;
        }
        // dx = rstd * (g*gamma - mg - xhat*mgx), as in the reference (kernels.cu:692)
        const f32x2 nmg01 = pk1(-mgv[0]), nmg23 = pk1(-mgv[GPT - 1]), nmx01 = pk1(-mgxv[0]), nmx23 = pk1(-mgxv[GPT - 1]);
        float* orow = dx + base + rowoff;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (FULL || rl + j * g.RSTEP < g.HW) {
                float4 o;
                unpk(pk_mul(rs01, pk_fma(xa[j], nmx01, pk_fma(da[j], ga01, nmg01))), o.x, o.y);
                unpk(pk_mul(rs23, pk_fma(xb[j], nmx23, pk_fma(db[j], ga23, nmg23))), o.z, o.w);
                __stcs(reinterpret_cast<float4*>(orow), o);
            }
            orow += jstride;
        }
        // (sharing this fold among all threads -- NW lanes per sum, xor shuffles -- instead of leaving it to Ct
        // threads of warp 0: backward 137 -> 153 us on [256,32,32,256])
        if (t < g.Ct) {  // one partial row per sample: [b][0:C] dgamma, [b][C:2C] dbeta
            const float* rcf = reinterpret_cast<const float*>(rc);
            float sa = 0.0f, sb = 0.0f;
#pragma unroll 8
            for (int w = 0; w < NW; ++w) {
                sa += rcf[(w * 2 + 0) * g.Ct + t];
                sb += rcf[(w * 2 + 1) * g.Ct + t];
            }
            float* dst = partials + (size_t)b * (2 * g.C) + c0 + t;
            dst[0] = sb;
            dst[g.C] = sa;
        }
    }
    if constexpr (!TMA)
        cp_async_wait_all();
    // (TMA: every box issued was also waited for, unless a wait ran out)
}

}  // namespace b200
