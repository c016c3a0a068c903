// Shared device/host helpers for the sm_100a layer kernels.
//
// Everything here is header-only and internal to the library; the public
// surface is include/b200_layer_kernels.h.
#pragma once

#include <atomic>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

namespace b200 {

// ---------------------------------------------------------------------------
// host side: error reporting, device properties, tunables
// ---------------------------------------------------------------------------

// Reports a usage / runtime error.  Default mode mirrors the reference's
// convention (src/nn.h:13-52): print to stderr and exit(1).  In record mode the
// message is kept and the launcher returns without launching.
void report_error(const char* file, int line, const char* fmt, ...);

#define B200_REQUIRE(cond, ...)                                  \
    do {                                                         \
        if (!(cond)) {                                           \
            ::b200::report_error(__FILE__, __LINE__, __VA_ARGS__); \
            return;                                              \
        }                                                        \
    } while (0)

#define B200_CUDA_OK(call)                                                            \
    do {                                                                              \
        cudaError_t e_ = (call);                                                      \
        if (e_ != cudaSuccess) {                                                      \
            ::b200::report_error(__FILE__, __LINE__, "%s -> %s", #call, cudaGetErrorString(e_)); \
            return;                                                                   \
        }                                                                             \
    } while (0)

// Checks the launch status of the kernel that was just enqueued.
#define B200_CHECK_LAUNCH()                                                           \
    do {                                                                              \
        cudaError_t e_ = cudaPeekAtLastError();                                       \
        if (e_ != cudaSuccess) {                                                      \
            (void)cudaGetLastError();                                                 \
            ::b200::report_error(__FILE__, __LINE__, "kernel launch failed: %s", cudaGetErrorString(e_)); \
        }                                                                             \
    } while (0)

int sm_count();              // SMs of the current device (cached per device)
int tune_lookup(const char* key, int dflt);  // value set through b200_tune_set, else dflt (locked map lookup)
unsigned tune_generation();                    // bumped by every b200_tune_set
void count_launch(int n = 1);  // increments the library's launch counter

// Launchers read tunables on every call and some hosts issue thousands of tiny launches per
// step, so each call site caches its value and re-reads the map only after a b200_tune_set.
struct TuneSite {
    std::atomic<unsigned> gen{ 0xffffffffu };
    std::atomic<int> value{ 0 };
    int get(const char* key, int dflt)
    {
        const unsigned g = tune_generation();
        if (gen.load(std::memory_order_acquire) != g) {
            value.store(tune_lookup(key, dflt), std::memory_order_relaxed);
            gen.store(g, std::memory_order_release);
        }
        return value.load(std::memory_order_relaxed);
    }
};
#define tune_get(key, dflt) ([&]() -> int { static ::b200::TuneSite site_; return site_.get(key, dflt); }())

// Scratch memory owned by the library, one arena per (device, stream).  Grows
// on demand (allocation happens only when a call needs more than is reserved);
// the contents are zero when first handed out and kernels that use counters
// restore them to zero before they finish.
struct Scratch {
    float* partials;       // at least `floats` floats
    unsigned int* tickets; // at least `ntickets` counters, all zero between kernels
};
bool scratch_get(cudaStream_t s, size_t floats, size_t ntickets, Scratch* out);
// out[c] = sum over `nparts` partial rows of `width` floats, fixed order; columns below `split`
// go to out_a, the rest to out_b (rownorm.cu).
void fold_partials(float* out_a, float* out_b, const float* partials, int nparts, int width, int split,
    cudaStream_t s);
// Set (per thread) while b200_groupnorm_describe walks the dispatcher: launch helpers then record what they would
// launch instead of launching, scratch_get hands out nothing, fold_partials does nothing.  No CUDA call is made.
bool planning_only();
void planning_only_set(bool on);
// Device address of the error word that kernels set when a bounded wait runs
// out (0 = healthy); one word per device.
int* device_error_word();

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Every kernel of the library is launched through launch_k.  With programmatic dependent launch (tunable
// "pdl": 1 = small launches only, the default; 2 = every launch; 0 = never) a kernel may be scheduled
// while the kernel before it on the stream is still draining: its CTAs take the SMs that fall free during
// the predecessor's last wave and stop at pdl_prologue() until the predecessor has completed and its
// writes are visible.  That removes the launch gap (1.5-3 us) between back-to-back kernels of this
// library, which is most of the run time of the small layers of a training step.  A predecessor that is
// not one of these kernels (cuBLAS, a copy) simply completes first, as in an ordinary launch; inside
// stream capture the dependency becomes a programmatic edge of the graph.
// Large launches are excluded because there it costs: back to back, the four big kernels of the
// benchmark step ([256,32,32,256]) take 0.485-0.490 ms with the attribute and 0.456-0.460 ms without
// (0.442 ms with this size rule; 0.452-0.459 ms when large grids also hold back the release of their
// dependents until their CTAs exit).
// (The likely cause: CTAs of a dependent grid are placed on SMs in the order in which the predecessor
// frees them rather than all at once, and the bandwidth the strided kernels reach depends on which CTAs
// run side by side -- see groupnorm_ostrip.cuh.)
// `threads` = CTAs x threads per CTA of the launch.
constexpr long PDL_MAX_THREADS = 98304;  // a third of the 148 x 2048 resident threads
inline void pdl_attribute(cudaLaunchAttribute* at, unsigned* n, long threads)
{
    const int mode = tune_get("pdl", 1);
    if (mode == 2 || (mode == 1 && threads <= PDL_MAX_THREADS)) {
        at[*n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[*n].val.programmaticStreamSerializationAllowed = 1;
        ++*n;
    }
}

template <class... KArgs, class... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    unsigned n = 0;
    pdl_attribute(at, &n, (long)grid.x * grid.y * grid.z * block.x * block.y * block.z);
    cfg.attrs = at;
    cfg.numAttrs = n;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // errors surface in B200_CHECK_LAUNCH
}

// ---------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// W consecutive floats moved as one access (W = 1 or 4).
template <int W>
struct alignas(4 * W) Pack {
    float v[W];
};

// Streaming (evict-first) loads and stores: every tensor on this path is
// touched once per kernel, so nothing is worth keeping in L1/L2.
template <int W>
__device__ __forceinline__ Pack<W> load_stream(const float* p)
{
    Pack<W> r;
    if constexpr (W == 4) {
        float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
        r.v[0] = __ldcs(p);
    }
    return r;
}

template <int W>
__device__ __forceinline__ void store_stream(float* p, const Pack<W>& r)
{
    if constexpr (W == 4) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
    } else {
        __stcs(p, r.v[0]);
    }
}

// Cached loads for small, re-used operands (gamma, beta, statistics).
template <int W>
__device__ __forceinline__ Pack<W> load_cached(const float* p)
{
    Pack<W> r;
    if constexpr (W == 4) {
        float4 t = __ldg(reinterpret_cast<const float4*>(p));
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
        r.v[0] = __ldg(p);
    }
    return r;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Sum over the whole CTA; every thread gets the result.  `buf` holds >= 32
// floats of shared memory and may be reused right after the call returns.
__device__ __forceinline__ float cta_sum(float v, float* buf)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // protects buf against a previous call's readers
    if (lane == 0)
        buf[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? buf[lane] : 0.0f;
    return warp_sum(t);
}

// --- activations -----------------------------------------------------------
// The reference's SiLU/GELU/tanh are built on a clamped (7,6) rational
// approximation of tanh (src/kernels.cu:6-17), which is part of its numerics;
// it is reproduced term for term.  The quotient uses the approximate divide
// (2 ulp), which is also what the reference's own build (--use_fast_math)
// executes; these kernels sit close enough to the issue-rate limit that the
// ~8 extra instructions of a correctly rounded divide are measurable.
enum : int { ACT_IDENTITY = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3, ACT_TANH = 4, ACT_MP_SILU = 5 };

__device__ __forceinline__ float rational_tanh(float x)
{
    const float x2 = x * x;
    const float num = x * (135135.0f + x2 * (17325.0f + x2 * (378.0f + x2)));
    const float den = 135135.0f + x2 * (62370.0f + x2 * (3150.0f + x2 * 28.0f));
    // den >= 135135, so the flush-to-zero approximate reciprocal is exact enough (1 ulp) and is a
    // single MUFU instruction; the non-ftz divide carries several instructions of range handling
    float rden;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rden) : "f"(den));
    return fmaxf(-1.0f, fminf(1.0f, num * rden));
}

// (tanh(x/2)+1)/2.  The reference clamps the result to [0,1] once more; with the
// tanh already clamped to [-1,1] that second clamp can never change the value
// ((t+1)*0.5 is exact at both ends and monotone), so it is not repeated here.
//
// tanh(x/2) is evaluated directly in x: with h = x/2 every coefficient below is
// the reference's coefficient times a power of two (135135/4, 17325/16, 378/64,
// 1/256 for the numerator; 135135/2, 62370/8, 3150/32, 28/128 for the
// denominator), all exactly representable, so each intermediate is the
// reference's intermediate scaled by a power of two and the quotient is
// bit-identical to rational_tanh(x * 0.5f) -- one multiply cheaper.
__device__ __forceinline__ float rational_sigmoid(float x)
{
    const float x2 = x * x;
    const float num = x * (33783.75f + x2 * (1082.8125f + x2 * (5.90625f + x2 * 0.00390625f)));
    const float den = 67567.5f + x2 * (7796.25f + x2 * (98.4375f + x2 * 0.21875f));
    float rden;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rden) : "f"(den));
    const float t = fmaxf(-1.0f, fminf(1.0f, num * rden));
    return fmaf(t, 0.5f, 0.5f);
}

#define B200_MP_SILU_SCALE (1.0f / 0.596f)

template <int ACT>
__device__ __forceinline__ float act_value(float v)
{
    if constexpr (ACT == ACT_RELU) {
        return v > 0.0f ? v : 0.0f;
    } else if constexpr (ACT == ACT_GELU) {
        return 0.5f * v * (1.0f + rational_tanh(0.7978845608f * (v + 0.044715f * v * v * v)));
    } else if constexpr (ACT == ACT_SILU) {
        return v * rational_sigmoid(v);
    } else if constexpr (ACT == ACT_MP_SILU) {
        return v * rational_sigmoid(v) * B200_MP_SILU_SCALE;
    } else if constexpr (ACT == ACT_TANH) {
        return rational_tanh(v);
    } else {
        return v;
    }
}

// derivative with respect to the pre-activation z (src/kernels.cu:40-68)
template <int ACT>
__device__ __forceinline__ float act_slope(float z)
{
    if constexpr (ACT == ACT_RELU) {
        return z > 0.0f ? 1.0f : 0.0f;
    } else if constexpr (ACT == ACT_TANH) {
        const float t = rational_tanh(z);
        return 1.0f - t * t;
    } else if constexpr (ACT == ACT_SILU) {
        const float s = rational_sigmoid(z);
        return s * (1.0f + z * (1.0f - s));
    } else if constexpr (ACT == ACT_MP_SILU) {
        const float s = rational_sigmoid(z);
        return s * (1.0f + z * (1.0f - s)) * B200_MP_SILU_SCALE;
    } else if constexpr (ACT == ACT_GELU) {
        const float c = 0.7978845608f;
        const float u = c * (z + 0.044715f * z * z * z);
        const float t = rational_tanh(u);
        const float du = c * (1.0f + 3.0f * 0.044715f * z * z);
        return 0.5f * (1.0f + t) + 0.5f * z * (1.0f - t * t) * du;
    } else {
        return 1.0f;
    }
}

// --- packed fp32 pairs -------------------------------------------------------
// sm_100 executes add/mul/fma on two fp32 values held in one 64-bit register
// (f32x2) as a single instruction.  The GroupNorm strip kernels are limited by
// instruction issue as much as by HBM, so their per-element arithmetic runs on
// pairs.  Each lane is an ordinary IEEE fp32 operation: results are bit-identical
// to the scalar forms.
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pk(float lo, float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pk1(float v) { return pk(v, v); }
__device__ __forceinline__ void unpk(f32x2 v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 pk_fma(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 pk_mul(f32x2 a, f32x2 b)
{
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 pk_add(f32x2 a, f32x2 b)
{
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// rational_sigmoid on a pair.  Differences from the scalar form, both below 1 ulp of the
// result: the numerator carries the final factor 1/2 (exact power-of-two scaling) so that
// t/2 + 1/2 is ONE fused multiply-add of numerator and reciprocal, and the clamp of t to
// [-1, 1] becomes the saturation of that result to [0, 1] (same value for every finite t).
__device__ __forceinline__ void rational_sigmoid_x2(f32x2 x, float& s0, float& s1)
{
    const f32x2 x2 = pk_mul(x, x);
    f32x2 n = pk_fma(x2, pk1(0.001953125f), pk1(2.953125f));
    n = pk_fma(n, x2, pk1(541.40625f));
    n = pk_fma(n, x2, pk1(16891.875f));
    n = pk_mul(n, x);
    f32x2 d = pk_fma(x2, pk1(0.21875f), pk1(98.4375f));
    d = pk_fma(d, x2, pk1(7796.25f));
    d = pk_fma(d, x2, pk1(67567.5f));
    float n0, n1, d0, d1, r0, r1;
    unpk(n, n0, n1);
    unpk(d, d0, d1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d1));
    asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(s0) : "f"(n0), "f"(r0));
    asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(s1) : "f"(n1), "f"(r1));
}

// act_value / act_slope on a pair of pre-activations (SiLU family on packed arithmetic,
// everything else through the scalar forms)
template <int ACT>
__device__ __forceinline__ f32x2 act_value_x2(f32x2 z)
{
    if constexpr (ACT == ACT_SILU || ACT == ACT_MP_SILU) {
        float s0, s1;
        rational_sigmoid_x2(z, s0, s1);
        f32x2 o = pk_mul(z, pk(s0, s1));
        if constexpr (ACT == ACT_MP_SILU)
            o = pk_mul(o, pk1(B200_MP_SILU_SCALE));
        return o;
    } else if constexpr (ACT == ACT_IDENTITY) {
        return z;
    } else {
        float z0, z1;
        unpk(z, z0, z1);
        return pk(act_value<ACT>(z0), act_value<ACT>(z1));
    }
}

template <int ACT>
__device__ __forceinline__ f32x2 act_slope_x2(f32x2 z)
{
    if constexpr (ACT == ACT_SILU || ACT == ACT_MP_SILU) {
        float s0, s1;
        rational_sigmoid_x2(z, s0, s1);
        const f32x2 s = pk(s0, s1);
        const f32x2 one = pk1(1.0f);
        // s * (1 + z * (1 - s))
        const f32x2 oms = pk_fma(s, pk1(-1.0f), one);
        f32x2 r = pk_mul(s, pk_fma(z, oms, one));
        if constexpr (ACT == ACT_MP_SILU)
            r = pk_mul(r, pk1(B200_MP_SILU_SCALE));
        return r;
    } else {
        float z0, z1;
        unpk(z, z0, z1);
        return pk(act_slope<ACT>(z0), act_slope<ACT>(z1));
    }
}

// First statement of every kernel: wait until the kernels this launch depends on have completed
// and flushed (a no-op for an ordinary launch), then let the next kernel on the stream be scheduled.
__device__ __forceinline__ void pdl_prologue()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// shared-memory address of a generic pointer (operand of cp.async)
__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// one butterfly step of a warp reduction on four lanes of data at once
__device__ __forceinline__ float4 shfl_xor4(float4 v, int off)
{
    v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
    v.z += __shfl_xor_sync(0xffffffffu, v.z, off);
    v.w += __shfl_xor_sync(0xffffffffu, v.w, off);
    return v;
}

#endif  // __CUDACC__

}  // namespace b200
