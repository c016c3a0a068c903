// Time / noise-level embeddings (reference: src/kernels.cu:385-394 mp_fourier,
// :444-456 sinusoidal, :459-485 learned table).
//
// The outputs are 100-500 KB, so these launches are latency-bound; the kernels
// are one thread per output pair, write coalesced, and compute each frequency
// once per (sample, j) pair instead of once per element.  Unlike the
// reference build (--use_fast_math) the transcendental functions are the
// full-range, accurate ones: with arguments up to ~1000 rad the fast
// intrinsics lose all but ~3 digits.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

namespace b200 {

__global__ void __launch_bounds__(256) mp_fourier_kernel(float* __restrict__ out, const float* __restrict__ x,
    const float* __restrict__ freqs, const float* __restrict__ phases, int total, int C)
{
    pdl_prologue();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int b = i / C, k = i - b * C;
        out[i] = 1.41421356237f * cosf(6.28318530718f * (__ldg(x + b) * __ldg(freqs + k) + __ldg(phases + k)));
    }
}

// one thread per (sample, j < half): writes sin to column j and cos to column half + j
__global__ void __launch_bounds__(256) sinusoidal_kernel(float* __restrict__ out, const float* __restrict__ t,
    int batch, int C, float log_max_period)
{
    pdl_prologue();
    const int half = C / 2;
    const int total = batch * half;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int b = i / half, j = i - b * half;
        const float freq = expf(-log_max_period * (float)j / (float)half);
        const float arg = __ldg(t + b) * freq;
        float sn, cs;
        sincosf(arg, &sn, &cs);
        out[(size_t)b * C + j] = sn;
        out[(size_t)b * C + half + j] = cs;
    }
}

__device__ __forceinline__ int table_row(float f, int T)
{
    const int r = (int)f;
    return r < 0 ? 0 : (r >= T ? T - 1 : r);
}

__global__ void __launch_bounds__(256) embed_gather_kernel(float* __restrict__ out, const float* __restrict__ table,
    const float* __restrict__ idx, int total, int C, int T)
{
    pdl_prologue();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int b = i / C, c = i - b * C;
        out[i] = __ldg(table + (size_t)table_row(__ldg(idx + b), T) * C + c);
    }
}

__global__ void __launch_bounds__(256) embed_scatter_kernel(float* __restrict__ grad_table,
    const float* __restrict__ grad_out, const float* __restrict__ idx, int total, int C, int T)
{
    pdl_prologue();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int b = i / C, c = i - b * C;
        atomicAdd(grad_table + (size_t)table_row(__ldg(idx + b), T) * C + c, grad_out[i]);
    }
}

static inline int small_grid(long n)
{
    long g = (n + 255) / 256;
    const long cap = (long)sm_count() * 8;
    if (g > cap)
        g = cap;
    return g < 1 ? 1 : (int)g;
}

}  // namespace b200

using namespace b200;

extern "C" {

void launch_mp_fourier(float* out, const float* x, const float* freqs, const float* phases, int batch, int C,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0 && (long)batch * C < 2147483648L, "mp_fourier: batch=%d C=%d", batch, C);
    if (batch == 0)
        return;
    launch_k(mp_fourier_kernel, small_grid((long)batch * C), 256, 0, s, out, x, freqs, phases, batch * C, C);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_sinusoidal(float* out, const float* t, int batch, int C, float log_max_period, cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0 && C % 2 == 0 && (long)batch * C < 2147483648L,
        "sinusoidal: batch=%d C=%d (C must be even)", batch, C);
    if (batch == 0)
        return;
    launch_k(sinusoidal_kernel, small_grid((long)batch * (C / 2)), 256, 0, s, out, t, batch, C, log_max_period);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_embed_gather(float* out, const float* table, const float* idx, int batch, int C, int T,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0 && T > 0 && (long)batch * C < 2147483648L, "embed_gather: bad extents");
    if (batch == 0)
        return;
    launch_k(embed_gather_kernel, small_grid((long)batch * C), 256, 0, s, out, table, idx, batch * C, C, T);
    count_launch();
    B200_CHECK_LAUNCH();
}

void launch_embed_scatter(float* grad_table, const float* grad_out, const float* idx, int batch, int C, int T,
    cudaStream_t s)
{
    B200_REQUIRE(batch >= 0 && C > 0 && T > 0 && (long)batch * C < 2147483648L, "embed_scatter: bad extents");
    if (batch == 0)
        return;
    launch_k(embed_scatter_kernel, small_grid((long)batch * C), 256, 0, s, grad_table, grad_out, idx, batch * C, C, T);
    count_launch();
    B200_CHECK_LAUNCH();
}

}  // extern "C"
