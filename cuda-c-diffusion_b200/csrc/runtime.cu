// Host-side runtime of the layer-kernel library: error reporting, tunables,
// launch counter, per-(device, stream) scratch arenas.
#include "dev_common.cuh"
#include "../../include/b200_layer_kernels.h"

#include <atomic>
#include <map>
#include <mutex>
#include <stdarg.h>
#include <stdlib.h>
#include <string>
#include <string.h>
#include <utility>
#include <vector>

namespace b200 {

__device__ int g_device_error = 0;

int* device_error_word()
{
    static int* cached[64] = { nullptr };
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_error) != cudaSuccess)
            return nullptr;
        cached[dev] = static_cast<int*>(p);
    }
    return cached[dev];
}

static std::mutex g_mu;
static int g_error_mode = 0;
static int g_error_count = 0;
static std::string g_last_error;
static std::map<std::string, int> g_tunables;
static std::atomic<long long> g_launches{ 0 };
static std::atomic<unsigned> g_tune_gen{ 0 };

void report_error(const char* file, int line, const char* fmt, ...)
{
    char msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof msg, fmt, ap);
    va_end(ap);
    const char* base = strrchr(file, '/');
    char full[640];
    snprintf(full, sizeof full, "b200 layer kernels %s:%d: %s", base ? base + 1 : file, line, msg);
    int mode;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_last_error = full;
        ++g_error_count;
        mode = g_error_mode;
    }
    if (mode == 0) {
        fprintf(stderr, "%s\n", full);
        exit(1);
    }
}

int sm_count()
{
    static int cached[64] = { 0 };
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Tunables can also come from the environment, for programs that only link the library:
// B200_TUNE="key=int,key=int" is read once, before the first lookup; b200_tune_set overrides it.
static void tune_from_environment_locked()
{
    static bool done = false;
    if (done)
        return;
    done = true;
    const char* env = getenv("B200_TUNE");
    if (!env)
        return;
    std::string all(env);
    size_t at = 0;
    while (at < all.size()) {
        size_t end = all.find(',', at);
        if (end == std::string::npos)
            end = all.size();
        const std::string item = all.substr(at, end - at);
        const size_t eq = item.find('=');
        if (eq != std::string::npos && eq > 0 && !g_tunables.count(item.substr(0, eq)))
            g_tunables[item.substr(0, eq)] = atoi(item.c_str() + eq + 1);
        at = end + 1;
    }
}

int tune_lookup(const char* key, int dflt)
{
    std::lock_guard<std::mutex> lk(g_mu);
    tune_from_environment_locked();
    auto it = g_tunables.find(key);
    return it == g_tunables.end() ? dflt : it->second;
}

unsigned tune_generation() { return g_tune_gen.load(std::memory_order_acquire); }

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// --- scratch arenas ----------------------------------------------------------
struct Arena {
    float* partials = nullptr;
    size_t floats = 0;
    unsigned int* tickets = nullptr;
    size_t ntickets = 0;
};
static std::map<std::pair<int, cudaStream_t>, Arena> g_arenas;
// Blocks that an arena has outgrown.  They are never released: a CUDA graph captured while a
// block was current keeps its address and may be replayed at any later time.
static std::vector<void*> g_retired;

// True while `s` is being captured into a graph (an allocation is not allowed then).
static bool stream_is_capturing(cudaStream_t s)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(s, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone;
}

static thread_local bool t_planning_only = false;
bool planning_only() { return t_planning_only; }
void planning_only_set(bool on) { t_planning_only = on; }

bool scratch_get(cudaStream_t s, size_t floats, size_t ntickets, Scratch* out)
{
    if (t_planning_only) {
        *out = Scratch();
        return true;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
        return false;
    std::lock_guard<std::mutex> lk(g_mu);
    Arena& a = g_arenas[std::make_pair(dev, s)];
    if (a.floats < floats) {
        // Growing.  Refused during stream capture (reserve the arena before capturing); the old
        // block is retired, not freed: kernels in flight and graphs captured earlier still use it.
        if (stream_is_capturing(s))
            return false;
        size_t want = floats < (1u << 18) ? (1u << 18) : floats;
        float* np = nullptr;
        if (cudaMalloc(&np, want * sizeof(float)) != cudaSuccess)
            return false;
        if (a.partials)
            g_retired.push_back(a.partials);
        a.partials = np;
        a.floats = want;
    }
    if (a.ntickets < ntickets) {
        if (stream_is_capturing(s))
            return false;
        size_t want = ntickets < 4096 ? 4096 : ntickets;
        unsigned int* nt = nullptr;
        if (cudaMalloc(&nt, want * sizeof(unsigned int)) != cudaSuccess)
            return false;
        if (cudaMemsetAsync(nt, 0, want * sizeof(unsigned int), s) != cudaSuccess)
            return false;
        if (a.tickets)
            g_retired.push_back(a.tickets);
        a.tickets = nt;
        a.ntickets = want;
    }
    out->partials = a.partials;
    out->tickets = a.tickets;
    return true;
}

}  // namespace b200

using namespace b200;

extern "C" {

void b200_set_error_mode(int mode)
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_error_mode = mode ? 1 : 0;
}

int b200_error_count(void)
{
    std::lock_guard<std::mutex> lk(g_mu);
    return g_error_count;
}

int b200_last_error(char* buf, int buflen)
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (buf && buflen > 0) {
        strncpy(buf, g_last_error.c_str(), (size_t)buflen - 1);
        buf[buflen - 1] = 0;
    }
    return (int)g_last_error.size();
}

void b200_clear_error(void)
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_error_count = 0;
    g_last_error.clear();
}

int b200_device_error_status(void)
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_device_error, sizeof(int)) != cudaSuccess)
        return -1;
    return v;
}

long long b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void b200_launch_count_reset(void) { g_launches.store(0, std::memory_order_relaxed); }

int b200_scratch_reserve(cudaStream_t s, long long bytes)
{
    Scratch sc;
    size_t floats = bytes > 0 ? (size_t)((bytes + 3) / 4) : 0;
    return scratch_get(s, floats, 4096, &sc) ? 0 : -1;
}

void b200_tune_set(const char* key, int value)
{
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_tunables[key] = value;
    }
    g_tune_gen.fetch_add(1, std::memory_order_release);
}

int b200_tune_get(const char* key, int dflt) { return tune_lookup(key, dflt); }

const char* b200_version(void) { return "b200-layer-kernels 0.1 (sm_100a)"; }

}  // extern "C"
