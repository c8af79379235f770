// Library-wide entry points: version, error text, cached device attributes.
#include "common.cuh"

#include <atomic>
#include <mutex>

namespace th {

char *last_error_buffer() {
    static thread_local char buffer[kErrorBufferBytes] = "";
    return buffer;
}

static std::atomic<long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
    static std::mutex guard;
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(guard);
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

}  // namespace th

extern "C" int th_version(void) { return 2; }

extern "C" long long th_launch_count(void) { return th::launches_so_far(); }

extern "C" const char *th_last_error_string(void) { return th::last_error_buffer(); }
