// Runtime underneath the operator layer: device enumeration, one in-order compute stream
// per device, a size-class caching allocator, copies, RNG state and error reporting.
//
// This is the CUDA counterpart of the reference's src/vulkan runtime:
//   VulkanContext   (src/vulkan/vulkan_context.cpp:107-151)  -> Runtime (lazy init, fork guard)
//   DeviceContext   (src/vulkan/device_context.cpp:7-90)     -> Device (stream, props, counters)
//   VulkanAllocator (src/vulkan/allocator.cpp:59-83,171-201) -> CachingAllocator
//   VulkanCache     (src/vulkan/cache.cpp:78-146)            -> size classes + free lists
//   VulkanGeneratorImpl (src/vulkan/generator.cpp:82-168)    -> RngState
// The deferred op list and hazard DAG (src/vulkan/shader.cpp:100-121, dispatch.cpp:65-169)
// have no counterpart: kernels launch eagerly and stream order is the dependency order.
#include "common.cuh"

#include <cuda.h>
#include <pthread.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace tvk {

// ---- errors -----------------------------------------------------------------
static thread_local std::string g_last_error;

int set_error(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}
void clear_error() { g_last_error.clear(); }

// ---- allocator --------------------------------------------------------------
static tvk_raw_alloc_fn g_raw_alloc = nullptr;
static tvk_raw_free_fn g_raw_free = nullptr;
static int g_fake_devices = 0;  // > 0: no CUDA calls at all (allocator unit tests on CPU)

static uint64_t round_size(uint64_t size) {
    const uint64_t kMin = 256;
    if (size <= kMin) return kMin;
    // size in (2^k, 2^(k+1)] -> next multiple of 2^(k-2): four classes per octave.
    int k = 63 - __builtin_clzll(size - 1);
    uint64_t step = uint64_t(1) << (k - 2);
    return (size + step - 1) / step * step;
}

// Blocks a captured graph refers to. A graph bakes device addresses into its nodes, so every block handed out while the
// capture ran belongs to the graph from then on: freed blocks are parked here (and reused only inside the same
// capture), never returned to the shared cache or to the driver while the graph exists. Without this a block freed
// during the capture could be handed to an unrelated allocation between two replays, and the next replay would write
// into it; tvk_empty_cache or the out-of-memory ladder could even cudaFree it under the graph.
struct GraphPool {
    std::map<uint64_t, std::vector<void*>> parked;   // freed blocks of this pool by size
    std::unordered_map<void*, uint64_t> owned;       // every block of the pool (live or parked) -> size
    uint64_t parked_bytes = 0;
};

class CachingAllocator {
public:
    int allocate(uint64_t bytes, void** out) {
        *out = nullptr;
        if (bytes == 0) return TVK_OK;
        const uint64_t rounded = round_size(bytes);
        std::lock_guard<std::mutex> lock(mu_);
        void* p = nullptr;
        if (capturing_) {
            auto pit = capturing_->parked.find(rounded);
            if (pit != capturing_->parked.end() && !pit->second.empty()) {
                p = pit->second.back();
                pit->second.pop_back();
                capturing_->parked_bytes -= rounded;
                parked_total_ -= rounded;
                ++stats_.num_cache_hits;
            }
        }
        auto it = free_.find(rounded);
        if (p) {
            // reused inside the capture
        } else if (it != free_.end() && !it->second.empty()) {
            p = it->second.back();  // newest first: it is the most likely to still sit in L2
            it->second.pop_back();
            cached_ -= rounded;
            ++stats_.num_cache_hits;
        } else {
            int rc = raw_alloc(&p, rounded);
            if (rc != 0 && capturing_) {
                // no retry ladder inside a capture: it would wait for the device and free blocks, both of which
                // invalidate the capture
                return set_error(TVK_ERR_OOM, "torchvulkan [ERROR]: out of memory during a graph capture: tried to allocate %llu bytes",
                                 (unsigned long long)rounded);
            }
            if (rc != 0) {
                // Ladder of VulkanAllocator::allocate: give the cache back to the driver, retry.
                ++stats_.num_oom_retries;
                release_cached_locked(/*sync=*/true);
                rc = raw_alloc(&p, rounded);
                if (rc != 0) {
                    return set_error(TVK_ERR_OOM,
                                     "torchvulkan [ERROR]: out of memory: tried to allocate %llu bytes "
                                     "(%llu allocated, %llu reserved)",
                                     (unsigned long long)rounded, (unsigned long long)stats_.allocated_bytes,
                                     (unsigned long long)(stats_.allocated_bytes + cached_));
                }
            }
            ++stats_.num_device_mallocs;
        }
        live_[p] = rounded;
        if (capturing_) {
            capturing_->owned[p] = rounded;
            owner_[p] = capturing_;
        }
        stats_.allocated_bytes += rounded;
        stats_.total_allocated_bytes += rounded;
        if (stats_.allocated_bytes > stats_.peak_allocated_bytes)
            stats_.peak_allocated_bytes = stats_.allocated_bytes;
        *out = p;
        return TVK_OK;
    }

    // Capture bracket of the device's graph: between the two calls every allocation joins a new pool.
    int begin_capture() {
        std::lock_guard<std::mutex> lock(mu_);
        if (capturing_) return set_error(TVK_ERR_INVALID, "tvk_graph_begin_capture: a capture is already running on this device");
        capturing_ = new GraphPool();
        return TVK_OK;
    }
    GraphPool* end_capture() {
        std::lock_guard<std::mutex> lock(mu_);
        GraphPool* pool = capturing_;
        capturing_ = nullptr;
        return pool;
    }
    // The graph is gone: its parked blocks go to the shared cache, its live blocks become ordinary blocks.
    void release_pool(GraphPool* pool) {
        if (!pool) return;
        std::lock_guard<std::mutex> lock(mu_);
        if (capturing_ == pool) capturing_ = nullptr;
        for (auto& kv : pool->owned) owner_.erase(kv.first);
        for (auto& kv : pool->parked)
            for (void* p : kv.second) {
                free_[kv.first].push_back(p);
                cached_ += kv.first;
                parked_total_ -= kv.first;
            }
        delete pool;
    }
    bool capturing() {
        std::lock_guard<std::mutex> lock(mu_);
        return capturing_ != nullptr;
    }

    int release(void* p) {
        if (!p) return TVK_OK;
        std::lock_guard<std::mutex> lock(mu_);
        auto it = live_.find(p);
        if (it == live_.end())
            return set_error(TVK_ERR_INVALID, "tvk_free: pointer %p was not allocated by tvk_malloc on this device", p);
        const uint64_t rounded = it->second;
        live_.erase(it);
        stats_.allocated_bytes -= rounded;
        stats_.total_freed_bytes += rounded;
        auto own = owner_.find(p);
        if (own != owner_.end()) {
            // a graph refers to this address: park it with the graph
            own->second->parked[rounded].push_back(p);
            own->second->parked_bytes += rounded;
            parked_total_ += rounded;
            return TVK_OK;
        }
        free_[rounded].push_back(p);
        cached_ += rounded;
        return TVK_OK;
    }

    void empty_cache() {
        std::lock_guard<std::mutex> lock(mu_);
        if (capturing_) return;      // waiting for the device or freeing blocks would invalidate the running capture
        release_cached_locked(/*sync=*/true);
    }

    void get_stats(tvk_mem_stats* s) {
        std::lock_guard<std::mutex> lock(mu_);
        *s = stats_;
        s->cached_bytes = cached_ + parked_total_;
        s->reserved_bytes = stats_.allocated_bytes + cached_ + parked_total_;
    }
    void reset_peak() {
        std::lock_guard<std::mutex> lock(mu_);
        stats_.peak_allocated_bytes = stats_.allocated_bytes;
    }

private:
    static int raw_alloc(void** p, uint64_t bytes) {
        if (g_raw_alloc) return g_raw_alloc(p, bytes);
        cudaError_t e = cudaMalloc(p, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();  // clear the sticky-free error
            return 1;
        }
        return 0;
    }
    static void raw_free(void* p) {
        if (g_raw_free) { g_raw_free(p); return; }
        cudaFree(p);
    }
    void release_cached_locked(bool sync) {
        // Cached blocks may still be read by kernels queued before the free; wait first.
        if (sync && !g_raw_alloc && g_fake_devices == 0) cudaDeviceSynchronize();
        for (auto& kv : free_)
            for (void* p : kv.second) raw_free(p);
        free_.clear();
        cached_ = 0;
    }

    std::mutex mu_;
    std::map<uint64_t, std::vector<void*>> free_;
    std::unordered_map<void*, uint64_t> live_;
    std::unordered_map<void*, GraphPool*> owner_;     // blocks that belong to a graph's pool
    GraphPool* capturing_ = nullptr;                  // the pool of the capture that is running, if any
    uint64_t parked_total_ = 0;
    uint64_t cached_ = 0;
    tvk_mem_stats stats_ = {};
};

// The shape of every device-side wait in this library, alone in a kernel: poll a flag (here one that nothing ever sets),
// give up after `polls` tries, record where in the status word and leave through the normal end of the kernel.
__device__ int g_never_set_flag = 0;
__global__ void bounded_wait_probe_kernel(int* status, int polls) {
    if (threadIdx.x != 0) return;
    volatile int* flag = &g_never_set_flag;
    for (int it = 0; it < polls; ++it) {
        if (*flag) return;
        __nanosleep(100);
    }
    if (atomicCAS(status, 0, 1) == 0) {
        status[1] = 99;           // site: the probe
        status[2] = (int)blockIdx.x;
        status[3] = polls;
    }
}

// ---- devices ------------------------------------------------------------------
struct RngState {
    std::mutex mu;
    uint64_t seed = 67280421310721ull;  // torch's default seed constant
    uint64_t offset = 0;
    // While a graph is being captured the random launches take their (seed, base offset) from these two words of device
    // memory plus an offset relative to the start of the capture; every launch of the graph first writes the generator's
    // current seed and offset there and advances the offset by what the graph consumes, so a replay draws new numbers.
    uint64_t* dev_state = nullptr;
    bool capturing = false;
    uint64_t capture_used = 0;
};

struct Device {
    int index = 0;
    cudaStream_t stream = nullptr;
    bool stream_ready = false;
    int* status_word = nullptr;
    int sms = 0;
    CachingAllocator alloc;
    RngState rng;
    std::mutex mu;
};

struct Runtime {
    std::vector<Device*> devices;
};

static std::mutex g_init_mu;
static std::atomic<bool> g_initialized{false};
static std::atomic<bool> g_bad_fork{false};
static Runtime* g_rt = nullptr;
static thread_local int g_current = 0;

static void on_fork_child() {
    if (g_initialized.load()) g_bad_fork.store(true);
}

static int ensure_init() {
    if (g_bad_fork.load())
        return set_error(TVK_ERR_BAD_FORK,
                         "torchvulkan [ERROR]: cannot re-initialize the device in a forked subprocess; "
                         "use the 'spawn' start method");
    if (g_initialized.load()) return TVK_OK;
    std::lock_guard<std::mutex> lock(g_init_mu);
    if (g_initialized.load()) return TVK_OK;
    int n = 0;
    if (g_fake_devices > 0) {
        n = g_fake_devices;
    } else {
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
    }
    Runtime* rt = new Runtime();
    for (int i = 0; i < n; ++i) {
        Device* d = new Device();
        d->index = i;
        rt->devices.push_back(d);
    }
    g_rt = rt;
    static bool fork_hook = false;
    if (!fork_hook) {
        pthread_atfork(nullptr, nullptr, on_fork_child);
        fork_hook = true;
    }
    g_initialized.store(true);
    return TVK_OK;
}

static int get_dev(int dev, Device** out) {
    int rc = ensure_init();
    if (rc) return rc;
    if (dev < 0 || dev >= (int)g_rt->devices.size())
        return set_error(TVK_ERR_INVALID, "torchvulkan [ERROR]: invalid device index %d (device count %d)", dev,
                         (int)g_rt->devices.size());
    *out = g_rt->devices[dev];
    return TVK_OK;
}

// Makes `dev` the CUDA-current device for the scope and restores the previous one after.
struct DeviceScope {
    int prev = -1;
    bool switched = false;
    int enter(int dev) {
        if (g_fake_devices > 0) return TVK_OK;
        TVK_CUDA_CHECK(cudaGetDevice(&prev));
        if (prev != dev) {
            TVK_CUDA_CHECK(cudaSetDevice(dev));
            switched = true;
        }
        return TVK_OK;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(prev);
    }
};

static int ensure_stream(Device* d) {
    if (d->stream_ready) return TVK_OK;
    if (g_fake_devices > 0) return TVK_OK;      // host-only unit tests: no CUDA calls at all
    std::lock_guard<std::mutex> lock(d->mu);
    if (d->stream_ready) return TVK_OK;
    DeviceScope scope;
    int rc = scope.enter(d->index);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
    TVK_CUDA_CHECK(cudaDeviceGetAttribute(&d->sms, cudaDevAttrMultiProcessorCount, d->index));
    d->stream_ready = true;
    return TVK_OK;
}

// Status words and SM counts are looked up by CUDA's current device, not by the tvk one,
// because kernel launchers run on whatever device the caller made current.
static std::mutex g_status_mu;
static int* g_status_words[64] = {};
static int g_sm_counts[64] = {};

int* device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (g_status_words[dev]) return g_status_words[dev];
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (!g_status_words[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 4 * sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 4 * sizeof(int));
        g_status_words[dev] = p;
    }
    return g_status_words[dev];
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sm_counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_counts[dev] = n;
    }
    return g_sm_counts[dev];
}

}  // namespace tvk

using namespace tvk;

extern "C" {

const char* tvk_last_error(void) { return g_last_error.c_str(); }
const char* tvk_version(void) { return "tvk 0.1 (sm_100a)"; }

int tvk_device_count(int* count) {
    if (!count) return set_error(TVK_ERR_INVALID, "tvk_device_count: null output");
    *count = 0;
    if (g_bad_fork.load()) return TVK_OK;
    int rc = ensure_init();
    if (rc) return rc;
    *count = (int)g_rt->devices.size();
    return TVK_OK;
}

int tvk_is_initialized(void) { return g_initialized.load() ? 1 : 0; }
int tvk_init(void) { return ensure_init(); }
int tvk_is_in_bad_fork(void) { return g_bad_fork.load() ? 1 : 0; }

int tvk_set_device(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    g_current = dev;
    if (g_fake_devices == 0) TVK_CUDA_CHECK(cudaSetDevice(dev));
    return TVK_OK;
}

int tvk_get_device(int* dev) {
    if (!dev) return set_error(TVK_ERR_INVALID, "tvk_get_device: null output");
    *dev = g_current;
    return TVK_OK;
}

int tvk_get_device_props(int dev, tvk_device_props* out) {
    if (!out) return set_error(TVK_ERR_INVALID, "tvk_get_device_props: null output");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    memset(out, 0, sizeof(*out));
    if (g_fake_devices > 0) {
        snprintf(out->name, sizeof(out->name), "fake device %d", dev);
        out->warp_size = 32;
        return TVK_OK;
    }
    cudaDeviceProp p;
    TVK_CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
    snprintf(out->name, sizeof(out->name), "%s", p.name);
    out->total_memory = p.totalGlobalMem;
    out->vendor_id = 0x10DE;
    out->device_id = (uint32_t)p.pciDeviceID;
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    cudaDriverGetVersion(&out->driver_version);
    cudaRuntimeGetVersion(&out->runtime_version);
    out->sm_count = p.multiProcessorCount;
    out->warp_size = p.warpSize;
    out->l2_bytes = p.l2CacheSize;
    out->max_smem_per_block = (int32_t)p.sharedMemPerBlockOptin;
    return TVK_OK;
}

int tvk_get_stream(int dev, void** stream) {
    if (!stream) return set_error(TVK_ERR_INVALID, "tvk_get_stream: null output");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (g_fake_devices > 0) { *stream = nullptr; return TVK_OK; }
    rc = ensure_stream(d);
    if (rc) return rc;
    *stream = (void*)d->stream;
    return TVK_OK;
}

int tvk_synchronize(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (g_fake_devices > 0) return TVK_OK;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaDeviceSynchronize());
    return TVK_OK;
}

int tvk_check_device_status(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (g_fake_devices > 0) return TVK_OK;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    int* w = device_status_word();
    if (!w) return set_error(TVK_ERR_CUDA, "could not allocate the device status word");
    if (d->alloc.capturing()) return TVK_OK;      // waiting for the device would invalidate the capture that is running
    TVK_CUDA_CHECK(cudaDeviceSynchronize());
    int host[4] = {0, 0, 0, 0};
    TVK_CUDA_CHECK(cudaMemcpy(host, w, sizeof(host), cudaMemcpyDeviceToHost));
    if (host[0] != 0) {
        TVK_CUDA_CHECK(cudaMemset(w, 0, sizeof(host)));
        if (host[0] == 1)
            return set_error(TVK_ERR_TIMEOUT,
                             "torchvulkan [ERROR]: a bounded device-side wait ran out (site %d, block %d, detail %d)",
                             host[1], host[2], host[3]);
        return set_error(TVK_ERR_INVALID,
                         "torchvulkan [ERROR]: a kernel reported an invalid input (code %d, site %d, detail %d/%d)",
                         host[0], host[1], host[2], host[3]);
    }
    return TVK_OK;
}

uint64_t tvk_round_size(uint64_t bytes) { return round_size(bytes); }

int tvk_debug_bounded_wait(int dev, int polls, void* stream) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    TVK_REQUIRE(polls >= 1 && polls <= 1000000, "tvk_debug_bounded_wait: %d polls outside [1, 1000000]", polls);
    if (g_fake_devices > 0) return TVK_OK;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    int* w = device_status_word();
    if (!w) return set_error(TVK_ERR_CUDA, "could not allocate the device status word");
    bounded_wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(w, polls);
    return launch_status("bounded-wait probe");
}

int tvk_malloc(int dev, uint64_t bytes, void** ptr) {
    if (!ptr) return set_error(TVK_ERR_INVALID, "tvk_malloc: null output");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    return d->alloc.allocate(bytes, ptr);
}

int tvk_free(int dev, void* ptr) {
    if (g_bad_fork.load()) return TVK_OK;  // deleter is a no-op in a forked child (allocator.cpp:73)
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    return d->alloc.release(ptr);
}

int tvk_empty_cache(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    d->alloc.empty_cache();
    return TVK_OK;
}

int tvk_mem_info(int dev, uint64_t* free_bytes, uint64_t* total_bytes) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    size_t f = 0, t = 0;
    if (g_fake_devices == 0) {
        DeviceScope scope;
        rc = scope.enter(dev);
        if (rc) return rc;
        TVK_CUDA_CHECK(cudaMemGetInfo(&f, &t));
    }
    // Cached blocks are reusable, so they count as free (DeviceContext::memoryFree).
    tvk_mem_stats s;
    d->alloc.get_stats(&s);
    if (free_bytes) *free_bytes = (uint64_t)f + s.cached_bytes;
    if (total_bytes) *total_bytes = (uint64_t)t;
    return TVK_OK;
}

int tvk_mem_get_stats(int dev, tvk_mem_stats* out) {
    if (!out) return set_error(TVK_ERR_INVALID, "tvk_mem_get_stats: null output");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    d->alloc.get_stats(out);
    return TVK_OK;
}

int tvk_mem_reset_peak(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    d->alloc.reset_peak();
    return TVK_OK;
}

int tvk_host_alloc(uint64_t bytes, void** host_ptr) {
    if (!host_ptr) return set_error(TVK_ERR_INVALID, "tvk_host_alloc: null output");
    *host_ptr = nullptr;
    if (bytes == 0) return TVK_OK;
    if (g_fake_devices > 0) {
        *host_ptr = malloc(bytes);
        return *host_ptr ? TVK_OK : set_error(TVK_ERR_OOM, "host allocation of %llu bytes failed", (unsigned long long)bytes);
    }
    cudaError_t e = cudaHostAlloc(host_ptr, bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(TVK_ERR_OOM, "pinned host allocation of %llu bytes failed: %s", (unsigned long long)bytes,
                         cudaGetErrorString(e));
    }
    return TVK_OK;
}

int tvk_host_free(void* host_ptr) {
    if (!host_ptr) return TVK_OK;
    if (g_fake_devices > 0) { free(host_ptr); return TVK_OK; }
    TVK_CUDA_CHECK(cudaFreeHost(host_ptr));
    return TVK_OK;
}

int tvk_debug_set_raw_allocator(tvk_raw_alloc_fn a, tvk_raw_free_fn f, int fake_device_count) {
    if (g_initialized.load() && ((a != nullptr) != (g_raw_alloc != nullptr)) && fake_device_count != g_fake_devices)
        return set_error(TVK_ERR_INVALID, "tvk_debug_set_raw_allocator: the device count can only be faked before first use");
    g_raw_alloc = a;
    g_raw_free = f;
    if (!g_initialized.load()) g_fake_devices = fake_device_count;
    return TVK_OK;
}

int tvk_memcpy_h2d(int dev, void* dst, const void* host_src, uint64_t bytes) {
    if (bytes == 0) return TVK_OK;
    TVK_REQUIRE(dst && host_src, "tvk_memcpy_h2d: null pointer");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    // Pageable sources are staged by the driver before the call returns, pinned ones are read
    // asynchronously: the caller keeps a pinned source alive until the next synchronize.
    TVK_CUDA_CHECK(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, d->stream));
    return TVK_OK;
}

int tvk_memcpy_d2h(int dev, void* host_dst, const void* src, uint64_t bytes) {
    if (bytes == 0) return TVK_OK;
    TVK_REQUIRE(host_dst && src, "tvk_memcpy_d2h: null pointer");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, d->stream));
    TVK_CUDA_CHECK(cudaStreamSynchronize(d->stream));
    return TVK_OK;
}

int tvk_memcpy_d2d(int dev, void* dst, const void* src, uint64_t bytes) {
    if (bytes == 0) return TVK_OK;
    TVK_REQUIRE(dst && src, "tvk_memcpy_d2d: null pointer");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (g_fake_devices > 0) {       // host-only unit tests: the fake raw allocator hands out host memory
        memmove(dst, src, (size_t)bytes);
        return TVK_OK;
    }
    rc = ensure_stream(d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, d->stream));
    return TVK_OK;
}

int tvk_memcpy_async(void* dst, const void* src, uint64_t bytes, void* stream) {
    if (bytes == 0) return TVK_OK;
    TVK_REQUIRE(dst && src, "tvk_memcpy_async: null pointer");
    TVK_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return TVK_OK;
}

int tvk_memcpy_peer(int dst_dev, void* dst, int src_dev, const void* src, uint64_t bytes) {
    if (bytes == 0) return TVK_OK;
    TVK_REQUIRE(dst && src, "tvk_memcpy_peer: null pointer");
    Device *dd, *sd;
    int rc = get_dev(dst_dev, &dd);
    if (rc) return rc;
    rc = get_dev(src_dev, &sd);
    if (rc) return rc;
    rc = ensure_stream(sd);
    if (rc) return rc;
    rc = ensure_stream(dd);
    if (rc) return rc;
    // Order after everything queued on the source, run on the destination's stream.
    DeviceScope scope;
    rc = scope.enter(src_dev);
    if (rc) return rc;
    cudaEvent_t ev;
    TVK_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    TVK_CUDA_CHECK(cudaEventRecord(ev, sd->stream));
    TVK_CUDA_CHECK(cudaStreamWaitEvent(dd->stream, ev, 0));
    TVK_CUDA_CHECK(cudaMemcpyPeerAsync(dst, dst_dev, src, src_dev, bytes, dd->stream));
    TVK_CUDA_CHECK(cudaEventDestroy(ev));
    return TVK_OK;
}

int tvk_pointer_device(const void* ptr, int* dev) {
    if (!dev) return set_error(TVK_ERR_INVALID, "tvk_pointer_device: null output");
    *dev = g_current;
    if (!ptr || g_fake_devices > 0) return TVK_OK;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(TVK_ERR_INVALID, "tvk_pointer_device: %p is not a device pointer (%s)", ptr, cudaGetErrorString(e));
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) *dev = attr.device;
    return TVK_OK;
}

// ---- sharing a buffer with the other ranks of the node ----------------------------------------
namespace {
struct OpenedIpc {
    unsigned char key[64];
    void* base;
    int refs;
};
std::mutex g_ipc_mutex;
std::vector<OpenedIpc> g_ipc_open;          // one mapping per exporting allocation, shared by every tvk_ipc_open of it
struct IpcView { void* ptr; void* base; };
std::vector<IpcView> g_ipc_views;
}  // namespace

int tvk_ipc_export(const void* ptr, tvk_ipc_handle* handle) {
    TVK_REQUIRE(ptr && handle, "tvk_ipc_export: null argument");
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    TVK_CUDA_CHECK(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
    TVK_REQUIRE(fn && q == cudaDriverEntryPointSuccess, "tvk_ipc_export: the driver does not provide cuMemGetAddressRange");
    CUdeviceptr base = 0;
    size_t size = 0;
    CUresult r = ((RangeFn)fn)(&base, &size, (CUdeviceptr)(uintptr_t)ptr);
    if (r != CUDA_SUCCESS) return set_error(TVK_ERR_INVALID, "tvk_ipc_export: %p is not inside a device allocation (driver code %d)", ptr, (int)r);
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    TVK_CUDA_CHECK(cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base));
    memcpy(handle->reserved, &h, 64);
    handle->offset = (uint64_t)((uintptr_t)ptr - (uintptr_t)base);
    return TVK_OK;
}

int tvk_ipc_open(const tvk_ipc_handle* handle, void** ptr) {
    TVK_REQUIRE(handle && ptr, "tvk_ipc_open: null argument");
    std::lock_guard<std::mutex> lock(g_ipc_mutex);
    void* base = nullptr;
    for (auto& o : g_ipc_open)
        if (memcmp(o.key, handle->reserved, 64) == 0) { base = o.base; ++o.refs; break; }
    if (!base) {
        cudaIpcMemHandle_t h;
        memcpy(&h, handle->reserved, 64);
        TVK_CUDA_CHECK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
        OpenedIpc o;
        memcpy(o.key, handle->reserved, 64);
        o.base = base;
        o.refs = 1;
        g_ipc_open.push_back(o);
    }
    *ptr = (uint8_t*)base + handle->offset;
    g_ipc_views.push_back({*ptr, base});
    return TVK_OK;
}

int tvk_ipc_close(void* ptr) {
    if (!ptr) return TVK_OK;
    std::lock_guard<std::mutex> lock(g_ipc_mutex);
    for (size_t i = 0; i < g_ipc_views.size(); ++i) {
        if (g_ipc_views[i].ptr != ptr) continue;
        void* base = g_ipc_views[i].base;
        g_ipc_views.erase(g_ipc_views.begin() + (long)i);
        for (size_t j = 0; j < g_ipc_open.size(); ++j) {
            if (g_ipc_open[j].base != base) continue;
            if (--g_ipc_open[j].refs == 0) {
                g_ipc_open.erase(g_ipc_open.begin() + (long)j);
                TVK_CUDA_CHECK(cudaIpcCloseMemHandle(base));
            }
            break;
        }
        return TVK_OK;
    }
    return set_error(TVK_ERR_INVALID, "tvk_ipc_close: %p was not returned by tvk_ipc_open", ptr);
}

int tvk_event_create(void** event) {
    if (!event) return set_error(TVK_ERR_INVALID, "tvk_event_create: null output");
    cudaEvent_t ev;
    TVK_CUDA_CHECK(cudaEventCreate(&ev));
    *event = (void*)ev;
    return TVK_OK;
}

int tvk_event_destroy(void* event) {
    if (!event) return TVK_OK;
    TVK_CUDA_CHECK(cudaEventDestroy((cudaEvent_t)event));
    return TVK_OK;
}

int tvk_event_record(int dev, void* event) {
    TVK_REQUIRE(event, "tvk_event_record: null event");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaEventRecord((cudaEvent_t)event, d->stream));
    return TVK_OK;
}

int tvk_event_wait(int dev, void* event) {
    TVK_REQUIRE(event, "tvk_event_wait: null event");
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (g_fake_devices > 0) return TVK_OK;
    rc = ensure_stream(d);
    if (rc) return rc;
    DeviceScope scope;
    rc = scope.enter(dev);
    if (rc) return rc;
    TVK_CUDA_CHECK(cudaStreamWaitEvent(d->stream, (cudaEvent_t)event, 0));
    return TVK_OK;
}

int tvk_event_synchronize(void* event) {
    TVK_REQUIRE(event, "tvk_event_synchronize: null event");
    TVK_CUDA_CHECK(cudaEventSynchronize((cudaEvent_t)event));
    return TVK_OK;
}

int tvk_event_query(void* event, int* done) {
    TVK_REQUIRE(event && done, "tvk_event_query: null pointer");
    cudaError_t e = cudaEventQuery((cudaEvent_t)event);
    if (e == cudaSuccess) { *done = 1; return TVK_OK; }
    if (e == cudaErrorNotReady) { cudaGetLastError(); *done = 0; return TVK_OK; }
    return set_error(TVK_ERR_CUDA, "cudaEventQuery failed: %s", cudaGetErrorString(e));
}

int tvk_event_elapsed_ms(void* start, void* end, float* ms) {
    TVK_REQUIRE(start && end && ms, "tvk_event_elapsed_ms: null pointer");
    TVK_CUDA_CHECK(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end));
    return TVK_OK;
}

// What tvk_graph_end_capture hands out: the executable graph and the memory pool its nodes point into.
struct GraphHandle {
    cudaGraphExec_t exec = nullptr;
    GraphPool* pool = nullptr;
    int device = 0;
    uint64_t rng_used = 0;       // generator offsets one launch of the graph consumes
};

__global__ void set_rng_state_kernel(uint64_t* state, uint64_t seed, uint64_t offset) {
    state[0] = seed;
    state[1] = offset;
}

int tvk_graph_begin_capture(int dev) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    rc = d->alloc.begin_capture();
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lock(d->rng.mu);
        d->rng.capturing = true;
        d->rng.capture_used = 0;
    }
    if (g_fake_devices > 0) return TVK_OK;
    if (!d->rng.dev_state) {
        DeviceScope scope;
        rc = scope.enter(dev);
        if (rc == TVK_OK && cudaMalloc((void**)&d->rng.dev_state, 2 * sizeof(uint64_t)) != cudaSuccess) {
            cudaGetLastError();
            d->rng.dev_state = nullptr;
            rc = set_error(TVK_ERR_OOM, "tvk_graph_begin_capture: no device memory for the generator state");
        }
        if (rc) {
            d->rng.capturing = false;
            d->alloc.release_pool(d->alloc.end_capture());
            return rc;
        }
    }
    // Relaxed: a cache miss of the allocator may still call cudaMalloc, from this thread or from autograd's
    cudaError_t e = cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) {
        d->rng.capturing = false;
        d->alloc.release_pool(d->alloc.end_capture());
        return set_error(TVK_ERR_CUDA, "cudaStreamBeginCapture failed: %s", cudaGetErrorString(e));
    }
    return TVK_OK;
}

int tvk_graph_end_capture(int dev, void** graph) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    if (!graph) return set_error(TVK_ERR_INVALID, "tvk_graph_end_capture: null output");
    *graph = nullptr;
    GraphPool* pool = d->alloc.end_capture();
    if (!pool) return set_error(TVK_ERR_INVALID, "tvk_graph_end_capture: no capture is running on device %d", dev);
    GraphHandle* h = new GraphHandle();
    h->pool = pool;
    h->device = dev;
    {
        std::lock_guard<std::mutex> lock(d->rng.mu);
        h->rng_used = d->rng.capture_used;
        d->rng.capturing = false;
        d->rng.capture_used = 0;
    }
    if (g_fake_devices > 0) {
        *graph = h;
        return TVK_OK;
    }
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(d->stream, &g);
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        d->alloc.release_pool(pool);
        delete h;
        return set_error(TVK_ERR_CUDA, "the capture was invalidated (a call that waits for the device, or a copy from pageable host memory, ran inside it): %s",
                         cudaGetErrorString(e));
    }
    e = cudaGraphInstantiate(&h->exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        cudaGetLastError();
        d->alloc.release_pool(pool);
        delete h;
        return set_error(TVK_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    *graph = (void*)h;
    return TVK_OK;
}

int tvk_graph_launch(int dev, void* graph) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    rc = ensure_stream(d);
    if (rc) return rc;
    if (!graph) return set_error(TVK_ERR_INVALID, "tvk_graph_launch: null graph");
    GraphHandle* h = (GraphHandle*)graph;
    if (h->device != dev) return set_error(TVK_ERR_INVALID, "tvk_graph_launch: the graph was captured on device %d, not %d", h->device, dev);
    if (g_fake_devices > 0) return TVK_OK;
    if (h->rng_used > 0 && d->rng.dev_state) {
        uint64_t seed, base;
        {
            std::lock_guard<std::mutex> lock(d->rng.mu);
            seed = d->rng.seed;
            base = d->rng.offset;
            d->rng.offset += h->rng_used;
        }
        set_rng_state_kernel<<<1, 1, 0, d->stream>>>(d->rng.dev_state, seed, base);
    }
    TVK_CUDA_CHECK(cudaGraphLaunch(h->exec, d->stream));
    return TVK_OK;
}

int tvk_graph_destroy(void* graph) {
    if (!graph) return TVK_OK;
    GraphHandle* h = (GraphHandle*)graph;
    Device* d;
    int rc = get_dev(h->device, &d);
    if (rc) return rc;
    if (h->exec) {
        // the graph may still be running: its blocks must not reach other users before it has finished
        if (g_fake_devices == 0) {
            DeviceScope scope;
            rc = scope.enter(h->device);
            if (rc) return rc;
            if (d->stream_ready) cudaStreamSynchronize(d->stream);
            cudaGraphExecDestroy(h->exec);
        }
    }
    d->alloc.release_pool(h->pool);
    delete h;
    return TVK_OK;
}

int tvk_rng_set_seed(int dev, uint64_t seed) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->rng.mu);
    d->rng.seed = seed;
    d->rng.offset = 0;
    return TVK_OK;
}

int tvk_rng_get_state(int dev, uint64_t* seed, uint64_t* offset) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->rng.mu);
    if (seed) *seed = d->rng.seed;
    if (offset) *offset = d->rng.offset;
    return TVK_OK;
}

int tvk_rng_set_state(int dev, uint64_t seed, uint64_t offset) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->rng.mu);
    d->rng.seed = seed;
    d->rng.offset = offset;
    return TVK_OK;
}

int tvk_rng_reserve_state(int dev, uint64_t count, uint64_t* seed, uint64_t* offset, const uint64_t** device_state) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    if (!device_state) return set_error(TVK_ERR_INVALID, "tvk_rng_reserve_state: null output");
    std::lock_guard<std::mutex> lock(d->rng.mu);
    if (seed) *seed = d->rng.seed;
    if (d->rng.capturing && d->rng.dev_state) {
        *device_state = d->rng.dev_state;
        if (offset) *offset = d->rng.capture_used;          // relative to what the graph's launch writes into device_state
        d->rng.capture_used += count;
        return TVK_OK;
    }
    *device_state = nullptr;
    if (offset) *offset = d->rng.offset;
    d->rng.offset += count;
    return TVK_OK;
}

int tvk_rng_reserve(int dev, uint64_t count, uint64_t* seed, uint64_t* offset) {
    Device* d;
    int rc = get_dev(dev, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->rng.mu);
    if (seed) *seed = d->rng.seed;
    if (offset) *offset = d->rng.offset;
    d->rng.offset += count;
    return TVK_OK;
}

}  // extern "C"
