// PrivateUse1 ("vulkan") device plumbing on top of the tvk C-ABI: device allocator, device guard,
// accelerator hooks, generator, and the helpers shared by the operator files.
//
// Counterparts in the reference: VulkanAllocator (src/vulkan/allocator.cpp:7-83, REGISTER_ALLOCATOR),
// VulkanGuardImpl (src/api/guard.cpp:19-100), VulkanHooksInterface + pinned allocator
// (src/api/hook.cpp:14-83), VulkanGeneratorImpl (src/vulkan/generator.cpp:41-168).
// Differences by design: a DataPtr carries the real device address (not a buffer object), there
// is one in-order compute stream per device (stream id 0), and events are device events.
#include "common.h"

#include <atomic>
#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

#include <ATen/core/GeneratorForPrivateuseone.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/CachingDeviceAllocator.h>
#include <c10/core/GeneratorImpl.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/util/Exception.h>

#include <cstring>
#include <map>
#include <mutex>

namespace tvk_aten {

void throw_status(int status, const char* what) {
    std::string msg = tvk_last_error();
    if (msg.empty()) msg = std::string("torchvulkan [ERROR]: ") + what + " failed";
    if (msg.rfind("torchvulkan", 0) != 0) msg = "torchvulkan [ERROR]: " + msg;
    if (status == TVK_ERR_OOM) {
        TORCH_CHECK_WITH(OutOfMemoryError, false, msg);
    }
    if (status == TVK_ERR_UNSUPPORTED) {
        TORCH_CHECK_NOT_IMPLEMENTED(false, msg);
    }
    TORCH_CHECK(false, msg);
}

const EnvFlags& env_flags() {
    static const EnvFlags flags = [] {
        auto set = [](const char* name) {
            const char* v = std::getenv(name);
            return v != nullptr && v[0] != '\0' && !(v[0] == '0' && v[1] == '\0');
        };
        EnvFlags f;
        f.profile = set("TORCHVULKAN_PROFILE");
        f.validation = set("TORCHVULKAN_VALIDATION");
        f.strict = true;     // TORCHVULKAN_STRICT: there is no CPU fallback to switch off
        return f;
    }();
    return flags;
}

static std::atomic<uint64_t> g_validation_errors{0};
uint64_t validation_error_count() { return g_validation_errors.load(); }

void profile_push(const char* name) {
    // "tvk_gemm(&d, ws.ptr, ...)" -> "tvk_gemm"
    char label[64];
    size_t n = 0;
    while (name[n] && name[n] != '(' && n + 1 < sizeof(label)) { label[n] = name[n]; ++n; }
    label[n] = '\0';
    nvtxRangePushA(label);
}
void profile_pop() { nvtxRangePop(); }

DeviceScope::DeviceScope(c10::DeviceIndex index) {
    TVK_CALL(tvk_get_device(&previous));
    device = index < 0 ? previous : (int)index;
    TVK_CALL(tvk_set_device(device));
    TVK_CALL(tvk_get_stream(device, &stream));
}
DeviceScope::~DeviceScope() {
    if (env_flags().validation) {
        // checked mode: the operator that just ran must have left neither a device-side status nor a CUDA error behind
        // (a destructor cannot raise: problems are warned about and counted)
        if (tvk_check_device_status(device) != TVK_OK) {
            g_validation_errors.fetch_add(1);
            TORCH_WARN("torchvulkan [WARNING]: validation: ", tvk_last_error());
        }
    }
    if (previous != device) tvk_set_device(previous);
}

Workspace::Workspace(int dev, uint64_t n) : bytes(n), device(dev) {
    if (n) TVK_CALL(tvk_malloc(dev, n, &ptr));
}
Workspace::~Workspace() {
    if (ptr) tvk_free(device, ptr);
}

// ---------------------------------------------------------------------------------------
// allocator
// ---------------------------------------------------------------------------------------
namespace {

struct Block {
    void* ptr;
    int device;
};

void delete_block(void* ctx) {
    auto* b = static_cast<Block*>(ctx);
    if (!b) return;
    tvk_free(b->device, b->ptr);  // a no-op in a forked child, as the reference's deleter
    delete b;
}

class TvkAllocator final : public c10::DeviceAllocator {
public:
    c10::DataPtr allocate(size_t nbytes) override {
        int dev = 0;
        TVK_CALL(tvk_get_device(&dev));
        c10::Device device(c10::DeviceType::PrivateUse1, (c10::DeviceIndex)dev);
        if (nbytes == 0) {
            int count = 0;
            TVK_CALL(tvk_device_count(&count));
            TORCH_CHECK(dev >= 0 && dev < count, "torchvulkan [ERROR]: current device ", dev, " out of range (", count, " devices)");
            return {nullptr, nullptr, &delete_block, device};
        }
        void* p = nullptr;
        TVK_CALL(tvk_malloc(dev, nbytes, &p));
        return {p, new Block{p, dev}, &delete_block, device};
    }
    c10::DeleterFnPtr raw_deleter() const override { return nullptr; }
    void copy_data(void* dest, const void* src, std::size_t count) const override {
        int dev = 0;
        TVK_CALL(tvk_pointer_device(src, &dev));
        TVK_CALL(tvk_memcpy_d2d(dev, dest, src, count));
    }
    bool initialized() override { return tvk_is_initialized() != 0; }
    void emptyCache(c10::MempoolId_t) override {
        int n = 0;
        TVK_CALL(tvk_device_count(&n));
        for (int i = 0; i < n; ++i) TVK_CALL(tvk_empty_cache(i));
    }
    void recordStream(const c10::DataPtr&, c10::Stream) override {}  // one stream per device
    c10::CachingDeviceAllocator::DeviceStats getDeviceStats(c10::DeviceIndex device) override {
        tvk_mem_stats s;
        TVK_CALL(tvk_mem_get_stats(device, &s));
        c10::CachingDeviceAllocator::DeviceStats out;
        auto set = [](c10::CachingAllocator::StatArray& a, uint64_t cur, uint64_t peak, uint64_t alloc, uint64_t freed) {
            for (auto& st : a) {
                st.current = (int64_t)cur;
                st.peak = (int64_t)peak;
                st.allocated = (int64_t)alloc;
                st.freed = (int64_t)freed;
            }
        };
        set(out.allocated_bytes, s.allocated_bytes, s.peak_allocated_bytes, s.total_allocated_bytes, s.total_freed_bytes);
        set(out.active_bytes, s.allocated_bytes, s.peak_allocated_bytes, s.total_allocated_bytes, s.total_freed_bytes);
        set(out.requested_bytes, s.allocated_bytes, s.peak_allocated_bytes, s.total_allocated_bytes, s.total_freed_bytes);
        set(out.reserved_bytes, s.reserved_bytes, s.reserved_bytes, s.reserved_bytes, 0);
        out.num_alloc_retries = (int64_t)s.num_oom_retries;
        out.num_device_alloc = (int64_t)s.num_device_mallocs;
        return out;
    }
    void resetAccumulatedStats(c10::DeviceIndex) override {}
    void resetPeakStats(c10::DeviceIndex device) override { TVK_CALL(tvk_mem_reset_peak(device)); }
    std::pair<size_t, size_t> getMemoryInfo(c10::DeviceIndex device) override {
        uint64_t f = 0, t = 0;
        TVK_CALL(tvk_mem_info(device, &f, &t));
        return {(size_t)f, (size_t)t};
    }
};

TvkAllocator g_allocator;

// ---------------------------------------------------------------------------------------
// pinned host allocator
// ---------------------------------------------------------------------------------------
class PinnedAllocator final : public c10::Allocator {
public:
    c10::DataPtr allocate(size_t nbytes) override {
        void* p = nullptr;
        if (nbytes) TVK_CALL(tvk_host_alloc(nbytes, &p));
        if (p) {
            std::lock_guard<std::mutex> lock(mu());
            blocks()[reinterpret_cast<uintptr_t>(p)] = nbytes;
        }
        return {p, p, &PinnedAllocator::free_block, c10::Device(c10::DeviceType::CPU)};
    }
    c10::DeleterFnPtr raw_deleter() const override { return &PinnedAllocator::free_block; }
    void copy_data(void* dest, const void* src, std::size_t count) const override { std::memcpy(dest, src, count); }
    static bool contains(const void* ptr) {
        std::lock_guard<std::mutex> lock(mu());
        const auto a = reinterpret_cast<uintptr_t>(ptr);
        auto it = blocks().upper_bound(a);
        if (it == blocks().begin()) return false;
        --it;
        return a < it->first + std::max<size_t>(it->second, 1);
    }

private:
    static void free_block(void* p) {
        if (!p) return;
        {
            std::lock_guard<std::mutex> lock(mu());
            blocks().erase(reinterpret_cast<uintptr_t>(p));
        }
        tvk_host_free(p);
    }
    static std::mutex& mu() { static std::mutex m; return m; }
    static std::map<uintptr_t, size_t>& blocks() { static auto* b = new std::map<uintptr_t, size_t>(); return *b; }
};

PinnedAllocator g_pinned;

// ---------------------------------------------------------------------------------------
// generator: 16-byte state (seed, offset) kept by the runtime per device
// ---------------------------------------------------------------------------------------
class TvkGeneratorImpl final : public c10::GeneratorImpl {
public:
    explicit TvkGeneratorImpl(c10::DeviceIndex index)
        : c10::GeneratorImpl(c10::Device(c10::DeviceType::PrivateUse1, index), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1)) {}
    void set_current_seed(uint64_t seed) override { TVK_CALL(tvk_rng_set_seed(device_.index(), seed)); }
    void set_offset(uint64_t offset) override {
        uint64_t s = 0, o = 0;
        TVK_CALL(tvk_rng_get_state(device_.index(), &s, &o));
        TVK_CALL(tvk_rng_set_state(device_.index(), s, offset));
    }
    uint64_t get_offset() const override {
        uint64_t s = 0, o = 0;
        TVK_CALL(tvk_rng_get_state(device_.index(), &s, &o));
        return o;
    }
    uint64_t current_seed() const override {
        uint64_t s = 0, o = 0;
        TVK_CALL(tvk_rng_get_state(device_.index(), &s, &o));
        return s;
    }
    uint64_t seed() override {
        const uint64_t s = c10::detail::getNonDeterministicRandom(true);
        set_current_seed(s);
        return s;
    }
    void set_state(const c10::TensorImpl& new_state) override {
        TORCH_CHECK(new_state.numel() * (int64_t)new_state.itemsize() == 16, "torchvulkan [ERROR]: RNG state must be 16 bytes");
        uint64_t v[2];
        std::memcpy(v, new_state.data(), 16);
        TVK_CALL(tvk_rng_set_state(device_.index(), v[0], v[1]));
    }
    c10::intrusive_ptr<c10::TensorImpl> get_state() const override {
        uint64_t v[2] = {0, 0};
        TVK_CALL(tvk_rng_get_state(device_.index(), &v[0], &v[1]));
        at::Tensor t = at::empty({16}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
        std::memcpy(t.data_ptr(), v, 16);
        return t.getIntrusivePtr();
    }
    static c10::DeviceType device_type() { return c10::DeviceType::PrivateUse1; }

private:
    TvkGeneratorImpl* clone_impl() const override { return new TvkGeneratorImpl(device_.index()); }
};

std::mutex g_gen_mu;
std::map<int, at::Generator> g_default_generators;

}  // namespace

const at::Generator& default_generator(c10::DeviceIndex index) {
    int dev = index;
    if (dev < 0) TVK_CALL(tvk_get_device(&dev));
    std::lock_guard<std::mutex> lock(g_gen_mu);
    auto it = g_default_generators.find(dev);
    if (it == g_default_generators.end())
        it = g_default_generators.emplace(dev, at::make_generator<TvkGeneratorImpl>((c10::DeviceIndex)dev)).first;
    return it->second;
}

at::Generator new_generator(c10::DeviceIndex index) {
    int dev = index;
    if (dev < 0) TVK_CALL(tvk_get_device(&dev));
    return at::make_generator<TvkGeneratorImpl>((c10::DeviceIndex)dev);
}

// ---------------------------------------------------------------------------------------
// device guard
// ---------------------------------------------------------------------------------------
namespace {

class TvkGuardImpl final : public c10::impl::DeviceGuardImplInterface {
public:
    c10::DeviceType type() const override { return c10::DeviceType::PrivateUse1; }
    c10::Device exchangeDevice(c10::Device d) const override {
        c10::Device old = getDevice();
        setDevice(d);
        return old;
    }
    c10::Device getDevice() const override {
        int dev = 0;
        tvk_get_device(&dev);
        return c10::Device(c10::DeviceType::PrivateUse1, (c10::DeviceIndex)dev);
    }
    void setDevice(c10::Device d) const override { TVK_CALL(tvk_set_device(d.index())); }
    void uncheckedSetDevice(c10::Device d) const noexcept override { tvk_set_device(d.index()); }
    c10::Stream getStream(c10::Device d) const noexcept override { return c10::Stream(c10::Stream::UNSAFE, indexed(d), 0); }
    c10::Stream getDefaultStream(c10::Device d) const override { return c10::Stream(c10::Stream::UNSAFE, indexed(d), 0); }
    c10::Stream getNewStream(c10::Device d, int) const override { return c10::Stream(c10::Stream::UNSAFE, indexed(d), 0); }
    c10::Stream getStreamFromGlobalPool(c10::Device d, bool) const override { return c10::Stream(c10::Stream::UNSAFE, indexed(d), 0); }
    c10::Stream exchangeStream(c10::Stream s) const noexcept override { return c10::Stream(c10::Stream::UNSAFE, s.device(), 0); }
    c10::DeviceIndex deviceCount() const noexcept override {
        int n = 0;
        if (tvk_device_count(&n) != TVK_OK) return 0;
        return (c10::DeviceIndex)n;
    }
    bool queryStream(const c10::Stream&) const override { return true; }
    void synchronizeStream(const c10::Stream& s) const override { TVK_CALL(tvk_synchronize(s.device_index())); }
    void synchronizeDevice(const c10::DeviceIndex index) const override { TVK_CALL(tvk_synchronize(index)); }

    void destroyEvent(void* event, const c10::DeviceIndex) const noexcept override { tvk_event_destroy(event); }
    void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index, const c10::EventFlag) const override {
        TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ", device_index,
                    " does not match recording stream's device index ", stream.device_index(), ".");
        if (*event == nullptr) TVK_CALL(tvk_event_create(event));
        TVK_CALL(tvk_event_record(stream.device_index(), *event));
    }
    void block(void* event, const c10::Stream& stream) const override {
        // each device has its own in-order stream: work submitted to `stream`'s device from here on follows the event,
        // on whichever device it was recorded
        if (event) TVK_CALL(tvk_event_wait(stream.device_index(), event));
    }
    bool queryEvent(void* event) const override {
        if (!event) return true;
        int done = 1;
        TVK_CALL(tvk_event_query(event, &done));
        return done != 0;
    }
    void synchronizeEvent(void* event) const override {
        if (event) TVK_CALL(tvk_event_synchronize(event));
    }
    double elapsedTime(void* e1, void* e2, const c10::DeviceIndex) const override {
        TORCH_CHECK(e1 && e2, "Both events must be recorded before calculating elapsed time.");
        TVK_CALL(tvk_event_synchronize(e2));
        float ms = 0.f;
        TVK_CALL(tvk_event_elapsed_ms(e1, e2, &ms));
        return ms;
    }

private:
    c10::Device indexed(c10::Device d) const { return d.has_index() ? d : getDevice(); }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, TvkGuardImpl);

// ---------------------------------------------------------------------------------------
// hooks
// ---------------------------------------------------------------------------------------
struct TvkHooks final : public at::PrivateUse1HooksInterface {
    bool isBuilt() const override { return true; }
    bool isAvailable() const override {
        int n = 0;
        return tvk_device_count(&n) == TVK_OK && n > 0;
    }
    bool hasPrimaryContext(c10::DeviceIndex index) const override {
        int n = 0;
        return tvk_device_count(&n) == TVK_OK && index < n;
    }
    c10::DeviceIndex deviceCount() const override {
        int n = 0;
        tvk_device_count(&n);
        return (c10::DeviceIndex)n;
    }
    void setCurrentDevice(c10::DeviceIndex device) const override { TVK_CALL(tvk_set_device(device)); }
    c10::DeviceIndex getCurrentDevice() const override {
        int d = 0;
        tvk_get_device(&d);
        return (c10::DeviceIndex)d;
    }
    c10::DeviceIndex exchangeDevice(c10::DeviceIndex device) const override {
        const c10::DeviceIndex old = getCurrentDevice();
        setCurrentDevice(device);
        return old;
    }
    c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex device) const override { return exchangeDevice(device); }
    at::Device getDeviceFromPtr(void* data) const override {
        int dev = 0;
        TVK_CALL(tvk_pointer_device(data, &dev));
        return c10::Device(c10::DeviceType::PrivateUse1, (c10::DeviceIndex)dev);
    }
    c10::Allocator* getPinnedMemoryAllocator() const override { return &g_pinned; }
    bool isPinnedPtr(const void* data) const override { return PinnedAllocator::contains(data); }
    void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override {
        c10::StorageImpl* impl = storage.unsafeGetStorageImpl();
        const size_t old = impl->nbytes();
        // the new block belongs on the storage's device, whichever device is current
        int current = 0;
        TVK_CALL(tvk_get_device(&current));
        const int target = storage.device().has_index() ? (int)storage.device().index() : current;
        if (target != current) TVK_CALL(tvk_set_device(target));
        c10::DataPtr fresh;
        try {
            fresh = g_allocator.allocate(newsize);
        } catch (...) {
            if (target != current) tvk_set_device(current);
            throw;
        }
        if (target != current) TVK_CALL(tvk_set_device(current));
        const size_t keep = std::min(old, newsize);
        if (keep) g_allocator.copy_data(fresh.get(), impl->data(), keep);
        impl->set_data_ptr_noswap(std::move(fresh));
        impl->set_nbytes(newsize);
    }
    const at::Generator& getDefaultGenerator(c10::DeviceIndex index) const override { return default_generator(index); }
    at::Generator getNewGenerator(c10::DeviceIndex index = -1) const override { return new_generator(index); }
};

TvkHooks g_hooks;
const bool g_hooks_registered = [] {
    at::RegisterPrivateUse1HooksInterface(&g_hooks);
    return true;
}();

}  // namespace

REGISTER_ALLOCATOR(c10::DeviceType::PrivateUse1, &g_allocator);

c10::Allocator* device_allocator() { return &g_allocator; }

}  // namespace tvk_aten
