// Shared helpers of the ATen operator layer: the PrivateUse1 ("vulkan") device registrations
// call the tvk C-ABI (include/tvk.h) through these.
#pragma once

#include <ATen/ATen.h>
#include <c10/core/Device.h>
#include <torch/library.h>

#include "../../include/tvk.h"

namespace tvk_aten {

// Converts a C-ABI status into the exception the reference would have raised
// (TORCH_CHECK / OutOfMemoryError, messages prefixed "torchvulkan [ERROR]:").
void throw_status(int status, const char* what);

// The reference's environment switches (src/vulkan/vulkan_context.cpp:195-248), read once:
//   TORCHVULKAN_PROFILE=1     every C-ABI call made by an operator is wrapped in an NVTX range named after the call (the
//                             reference captures pipeline statistics per dispatch, src/vulkan/shader.cpp:428-431)
//   TORCHVULKAN_VALIDATION=1  checked mode: after every operator the device is synchronised and its status word and CUDA's
//                             error state are read; problems are warned about and counted (_validation_error_count), as
//                             the reference counts the messages of the Vulkan validation layer
//   TORCHVULKAN_STRICT        accepted; this backend never falls back to the CPU, so it is always strict
struct EnvFlags {
    bool profile = false, validation = false, strict = true;
};
const EnvFlags& env_flags();
uint64_t validation_error_count();
void profile_push(const char* name);
void profile_pop();
struct ProfileRange {
    explicit ProfileRange(const char* name) : on(env_flags().profile) { if (on) profile_push(name); }
    ~ProfileRange() { if (on) profile_pop(); }
    bool on;
};

#define TVK_CALL(expr)                                        \
    do {                                                      \
        ::tvk_aten::ProfileRange _tvk_range(#expr);           \
        int _tvk_rc = (expr);                                 \
        if (_tvk_rc != TVK_OK) ::tvk_aten::throw_status(_tvk_rc, #expr); \
    } while (0)

inline bool is_vulkan(const at::Tensor& t) { return t.device().type() == c10::DeviceType::PrivateUse1; }

// Same shape and the same element order in memory: strides are compared only along dimensions longer than one (a
// [128, 64, 1, 1] filter is the same bytes in contiguous and in channels-last strides).
inline bool same_layout(const at::Tensor& a, const at::Tensor& b) {
    if (a.sizes() != b.sizes()) return false;
    for (int64_t d = 0; d < a.dim(); ++d)
        if (a.size(d) > 1 && a.stride(d) != b.stride(d)) return false;
    return true;
}

inline int to_tvk_dtype(at::ScalarType st) {
    switch (st) {
        case at::kFloat: return TVK_F32;
        case at::kHalf: return TVK_F16;
        case at::kBFloat16: return TVK_BF16;
        case at::kLong: return TVK_I64;
        case at::kInt: return TVK_I32;
        case at::kByte: case at::kBool: case at::kChar: return TVK_U8;
        case at::kDouble: return TVK_F64;
        default: return -1;
    }
}

inline bool is_hot_float(at::ScalarType st) { return st == at::kFloat || st == at::kHalf || st == at::kBFloat16; }

// Ops on the hot path never fall back to the CPU: unsupported dtypes raise.
#define TVK_NOT_IMPLEMENTED(...) TORCH_CHECK(false, "torchvulkan [NOT IMPLEMENTED]: ", __VA_ARGS__)

// Makes the tensor's device current for tvk (and CUDA) for the scope, returns its compute stream.
struct DeviceScope {
    explicit DeviceScope(const at::Tensor& t) : DeviceScope(t.device().index()) {}
    explicit DeviceScope(c10::DeviceIndex index);
    ~DeviceScope();
    void* stream = nullptr;
    int device = 0;
    int previous = 0;
};

// Scratch from the caching allocator, released (stream-ordered) at scope exit.
struct Workspace {
    Workspace(int device, uint64_t bytes);
    ~Workspace();
    Workspace(const Workspace&) = delete;
    void* ptr = nullptr;
    uint64_t bytes = 0;
    int device = 0;
};

at::Tensor empty_vulkan(at::IntArrayRef sizes, at::ScalarType dtype, c10::Device device);
at::Tensor empty_like_contig(const at::Tensor& t);
// A contiguous tensor with the same values (the tensor itself when it already is).
at::Tensor contiguous_vulkan(const at::Tensor& t);
// Fills a tvk_iter for `out` and up to three inputs broadcast to out's shape.
void make_iter(tvk_iter* it, const at::Tensor& out, std::initializer_list<const at::Tensor*> inputs);

}  // namespace tvk_aten
