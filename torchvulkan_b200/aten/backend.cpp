// Python module `_C`: the functions torchvulkan/__init__.py calls, with the reference's names and
// argument meaning (src/api/backend.cpp:12-129), implemented over the tvk C-ABI.
#include <torch/csrc/Generator.h>
#include <torch/extension.h>

#include "common.h"

namespace tvk_aten {
const at::Generator& default_generator(c10::DeviceIndex index);
}

namespace py = pybind11;
using tvk_aten::throw_status;

static int device_count_nothrow() {
    int n = 0;
    if (tvk_device_count(&n) != TVK_OK) return 0;
    return n;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "torchvulkan backend (B200-native runtime)";

    m.def("is_available", []() -> bool { return device_count_nothrow() > 0; });
    m.def("device_count", []() -> int64_t { return device_count_nothrow(); });
    m.def("current_device", []() -> int64_t {
        int d = 0;
        TVK_CALL(tvk_get_device(&d));
        return d;
    });
    m.def("synchronize", [](int64_t device_index) {
        TVK_CALL(tvk_synchronize((int)device_index));
        // A bounded device-side wait that ran out, or a kernel that saw an invalid index, surfaces here.
        TVK_CALL(tvk_check_device_status((int)device_index));
    }, py::call_guard<py::gil_scoped_release>());
    m.def("_default_generator", [](int64_t device_index) {
        return py::reinterpret_steal<py::object>(THPGenerator_initDefaultGenerator(tvk_aten::default_generator((c10::DeviceIndex)device_index)));
    });
    m.def("_manual_seed", [](int64_t device_index, uint64_t seed) { TVK_CALL(tvk_rng_set_seed((int)device_index, seed)); });
    m.def("_manual_seed_all", [](uint64_t seed) {
        const int n = device_count_nothrow();
        for (int i = 0; i < n; ++i) TVK_CALL(tvk_rng_set_seed(i, seed));
    });
    m.def("_is_in_bad_fork", []() -> bool { return tvk_is_in_bad_fork() != 0; });
    m.def("empty_cache", []() {
        const int n = device_count_nothrow();
        for (int i = 0; i < n; ++i) TVK_CALL(tvk_empty_cache(i));
    }, py::call_guard<py::gil_scoped_release>());
    // Kernels are compiled ahead of time: there is no pipeline cache to save.
    m.def("_save_pipeline_caches", []() {});
    m.def("_amp_supported_dtypes", [](int64_t) {
        std::vector<py::object> dtypes;
        dtypes.push_back(py::reinterpret_borrow<py::object>(reinterpret_cast<PyObject*>(torch::getTHPDtype(at::kHalf))));
        dtypes.push_back(py::reinterpret_borrow<py::object>(reinterpret_cast<PyObject*>(torch::getTHPDtype(at::kBFloat16))));
        return dtypes;
    });
    auto stats = [](int64_t device_index) {
        tvk_mem_stats s;
        TVK_CALL(tvk_mem_get_stats((int)device_index, &s));
        return s;
    };
    m.def("_memory_usage", [stats](int64_t d) -> uint64_t { return stats(d).reserved_bytes; });
    m.def("_memory_reserved", [stats](int64_t d) -> uint64_t { return stats(d).reserved_bytes; });
    m.def("_memory_allocated", [stats](int64_t d) -> uint64_t { return stats(d).allocated_bytes; });
    m.def("_max_memory_allocated", [stats](int64_t d) -> uint64_t { return stats(d).peak_allocated_bytes; });
    m.def("_reset_peak_memory_stats", [](int64_t d) { TVK_CALL(tvk_mem_reset_peak((int)d)); });
    m.def("_mem_get_info", [](int64_t d) -> std::pair<uint64_t, uint64_t> {
        uint64_t f = 0, t = 0;
        TVK_CALL(tvk_mem_info((int)d, &f, &t));
        return {f, t};
    });
    // Storage slices own nothing on this backend (a DataPtr is a plain device address).
    m.def("_record_storage_slice_deleter", [](const at::Tensor&) {});
    m.def("_is_initialized", []() -> bool { return tvk_is_initialized() != 0; });
    m.def("_lazy_init", []() { TVK_CALL(tvk_init()); });
    m.def("_device_properties", [](int64_t device_index) {
        tvk_device_props p;
        TVK_CALL(tvk_get_device_props((int)device_index, &p));
        py::dict info;
        info["name"] = std::string(p.name);
        info["total_memory"] = p.total_memory;
        info["vendor_id"] = p.vendor_id;
        info["device_id"] = p.device_id;
        info["api_version"] = "CUDA " + std::to_string(p.runtime_version / 1000) + "." + std::to_string(p.runtime_version % 1000 / 10) +
                              " sm_" + std::to_string(p.cc_major) + std::to_string(p.cc_minor);
        info["driver_version"] = p.driver_version;
        info["subgroup_size"] = p.warp_size;
        info["has_fp64"] = true;   // copies, fills and casts only
        info["has_int64"] = true;
        info["has_fp16"] = true;
        info["has_bf16"] = true;
        info["has_int16"] = false;
        info["has_int8"] = true;
        return info;
    });
    // the number of problems the checked mode (TORCHVULKAN_VALIDATION=1) has seen: the counterpart of the reference's count of
    // validation-layer messages (src/api/backend.cpp:127-129)
    m.def("_validation_error_count", []() -> uint64_t { return tvk_aten::validation_error_count(); });
}
