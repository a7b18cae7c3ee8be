// Allocation, copies, casts, scalar read-back and views for the "vulkan" device.
//
// Counterparts in the reference: empty_memory_format_vulkan / empty_strided_vulkan / resize / clone /
// set_ (src/api/tensor/allocation.cpp:35-247), copy_vulkan / _local_scalar_dense
// (src/api/tensor/transfer.cpp:292-398), dispatch_copy_shader (transfer.cpp:16-56),
// dispatch_cast_shader (src/api/tensor/cast.cpp:8-55) and the metadata-only views
// (src/api/tensor/views.cpp:14-159). Tensors are ordinary strided TensorImpls whose storage
// holds a device pointer from the tvk caching allocator; views never touch the device.
#include "common.h"

#include <ATen/EmptyTensor.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorShape.h>
#include <ATen/ops/_reshape_alias_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/unfold_native.h>
#include <ATen/ops/view_native.h>
#include <c10/core/DeviceGuard.h>

namespace tvk_aten {

c10::Allocator* device_allocator();

namespace {

constexpr c10::DispatchKeySet kKeys(c10::DispatchKey::PrivateUse1);

struct CurrentDevice {  // allocations land on tvk's current device
    explicit CurrentDevice(c10::optional<at::Device> device) {
        TVK_CALL(tvk_get_device(&prev));
        if (device.has_value() && device->has_index() && device->index() != prev) {
            TVK_CALL(tvk_set_device(device->index()));
            switched = true;
        }
    }
    ~CurrentDevice() {
        if (switched) tvk_set_device(prev);
    }
    int prev = 0;
    bool switched = false;
};

at::Tensor empty_memory_format(c10::SymIntArrayRef size, c10::optional<at::ScalarType> dtype, c10::optional<at::Layout> layout,
                               c10::optional<at::Device> device, c10::optional<bool>, c10::optional<at::MemoryFormat> memory_format) {
    TORCH_CHECK(layout.value_or(at::kStrided) == at::kStrided, "torchvulkan [ERROR]: Only Strided layout is supported");
    CurrentDevice scope(device);
    const auto st = dtype.value_or(c10::typeMetaToScalarType(at::get_default_dtype()));
    return at::detail::empty_generic(C10_AS_INTARRAYREF_SLOW(size), device_allocator(), kKeys, st, memory_format);
}

at::Tensor empty_strided(c10::SymIntArrayRef size, c10::SymIntArrayRef stride, c10::optional<at::ScalarType> dtype,
                         c10::optional<at::Layout>, c10::optional<at::Device> device, c10::optional<bool>) {
    CurrentDevice scope(device);
    const auto st = dtype.value_or(c10::typeMetaToScalarType(at::get_default_dtype()));
    return at::detail::empty_strided_generic(C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride), device_allocator(), kKeys, st);
}

}  // namespace

at::Tensor empty_vulkan(at::IntArrayRef sizes, at::ScalarType dtype, c10::Device device) {
    CurrentDevice scope(device);
    return at::detail::empty_generic(sizes, device_allocator(), kKeys, dtype, c10::nullopt);
}

at::Tensor empty_like_contig(const at::Tensor& t) { return empty_vulkan(t.sizes(), t.scalar_type(), t.device()); }

void make_iter(tvk_iter* it, const at::Tensor& out, std::initializer_list<const at::Tensor*> inputs) {
    const int64_t nd = out.dim();
    TORCH_CHECK(nd <= TVK_MAX_DIMS, "torchvulkan [NOT IMPLEMENTED]: tensors with more than ", TVK_MAX_DIMS, " dimensions");
    it->ndim = (int32_t)nd;
    it->noperands = (int32_t)inputs.size() + 1;
    for (int64_t d = 0; d < nd; ++d) {
        it->sizes[d] = out.size(d);
        it->strides[0][d] = out.stride(d);
    }
    int o = 1;
    for (const at::Tensor* in : inputs) {
        // right-aligned broadcast of `in` against out's shape
        const int64_t off = nd - in->dim();
        TORCH_CHECK(off >= 0, "torchvulkan [ERROR]: operand has more dimensions than the output");
        for (int64_t d = 0; d < nd; ++d) {
            int64_t s = 0;
            if (d >= off) {
                const int64_t sz = in->size(d - off);
                TORCH_CHECK(sz == out.size(d) || sz == 1, "The size of tensor a (", sz, ") must match the size of tensor b (", out.size(d),
                            ") at non-singleton dimension ", d);
                s = sz == 1 ? 0 : in->stride(d - off);
            }
            it->strides[o][d] = s;
        }
        ++o;
    }
}

namespace {

// dst (vulkan, any strides) <- src (vulkan, same device, any strides, any supported dtype)
void device_copy(const at::Tensor& dst, const at::Tensor& src) {
    if (dst.numel() == 0) return;
    int ddt = to_tvk_dtype(dst.scalar_type()), sdt = to_tvk_dtype(src.scalar_type());
    if (dst.scalar_type() == src.scalar_type() && ddt < 0) {
        // a same-type copy does not interpret the values: types the kernels have no arithmetic for (float8, int16, ...)
        // move as integers of their width
        switch (dst.element_size()) {
            case 1: ddt = sdt = TVK_U8; break;
            case 4: ddt = sdt = TVK_I32; break;
            case 8: ddt = sdt = TVK_I64; break;
            default: break;
        }
    }
    TORCH_CHECK(ddt >= 0 && sdt >= 0, "torchvulkan [NOT IMPLEMENTED]: copy between ", src.scalar_type(), " and ", dst.scalar_type());
    DeviceScope scope(dst);
    // bool <-> number conversions are not plain byte copies
    const bool bool_mix = (dst.scalar_type() == at::kBool) != (src.scalar_type() == at::kBool);
    if (dst.is_contiguous() && src.is_contiguous() && src.sizes() == dst.sizes() && !bool_mix) {
        if (ddt == sdt) TVK_CALL(tvk_memcpy_d2d(scope.device, dst.data_ptr(), src.data_ptr(), dst.nbytes()));
        else TVK_CALL(tvk_cast(ddt, dst.data_ptr(), sdt, src.data_ptr(), dst.numel(), scope.stream));
        return;
    }
    if (bool_mix && dst.scalar_type() == at::kBool) {
        // number -> bool is (x != 0)
        at::Tensor zero = at::zeros({}, src.options());
        at::Tensor ne = at::ne(src, zero);
        device_copy(dst, ne);
        return;
    }
    tvk_iter it;
    make_iter(&it, dst, {&src});
    TVK_CALL(tvk_copy_strided(ddt, dst.data_ptr(), sdt, src.data_ptr(), &it, scope.stream));
}

at::Tensor copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
    TORCH_CHECK(self.sizes() == dst.sizes() || self.numel() == dst.numel() || self.dim() <= dst.dim(),
                "torchvulkan [ERROR]: copy_ shape mismatch");
    if (is_vulkan(self) && is_vulkan(dst)) {
        if (self.device() == dst.device()) {
            at::Tensor src = self.sizes() == dst.sizes() ? self : self.expand(dst.sizes());
            device_copy(dst, src);
        } else {
            // cross-device: contiguous staging on the source device, peer copy, then layout on the destination
            at::Tensor src = self.expand(dst.sizes()).contiguous();
            at::Tensor landing = (dst.is_contiguous() && dst.scalar_type() == src.scalar_type()) ? dst : empty_vulkan(dst.sizes(), src.scalar_type(), dst.device());
            TVK_CALL(tvk_memcpy_peer(dst.device().index(), landing.data_ptr(), src.device().index(), src.data_ptr(), src.nbytes()));
            TVK_CALL(tvk_synchronize(dst.device().index()));  // src may be freed by the caller right after
            if (!landing.is_same(dst)) device_copy(dst, landing);
        }
        return dst;
    }
    if (is_vulkan(dst)) {
        // host -> device. The bytes go up in the source dtype; any cast or re-layout runs on the device.
        TORCH_CHECK(self.device().is_cpu(), "torchvulkan [ERROR]: copies between vulkan and ", self.device().type(), " go through the CPU");
        at::Tensor src = self.expand(dst.sizes()).contiguous();
        const bool direct = dst.is_contiguous() && dst.scalar_type() == src.scalar_type();
        const bool castable = to_tvk_dtype(src.scalar_type()) >= 0 && src.scalar_type() != at::kBool && dst.scalar_type() != at::kBool;
        if (!direct && !castable) src = src.to(dst.scalar_type());
        at::Tensor landing = (dst.is_contiguous() && dst.scalar_type() == src.scalar_type()) ? dst : empty_vulkan(dst.sizes(), src.scalar_type(), dst.device());
        if (src.nbytes()) {
            TVK_CALL(tvk_memcpy_h2d(dst.device().index(), landing.data_ptr(), src.data_ptr(), src.nbytes()));
            // A pinned source is read asynchronously: finish before the temporary `src` can die.
            if (src.is_pinned() && !(non_blocking && src.is_same(self))) TVK_CALL(tvk_synchronize(dst.device().index()));
        }
        if (!landing.is_same(dst)) device_copy(dst, landing);
        return dst;
    }
    // device -> host
    TORCH_CHECK(dst.device().is_cpu(), "torchvulkan [ERROR]: copies between vulkan and ", dst.device().type(), " go through the CPU");
    at::Tensor src = self.sizes() == dst.sizes() ? self : self.expand(dst.sizes());
    const bool castable = to_tvk_dtype(dst.scalar_type()) >= 0 && dst.scalar_type() != at::kBool && src.scalar_type() != at::kBool;
    at::Tensor staged = src;
    if (!src.is_contiguous() || (src.scalar_type() != dst.scalar_type() && castable)) {
        staged = empty_vulkan(src.sizes(), castable ? dst.scalar_type() : src.scalar_type(), src.device());
        device_copy(staged, src);
    }
    if (dst.is_contiguous() && dst.scalar_type() == staged.scalar_type()) {
        if (staged.nbytes()) TVK_CALL(tvk_memcpy_d2h(staged.device().index(), dst.data_ptr(), staged.data_ptr(), staged.nbytes()));
    } else {
        at::Tensor host = at::empty(staged.sizes(), staged.options().device(at::kCPU));
        if (staged.nbytes()) TVK_CALL(tvk_memcpy_d2h(staged.device().index(), host.data_ptr(), staged.data_ptr(), staged.nbytes()));
        dst.copy_(host);
    }
    return dst;
}

at::Tensor copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
    dst.resize_(self.sizes());
    return copy_from(self, dst, false);
}

at::Scalar local_scalar_dense(const at::Tensor& self) {
    TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
    at::Tensor host = at::empty({}, self.options().device(at::kCPU));
    TVK_CALL(tvk_memcpy_d2h(self.device().index(), host.data_ptr(), self.data_ptr(), self.itemsize()));
    return host.item();
}

const at::Tensor& resize_(const at::Tensor& self, c10::SymIntArrayRef size, c10::optional<at::MemoryFormat> memory_format) {
    auto sizes = C10_AS_INTARRAYREF_SLOW(size);
    auto* impl = self.unsafeGetTensorImpl();
    impl->set_sizes_contiguous(sizes);
    if (memory_format.has_value() && *memory_format != at::MemoryFormat::Preserve) impl->empty_tensor_restride(*memory_format);
    const size_t need = (size_t)(impl->storage_offset() + at::detail::computeStorageNbytesContiguous(sizes, self.itemsize()) / std::max<size_t>(self.itemsize(), 1)) * self.itemsize();
    const c10::Storage& storage = impl->unsafe_storage();
    if (storage && need > storage.nbytes()) at::detail::getPrivateUse1Hooks().resizePrivateUse1Bytes(storage, need);
    return self;
}

at::Tensor clone(const at::Tensor& self, c10::optional<at::MemoryFormat> memory_format) {
    const auto mf = memory_format.value_or(at::MemoryFormat::Preserve);
    at::Tensor out;
    if (mf == at::MemoryFormat::Preserve && self.is_non_overlapping_and_dense()) {
        out = at::empty_strided(self.sizes(), self.strides(), self.options());
    } else {
        out = at::empty(self.sizes(), self.options(), mf == at::MemoryFormat::Preserve ? at::MemoryFormat::Contiguous : mf);
    }
    device_copy(out, self);
    return out;
}

at::Tensor& set_storage_offset(at::Tensor& self, at::Storage source, c10::SymInt offset, c10::SymIntArrayRef size, c10::SymIntArrayRef stride) {
    auto* impl = self.unsafeGetTensorImpl();
    impl->set_storage_keep_dtype(std::move(source));
    impl->set_storage_offset(offset.guard_int(__FILE__, __LINE__));
    auto sizes = C10_AS_INTARRAYREF_SLOW(size);
    if (stride.empty() && !sizes.empty()) impl->set_sizes_contiguous(sizes);
    else impl->set_sizes_and_strides(sizes, C10_AS_INTARRAYREF_SLOW(stride));
    return self;
}

at::Tensor& set_storage(at::Tensor& self, at::Storage source) {
    const int64_t n = (int64_t)(source.nbytes() / std::max<size_t>(self.itemsize(), 1));
    auto* impl = self.unsafeGetTensorImpl();
    impl->set_storage_keep_dtype(std::move(source));
    impl->set_storage_offset(0);
    impl->set_sizes_contiguous({n});
    return self;
}

at::Tensor& set_tensor(at::Tensor& self, const at::Tensor& source) {
    if (self.unsafeGetTensorImpl() == source.unsafeGetTensorImpl()) return self;
    auto* impl = self.unsafeGetTensorImpl();
    impl->set_storage_keep_dtype(source.storage());
    impl->set_storage_offset(source.storage_offset());
    impl->set_sizes_and_strides(source.sizes(), source.strides());
    return self;
}

at::Tensor& set_empty(at::Tensor& self) {
    c10::Storage storage(c10::Storage::use_byte_size_t(), 0, device_allocator(), true);
    return set_storage(self, std::move(storage));
}

// Module.to("vulkan") asks this before it swaps `param.data`; answering yes for dense CPU <-> vulkan
// tensors keeps the Parameter objects (and with them tied weights) instead of replacing them
// (src/api/tensor/transfer.cpp:383-388).
bool has_compatible_shallow_copy_type(const at::Tensor& self, const at::Tensor& from) {
    auto dense = [](const at::Tensor& t) { return t.layout() == at::kStrided && (t.device().is_cpu() || is_vulkan(t)); };
    return dense(self) && dense(from);
}

}  // namespace

at::Tensor contiguous_vulkan(const at::Tensor& t) {
    if (t.is_contiguous()) return t;
    at::Tensor out = empty_like_contig(t);
    device_copy(out, t);
    return out;
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("empty.memory_format", &empty_memory_format);
    m.impl("empty_strided", &empty_strided);
    m.impl("resize_", &resize_);
    m.impl("clone", &clone);
    m.impl("set_.source_Storage_storage_offset", &set_storage_offset);
    m.impl("set_.source_Storage", &set_storage);
    m.impl("set_.source_Tensor", &set_tensor);
    m.impl("set_", &set_empty);
    m.impl("_copy_from", &copy_from);
    m.impl("_copy_from_and_resize", &copy_from_and_resize);
    m.impl("_local_scalar_dense", &local_scalar_dense);
    m.impl("_has_compatible_shallow_copy_type", &has_compatible_shallow_copy_type);
    // Views are pure metadata: ATen's device-independent implementations apply as they are.
    m.impl("as_strided", &at::native::as_strided_tensorimpl);
    m.impl("view", &at::native::view);
    m.impl("_reshape_alias", &at::native::_reshape_alias);
    m.impl("unfold", &at::native::unfold);
}

}  // namespace tvk_aten
