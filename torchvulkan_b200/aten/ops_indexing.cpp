// The gather family on the "vulkan" device, built on the row-gather (embedding) kernel and its deterministic backward:
// index_select / index_add, gather / scatter_add, x[idx] with one index tensor and its accumulate-put, flip, roll,
// scatter of a value (one_hot), prod, equal.
//
// Counterparts in the reference: src/api/ops/indexing.cpp:100-298 and 416-423 (gather, index_select, index, scatter through
// one indexing shader family), src/api/ops/shape.cpp (flip, roll), src/api/ops/reduce.cpp (prod). Here every selection is
// reduced to "pick rows of a 2-D table": the selected dimension is moved first and the rest is folded into the row, which
// is what tvk_embedding_forward does at full bandwidth; the adjoint is tvk_embedding_backward, which sums the rows of each
// index in a fixed order (no atomics). Element-wise selections (gather) use rows of one element through flat indices: they
// are correct for any shape but are not a tuned path. Floating tensors only; integer tables raise.
#include "common.h"

namespace tvk_aten {
namespace {

void require_table(const at::Tensor& t, const char* op) {
    if (!is_hot_float(t.scalar_type())) TVK_NOT_IMPLEMENTED(op, " for dtype ", t.scalar_type(), " on the vulkan device (floating tensors are supported)");
}
// selections only move values: integer, boolean and float64 tensors are gathered bit for bit
void require_gatherable(const at::Tensor& t, const char* op) {
    const at::ScalarType st = t.scalar_type();
    if (!(is_hot_float(st) || st == at::kLong || st == at::kInt || st == at::kBool || st == at::kByte || st == at::kDouble))
        TVK_NOT_IMPLEMENTED(op, " for dtype ", st, " on the vulkan device");
}
at::Tensor long_index(const at::Tensor& index, const char* op) {
    TORCH_CHECK(index.scalar_type() == at::kLong || index.scalar_type() == at::kInt, op, "(): Expected dtype int32/int64 for index");
    return index.scalar_type() == at::kLong ? index : index.to(at::kLong);
}
at::Tensor& into(at::Tensor& out, const at::Tensor& value) {
    if (out.sizes() != value.sizes()) out.resize_(value.sizes());
    out.copy_(value);
    return out;
}

// rows of self along `dim` picked by a Long tensor of any shape: result shape = self[:dim] + index.shape + self[dim+1:]
at::Tensor take_along(const at::Tensor& self, int64_t dim, const at::Tensor& index) {
    const int64_t n = self.size(dim);
    int64_t rest = 1;
    std::vector<int64_t> moved_shape(index.sizes().begin(), index.sizes().end());
    for (int64_t d = 0; d < self.dim(); ++d)
        if (d != dim) { moved_shape.push_back(self.size(d)); rest *= self.size(d); }
    if (n == 0 || rest == 0 || index.numel() == 0) {                 // nothing to gather (an index into an empty dimension must be empty)
        TORCH_CHECK(index.numel() == 0 || n > 0, "index out of range in self");
        std::vector<int64_t> shape;
        for (int64_t d = 0; d < dim; ++d) shape.push_back(self.size(d));
        for (int64_t d = 0; d < index.dim(); ++d) shape.push_back(index.size(d));
        for (int64_t d = dim + 1; d < self.dim(); ++d) shape.push_back(self.size(d));
        return at::empty(shape, self.options());
    }
    at::Tensor table = contiguous_vulkan(self.movedim(dim, 0)).reshape({n, rest});
    // The row gather copies bits, so integer and boolean tables ride it as fp32 words: Int as it is, Long as two words per
    // element, Bool / Byte widened to Int first (exact) and narrowed afterwards.
    const at::ScalarType st = self.scalar_type();
    at::Tensor rows;
    if (is_hot_float(st)) {
        rows = at::embedding(table, index.reshape({-1}));
    } else {
        const at::ScalarType word = (st == at::kLong || st == at::kDouble) ? st : at::kInt;
        at::Tensor words = (word == st ? table : table.to(at::kInt)).view(at::kFloat);
        rows = at::embedding(words, index.reshape({-1})).view(word);
        if (word != st) rows = rows.to(st);
    }
    rows = rows.reshape(moved_shape);                                                       // [index..., rest...]
    // bring the index dimensions back to position dim
    const int64_t k = index.dim(), nd = (int64_t)moved_shape.size();
    std::vector<int64_t> perm;
    for (int64_t d = 0; d < dim; ++d) perm.push_back(k + d);
    for (int64_t d = 0; d < k; ++d) perm.push_back(d);
    for (int64_t d = k + dim; d < nd; ++d) perm.push_back(d);
    return contiguous_vulkan(rows.permute(perm));
}
// the adjoint: a zero tensor of `sizes` with the slices of `source` (shaped like take_along's result) added at index
at::Tensor add_along(at::IntArrayRef sizes, int64_t dim, const at::Tensor& index, const at::Tensor& source) {
    const int64_t n = sizes[dim], k = index.dim(), nd = source.dim();
    std::vector<int64_t> perm;                                   // source -> [index..., rest...]
    for (int64_t d = 0; d < k; ++d) perm.push_back(dim + d);
    for (int64_t d = 0; d < dim; ++d) perm.push_back(d);
    for (int64_t d = dim + k; d < nd; ++d) perm.push_back(d);
    int64_t rest = 1;
    std::vector<int64_t> moved_sizes{n};
    for (int64_t d = 0; d < (int64_t)sizes.size(); ++d)
        if (d != dim) { rest *= sizes[d]; moved_sizes.push_back(sizes[d]); }
    if (n == 0 || rest == 0 || index.numel() == 0) return at::zeros(sizes, source.options());
    at::Tensor g = contiguous_vulkan(source.permute(perm)).reshape({index.numel(), rest});
    at::Tensor table = at::embedding_dense_backward(g, index.reshape({-1}), n, -1, false);      // [n, rest]
    return contiguous_vulkan(table.reshape(moved_sizes).movedim(0, dim));
}

at::Tensor vk_index_select(const at::Tensor& self, int64_t dim, const at::Tensor& index_in) {
    require_gatherable(self, "index_select");
    TORCH_CHECK(index_in.dim() <= 1, "index_select(): Index is supposed to be a vector, but got dim: ", index_in.dim());
    at::Tensor index = long_index(index_in, "index_select");
    if (self.dim() == 0) {
        TORCH_CHECK(index.numel() == 1, "index_select(): Index to scalar can have only 1 value, got ", index.numel(), " value(s)");
        return self.clone();
    }
    dim = at::maybe_wrap_dim(dim, self.dim());
    return take_along(self, dim, index.reshape({-1}));
}
at::Tensor& vk_index_select_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor& out) { return into(out, vk_index_select(self, dim, index)); }

at::Tensor vk_index_add(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, const at::Tensor& source, const at::Scalar& alpha) {
    require_table(self, "index_add");
    at::Tensor index = long_index(index_in, "index_add");
    dim = at::maybe_wrap_dim(dim, std::max<int64_t>(self.dim(), 1));
    if (self.dim() == 0) return self + source.reshape({}) * alpha;
    TORCH_CHECK(index.dim() <= 1 && source.dim() == self.dim() && source.size(dim) == index.numel(), "index_add(): source and index do not fit self along dim ", dim);
    at::Tensor delta = add_along(self.sizes(), dim, index.reshape({-1}), source.to(self.scalar_type()));
    return alpha.toDouble() == 1.0 ? self + delta : self + delta * alpha;
}
at::Tensor& vk_index_add_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& source, const at::Scalar& alpha, at::Tensor& out) {
    return into(out, vk_index_add(self, dim, index, source, alpha));
}
at::Tensor& vk_index_add_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& source, const at::Scalar& alpha) {
    self.copy_(vk_index_add(self, dim, index, source, alpha));
    return self;
}

// flat element offsets (into a contiguous tensor of `sizes`) of the elements gather / scatter address: index along dim,
// the running coordinate along every other dimension
at::Tensor flat_offsets(at::IntArrayRef sizes, int64_t dim, const at::Tensor& index) {
    const int64_t nd = (int64_t)sizes.size();
    std::vector<int64_t> strides(nd, 1);
    for (int64_t d = nd - 2; d >= 0; --d) strides[d] = strides[d + 1] * sizes[d + 1];
    at::Tensor flat = index * strides[dim];
    for (int64_t d = 0; d < nd; ++d) {
        if (d == dim) continue;
        std::vector<int64_t> view(nd, 1);
        view[d] = index.size(d);
        at::Tensor coord = at::arange(index.size(d), at::TensorOptions().dtype(at::kLong).device(at::kCPU)).mul_(strides[d]).to(index.device());
        flat = flat + coord.view(view);
    }
    return flat;
}
at::Tensor vk_gather(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, bool) {
    require_gatherable(self, "gather");
    at::Tensor index = long_index(index_in, "gather");
    if (self.dim() == 0) return self.expand(index.sizes()).clone();
    dim = at::maybe_wrap_dim(dim, self.dim());
    TORCH_CHECK(index.dim() == self.dim(), "Index tensor must have the same number of dimensions as input tensor");
    for (int64_t d = 0; d < self.dim(); ++d)
        TORCH_CHECK(d == dim || index.size(d) <= self.size(d), "Size does not match at dimension ", d, " expected index ", index.sizes(), " to be no larger than self ", self.sizes(), " apart from dimension ", dim);
    if (index.numel() == 0) return at::empty(index.sizes(), self.options());
    at::Tensor flat = flat_offsets(self.sizes(), dim, index);
    return take_along(contiguous_vulkan(self).reshape({-1}), 0, flat.reshape({-1})).reshape(index.sizes());
}
at::Tensor& vk_gather_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, bool sparse_grad, at::Tensor& out) { return into(out, vk_gather(self, dim, index, sparse_grad)); }

at::Tensor vk_scatter_add(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, const at::Tensor& src) {
    require_table(self, "scatter_add");
    at::Tensor index = long_index(index_in, "scatter_add");
    if (index.numel() == 0) return self.clone();
    dim = at::maybe_wrap_dim(dim, std::max<int64_t>(self.dim(), 1));
    TORCH_CHECK(self.dim() > 0 && index.dim() == self.dim() && src.dim() == self.dim(), "scatter_add(): self, index and src must have the same number of dimensions");
    at::Tensor flat = flat_offsets(self.sizes(), dim, index);
    at::Tensor s = src;
    for (int64_t d = 0; d < src.dim(); ++d) s = s.narrow(d, 0, index.size(d));              // only the part of src the index covers is read
    at::Tensor delta = at::embedding_dense_backward(contiguous_vulkan(s.to(self.scalar_type())).reshape({-1, 1}), flat.reshape({-1}), self.numel(), -1, false);
    return self + delta.reshape(self.sizes());
}
at::Tensor& vk_scatter_add_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src, at::Tensor& out) {
    return into(out, vk_scatter_add(self, dim, index, src));
}
at::Tensor& vk_scatter_add_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src) {
    self.copy_(vk_scatter_add(self, dim, index, src));
    return self;
}

// scatter of a source tensor: the addressed elements take the source value, the others keep self. It is built from two
// additive scatters (the values and a hit count); where several source elements address one position, for which ATen
// promises no particular winner, the result is their mean.
at::Tensor vk_scatter_src(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, const at::Tensor& src) {
    require_table(self, "scatter");
    at::Tensor index = long_index(index_in, "scatter");
    if (index.numel() == 0) return self.clone();
    TORCH_CHECK(src.scalar_type() == self.scalar_type(), "scatter(): Expected self.dtype to be equal to src.dtype");
    at::Tensor zero = at::zeros_like(self, at::MemoryFormat::Contiguous);
    at::Tensor count = vk_scatter_add(zero, dim, index, at::ones(index.sizes(), self.options()));
    at::Tensor sum = vk_scatter_add(zero, dim, index, src);
    return at::where(at::gt(count, 0), sum / at::clamp_min(count, 1.0), self);
}
at::Tensor& vk_scatter_src_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src, at::Tensor& out) {
    return into(out, vk_scatter_src(self, dim, index, src));
}
at::Tensor& vk_scatter_src_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src) {
    self.copy_(vk_scatter_src(self, dim, index, src));
    return self;
}

// index_copy: the slices of self named by index are replaced by the slices of source. Like scatter with a source it is two
// additive passes (values and a hit count); slices named more than once, for which ATen promises no winner, average.
at::Tensor vk_index_copy(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, const at::Tensor& source) {
    require_table(self, "index_copy");
    at::Tensor index = long_index(index_in, "index_copy");
    TORCH_CHECK(index.dim() <= 1, "index_copy_(): Index should have dimension 1 or 0, actual = ", index.dim());
    TORCH_CHECK(source.scalar_type() == self.scalar_type(), "index_copy_(): self and source expected to have the same dtype");
    if (index.numel() == 0) return self.clone();
    if (self.dim() == 0) return source.reshape({}).clone();
    dim = at::maybe_wrap_dim(dim, self.dim());
    at::Tensor idx = index.reshape({-1});
    TORCH_CHECK(source.dim() == self.dim() && source.size(dim) == idx.numel(), "index_copy_(): Number of indices (", idx.numel(), ") should be equal to source.size(dim)");
    at::Tensor zero = at::zeros_like(self, at::MemoryFormat::Contiguous);
    at::Tensor sum = zero.index_add(dim, idx, source), count = zero.index_add(dim, idx, at::ones_like(source));
    return at::where(at::gt(count, 0), sum / at::clamp_min(count, 1.0), self);
}
at::Tensor& vk_index_copy_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& source, at::Tensor& out) {
    return into(out, vk_index_copy(self, dim, index, source));
}
at::Tensor& vk_index_copy_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& source) {
    self.copy_(vk_index_copy(self, dim, index, source));
    return self;
}

// scatter of one value: out = self with `value` at the addressed elements. The addressed set is the union over the index
// entries along dim, found by comparing a coordinate ramp with each index slice (one_hot is the case of one slice).
at::Tensor vk_scatter_value(const at::Tensor& self, int64_t dim, const at::Tensor& index_in, const at::Scalar& value) {
    at::Tensor index = long_index(index_in, "scatter");
    dim = at::maybe_wrap_dim(dim, std::max<int64_t>(self.dim(), 1));
    TORCH_CHECK(self.dim() > 0 && index.dim() == self.dim(), "scatter(): Index tensor must have the same number of dimensions as self tensor");
    for (int64_t d = 0; d < self.dim(); ++d)
        if (d != dim && index.size(d) != self.size(d)) TVK_NOT_IMPLEMENTED("scatter with an index smaller than self outside the scattered dimension");
    std::vector<int64_t> view(self.dim(), 1);
    view[dim] = self.size(dim);
    at::Tensor ramp = at::arange(self.size(dim), at::TensorOptions().dtype(at::kLong).device(at::kCPU)).to(self.device()).view(view);
    at::Tensor hit;
    for (int64_t j = 0; j < index.size(dim); ++j) {
        at::Tensor h = at::eq(ramp, index.narrow(dim, j, 1));
        hit = hit.defined() ? at::logical_or(hit, h) : h;
    }
    if (!hit.defined()) return self.clone();
    at::Tensor result;
    if (is_hot_float(self.scalar_type())) {
        at::Tensor v = at::empty({}, self.options());
        v.fill_(value);
        return at::where(hit, v, self);
    }
    // integer tensors (one_hot builds a Long tensor): out = self * (1 - hit) + value * hit in 64-bit integers
    TORCH_CHECK(self.scalar_type() == at::kLong || self.scalar_type() == at::kInt, "torchvulkan [NOT IMPLEMENTED]: scatter for dtype ", self.scalar_type());
    at::Tensor h = hit.to(self.scalar_type());
    return self - self * h + h * value;
}
at::Tensor& vk_scatter_value_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Scalar& value, at::Tensor& out) {
    return into(out, vk_scatter_value(self, dim, index, value));
}
at::Tensor& vk_scatter_value_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Scalar& value) {
    self.copy_(vk_scatter_value(self, dim, index, value));
    return self;
}

// Row-major positions of the true entries of a boolean mask, as a Long vector. The count is read back (the length depends
// on the data: one synchronisation, as on any backend); the selection stays on the device: a stable sort of the negated
// mask lists the selected positions first and in order.
at::Tensor selected_positions(const at::Tensor& mask) {
    at::Tensor m = contiguous_vulkan(mask).reshape({-1});
    const int64_t count = m.numel() ? m.sum().item<int64_t>() : 0;
    if (count == 0) return at::empty({0}, mask.options().dtype(at::kLong));
    at::Tensor order = std::get<1>(at::sort(at::logical_not(m).to(at::kFloat), /*stable=*/true, /*dim=*/0, /*descending=*/false));
    return order.narrow(0, 0, count);
}
// self with the dimensions a mask at position pos covers folded into one
at::Tensor fold_masked_dims(const at::Tensor& self, int64_t pos, const at::Tensor& mask) {
    TORCH_CHECK(pos + mask.dim() <= self.dim(), "too many indices for tensor of dimension ", self.dim());
    std::vector<int64_t> shape;
    for (int64_t d = 0; d < pos; ++d) shape.push_back(self.size(d));
    for (int64_t d = 0; d < mask.dim(); ++d)
        TORCH_CHECK(mask.size(d) == self.size(pos + d), "The shape of the mask ", mask.sizes(), " at index ", d, " does not match the shape of the indexed tensor ", self.sizes(),
                    " at index ", pos + d);
    shape.push_back(mask.numel());
    for (int64_t d = pos + mask.dim(); d < self.dim(); ++d) shape.push_back(self.size(d));
    return contiguous_vulkan(self).reshape(shape);
}

// x[idx]: one index tensor at one position, the others absent (basic slices are views taken before the call). A Long index
// picks slices along its dimension; a boolean mask picks the slices where it is true over the dimensions it covers.
int64_t single_index_position(const c10::List<c10::optional<at::Tensor>>& indices, at::Tensor* index) {
    int64_t pos = -1;
    for (size_t i = 0; i < indices.size(); ++i) {
        c10::optional<at::Tensor> t = indices.get(i);
        if (!t.has_value() || !t->defined()) continue;
        if (pos >= 0) TVK_NOT_IMPLEMENTED("indexing with more than one index tensor");
        pos = (int64_t)i;
        *index = *t;
    }
    TORCH_CHECK(pos >= 0, "index(): no index tensor");
    return pos;
}
at::Tensor vk_index_tensor(const at::Tensor& self, const c10::List<c10::optional<at::Tensor>>& indices) {
    require_gatherable(self, "index");
    at::Tensor index;
    const int64_t pos = single_index_position(indices, &index);
    if (index.scalar_type() == at::kBool || index.scalar_type() == at::kByte) {
        at::Tensor mask = (is_vulkan(index) ? index : index.to(self.device())).to(at::kBool);
        return take_along(fold_masked_dims(self, pos, mask), pos, selected_positions(mask));
    }
    index = long_index(index, "index");
    at::Tensor idx = is_vulkan(index) ? index : index.to(self.device());
    // negative indices count from the end
    idx = at::where(at::lt(idx, 0), idx + self.size(pos), idx);
    return take_along(self, pos, idx);
}
at::Tensor& vk_index_tensor_out(const at::Tensor& self, const c10::List<c10::optional<at::Tensor>>& indices, at::Tensor& out) { return into(out, vk_index_tensor(self, indices)); }
at::Tensor& vk_index_put_impl_(at::Tensor& self, const c10::List<c10::optional<at::Tensor>>& indices, const at::Tensor& values, bool accumulate, bool) {
    require_table(self, "index_put_");
    at::Tensor index;
    const int64_t pos = single_index_position(indices, &index);
    if (index.scalar_type() == at::kBool || index.scalar_type() == at::kByte) {
        at::Tensor mask = (is_vulkan(index) ? index : index.to(self.device())).to(at::kBool);
        if (!accumulate) {
            // x[mask] = value with one value: a masked fill (the mask is aligned to the dimensions it covers)
            if (values.numel() != 1) TVK_NOT_IMPLEMENTED("assignment of more than one value through a boolean mask");
            std::vector<int64_t> view(self.dim(), 1);
            TORCH_CHECK(pos + mask.dim() <= self.dim(), "too many indices for tensor of dimension ", self.dim());
            for (int64_t d = 0; d < mask.dim(); ++d) view[pos + d] = mask.size(d);
            self.masked_fill_(mask.reshape(view), values.reshape({}).to(self.scalar_type()));
            return self;
        }
        at::Tensor rows = selected_positions(mask);
        at::Tensor folded = fold_masked_dims(self, pos, mask);
        std::vector<int64_t> shape(folded.sizes().begin(), folded.sizes().end());
        shape[pos] = rows.numel();
        at::Tensor delta = add_along(folded.sizes(), pos, rows, values.to(self.scalar_type()).expand(shape));
        self.add_(delta.reshape(self.sizes()));
        return self;
    }
    index = long_index(index, "index_put_");
    at::Tensor idx = is_vulkan(index) ? index : index.to(self.device());
    idx = at::where(at::lt(idx, 0), idx + self.size(pos), idx);
    std::vector<int64_t> shape;
    for (int64_t d = 0; d < pos; ++d) shape.push_back(self.size(d));
    for (int64_t d = 0; d < idx.dim(); ++d) shape.push_back(idx.size(d));
    for (int64_t d = pos + 1; d < self.dim(); ++d) shape.push_back(self.size(d));
    at::Tensor src = values.to(self.scalar_type()).expand(shape);
    at::Tensor delta = add_along(self.sizes(), pos, idx, src);
    if (accumulate) {
        self.add_(delta);
        return self;
    }
    // assignment: the addressed slices take the new values, the others stay. (An index that names a slice twice is left
    // undefined by ATen - one of the values wins; here they add up.)
    std::vector<int64_t> view(self.dim(), 1);
    view[pos] = self.size(pos);
    at::Tensor hit = at::gt(add_along({self.size(pos)}, 0, idx.reshape({-1}), at::ones({idx.numel()}, self.options())), 0).view(view);
    self.copy_(at::where(hit, delta, self));
    return self;
}

// ---- masked_select ------------------------------------------------------------------------------
// The elements of self where mask is true, in row-major order (selected_positions, then a row gather). Printing a floating
// tensor goes through this: torch's formatter selects the finite non-zero values.
at::Tensor vk_masked_select(const at::Tensor& self, const at::Tensor& mask) {
    require_gatherable(self, "masked_select");
    TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_select: expected BoolTensor for mask");
    const auto shape = at::infer_size(self.sizes(), mask.sizes());
    at::Tensor xs = contiguous_vulkan(self.expand(shape)).reshape({-1});
    if (xs.numel() == 0) return at::empty({0}, self.options());
    at::Tensor rows = selected_positions(mask.expand(shape));
    if (rows.numel() == 0) return at::empty({0}, self.options());
    return take_along(xs, 0, rows);
}
at::Tensor& vk_masked_select_out(const at::Tensor& self, const at::Tensor& mask, at::Tensor& out) { return into(out, vk_masked_select(self, mask)); }

// nonzero: the positions from selected_positions, unravelled into one column per dimension with exact integer division
at::Tensor vk_nonzero(const at::Tensor& self) {
    at::Tensor mask = self.scalar_type() == at::kBool ? self : at::ne(self, 0);
    at::Tensor flat = selected_positions(mask);
    const int64_t nd = self.dim();
    if (nd == 0) return at::empty({flat.numel(), 0}, flat.options());
    std::vector<at::Tensor> cols(nd);
    at::Tensor rest = flat;
    for (int64_t d = nd - 1; d >= 0; --d) {
        const int64_t size = std::max<int64_t>(self.size(d), 1);
        cols[d] = at::remainder(rest, size);
        rest = at::floor_divide(rest, size);
    }
    return at::stack(cols, 1);
}
at::Tensor& vk_nonzero_out(const at::Tensor& self, at::Tensor& out) { return into(out, vk_nonzero(self)); }

// ---- flip, roll --------------------------------------------------------------------------------
at::Tensor vk_flip(const at::Tensor& self, at::IntArrayRef dims) {
    require_gatherable(self, "flip");
    at::Tensor r = self;
    for (int64_t d : dims) {
        d = at::maybe_wrap_dim(d, self.dim());
        const int64_t n = self.size(d);
        if (n <= 1) continue;
        at::Tensor rev = at::arange(n - 1, -1, -1, at::TensorOptions().dtype(at::kLong).device(at::kCPU)).to(self.device());
        r = take_along(r, d, rev);
    }
    return r.is_same(self) ? self.clone() : r;
}
at::Tensor vk_roll(const at::Tensor& self, at::IntArrayRef shifts, at::IntArrayRef dims) {
    if (dims.empty()) {
        TORCH_CHECK(shifts.size() == 1, "roll(): without dims, shifts must be one number");
        return vk_roll(contiguous_vulkan(self).reshape({-1}), shifts, {0}).reshape(self.sizes());
    }
    TORCH_CHECK(shifts.size() == dims.size(), "shifts and dimensions must align. shifts: ", shifts.size(), ", dims:", dims.size());
    at::Tensor r = self;
    for (size_t i = 0; i < dims.size(); ++i) {
        const int64_t d = at::maybe_wrap_dim(dims[i], self.dim()), n = self.size(d);
        if (n == 0) continue;
        const int64_t s = ((shifts[i] % n) + n) % n;
        if (s == 0) continue;
        r = at::cat({r.narrow(d, n - s, s), r.narrow(d, 0, n - s)}, d);
    }
    return r.is_same(self) ? self.clone() : r;
}

// ---- prod, equal ---------------------------------------------------------------------------------
// the running product's last element (cumprod is the scan kernel with fp32 accumulation)
at::Tensor vk_prod_dim(const at::Tensor& self, int64_t dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
    require_table(self, "prod");
    at::Tensor x = dtype.has_value() ? self.to(*dtype) : self;
    if (x.dim() == 0) return x.clone();
    dim = at::maybe_wrap_dim(dim, x.dim());
    if (x.size(dim) == 0) {
        std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
        shape[dim] = 1;
        at::Tensor one = at::ones(shape, x.options());
        return keepdim ? one : one.squeeze(dim);
    }
    at::Tensor last = at::cumprod(x, dim).narrow(dim, x.size(dim) - 1, 1);
    return contiguous_vulkan(keepdim ? last : last.squeeze(dim));
}
at::Tensor vk_prod_all(const at::Tensor& self, c10::optional<at::ScalarType> dtype) {
    return vk_prod_dim(contiguous_vulkan(self).reshape({-1}), 0, false, dtype);
}
at::Tensor& vk_prod_int_out(const at::Tensor& self, int64_t dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    return into(out, vk_prod_dim(self, dim, keepdim, dtype));
}
// k-th smallest value along dim and its index (k counts from 1): the k-th column of the sort. median = the lower middle one.
std::tuple<at::Tensor, at::Tensor> vk_kthvalue(const at::Tensor& self, int64_t k, int64_t dim, bool keepdim) {
    require_table(self, "kthvalue");
    at::Tensor x = self.dim() == 0 ? self.reshape({1}) : self;
    dim = at::maybe_wrap_dim(dim, x.dim());
    TORCH_CHECK(k >= 1 && k <= x.size(dim), "kthvalue(): selected number k out of range for dimension ", dim);
    at::Tensor values, indices;
    std::tie(values, indices) = at::sort(x, /*stable=*/true, dim, false);
    values = contiguous_vulkan(values.narrow(dim, k - 1, 1));
    indices = contiguous_vulkan(indices.narrow(dim, k - 1, 1));
    if (self.dim() == 0) return {values.reshape({}), indices.reshape({})};
    if (!keepdim) return {values.squeeze(dim), indices.squeeze(dim)};
    return {values, indices};
}
std::tuple<at::Tensor, at::Tensor> vk_median_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
    const int64_t n = self.dim() == 0 ? 1 : self.size(at::maybe_wrap_dim(dim, self.dim()));
    TORCH_CHECK(n > 0, "median(): Expected reduction dim ", dim, " to have non-zero size.");
    return vk_kthvalue(self, (n + 1) / 2, dim, keepdim);
}
at::Tensor vk_median(const at::Tensor& self) {
    TORCH_CHECK(self.numel() > 0, "median(): cannot compute the median of an empty tensor");
    return std::get<0>(vk_median_dim(contiguous_vulkan(self).reshape({-1}), 0, false));
}

bool vk_equal(const at::Tensor& a, const at::Tensor& b) {
    if (a.sizes() != b.sizes()) return false;
    if (a.numel() == 0) return true;
    return at::eq(a, b).all().item<bool>();
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("index_select", &vk_index_select);
    m.impl("index_select.out", &vk_index_select_out);
    m.impl("index_add", &vk_index_add);
    m.impl("index_add.out", &vk_index_add_out);
    m.impl("index_add_", &vk_index_add_);
    m.impl("gather", &vk_gather);
    m.impl("gather.out", &vk_gather_out);
    m.impl("scatter_add", &vk_scatter_add);
    m.impl("scatter_add.out", &vk_scatter_add_out);
    m.impl("scatter_add_", &vk_scatter_add_);
    m.impl("index_copy", &vk_index_copy);
    m.impl("index_copy.out", &vk_index_copy_out);
    m.impl("index_copy_", &vk_index_copy_);
    m.impl("scatter.src", &vk_scatter_src);
    m.impl("scatter.src_out", &vk_scatter_src_out);
    m.impl("scatter_.src", &vk_scatter_src_);
    m.impl("scatter.value", &vk_scatter_value);
    m.impl("scatter.value_out", &vk_scatter_value_out);
    m.impl("scatter_.value", &vk_scatter_value_);
    m.impl("index.Tensor", &vk_index_tensor);
    m.impl("index.Tensor_out", &vk_index_tensor_out);
    m.impl("_index_put_impl_", &vk_index_put_impl_);
    m.impl("nonzero", &vk_nonzero);
    m.impl("nonzero.out", &vk_nonzero_out);
    m.impl("masked_select", &vk_masked_select);
    m.impl("masked_select.out", &vk_masked_select_out);
    m.impl("flip", &vk_flip);
    m.impl("roll", &vk_roll);
    m.impl("prod", &vk_prod_all);
    m.impl("prod.dim_int", &vk_prod_dim);
    m.impl("prod.int_out", &vk_prod_int_out);
    m.impl("equal", &vk_equal);
    m.impl("kthvalue", &vk_kthvalue);
    m.impl("median", &vk_median);
    m.impl("median.dim", &vk_median_dim);
}

}  // namespace tvk_aten
