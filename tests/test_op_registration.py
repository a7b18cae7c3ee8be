"""CPU-only check of the ATen extension's operator table: every operator a script on the "vulkan" device is documented to
reach must resolve for the PrivateUse1 key, either to a kernel of this backend, to one of ATen's composite kernels (which
decompose into operators that are checked here too), or, for structured operators, through the registered out= variant.
No tensor is created on the device, so this runs without a GPU and catches a registration that was lost or misspelt."""
import pytest
import torch


def _resolves(name):
    C = torch._C
    has = C._dispatch_has_kernel_for_dispatch_key
    if has(name, "PrivateUse1") or has(name, "CompositeImplicitAutograd") or has(name, "CompositeExplicitAutograd"):
        return True
    if has(name, "CompositeExplicitAutogradNonFunctional"):          # structured: the functional form writes through out=
        base, _, overload = name.partition(".")
        base = base[:-1] if base.endswith("_") and not base.endswith("__") else base
        for cand in (base + ".out", f"{base}.{overload}_out" if overload else None, f"{base}.out_{overload}" if overload else None):
            if cand and has(cand, "PrivateUse1"):
                return True
    return False


OPERATORS = """
mm bmm addmm baddbmm addmv dot vdot matmul linear _scaled_mm convolution_overrideable convolution_backward_overrideable
_scaled_dot_product_fused_attention_overrideable _scaled_dot_product_fused_attention_overrideable_backward
_native_multi_head_attention _transformer_encoder_layer_fwd _nested_tensor_from_mask_left_aligned
native_layer_norm native_layer_norm_backward native_group_norm native_group_norm_backward native_batch_norm native_batch_norm_backward
_softmax _softmax_backward_data _log_softmax _log_softmax_backward_data nll_loss_forward nll_loss_backward nll_loss2d_forward nll_loss2d_backward
embedding embedding_dense_backward _embedding_bag _embedding_bag_forward_only _embedding_bag_backward _embedding_bag_per_sample_weights_backward
native_dropout native_dropout_backward uniform_ normal_ bernoulli_.float bernoulli_.Tensor exponential_ multinomial normal.Tensor_Tensor normal.Tensor_float normal.float_Tensor
add.Tensor sub.Tensor mul.Tensor div.Tensor pow.Tensor_Tensor pow_.Tensor pow.Tensor_Scalar pow.Scalar maximum minimum atan2 fmod.Tensor remainder.Tensor
relu gelu gelu_backward silu silu_backward sigmoid tanh exp log sqrt rsqrt abs neg erf erfinv sin cos floor ceil round trunc sign sgn
eq.Tensor ne.Tensor lt.Tensor le.Tensor gt.Tensor ge.Tensor eq.Scalar logical_and logical_or logical_not logical_xor isnan where.self
clamp clamp_min clamp_max lerp.Tensor lerp.Scalar addcmul addcdiv masked_fill_.Scalar masked_fill_.Tensor fill_.Scalar
sum.dim_IntList mean.dim amax amin aminmax prod.dim_int var.correction std.correction argmax argmin max.dim min.dim all.dim any.dim nansum
cumsum cumprod logcumsumexp _cummax_helper _cummin_helper sort topk kthvalue median _unique2 bincount
index_select gather scatter_add scatter.value scatter.src index_add index_copy index.Tensor index_put_ masked_select nonzero flip roll cat
tril triu tril_indices triu_indices arange.start_out linspace.out eye.m_out
max_pool2d_with_indices max_pool2d_with_indices_backward avg_pool2d avg_pool2d_backward
max_pool3d_with_indices max_pool3d_with_indices_backward avg_pool3d avg_pool3d_backward
_adaptive_avg_pool2d _adaptive_avg_pool2d_backward adaptive_max_pool2d adaptive_max_pool2d_backward _adaptive_avg_pool3d _adaptive_avg_pool3d_backward max_unpool2d
upsample_nearest1d upsample_nearest2d upsample_nearest3d _upsample_nearest_exact2d upsample_linear1d upsample_bilinear2d upsample_trilinear3d
upsample_bilinear2d_backward upsample_bicubic2d upsample_bicubic2d_backward grid_sampler_2d grid_sampler_2d_backward
reflection_pad1d reflection_pad2d reflection_pad3d replication_pad1d replication_pad2d replication_pad3d im2col col2im
_thnn_fused_lstm_cell _thnn_fused_gru_cell _weight_norm_interface _cdist_forward _cdist_backward bucketize.Tensor searchsorted.Tensor
linalg_vector_norm linalg_cross isin.Tensor_Tensor logit logit_backward channel_shuffle repeat_interleave.Tensor
mse_loss mse_loss_backward binary_cross_entropy binary_cross_entropy_backward smooth_l1_loss huber_loss
_amp_foreach_non_finite_check_and_unscale_ _amp_update_scale_ _fused_adam_ _fused_adamw_ _fused_sgd_
_local_scalar_dense _copy_from empty.memory_format empty_strided as_strided view _reshape_alias resize_
""".split()


@pytest.fixture(scope="module")
def backend():
    import torchvulkan  # noqa: F401  (loads the extension; registering the device needs no GPU)

    assert torch._C._get_privateuse1_backend_name() == "vulkan"


@pytest.mark.parametrize("op", OPERATORS)
def test_operator_resolves_on_the_device_key(backend, op):
    name = "aten::" + op
    assert name in set(torch._C._dispatch_get_all_op_names()), f"{name} is not an ATen operator of this PyTorch"
    assert _resolves(name), f"{name} has no kernel for the vulkan (PrivateUse1) key"
