"""BASELINE config 2 (MLP fwd+bwd fp16 + AdamW) through the C-ABI against the fp64 oracle.

Bar: relative Frobenius error <= 1e-2 for every fp16 result (loss, logits, each gradient, each
parameter after the step) against the oracle evaluated in float64 on the same fp16 parameter and
input values.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_fro

pytestmark = pytest.mark.gpu


def f64(t):
    return t.detach().float().cpu().double().numpy()


def run(cuda, sizes, batch, seed=0, fused=False, fuse_forward=False):
    from torchvulkan_b200.workloads import MLPStep

    step = MLPStep(sizes=sizes, batch=batch, dtype=torch.float16, device=cuda, seed=seed, fused=fused, fuse_forward=fuse_forward)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, sizes[0], generator=g).half()
    labels = torch.randint(0, sizes[-1], (batch,), generator=g)
    w0 = [f64(w) for w in step.w]
    b0 = [f64(b) for b in step.b]
    loss = step.forward_backward(x.to(cuda), labels.to(cuda))
    from torchvulkan_b200 import cuda_ops
    cuda_ops.check_device_status()
    rl, rlogits, rgw, rgb = oracle.mlp_step(f64(x), labels.numpy(), w0, b0)
    assert abs(float(loss) - rl) / abs(rl) <= 1e-2
    assert rel_fro(f64(step.z[-1]), rlogits) <= 1e-2
    for i in range(step.nl):
        assert rel_fro(f64(step.gw[i]), rgw[i]) <= 1e-2, f"grad W{i}"
        assert rel_fro(f64(step.gb[i]), rgb[i]) <= 1e-2, f"grad b{i}"
    # AdamW from the device's own gradients (so the check isolates the optimizer arithmetic)
    grads = [t.clone() for t in step.grads]
    params0 = [p.clone() for p in step.params]
    step.optimizer_step()
    for p0, g_, p1 in zip(params0, grads, step.params):
        rp, _, _ = oracle.adam_step(p0.float().cpu().numpy(), g_.float().cpu().numpy(), 0.0 * p0.float().cpu().numpy(),
                                    0.0 * p0.float().cpu().numpy(), 1)
        # the update is ~lr per element: compare the change, not only the value
        d_ref = rp.astype(np.float64) - f64(p0)
        d_got = f64(p1) - f64(p0)
        assert rel_fro(f64(p1), rp) <= 1e-3
        assert np.max(np.abs(d_got - d_ref)) <= 1e-3 * 1.5  # one fp16 ulp of the parameter scale at most
    return step


def test_mlp_step_small(cuda):
    run(cuda, (72, 136, 136, 10), 48)


@pytest.mark.parametrize("sizes,batch", [((72, 136, 136, 10), 48), ((784, 8192, 8192, 10), 256)])
def test_mlp_step_with_fused_epilogues(cuda, sizes, batch):
    """The step with gelu written by the addmm epilogue and gelu_backward applied by the input-gradient epilogue: the same
    bars against the fp64 oracle, a launch count four lower, and results that stay within fp16 rounding of the step issued
    operator by operator (the fused input gradient skips one rounding to fp16)."""
    fused = run(cuda, sizes, batch, fused=True, fuse_forward=True)
    run(cuda, sizes, batch, fused=True)
    plain = run(cuda, sizes, batch, fused=False)
    saved = sum(fused._fused_fwd) + sum(fused._fused_bwd) + 2      # and the cross-entropy: two launches instead of four
    assert fused.launches_per_step == plain.launches_per_step - saved and saved >= (5 if batch == 256 else 4)
    for a, b in zip(fused.h, plain.h):
        # gelu of the fp32 accumulator against gelu of its fp16 rounding: one rounding apart
        assert rel_fro(f64(a), f64(b)) <= 1e-3
    for a, b in zip(fused.grads, plain.grads):
        # gradients of a mean loss over the batch sit in fp16's subnormal range (spacing 6e-8 at values of 1e-5): the two
        # orders of rounding differ by that quantisation; both are held to 1e-2 against the fp64 oracle by run()
        assert rel_fro(f64(a), f64(b)) <= 1e-2


def test_mlp_step_config2(cuda):
    step = run(cuda, (784, 8192, 8192, 10), 256)
    assert step.num_params() == 73_629_706
    assert step.gemm_flops() == 109_781_712_896


@pytest.mark.parametrize("sizes,batch", [((72, 136, 136, 10), 48), ((784, 8192, 8192, 10), 256)])
def test_graph_replay_matches_eager_steps(cuda, sizes, batch):
    """Three steps issued launch by launch (one Adam launch per tensor, host step count) and three replays of a
    captured step (one list launch, step count in device memory) end with the same bits."""
    from torchvulkan_b200 import cuda_ops
    from torchvulkan_b200.workloads import MLPStep

    eager = MLPStep(sizes=sizes, batch=batch, dtype=torch.float16, device=cuda, seed=3)
    graph = MLPStep(sizes=sizes, batch=batch, dtype=torch.float16, device=cuda, seed=3, list_optimizer=True)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(batch, sizes[0], generator=g).half().to(cuda)
    labels = torch.randint(0, sizes[-1], (batch,), generator=g).to(cuda)
    for _ in range(3):
        eager.step(x, labels)
    graph.step(x, labels)                     # one ordinary step first, then capture and replay two more
    torch.cuda.synchronize()
    graph.capture(x, labels)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    cuda_ops.check_device_status()
    assert graph.step_count == 3 and float(graph.step_dev) == 3.0
    assert torch.equal(graph.loss, eager.loss)
    for a, b in zip(graph.params, eager.params):
        assert torch.equal(a, b)
    for a, b in zip(graph.m + graph.v, eager.m + eager.v):
        assert torch.equal(a, b)
