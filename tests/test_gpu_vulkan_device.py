"""The reference-facing surface: `import torchvulkan`, tensors on the "vulkan" device, ATen ops
dispatched to the B200 kernels. Mirrors the reference's own strategy (tests/test_pytorch_ops.py):
run on the device and on ATen CPU from the same seeded inputs and compare with its tolerance ladder
(fp16/bf16 matmul-like atol=1e-1 rtol=3e-1 at most; here the tighter BASELINE bars are used:
relative Frobenius 1e-2 for half types, 1e-4 for fp32, exact for indices)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_fro

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vk(cuda):
    import torchvulkan

    assert torchvulkan.is_available() and torchvulkan.device_count() >= 1
    return torch.device("vulkan:0")


def close(dev_t, cpu_t, tol):
    a = dev_t.detach().cpu().double().numpy()
    b = cpu_t.detach().double().numpy()
    assert a.shape == b.shape, (a.shape, b.shape)
    assert rel_fro(a, b) <= tol, rel_fro(a, b)


def test_module_api(vk):
    import torchvulkan

    assert torch.vulkan is torchvulkan or torch.vulkan.is_available()
    p = torchvulkan.get_device_properties(0)
    assert "B200" in p.name and p.subgroup_size == 32 and p.has_fp16 and p.has_bf16
    torchvulkan.synchronize()
    before = torchvulkan.memory_allocated()
    t = torch.empty(1 << 20, device=vk)
    assert torchvulkan.memory_allocated() >= before + (4 << 20)
    assert torchvulkan.max_memory_allocated() >= torchvulkan.memory_allocated()
    del t
    assert torchvulkan.memory_allocated() == before
    assert torchvulkan.memory_reserved() >= before
    torchvulkan.empty_cache()
    free, total = torchvulkan.mem_get_info()
    assert 0 < free <= total
    torchvulkan.manual_seed(7)
    assert torchvulkan.initial_seed() == 7
    assert torch.ones(2).vulkan().is_vulkan and torch.ones(2, device=vk).device.type == "vulkan"


def test_copies_views_casts(vk):
    x = torch.randn(37, 53)
    d = x.to(vk)
    assert torch.equal(d.cpu(), x)
    assert torch.equal(d.t().cpu(), x.t())                       # strided device -> host
    assert torch.equal(d[3:20:2, 1::3].contiguous().cpu(), x[3:20:2, 1::3])
    assert torch.equal(d.view(53, 37).cpu(), x.view(53, 37))
    assert torch.equal(d.half().cpu(), x.half()) and torch.equal(d.to(torch.bfloat16).cpu(), x.to(torch.bfloat16))
    assert torch.equal(d.to(torch.int64).cpu(), x.to(torch.int64))
    e = torch.empty(53, 37, device=vk)
    e.copy_(d.t())
    assert torch.equal(e.cpu(), x.t())
    e.t().copy_(x)                                                # host -> strided device
    assert torch.equal(e.cpu(), x.t())
    assert d[5, 7].item() == x[5, 7].item()
    assert torch.equal(d.clone().cpu(), x) and torch.equal(torch.zeros(5, device=vk).cpu(), torch.zeros(5))
    assert torch.equal(torch.full((3, 4), 2.5, device=vk).cpu(), torch.full((3, 4), 2.5))
    i = torch.arange(10).to(vk)
    i += 1
    assert torch.equal(i.cpu(), torch.arange(10) + 1)


def test_config1_script(vk):
    """README-style script: seeded CPU inputs, .to('vulkan'), (x @ y).relu().sum()."""
    torch.manual_seed(0)
    x, y = torch.randn(1024, 1024), torch.randn(1024, 1024)
    z = (x.to(vk) @ y.to(vk)).relu()
    s = z.sum().item()
    ref = (x.double() @ y.double()).relu()
    assert abs(s - ref.sum().item()) / ref.sum().item() <= 1e-4
    assert torch.allclose(z.cpu(), (x @ y).relu(), atol=1e-4, rtol=1e-3)   # tests/test_pytorch_ops.py:322-327


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3), (torch.bfloat16, 1e-2)])
def test_elementwise_ops(vk, dtype, tol):
    torch.manual_seed(1)
    a, b = torch.randn(33, 65).to(dtype), torch.randn(33, 65).to(dtype)
    row = torch.randn(65).to(dtype)
    da, db, drow = a.to(vk), b.to(vk), row.to(vk)
    f = lambda t: t.float()  # noqa: E731
    close(da + db, f(a) + f(b), tol); close(da - db * 2, f(a) - f(b) * 2, tol); close(da * drow, f(a) * f(row), tol)
    close(da / (db.abs() + 1), f(a) / (f(b).abs() + 1), tol); close(torch.add(da, db, alpha=0.5), f(a) + 0.5 * f(b), tol)
    close(da * 3.0, f(a) * 3.0, tol); close(2.0 - da, 2.0 - f(a), tol); close(da.t() + db.t(), (f(a) + f(b)).t(), tol)
    close(torch.maximum(da, db), torch.maximum(f(a), f(b)), tol); close(da.pow(2), f(a).pow(2), tol)
    gelu_tanh = lambda t: F.gelu(t, approximate="tanh")  # noqa: E731
    for fn in (torch.exp, torch.sigmoid, torch.tanh, torch.relu, F.gelu, gelu_tanh, F.silu, torch.neg, torch.abs):
        close(fn(da), fn(f(a)), tol)
    xg, xc = da.clone().requires_grad_(), f(a).clone().requires_grad_()
    gelu_tanh(xg).backward(db); gelu_tanh(xc).backward(f(b))
    close(xg.grad, xc.grad, tol)
    close((da.abs() + 0.1).sqrt(), (f(a).abs() + 0.1).sqrt(), tol); close((da.abs() + 0.1).rsqrt(), (f(a).abs() + 0.1).rsqrt(), tol)
    close(torch.addcmul(da, db, drow, value=0.3), torch.addcmul(f(a), f(b), f(row), value=0.3), tol)
    close(torch.lerp(da, db, 0.25), torch.lerp(f(a), f(b), 0.25), tol)
    assert torch.equal((da > db).cpu(), a > b) and torch.equal((da == da).cpu(), a == a) and torch.equal((da <= 0.5).cpu(), a <= 0.5)
    assert torch.equal(torch.where(da > 0, da, db).cpu(), torch.where(a > 0, a, b))
    c = da.clone(); c += db; c *= 2; c.sub_(drow)
    close(c, ((f(a) + f(b)).to(dtype).float() * 2).to(dtype).float() - f(row), tol * 2)
    close(torch.cat([da, db], 1), torch.cat([a, b], 1).float(), 0)
    close(torch.cat([da, db], 0), torch.cat([a, b], 0).float(), 0)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3)])
def test_reductions_sort(vk, dtype, tol):
    torch.manual_seed(2)
    x = torch.randn(12, 34, 56).to(dtype)
    d = x.to(vk)
    f = x.float()
    close(d.sum(), f.sum(), tol * 10); close(d.sum(1), f.sum(1), tol); close(d.sum((0, 2)), f.sum((0, 2)), tol); close(d.mean((1, 2)), f.mean((1, 2)), tol)
    close(d.mean(-1, keepdim=True), f.mean(-1, keepdim=True), tol); close(d.amax(1), f.amax(1), 0); close(d.sum(0, dtype=torch.float32), f.sum(0), 1e-5)
    assert torch.equal(d.argmax().cpu(), x.argmax()) and torch.equal(d.argmax(1).cpu(), x.argmax(1)) and torch.equal(d.argmin(2, keepdim=True).cpu(), x.argmin(2, keepdim=True))
    v, i = torch.topk(d, 5, dim=1)
    rv, ri = torch.sort(x, dim=1, descending=True, stable=True)
    assert torch.equal(v.cpu(), rv[:, :5]) and torch.equal(i.cpu(), ri[:, :5])
    v, i = torch.sort(d, dim=-1, stable=True)
    rv, ri = torch.sort(x, dim=-1, stable=True)
    assert torch.equal(v.cpu(), rv) and torch.equal(i.cpu(), ri)


def test_nn_ops_forward_backward(vk):
    torch.manual_seed(3)
    # cross entropy (log_softmax + nll) fwd/bwd
    logits = torch.randn(64, 10, requires_grad=True)
    target = torch.randint(0, 10, (64,))
    dl = logits.detach().to(vk).requires_grad_()
    loss = F.cross_entropy(dl, target.to(vk)); loss.backward()
    ref = F.cross_entropy(logits, target); ref.backward()
    close(loss, ref, 1e-5); close(dl.grad, logits.grad, 1e-5)
    close(F.softmax(dl, -1), F.softmax(logits, -1), 1e-5); close(F.softmax(dl, 0), F.softmax(logits, 0), 1e-5)
    # rms_norm
    x = torch.randn(40, 96, requires_grad=True); w = (torch.rand(96) + 0.5).requires_grad_()
    dx, dw = x.detach().to(vk).requires_grad_(), w.detach().to(vk).requires_grad_()
    g = torch.randn(40, 96)
    F.rms_norm(dx, (96,), dw).backward(g.to(vk)); F.rms_norm(x, (96,), w).backward(g)
    close(dx.grad, x.grad, 1e-5); close(dw.grad, w.grad, 1e-5)
    # batch norm (training) with running statistics
    bn_c, bn_d = torch.nn.BatchNorm2d(16), torch.nn.BatchNorm2d(16).to(vk)
    xi = torch.randn(8, 16, 6, 6, requires_grad=True); di = xi.detach().to(vk).requires_grad_()
    gi = torch.randn(8, 16, 6, 6)
    bn_d(di).backward(gi.to(vk)); bn_c(xi).backward(gi)
    close(di.grad, xi.grad, 1e-4); close(bn_d.weight.grad, bn_c.weight.grad, 1e-4); close(bn_d.bias.grad, bn_c.bias.grad, 1e-5)
    close(bn_d.running_mean, bn_c.running_mean, 1e-5); close(bn_d.running_var, bn_c.running_var, 1e-5)
    assert bn_d.num_batches_tracked.item() == 1
    # embedding
    emb_c = torch.nn.Embedding(50, 32); emb_d = torch.nn.Embedding(50, 32).to(vk)
    emb_d.weight.data.copy_(emb_c.weight.data)
    idx = torch.randint(0, 50, (7, 9)); ge = torch.randn(7, 9, 32)
    emb_d(idx.to(vk)).backward(ge.to(vk)); emb_c(idx).backward(ge)
    close(emb_d.weight.grad, emb_c.weight.grad, 1e-6)
    # linear fwd/bwd (addmm + the transposed mm products autograd issues)
    lin_c = torch.nn.Linear(72, 40); lin_d = torch.nn.Linear(72, 40).to(vk)
    lin_d.load_state_dict(lin_c.state_dict())
    xi = torch.randn(33, 72, requires_grad=True); di = xi.detach().to(vk).requires_grad_()
    F.gelu(lin_d(di)).sum().backward(); F.gelu(lin_c(xi)).sum().backward()
    close(di.grad, xi.grad, 1e-5); close(lin_d.weight.grad, lin_c.weight.grad, 1e-5); close(lin_d.bias.grad, lin_c.bias.grad, 1e-5)
    close(torch.bmm(torch.ones(3, 4, 5, device=vk), torch.ones(3, 5, 6, device=vk)), torch.full((3, 4, 6), 5.0), 0)


@pytest.mark.parametrize("L,S", [(12, 24), (24, 16), (256, 128), (64, 384)])
def test_sdpa_causal_with_unequal_lengths_matches_aten(vk, L, S):
    """is_causal hides key > row whatever L and S are (src/api/ops/attention.cpp:107-112), which is ATen's rule too:
    out and all three gradients against ATen CPU in fp32 on the same fp16-rounded inputs."""
    torch.manual_seed(11)
    q, k, v = torch.randn(2, 4, L, 64).half(), torch.randn(2, 2, S, 64).half(), torch.randn(2, 2, S, 64).half()
    g = torch.randn(2, 4, L, 64).half()
    dq, dk, dv = (t.to(vk).requires_grad_() for t in (q, k, v))
    cq, ck, cv = (t.float().requires_grad_() for t in (q, k, v))
    out = F.scaled_dot_product_attention(dq, dk, dv, is_causal=True, enable_gqa=True)
    ref = F.scaled_dot_product_attention(cq, ck, cv, is_causal=True, enable_gqa=True)
    out.backward(g.to(vk)); ref.backward(g.float())
    close(out, ref, 1e-2)
    close(dq.grad, cq.grad, 1e-2); close(dk.grad, ck.grad, 1e-2); close(dv.grad, cv.grad, 1e-2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 3e-3)])
def test_layer_norm_group_norm_and_scans(vk, dtype, tol):
    """native_layer_norm / native_group_norm forward and backward, cumsum / cumprod / logcumsumexp (the row kernels next
    to softmax and RMSNorm; src/api/ops/norm.cpp:264-325, src/api/ops/scan.cpp:104-126) against ATen CPU in fp32."""
    torch.manual_seed(21)
    x = torch.randn(6, 17, 96).to(dtype)
    ln_c, ln_d = torch.nn.LayerNorm(96), torch.nn.LayerNorm(96).to(dtype).to(vk)
    with torch.no_grad():
        ln_c.weight.copy_(torch.rand(96) + 0.5); ln_c.bias.copy_(torch.randn(96))
        ln_d.weight.copy_(ln_c.weight.to(dtype)); ln_d.bias.copy_(ln_c.bias.to(dtype))
        ln_c.weight.copy_(ln_d.weight.cpu().float()); ln_c.bias.copy_(ln_d.bias.cpu().float())
    xc, xd = x.float().clone().requires_grad_(), x.detach().to(vk).requires_grad_()
    g = torch.randn(6, 17, 96).to(dtype)
    ln_d(xd).backward(g.to(vk)); ln_c(xc).backward(g.float())
    close(ln_d(xd), ln_c(xc), tol); close(xd.grad, xc.grad, tol); close(ln_d.weight.grad, ln_c.weight.grad, tol); close(ln_d.bias.grad, ln_c.bias.grad, tol)
    close(F.layer_norm(xd, (17, 96)), F.layer_norm(xc, (17, 96)), tol)                     # two trailing axes, no affine
    xi = torch.randn(4, 12, 6, 5).to(dtype)
    gn_c, gn_d = torch.nn.GroupNorm(4, 12), torch.nn.GroupNorm(4, 12).to(dtype).to(vk)
    with torch.no_grad():
        gn_c.weight.copy_(torch.rand(12) + 0.5); gn_c.bias.copy_(torch.randn(12))
        gn_d.weight.copy_(gn_c.weight.to(dtype)); gn_d.bias.copy_(gn_c.bias.to(dtype))
        gn_c.weight.copy_(gn_d.weight.cpu().float()); gn_c.bias.copy_(gn_d.bias.cpu().float())
    ic, idv = xi.float().clone().requires_grad_(), xi.detach().to(vk).requires_grad_()
    gi = torch.randn(4, 12, 6, 5).to(dtype)
    gn_d(idv).backward(gi.to(vk)); gn_c(ic).backward(gi.float())
    close(gn_d(idv), gn_c(ic), tol); close(idv.grad, ic.grad, tol); close(gn_d.weight.grad, gn_c.weight.grad, tol); close(gn_d.bias.grad, gn_c.bias.grad, tol)
    s = (torch.randn(5, 40, 3) * 0.5).to(dtype)
    for d in (0, 1, 2, -1):
        close(torch.cumsum(s.to(vk), d), torch.cumsum(s.float(), d), tol * 4)
        close(torch.logcumsumexp(s.to(vk), d), torch.logcumsumexp(s.float(), d), tol * 4)
    p = (1 + torch.randn(5, 40) * 0.05).to(dtype)
    close(torch.cumprod(p.to(vk), 1), torch.cumprod(p.float(), 1), tol * 4)
    i = torch.randint(-4, 5, (7, 33))
    assert torch.equal(torch.cumsum(i.to(vk), 1).cpu(), torch.cumsum(i, 1)) and torch.equal(i.to(vk).cumsum(0).cpu(), i.cumsum(0))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3), (torch.bfloat16, 1e-2)])
def test_addbmm_mv_dot_and_add_relu(vk, dtype, tol):
    """The remaining matmul-shaped entry points on the same product kernel (addbmm, addmv / mv, dot:
    src/api/decompositions.cpp:46-58, 109-124, 1114-1129) and _add_relu as one kernel (src/api/ops/binary.cpp:655-673)."""
    torch.manual_seed(31)
    f = lambda t: t.float()  # noqa: E731
    b1, b2, inp = torch.randn(5, 40, 72).to(dtype), torch.randn(5, 72, 56).to(dtype), torch.randn(40, 56).to(dtype)
    close(torch.addbmm(inp.to(vk), b1.to(vk), b2.to(vk), beta=0.5, alpha=2.0), torch.addbmm(f(inp), f(b1), f(b2), beta=0.5, alpha=2.0), tol)
    close(torch.addbmm(inp[0].to(vk), b1.to(vk), b2.to(vk)), torch.addbmm(f(inp[0]), f(b1), f(b2)), tol)          # broadcast row
    mat, vec, v0 = torch.randn(300, 520).to(dtype), torch.randn(520).to(dtype), torch.randn(300).to(dtype)
    close(torch.mv(mat.to(vk), vec.to(vk)), torch.mv(f(mat), f(vec)), tol)
    close(torch.addmv(v0.to(vk), mat.to(vk), vec.to(vk), beta=0.25, alpha=1.5), torch.addmv(f(v0), f(mat), f(vec), beta=0.25, alpha=1.5), tol)
    close(torch.mv(mat.t()[:256].to(vk), v0[:300].to(vk)), torch.mv(f(mat.t()[:256]), f(v0[:300])), tol)          # transposed matrix
    x, y = torch.randn(70001).to(dtype), torch.randn(70001).to(dtype)
    ref = torch.dot(f(x), f(y))
    assert abs(torch.dot(x.to(vk), y.to(vk)).item() - ref.item()) <= max(tol, 1e-4) * (f(x).abs() * f(y).abs()).sum().item() ** 0.5 * 4
    a, b = torch.randn(33, 65).to(dtype), torch.randn(33, 65).to(dtype)
    close(torch._add_relu(a.to(vk), b.to(vk)), torch.relu(f(a) + f(b)), tol)
    c = a.to(vk).clone()
    torch._add_relu_(c, b.to(vk), alpha=0.5)
    close(c, torch.relu(f(a) + 0.5 * f(b)), tol)


def make_mlp(sizes):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(torch.nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(torch.nn.GELU())
    return torch.nn.Sequential(*layers)


@pytest.mark.parametrize("sizes,batch,dtype,fused", [((72, 136, 136, 10), 48, torch.float32, False), ((72, 136, 136, 10), 48, torch.float16, True),
                                                     ((784, 8192, 8192, 10), 256, torch.float16, True)])
def test_mlp_training_script(vk, sizes, batch, dtype, fused):
    """examples/mlp.py-shaped training steps written against the public API only (BASELINE config 2).
    fp16 parameters use AdamW(fused=True): the foreach path does its arithmetic in the parameter dtype,
    where eps = 1e-8 underflows to zero (on any backend); fp32 parameters take the default foreach path."""
    torch.manual_seed(0)
    ref = make_mlp(sizes)                                   # fp32 CPU model holding the device model's values
    dev = make_mlp(sizes)
    dev.load_state_dict(ref.state_dict())
    dev = dev.to(dtype).to(vk)
    with torch.no_grad():
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            p_ref.copy_(p_dev.cpu().float())
    x = torch.randn(batch, sizes[0]).to(dtype)
    y = torch.randint(0, sizes[-1], (batch,))
    opt_d = torch.optim.AdamW(dev.parameters(), lr=1e-3, weight_decay=1e-2, fused=fused)
    opt_c = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=1e-2)
    gtol = 1e-2 if dtype == torch.float16 else 1e-4
    # fp16: BASELINE config 2 checks the parameters after one step. (With fp16 moments a second step
    # divides by second moments that underflowed, on this and on the reference backend alike, which
    # turns one-ulp differences into large ones.)
    for _ in range(1 if dtype == torch.float16 else 2):
        opt_d.zero_grad(set_to_none=True); opt_c.zero_grad(set_to_none=True)
        loss_d = F.cross_entropy(dev(x.to(vk)), y.to(vk)); loss_d.backward()
        loss_c = F.cross_entropy(ref(x.float()), y); loss_c.backward()
        assert abs(loss_d.item() - loss_c.item()) / abs(loss_c.item()) <= gtol
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            close(p_dev.grad, p_ref.grad, gtol)
            # Adam normalises the update, so it amplifies the rounding of tiny fp16 gradients: give the
            # reference optimizer the device's gradient values to check the optimizer arithmetic itself.
            p_ref.grad = p_dev.grad.cpu().float()
        opt_d.step(); opt_c.step()
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            diff = (p_dev.detach().cpu().float() - p_ref.detach()).abs().max().item()
            assert diff <= (1.3e-4 if dtype == torch.float16 else 2e-6), diff   # at most ~1 ulp of the storage type
            if dtype == torch.float16:
                # The device keeps parameters and both moments in fp16 (as the reference does,
                # src/api/ops/optim.cpp:72-73): round the fp32 reference's copies the same way so the next
                # step starts from identical state (second moments of tiny gradients underflow to zero).
                with torch.no_grad():
                    p_ref.copy_(p_dev.detach().cpu().float())
                    st = opt_c.state[p_ref]
                    st["exp_avg"].copy_(st["exp_avg"].half().float())
                    st["exp_avg_sq"].copy_(st["exp_avg_sq"].half().float())
    import torchvulkan
    torchvulkan.synchronize()


@pytest.mark.parametrize("cfg", [dict(vocab=64, seq=64, layers=2, width=128, heads=4, kv_heads=2, hidden=352, batch=4),
                                 dict(vocab=128, seq=256, layers=6, width=512, heads=8, kv_heads=2, hidden=1376, batch=32)])
def test_decoder_training_step(vk, cfg):
    """BASELINE config 3 (and a reduced copy): decoder-only transformer fwd+bwd in fp16 on the device against
    the same weights in fp32 on ATen CPU. Bar: loss within 1e-2 relative, every gradient within 1e-2
    relative Frobenius (a few of the deepest, smallest gradients are allowed 3e-2: fp16 activations)."""
    from models import Decoder

    torch.manual_seed(0)
    batch = cfg.pop("batch")
    ref = Decoder(**cfg)
    dev = Decoder(**cfg)
    dev.load_state_dict(ref.state_dict())
    dev = dev.half().to(vk)
    with torch.no_grad():
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            p_ref.copy_(p_dev.cpu().float())
    ids = torch.randint(0, cfg["vocab"], (batch, cfg["seq"]))
    tgt = torch.randint(0, cfg["vocab"], (batch * cfg["seq"],))
    # The mean over 8192 tokens makes the gradients that reach the attention inputs ~1e-8, below fp16's
    # range on any backend: the backward pass runs on the loss times a power of two (plain static loss
    # scaling, the same factor on both sides, so the gradients compare directly).
    loss_scale = 4096.0 if batch * cfg["seq"] >= 4096 else 1.0
    loss_d = F.cross_entropy(dev(ids.to(vk)).view(-1, cfg["vocab"]), tgt.to(vk)); (loss_d * loss_scale).backward()
    loss_c = F.cross_entropy(ref(ids).view(-1, cfg["vocab"]), tgt); (loss_c * loss_scale).backward()
    assert abs(loss_d.item() - loss_c.item()) / abs(loss_c.item()) <= 1e-2
    errs = {n: rel_fro(pd.grad.cpu().double().numpy(), pr.grad.double().numpy())
            for (n, pr), (_, pd) in zip(ref.named_parameters(), dev.named_parameters())}
    worst = sorted(errs.items(), key=lambda kv: -kv[1])[:3]
    assert all(e <= 3e-2 for e in errs.values()), worst
    assert sum(e <= 1e-2 for e in errs.values()) >= 0.9 * len(errs), worst
    import torchvulkan
    torchvulkan.synchronize()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 0, 1)])
def test_conv2d_autograd(vk, dtype, stride, pad, k):
    """F.conv2d forward, bias, and all three gradients through convolution_overrideable(+backward)."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 24, 13, 10, generator=g).to(dtype)
    w = (torch.randn(40, 24, k, k, generator=g) / (24 * k * k) ** 0.5).to(dtype)
    b = torch.randn(40, generator=g).to(dtype)
    xd, wd, bd = (t.to(vk).requires_grad_() for t in (x, w, b))
    xc, wc, bc = (t.double().requires_grad_() for t in (x, w, b))
    yd = F.conv2d(xd, wd, bd, stride=stride, padding=pad)
    yc = F.conv2d(xc, wc, bc, stride=stride, padding=pad)
    gy = torch.randn(yc.shape, generator=g).to(dtype)
    yd.backward(gy.to(vk)); yc.backward(gy.double())
    for name, d, c in (("y", yd, yc), ("gx", xd.grad, xc.grad), ("gw", wd.grad, wc.grad), ("gb", bd.grad, bc.grad)):
        assert rel_fro(d.detach().cpu().double().numpy(), c.detach().numpy()) <= (1e-2 if dtype != torch.float32 else 1e-5), name


def _conv_family_check(fn, tensors, dtype, **kw):
    """fn(*tensors, **kw) on the device against ATen CPU in float64: the output and the gradient of every tensor."""
    dev = [t.to("vulkan:0").requires_grad_() for t in tensors]
    cpu = [t.double().requires_grad_() for t in tensors]
    yd, yc = fn(*dev, **kw), fn(*cpu, **kw)
    assert yd.shape == yc.shape
    gy = torch.randn(yc.shape, generator=torch.Generator().manual_seed(9)).to(dtype)
    yd.backward(gy.to("vulkan:0")); yc.backward(gy.double())
    tol = 1e-2 if dtype != torch.float32 else 1e-4
    assert rel_fro(yd.detach().cpu().double().numpy(), yc.detach().numpy()) <= tol, "output"
    for i, (d, c) in enumerate(zip(dev, cpu)):
        assert d.grad.shape == c.grad.shape
        assert rel_fro(d.grad.cpu().double().numpy(), c.grad.numpy()) <= tol, f"gradient of argument {i}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("groups,cin,cout", [(2, 24, 40), (4, 16, 16), (24, 24, 24), (24, 24, 72)])
def test_grouped_and_depthwise_conv2d(vk, dtype, groups, cin, cout):
    """groups > 1 through convolution_overrideable(+backward): depthwise (groups == cin, with and without a channel
    multiplier) on the direct kernels, other groupings group by group on the tensor-core kernels."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, cin, 11, 9, generator=g).to(dtype)
    w = (torch.randn(cout, cin // groups, 3, 3, generator=g) / 3.0).to(dtype)
    b = torch.randn(cout, generator=g).to(dtype)
    for stride, pad in ((1, 1), (2, 1)):
        _conv_family_check(F.conv2d, (x, w, b), dtype, stride=stride, padding=pad, groups=groups)
    if groups == cin:          # the direct kernels also take dilation and unequal strides
        _conv_family_check(F.conv2d, (x, w, b), dtype, stride=(2, 1), padding=(2, 0), dilation=(2, 1), groups=groups)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_conv_transpose2d(vk, dtype):
    """Transposed convolution = the input-gradient product of the forward one; stride 2 with output_padding, and groups."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 16, 7, 6, generator=g).to(dtype)
    w = (torch.randn(16, 24, 3, 3, generator=g) / 12.0).to(dtype)
    b = torch.randn(24, generator=g).to(dtype)
    _conv_family_check(F.conv_transpose2d, (x, w, b), dtype, stride=1, padding=1)
    _conv_family_check(F.conv_transpose2d, (x, w, b), dtype, stride=2, padding=1, output_padding=1)
    w2 = (torch.randn(16, 6, 3, 3, generator=g) / 6.0).to(dtype)              # groups 2: 16 -> 12 channels
    _conv_family_check(F.conv_transpose2d, (x, w2), dtype, stride=2, padding=1, output_padding=1, groups=2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_conv2d_dilation_and_other_strides(vk, dtype):
    """Dilation, strides above 2, unequal strides and filters of many taps (the reference's one convolution entry takes any
    geometry, src/api/ops/conv.cpp:1088-1117): unfold + tensor-core GEMM + fold in the tensors' dtype."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(3, 16, 19, 17, generator=g).to(dtype)
    w = (torch.randn(24, 16, 3, 3, generator=g) / 12.0).to(dtype)
    b = torch.randn(24, generator=g).to(dtype)
    _conv_family_check(F.conv2d, (x, w, b), dtype, stride=1, padding=2, dilation=2)
    _conv_family_check(F.conv2d, (x, w, b), dtype, stride=3, padding=1)
    _conv_family_check(F.conv2d, (x, w, b), dtype, stride=(1, 2), padding=(0, 1))
    _conv_family_check(F.conv2d, (x, w, b), dtype, stride=(2, 1), padding=(3, 1), dilation=(3, 1))
    _conv_family_check(F.conv2d, (x.contiguous(memory_format=torch.channels_last), w, b), dtype, stride=2, padding=2, dilation=2)
    w9 = (torch.randn(8, 16, 9, 9, generator=g) / 36.0).to(dtype)             # 81 taps
    _conv_family_check(F.conv2d, (x, w9), dtype, stride=1, padding=4)
    # transposed and grouped convolutions reach the same route through the dense entry
    wt = (torch.randn(16, 6, 3, 3, generator=g) / 12.0).to(dtype)
    _conv_family_check(F.conv_transpose2d, (x, wt), dtype, stride=3, padding=1, output_padding=2)
    wg = (torch.randn(24, 8, 3, 3, generator=g) / 8.0).to(dtype)
    _conv_family_check(F.conv2d, (x, wg), dtype, stride=1, padding=2, dilation=2, groups=2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_conv_transpose3d(vk, dtype):
    """Transposed 3-D convolution (slow_conv_transpose3d in the reference, src/api/ops/conv.cpp:1196-1220, 1307): one
    transposed 2-D convolution per depth tap; gradients from the forward 3-D convolution with the roles swapped."""
    g = torch.Generator().manual_seed(8)
    x = torch.randn(2, 8, 4, 7, 5, generator=g).to(dtype)
    w = (torch.randn(8, 12, 3, 3, 3, generator=g) / 14.0).to(dtype)           # [cin, cout / groups, kd, kh, kw]
    b = torch.randn(12, generator=g).to(dtype)
    _conv_family_check(F.conv_transpose3d, (x, w, b), dtype, stride=1, padding=1)
    _conv_family_check(F.conv_transpose3d, (x, w, b), dtype, stride=2, padding=1, output_padding=1)
    _conv_family_check(F.conv_transpose3d, (x, w, b), dtype, stride=(1, 2, 2), padding=(0, 1, 1), output_padding=(0, 1, 1))
    _conv_family_check(F.conv_transpose3d, (x, w, b), dtype, stride=(2, 1, 1), padding=(1, 1, 1), output_padding=(1, 0, 0))
    w2 = (torch.randn(8, 3, 2, 3, 3, generator=g) / 8.0).to(dtype)            # groups 2: 8 -> 6 channels
    _conv_family_check(F.conv_transpose3d, (x, w2), dtype, stride=2, padding=(0, 1, 1), groups=2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_conv3d(vk, dtype):
    """3-D convolution: one 2-D convolution per depth tap over the batch n * depths."""
    g = torch.Generator().manual_seed(7)
    x = torch.randn(2, 8, 6, 9, 7, generator=g).to(dtype)
    w = (torch.randn(12, 8, 3, 3, 3, generator=g) / 14.0).to(dtype)
    b = torch.randn(12, generator=g).to(dtype)
    _conv_family_check(F.conv3d, (x, w, b), dtype, stride=1, padding=1)
    _conv_family_check(F.conv3d, (x, w, b), dtype, stride=2, padding=1)
    _conv_family_check(F.conv3d, (x, w, b), dtype, stride=(2, 1, 1), padding=(0, 1, 1))
    w2 = (torch.randn(12, 4, 2, 3, 3, generator=g) / 8.0).to(dtype)
    _conv_family_check(F.conv3d, (x, w2), dtype, stride=1, padding=(1, 1, 1), groups=2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_conv1d_and_conv_transpose1d(vk, dtype):
    """1-D convolutions run as 2-D ones of height 1."""
    g = torch.Generator().manual_seed(6)
    x = torch.randn(4, 16, 37, generator=g).to(dtype)
    w = (torch.randn(24, 16, 5, generator=g) / 9.0).to(dtype)
    b = torch.randn(24, generator=g).to(dtype)
    _conv_family_check(F.conv1d, (x, w, b), dtype, stride=1, padding=2)
    _conv_family_check(F.conv1d, (x, w, b), dtype, stride=2, padding=1)
    wd = (torch.randn(16, 1, 5, generator=g) / 2.0).to(dtype)                 # depthwise
    _conv_family_check(F.conv1d, (x, wd), dtype, stride=1, padding=2, groups=16)
    wt = (torch.randn(16, 8, 4, generator=g) / 8.0).to(dtype)
    _conv_family_check(F.conv_transpose1d, (x, wt), dtype, stride=2, padding=1)


@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("width,batch,size", [(16, 8, 16), (64, 256, 32)])
def test_resnet_training_step(vk, width, batch, size, channels_last):
    """BASELINE config 4 (and a reduced copy): ResNet fwd+bwd in fp16 and an SGD-momentum step on the device against
    the same weights in fp32 on ATen CPU.

    Layer by layer (every Conv2d, BatchNorm2d and Linear): the CPU layer is fed the tensors the device layer saw
    (its input and its incoming gradient), and its output, input gradient and parameter gradients must match the
    device's within 1e-2 relative Frobenius. End to end the bar is looser: a ReLU whose fp16 pre-activation rounds
    to the other side of zero flips a whole gradient path, so fp16 and fp32 runs of any backend drift apart by a
    few percent per block; the loss must agree within 1e-2 and every gradient within 0.25. The backward pass runs
    on the loss times 1024 (static loss scaling, same factor on both sides): with a mean over 256 images the
    stage-1 activation gradients are otherwise below fp16's normal range.

    With channels_last the model and its input use torch.channels_last memory (the layout the convolution and
    batch-norm kernels read and write in place); the activations must keep that format through the network."""
    import copy

    from models import SmallResNet

    torch.manual_seed(0)
    ref, dev = SmallResNet(width), SmallResNet(width)
    dev.load_state_dict(ref.state_dict())
    dev = dev.half().to(vk)
    if channels_last:
        dev = dev.to(memory_format=torch.channels_last)
    with torch.no_grad():
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            p_ref.copy_(p_dev.cpu().float())
    pristine = copy.deepcopy(ref)
    seen = {}
    for name, mod in dev.named_modules():
        if isinstance(mod, (torch.nn.Conv2d, torch.nn.BatchNorm2d, torch.nn.Linear)):
            seen[name] = {}
            mod.register_forward_hook(lambda m, inp, out, name=name: seen[name].update(x=inp[0].detach(), y=out.detach()))
            mod.register_full_backward_hook(lambda m, gin, gout, name=name: seen[name].update(gx=gin[0], gy=gout[0]))
    x = torch.randn(batch, 3, size, size).half()
    y = torch.randint(0, 10, (batch,))
    lr, loss_scale = 0.05, 1024.0
    # the channels-last run also takes the fused (list) optimizer: 1x1 filters and their gradients then differ in strides
    # along their unit dimensions only, which the list kernels must accept as one layout
    opt_d = torch.optim.SGD(dev.parameters(), lr=lr / loss_scale, momentum=0.9, fused=bool(channels_last))
    opt_c = torch.optim.SGD(ref.parameters(), lr=lr / loss_scale, momentum=0.9)
    x_dev = x.to(vk).contiguous(memory_format=torch.channels_last) if channels_last else x.to(vk)
    loss_d = F.cross_entropy(dev(x_dev), y.to(vk)); (loss_d * loss_scale).backward()
    loss_c = F.cross_entropy(ref(x.float()), y); (loss_c * loss_scale).backward()
    assert abs(loss_d.item() - loss_c.item()) / abs(loss_c.item()) <= 1e-2
    if channels_last:
        kept = [n for n, rec in seen.items() if rec["y"].dim() == 4 and rec["y"].is_contiguous(memory_format=torch.channels_last)]
        assert len(kept) >= sum(rec["y"].dim() == 4 for rec in seen.values()) - 1, "activations fell out of channels-last memory"

    cpu64 = lambda t: t.detach().cpu().double().numpy()  # noqa: E731
    bad = []
    for name, rec in seen.items():
        layer = copy.deepcopy(pristine.get_submodule(name))
        xin = rec["x"].cpu().float().requires_grad_()
        out = layer(xin)
        out.backward(rec["gy"].cpu().float())
        checks = [("out", rec["y"], out)]
        if rec.get("gx") is not None:
            checks.append(("grad_input", rec["gx"], xin.grad))
        dev_layer = dev.get_submodule(name)
        for pname, p in layer.named_parameters():
            checks.append((pname + ".grad", getattr(dev_layer, pname).grad, p.grad))
        for what, got, want in checks:
            err = rel_fro(cpu64(got), cpu64(want))
            if not err <= 1e-2:
                bad.append((name, what, round(float(err), 4)))
    assert not bad, bad

    errs = {n: rel_fro(cpu64(pd.grad), cpu64(pr.grad)) for (n, pr), (_, pd) in zip(ref.named_parameters(), dev.named_parameters())}
    assert all(e <= 0.25 for e in errs.values()), sorted(errs.items(), key=lambda kv: -kv[1])[:3]
    # the optimizer step itself: same gradients in, same parameters out
    with torch.no_grad():
        for p_ref, p_dev in zip(ref.parameters(), dev.parameters()):
            p_ref.grad.copy_(p_dev.grad.cpu().float())
    opt_d.step(); opt_c.step()
    for (n, pr), (_, pd) in zip(ref.named_parameters(), dev.named_parameters()):
        # fp16 storage: one rounding (2^-11 relative), or one subnormal step (2^-24) for the freshly moved zero biases
        np.testing.assert_allclose(cpu64(pd), cpu64(pr), rtol=1e-3, atol=1.2e-7, err_msg=n)
    for (n, br), (_, bd) in zip(ref.named_buffers(), dev.named_buffers()):
        if br.dtype.is_floating_point:
            assert rel_fro(cpu64(bd), cpu64(br)) <= 1e-2, n
    import torchvulkan
    torchvulkan.synchronize()


@pytest.mark.parametrize("channels_last", [False, True])
def test_resnet_fp32_training_step(vk, channels_last):
    """The ResNet of config 4 in fp32 (convolutions through unfold + 3xTF32 GEMM): loss, every gradient and the
    parameters after one SGD step against ATen CPU fp32."""
    from models import SmallResNet

    torch.manual_seed(0)
    ref, dev = SmallResNet(16), SmallResNet(16)
    dev.load_state_dict(ref.state_dict())
    dev = dev.to(vk)
    if channels_last:
        dev = dev.to(memory_format=torch.channels_last)
    x, y = torch.randn(8, 3, 16, 16), torch.randint(0, 10, (8,))
    # the optimizer of the reference's example (examples/conv.py:64): Nesterov momentum with weight decay; two steps, so
    # that the second one runs with momentum buffers in place
    kw = dict(lr=0.05, momentum=0.9, nesterov=True, weight_decay=5e-4)
    opt_d = torch.optim.SGD(dev.parameters(), **kw)
    opt_c = torch.optim.SGD(ref.parameters(), **kw)
    xd = x.to(vk).contiguous(memory_format=torch.channels_last) if channels_last else x.to(vk)
    for _ in range(2):
        opt_d.zero_grad(set_to_none=True); opt_c.zero_grad(set_to_none=True)
        loss_d = F.cross_entropy(dev(xd), y.to(vk)); loss_d.backward()
        loss_c = F.cross_entropy(ref(x), y); loss_c.backward()
        assert abs(loss_d.item() - loss_c.item()) <= 1e-4 * abs(loss_c.item())
        for (n, pr), (_, pd) in zip(ref.named_parameters(), dev.named_parameters()):
            assert rel_fro(pd.grad.cpu().double().numpy(), pr.grad.double().numpy()) <= 1e-3, n
        opt_d.step(); opt_c.step()
    for (n, pr), (_, pd) in zip(ref.named_parameters(), dev.named_parameters()):
        assert rel_fro(pd.detach().cpu().double().numpy(), pr.detach().double().numpy()) <= 1e-4, n


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3)])
@pytest.mark.parametrize("channels_last", [False, True])
def test_batch_norm_evaluation_mode(vk, dtype, tol, channels_last):
    """model.eval(): batch norm with the running statistics (2-D and 4-D inputs, both memory formats), and a whole
    ResNet forward in evaluation mode against ATen CPU."""
    from models import SmallResNet

    torch.manual_seed(0)
    bn = torch.nn.BatchNorm2d(24)
    bn.running_mean.normal_(); bn.running_var.uniform_(0.5, 2.0); bn.weight.data.normal_(); bn.bias.data.normal_()
    bn.eval()
    x = torch.randn(3, 24, 7, 5)
    dev = torch.nn.BatchNorm2d(24).to(dtype).to(vk).eval()
    dev.load_state_dict({k: v.to(dtype) if v.is_floating_point() else v for k, v in bn.state_dict().items()})
    xd = x.to(dtype).to(vk)
    if channels_last:
        xd = xd.contiguous(memory_format=torch.channels_last)
    yd = dev(xd)
    assert yd.is_contiguous(memory_format=torch.channels_last if channels_last else torch.contiguous_format)
    ref = bn.double()(x.to(dtype).double())
    assert rel_fro(yd.detach().cpu().double().numpy(), ref.detach().numpy()) <= tol
    # gradients through a frozen layer (the statistics are constants): input, weight and bias
    xg, xc = xd.detach().clone().requires_grad_(), x.to(dtype).double().requires_grad_()
    gy = torch.randn(3, 24, 7, 5).to(dtype)
    dev(xg).backward(gy.to(vk)); bn(xc).backward(gy.double())
    btol = max(tol, 5e-3 if dtype == torch.float16 else tol)
    for got, want in ((xg.grad, xc.grad), (dev.weight.grad, bn.weight.grad), (dev.bias.grad, bn.bias.grad)):
        assert rel_fro(got.cpu().double().numpy(), want.numpy()) <= btol
    bn1 = torch.nn.BatchNorm1d(24).eval()
    d1 = torch.nn.BatchNorm1d(24).to(dtype).to(vk).eval()
    x1 = torch.randn(9, 24)
    assert rel_fro(d1(x1.to(dtype).to(vk)).detach().cpu().double().numpy(), bn1.double()(x1.to(dtype).double()).detach().numpy()) <= tol
    if dtype == torch.float16:
        net = SmallResNet(16).eval()
        with torch.no_grad():
            for m in net.modules():
                if isinstance(m, torch.nn.BatchNorm2d):
                    m.running_mean.normal_(0, 0.1); m.running_var.uniform_(0.8, 1.2)
        dnet = SmallResNet(16)
        dnet.load_state_dict(net.state_dict())
        dnet = dnet.half().to(vk).eval()
        if channels_last:
            dnet = dnet.to(memory_format=torch.channels_last)
        img = torch.randn(4, 3, 16, 16).half()
        with torch.no_grad():
            out_d = dnet(img.to(vk).contiguous(memory_format=torch.channels_last) if channels_last else img.to(vk))
            out_c = net(img.float())
        assert rel_fro(out_d.cpu().double().numpy(), out_c.double().numpy()) <= 2e-2


@pytest.mark.parametrize("kind", ["mlp", "decoder"])
def test_graph_replay_equals_eager_steps(vk, kind):
    """torchvulkan.Graph: a training step captured once and replayed must leave exactly the parameters that the same
    number of eager steps leaves (same kernels in the same order; the optimizer's step count lives on the device)."""
    import copy

    import torchvulkan
    from models import Decoder

    torch.manual_seed(0)
    if kind == "mlp":
        base = torch.nn.Sequential(torch.nn.Linear(72, 136), torch.nn.GELU(), torch.nn.Linear(136, 10))
        x, y = torch.randn(48, 72).half().to(vk), torch.randint(0, 10, (48,)).to(vk)
        loss_of = lambda m: F.cross_entropy(m(x), y)  # noqa: E731
    else:
        base = Decoder(vocab=64, seq=128, layers=2, width=128, heads=4, kv_heads=2, hidden=352)
        ids, tgt = torch.randint(0, 64, (2, 128)).to(vk), torch.randint(0, 64, (2 * 128,)).to(vk)
        loss_of = lambda m: F.cross_entropy(m(ids).view(-1, 64), tgt) * 256.0  # noqa: E731
    models = [copy.deepcopy(base).half().to(vk) for _ in range(2)]
    opts = [torch.optim.AdamW(m.parameters(), lr=1e-3, fused=True) for m in models]
    losses = [None, None]

    def step(i):
        opts[i].zero_grad(set_to_none=True)
        losses[i] = loss_of(models[i])
        losses[i].backward()
        opts[i].step()

    for _ in range(7):
        step(0)                                   # seven eager steps
    for _ in range(3):
        step(1)                                   # three eager steps, ...
    g = torchvulkan.Graph()
    with g.capture():
        step(1)                                   # ... one recorded (not run) ...
    junk = []
    for r in range(4):
        g.replay()                                # ... and four replays of it
        # Work between the replays must not disturb the graph: its temporaries are parked in a pool of its own, so
        # neither fresh allocations (of the sizes the step uses) nor empty_cache() can be given, or free, its memory.
        junk.append([torch.full_like(p, float(r)) for p in models[1].parameters()])
        junk.append(torch.randn(48, 136).half().to(vk).float().half())
        if r == 1:
            torchvulkan.empty_cache()
        if r == 2:
            junk.clear()
    torchvulkan.synchronize()
    for (n, p0), (_, p1) in zip(models[0].named_parameters(), models[1].named_parameters()):
        assert torch.equal(p0.cpu(), p1.cpu()), n
    assert torch.equal(losses[0].cpu(), losses[1].cpu())
    with pytest.raises(RuntimeError):
        torchvulkan.Graph().replay()


def test_hot_ops_raise_instead_of_falling_back(vk):
    a = torch.ones(4, 4, dtype=torch.int64).to(vk)
    with pytest.raises((RuntimeError, NotImplementedError), match="NOT IMPLEMENTED"):
        a @ a
    with pytest.raises(RuntimeError, match="cannot be multiplied"):
        torch.ones(3, 4, device=vk) @ torch.ones(5, 6, device=vk)


def test_environment_switches_of_the_reference(vk):
    """TORCHVULKAN_VALIDATION / TORCHVULKAN_PROFILE / TORCHVULKAN_STRICT (src/vulkan/vulkan_context.cpp:195-248) in a fresh
    process: the checked mode counts nothing on healthy operators, counts the time-out a bounded wait leaves behind (made
    on purpose by the test hook that polls a flag nothing sets) and the device stays usable; the NVTX ranges of the profile
    switch and the strict switch change no result."""
    import os
    import subprocess
    import sys
    import textwrap
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    code = textwrap.dedent("""
        import torch, torchvulkan
        from torchvulkan_b200 import capi
        C = torchvulkan._load_backend()
        vk = torch.device("vulkan:0")
        x = torch.randn(300, 200).to(vk)
        y = (x @ x.t()).relu().sum().item()
        assert C._validation_error_count() == 0
        capi.call("tvk_debug_bounded_wait", 0, 2000, None)       # legacy stream: ordered with the device's own stream by the check's synchronize
        import warnings
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter("always")
            z = (x + 1).sum().item()
        assert C._validation_error_count() == 1, C._validation_error_count()
        assert any("bounded device-side wait ran out" in str(w.message) for w in seen)
        assert abs((x + 1).sum().item() - z) < 1e-3 and C._validation_error_count() == 1
        print("ENV-OK", y)
    """)
    env = dict(os.environ, PYTHONPATH=str(root), TORCHVULKAN_VALIDATION="1", TORCHVULKAN_PROFILE="1", TORCHVULKAN_STRICT="1")
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "ENV-OK" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


@pytest.mark.parametrize("dtype,mask_kind,causal,gqa,L,S", [
    (torch.float32, None, True, False, 48, 48),
    (torch.float32, None, False, False, 40, 56),
    (torch.float16, "bool", False, False, 40, 56),
    (torch.float16, "float", False, False, 40, 56),
    (torch.float32, "bool", False, True, 40, 56),
    (torch.bfloat16, "float", False, True, 24, 40),
    (torch.float16, None, False, False, 37, 53),
    (torch.float16, None, True, True, 37, 53),
])
def test_attention_with_masks_fp32_and_odd_lengths(vk, dtype, mask_kind, causal, gqa, L, S):
    """F.scaled_dot_product_attention for the cases outside the attention kernels (an additive or boolean mask, fp32, key
    counts that are not multiples of 8): the same overrideable operator composes them from this backend's launches
    (the reference's fused path takes the mask as an additive bias, src/api/ops/attention.cpp:698-722). Output, the
    gradients of q, k, v and of a floating mask against ATen CPU in float64; a query row whose mask hides every key
    gives 0 (attention_coop.slang:164-222)."""
    g = torch.Generator().manual_seed(17)
    B, H, D = 2, 4, 32
    Hk = 2 if gqa else H
    q, k, v = (torch.randn(B, h, n, D, generator=g).to(dtype) for h, n in ((H, L), (Hk, S), (Hk, S)))
    mask = None
    if mask_kind == "bool":
        mask = torch.rand(B, 1, L, S, generator=g) > 0.3
        mask[..., 0] = True
        mask[0, 0, 3, :] = False                                         # one row sees nothing
    elif mask_kind == "float":
        mask = (torch.randn(1, H, L, S, generator=g) * 0.5).to(dtype)
    qd, kd, vd = (t.to(vk).requires_grad_() for t in (q, k, v))
    qc, kc, vc = (t.double().requires_grad_() for t in (q, k, v))
    md = mc = None
    if mask is not None:
        md = mask.to(vk)
        mc = mask if mask.dtype == torch.bool else mask.double()
        if mask_kind == "float":
            md.requires_grad_(); mc.requires_grad_()
    od = F.scaled_dot_product_attention(qd, kd, vd, attn_mask=md, is_causal=causal, enable_gqa=gqa)
    oc = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=mc, is_causal=causal, enable_gqa=gqa)
    assert od.dtype == dtype and od.shape == oc.shape
    gy = torch.randn(oc.shape, generator=g).to(dtype)
    od.backward(gy.to(vk)); oc.backward(gy.double())
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    if mask_kind == "bool":
        assert float(od[0, :, 3].detach().abs().max().cpu()) == 0.0
        oc = oc.detach().clone(); oc[0, :, 3] = 0                        # (ATen's CPU kernel leaves NaN or 0 there, by version)
        for t in (qc.grad, kc.grad, vc.grad):
            t.nan_to_num_(0.0)
    assert rel_fro(od.detach().cpu().double().numpy(), oc.detach().numpy()) <= tol
    pairs = [(qd.grad, qc.grad), (kd.grad, kc.grad), (vd.grad, vc.grad)] + ([(md.grad, mc.grad)] if mask_kind == "float" else [])
    for got, want in pairs:
        assert got.shape == want.shape
        assert rel_fro(got.cpu().double().numpy(), want.numpy()) <= tol


@pytest.mark.parametrize("rowwise", [False, True])
@pytest.mark.parametrize("kinds", [("e4m3", "e4m3"), ("e4m3", "e5m2")])
def test_scaled_mm(vk, rowwise, kinds):
    """torch._scaled_mm on float8 operands against the emulation the reference follows (src/api/ops/matmul.cpp:706-747):
    upcast, scale, fp32 product, bias, cast. The products of float8 values are exact in fp32 on both sides, so the
    results differ only by the order of the fp32 additions."""
    f8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
    g = torch.Generator().manual_seed(21)
    # k a multiple of 16: the operands are read in place by the float8 kernel (ragged blocks, aligned and unaligned output
    # pitches); other k: the widened route
    for m, k, n in ((48, 72, 40), (33, 70, 37), (256, 512, 128), (200, 272, 136), (130, 144, 100), (300, 1040, 520)):
        a = torch.randn(m, k, generator=g).to(f8[kinds[0]])
        b = torch.randn(n, k, generator=g).to(f8[kinds[1]]).t()              # column-major, as torch's CUDA op wants it
        sa = (torch.rand(m, 1, generator=g) + 0.5) if rowwise else torch.tensor(0.75)
        sb = (torch.rand(1, n, generator=g) + 0.5) if rowwise else torch.tensor(1.5)
        bias = torch.randn(n, generator=g).bfloat16()
        ref = (a.float() * sa) @ (b.float() * sb)
        for out_dtype, with_bias in ((torch.bfloat16, True), (torch.float32, False), (torch.float16, False)):
            got = torch._scaled_mm(a.to(vk), b.to(vk), sa.to(vk), sb.to(vk), bias.to(vk) if with_bias else None, None, out_dtype)
            assert got.dtype == out_dtype and got.shape == (m, n) and got.is_contiguous()
            want = (ref + bias.float()) if with_bias else ref
            tol = {torch.float32: 1e-5, torch.float16: 1e-3, torch.bfloat16: 1e-2}[out_dtype]
            assert rel_fro(got.cpu().double().numpy(), want.double().numpy()) <= tol, (m, k, n, out_dtype)
        # a row-major second operand is consumed through its strides as well
        got = torch._scaled_mm(a.to(vk), b.contiguous().to(vk), sa.to(vk), sb.to(vk), None, None, torch.float32)
        assert rel_fro(got.cpu().double().numpy(), ref.double().numpy()) <= 1e-5
        # float8 output: divided by scale_result, cast without saturation
        sr = torch.tensor(4.0)
        got8 = torch._scaled_mm(a.to(vk), b.to(vk), sa.to(vk), sb.to(vk), None, sr.to(vk), torch.float8_e4m3fn)
        want8 = (ref / sr).to(torch.float8_e4m3fn)
        assert got8.dtype == torch.float8_e4m3fn
        g8, w8 = got8.cpu().float(), want8.float()
        # identical except where the fp32 sums differ in the last place right at a rounding boundary of the 3-bit mantissa
        same = (g8 == w8) | (g8.isnan() & w8.isnan())
        assert same.float().mean() >= 0.995
        assert rel_fro(g8.nan_to_num(0.0).double().numpy(), w8.nan_to_num(0.0).double().numpy()) <= 2e-2
    with pytest.raises(ValueError, match="Invalid scaling configuration"):
        torch._scaled_mm(a.to(vk), b.to(vk), torch.ones(3).to(vk), torch.ones(1).to(vk), None, None, torch.bfloat16)
    with pytest.raises(ValueError, match="must be fp8"):
        torch._scaled_mm(a.float().to(vk), b.to(vk), torch.ones(()).to(vk), torch.ones(()).to(vk), None, None, torch.bfloat16)


def test_conv_bn_folding_for_inference_runs_on_the_device(vk):
    """Evaluation-mode Conv2d + BatchNorm2d folded into one convolution by torch's own utility
    (torch.nn.utils.fusion.fuse_conv_bn_eval): the folding arithmetic runs on the device's elementwise kernels, and the
    folded convolution gives the unfolded pair's output."""
    from torch.nn.utils.fusion import fuse_conv_bn_eval

    torch.manual_seed(31)
    conv, bn = torch.nn.Conv2d(16, 24, 3, padding=1), torch.nn.BatchNorm2d(24)
    with torch.no_grad():
        bn.running_mean.uniform_(-0.5, 0.5); bn.running_var.uniform_(0.5, 2.0); bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-0.3, 0.3)
    x = torch.randn(4, 16, 12, 10)
    ref = bn.eval()(conv.eval()(x))
    dconv, dbn = torch.nn.Conv2d(16, 24, 3, padding=1), torch.nn.BatchNorm2d(24)
    dconv.load_state_dict(conv.state_dict()); dbn.load_state_dict(bn.state_dict())
    dconv, dbn = dconv.to(vk).eval(), dbn.to(vk).eval()
    with torch.no_grad():
        fused = fuse_conv_bn_eval(dconv, dbn)
        assert fused.weight.device.type == "vulkan"
        out = fused(x.to(vk))
        pair = dbn(dconv(x.to(vk)))
    close(out, ref, 1e-4)
    close(pair, ref, 1e-4)


def test_language_model_script_flow(vk):
    """What the reference's language-model example does around its model (examples/llm.py:100-135), in fp32 against the same
    run on ATen CPU: AdamW with its default settings, clip_grad_norm_, loss.item(); then eval(), a sampling loop with
    torch.multinomial over softmax(logits / temperature), torch.cat of the sampled ids, .tolist()."""
    from models import Decoder

    def run(device):
        torch.manual_seed(0)
        model = Decoder(vocab=64, seq=32, layers=2, width=64, heads=4, kv_heads=2, hidden=96).to(device)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
        g = torch.Generator().manual_seed(1)
        losses, norms = [], []
        model.train()
        for _ in range(4):
            windows = torch.randint(0, 64, (8, 33), generator=g)
            inputs, targets = windows[:, :-1].to(device), windows[:, 1:].to(device)
            logits = model(inputs)
            loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1))
            opt.zero_grad()
            loss.backward()
            norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)))
            opt.step()
            losses.append(loss.item())
        return model, losses, norms

    md, ld, nd = run(vk)
    mc, lc, nc = run(torch.device("cpu"))
    assert np.allclose(ld, lc, rtol=2e-4, atol=1e-5), (ld, lc)
    assert np.allclose(nd, nc, rtol=2e-3), (nd, nc)
    for pd, pc in zip(md.parameters(), mc.parameters()):
        assert rel_fro(pd.detach().cpu().double().numpy(), pc.detach().double().numpy()) <= 1e-4
    md.eval()
    idx = torch.tensor([[3, 1, 4, 1]], device=vk)
    assert idx.device.type == "vulkan"
    with torch.no_grad():
        for _ in range(6):
            logits = md(idx[:, -32:])[:, -1] / 0.8
            idx = torch.cat((idx, torch.multinomial(logits.softmax(-1), 1)), dim=1)
    sample = idx[0].tolist()
    assert len(sample) == 10 and sample[:4] == [3, 1, 4, 1] and all(0 <= t < 64 for t in sample)


def test_image_classifier_script_flow(vk):
    """What the reference's convolution example does around its model (examples/conv.py:58-86), in fp32 against ATen CPU:
    SGD with momentum, Nesterov and weight decay under a OneCycleLR schedule, then eval() and the accuracy count
    (argmax == targets).sum().item()."""
    from models import SmallResNet

    def run(device):
        torch.manual_seed(0)
        model = SmallResNet(8).to(device)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, nesterov=True, weight_decay=5e-4)
        sched = torch.optim.lr_scheduler.OneCycleLR(opt, max_lr=0.1, total_steps=4)
        crit = torch.nn.CrossEntropyLoss()
        g = torch.Generator().manual_seed(2)
        losses = []
        model.train()
        for _ in range(4):
            data, targets = torch.randn(16, 3, 16, 16, generator=g), torch.randint(0, 10, (16,), generator=g)
            loss = crit(model(data.to(device)), targets.to(device))
            opt.zero_grad()
            loss.backward()
            opt.step()
            sched.step()
            losses.append(loss.item())
        model.eval()
        data, targets = torch.randn(64, 3, 16, 16, generator=g), torch.randint(0, 10, (64,), generator=g)
        with torch.no_grad():
            out = model(data.to(device))
            correct = (out.argmax(dim=1) == targets.to(device)).sum().item()
        return losses, out.cpu(), correct

    ld, od, cd = run(vk)
    lc, oc, cc = run(torch.device("cpu"))
    assert np.allclose(ld, lc, rtol=2e-3, atol=1e-4), (ld, lc)
    assert rel_fro(od.double().numpy(), oc.double().numpy()) <= 2e-2
    assert isinstance(cd, int) and abs(cd - cc) <= 3


def test_mixed_precision_training_loops(vk):
    """The usual mixed-precision recipes end to end on the device: a small decoder with dropout under fp16 autocast with
    GradScaler, gradient clipping after unscale_ and the fused AdamW (which receives the scaler's found_inf); a small ResNet in
    channels-last under bf16 autocast with momentum SGD. The losses stay finite and go down."""
    from models import Decoder, SmallResNet

    torch.manual_seed(0)
    model = torch.nn.Sequential(Decoder(vocab=64, seq=64, layers=2, width=128, heads=4, kv_heads=2, hidden=256), torch.nn.Dropout(0.1)).to(vk)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, fused=True)
    scaler = torch.amp.GradScaler("vulkan")
    g = torch.Generator().manual_seed(1)
    data = torch.randint(0, 64, (16, 65), generator=g)
    losses = []
    for _ in range(16):
        x, y = data[:, :-1].to(vk), data[:, 1:].to(vk)
        with torch.autocast("vulkan", dtype=torch.float16):
            loss = F.cross_entropy(model(x).view(-1, 64), y.reshape(-1))
        opt.zero_grad(set_to_none=True)
        scaler.scale(loss).backward()
        scaler.unscale_(opt)
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        scaler.step(opt); scaler.update()
        losses.append(loss.item())
    assert all(np.isfinite(losses)) and losses[-1] < losses[0] - 0.3, losses
    # the scaler without unscale_(): the fused optimizer divides the gradients by grad_scale itself
    w = torch.nn.Parameter(torch.ones(8, device=vk))
    o2 = torch.optim.AdamW([w], lr=0.1, fused=True, weight_decay=0.0)
    s2 = torch.amp.GradScaler("vulkan", init_scale=256.0)
    s2.scale((w * torch.arange(8.0, device=vk)).sum()).backward()
    s2.step(o2); s2.update()
    assert torch.allclose(w.grad.cpu(), torch.arange(8.0)) and float(w.detach().cpu()[1]) < 1.0 and float(w.detach().cpu()[0]) == 1.0
    net = torch.nn.Sequential(SmallResNet(8), torch.nn.Dropout(0.2)).to(vk).to(memory_format=torch.channels_last)
    o3 = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    img, lab = torch.randn(32, 3, 16, 16, generator=g), torch.randint(0, 10, (32,), generator=g)
    ls = []
    for _ in range(12):
        with torch.autocast("vulkan", dtype=torch.bfloat16):
            loss = F.cross_entropy(net(img.to(vk).contiguous(memory_format=torch.channels_last)), lab.to(vk))
        o3.zero_grad(); loss.backward(); o3.step(); ls.append(loss.item())
    assert all(np.isfinite(ls)) and ls[-1] < ls[0], ls


def _module_matches_cpu(vk, make, inputs, tol=2e-4, loss=None):
    """The same module (same initial state) on the device and on ATen CPU: output and every gradient."""
    torch.manual_seed(0)
    ref = make()
    dev = make()
    dev.load_state_dict(ref.state_dict())
    dev = dev.to(vk)
    xs_c = [t.clone().requires_grad_(t.is_floating_point()) for t in inputs]
    xs_d = [t.to(vk).requires_grad_(t.is_floating_point()) for t in inputs]
    loss = loss or (lambda o: (o[0] if isinstance(o, tuple) else o).pow(2).mean())
    lc, ld = loss(ref(*xs_c)), loss(dev(*xs_d))
    assert abs(lc.item() - ld.item()) <= tol * (1 + abs(lc.item())), (lc.item(), ld.item())
    lc.backward(); ld.backward()
    def close(d, c, what):
        # relative to the gradient's own size, with a floor: a gradient that is numerically zero (1e-9) is compared absolutely
        d, c = d.cpu().double(), c.double()
        err = float((d - c).norm()) / max(float(c.norm()), 1e-5 * c.numel() ** 0.5)
        assert err <= 50 * tol, (what, err)

    for (n, pc), pd in zip(ref.named_parameters(), dev.parameters()):
        close(pd.grad, pc.grad, n)
    for c, d in zip(xs_c, xs_d):
        if c.grad is not None:
            close(d.grad, c.grad, "input")


def test_recurrent_transformer_and_padding_modules_match_cpu(vk):
    """nn.LSTM / nn.GRU (the fused cells every non-CPU device is routed to), nn.TransformerEncoderLayer in training mode,
    MultiheadAttention with a padding mask, reflection / replication padding, the 4-D cross-entropy of a segmentation head and
    weight normalisation, each against the same module on ATen CPU in fp32."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 10, 32, generator=g)
    img = torch.randn(2, 8, 12, 10, generator=g)
    _module_matches_cpu(vk, lambda: torch.nn.LSTM(32, 24, num_layers=2, batch_first=True), [x])
    _module_matches_cpu(vk, lambda: torch.nn.GRU(32, 24, batch_first=True, bidirectional=True), [x])
    _module_matches_cpu(vk, lambda: torch.nn.LSTM(32, 24, bias=False), [x])
    _module_matches_cpu(vk, lambda: torch.nn.TransformerEncoderLayer(32, 4, 64, dropout=0.0, batch_first=True), [x])
    _module_matches_cpu(vk, lambda: torch.nn.TransformerDecoderLayer(32, 4, 64, dropout=0.0, batch_first=True, norm_first=True), [x, x.flip(0)])
    pad_mask = (torch.arange(10)[None] > 6).expand(4, 10)

    class Mha(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.m = torch.nn.MultiheadAttention(32, 4, batch_first=True)

        def forward(self, t):
            return self.m(t, t, t, key_padding_mask=pad_mask.to(t.device), need_weights=False)[0]

    _module_matches_cpu(vk, Mha, [x])
    _module_matches_cpu(vk, lambda: torch.nn.Sequential(torch.nn.ReflectionPad2d((2, 1, 0, 3)), torch.nn.Conv2d(8, 4, 3)), [img])
    _module_matches_cpu(vk, lambda: torch.nn.Sequential(torch.nn.ReplicationPad2d(2), torch.nn.Conv2d(8, 4, 3)), [img])
    _module_matches_cpu(vk, lambda: torch.nn.Sequential(torch.nn.ReflectionPad1d(3), torch.nn.Conv1d(10, 6, 3)), [x])
    _module_matches_cpu(vk, lambda: torch.nn.utils.parametrizations.weight_norm(torch.nn.Linear(32, 16)), [x])
    tgt = torch.randint(0, 8, (2, 12, 10), generator=g)
    tgt[0, :2] = -100
    for red in ("mean", "sum", "none"):
        _module_matches_cpu(vk, lambda: torch.nn.Conv2d(8, 8, 1), [img],
                            loss=lambda o, red=red: F.cross_entropy(o, tgt.to(o.device), reduction=red, ignore_index=-100).sum())


def test_unfold_fold_embedding_renorm_and_triangle_indices(vk):
    g = torch.Generator().manual_seed(6)
    img = torch.randn(2, 3, 9, 8, generator=g)
    for kw in (dict(kernel_size=3), dict(kernel_size=(3, 2), stride=2, padding=1), dict(kernel_size=2, dilation=2, padding=(1, 0), stride=(1, 2))):
        xd, xc = img.to(vk).requires_grad_(), img.clone().requires_grad_()
        cd, cc = F.unfold(xd, **kw), F.unfold(xc, **kw)
        assert rel_fro(cd.detach().cpu().double().numpy(), cc.detach().double().numpy()) == 0.0
        gy = torch.randn(cc.shape, generator=g)
        cd.backward(gy.to(vk)); cc.backward(gy)
        assert rel_fro(xd.grad.cpu().double().numpy(), xc.grad.double().numpy()) <= 1e-6
        fd, fc = F.fold(gy.to(vk), (9, 8), **kw), F.fold(gy, (9, 8), **kw)
        assert rel_fro(fd.cpu().double().numpy(), fc.double().numpy()) <= 1e-6
    torch.manual_seed(0)
    emb_c = torch.nn.Embedding(12, 6, max_norm=1.0)
    emb_d = torch.nn.Embedding(12, 6, max_norm=1.0)
    emb_d.load_state_dict(emb_c.state_dict())
    emb_d = emb_d.to(vk)
    ids = torch.tensor([[1, 5, 5], [9, 0, 1]])
    out_d, out_c = emb_d(ids.to(vk)), emb_c(ids)
    assert rel_fro(out_d.detach().cpu().double().numpy(), out_c.detach().double().numpy()) <= 1e-6
    assert rel_fro(emb_d.weight.detach().cpu().double().numpy(), emb_c.weight.detach().double().numpy()) <= 1e-6   # only the rows that were looked up shrank
    m = torch.randn(5, 5, generator=g)
    assert abs(float(m.to(vk).trace().cpu()) - float(m.trace())) < 1e-5
    assert torch.equal(torch.tril_indices(4, 5, -1, device=vk).cpu(), torch.tril_indices(4, 5, -1))
    assert torch.equal(torch.triu_indices(4, 5, 1, device=vk).cpu(), torch.triu_indices(4, 5, 1))


@pytest.mark.parametrize("mode,padding_mode,align", [("bilinear", "zeros", False), ("bilinear", "zeros", True), ("bilinear", "border", False), ("nearest", "zeros", False)])
def test_grid_sample(vk, mode, padding_mode, align):
    """F.grid_sample (2-D) on the device against ATen CPU: output, the gradient of the input and, for bilinear sampling, of
    the grid; sampling positions reach outside the image."""
    g = torch.Generator().manual_seed(8)
    x = torch.randn(2, 3, 7, 6, generator=g)
    grid = torch.rand(2, 5, 4, 2, generator=g) * 2.6 - 1.3
    xd, xc = x.to(vk).requires_grad_(), x.clone().requires_grad_()
    gd, gc = grid.to(vk).requires_grad_(), grid.clone().requires_grad_()
    yd = F.grid_sample(xd, gd, mode=mode, padding_mode=padding_mode, align_corners=align)
    yc = F.grid_sample(xc, gc, mode=mode, padding_mode=padding_mode, align_corners=align)
    assert rel_fro(yd.detach().cpu().double().numpy(), yc.detach().double().numpy()) <= 1e-5
    gy = torch.randn(yc.shape, generator=g)
    yd.backward(gy.to(vk)); yc.backward(gy)
    assert rel_fro(xd.grad.cpu().double().numpy(), xc.grad.double().numpy()) <= 1e-5
    if mode == "bilinear":
        assert rel_fro(gd.grad.cpu().double().numpy(), gc.grad.double().numpy()) <= 1e-4


def test_cdist_bucketize_searchsorted(vk):
    g = torch.Generator().manual_seed(9)
    a, b = torch.randn(2, 5, 7, generator=g), torch.randn(2, 6, 7, generator=g)
    ad, ac = a.to(vk).requires_grad_(), a.clone().requires_grad_()
    bd, bc = b.to(vk).requires_grad_(), b.clone().requires_grad_()
    dd, dc = torch.cdist(ad, bd), torch.cdist(ac, bc)
    assert rel_fro(dd.detach().cpu().double().numpy(), dc.detach().double().numpy()) <= 1e-5
    gy = torch.randn(dc.shape, generator=g)
    dd.backward(gy.to(vk)); dc.backward(gy)
    assert rel_fro(ad.grad.cpu().double().numpy(), ac.grad.double().numpy()) <= 1e-4 and rel_fro(bd.grad.cpu().double().numpy(), bc.grad.double().numpy()) <= 1e-4
    for p in (1.0, float("inf"), 3.0):
        assert rel_fro(torch.cdist(a.to(vk), b.to(vk), p=p).cpu().double().numpy(), torch.cdist(a, b, p=p).double().numpy()) <= 1e-5
    codes = torch.randn(32, 7, generator=g)                                  # the nearest-code search of a vector quantiser
    assert torch.equal(torch.cdist(a[0].to(vk), codes.to(vk)).argmin(1).cpu(), torch.cdist(a[0], codes).argmin(1))
    bnd = torch.tensor([0.1, 0.5, 0.5, 2.0]); v = torch.tensor([[0.0, 0.1, 0.3], [0.5, 2.0, 3.0]])
    seq = torch.sort(torch.randn(3, 8, generator=g), dim=1).values; q = torch.randn(3, 4, generator=g)
    for right in (False, True):
        assert torch.equal(torch.bucketize(v.to(vk), bnd.to(vk), right=right).cpu(), torch.bucketize(v, bnd, right=right))
        assert torch.equal(torch.searchsorted(seq.to(vk), q.to(vk), right=right).cpu(), torch.searchsorted(seq, q, right=right))
    assert torch.bucketize(v.to(vk), bnd.to(vk), out_int32=True).dtype == torch.int32


def test_attention_modules_in_eval_mode_take_the_one_operator_path(vk, monkeypatch):
    """In eval mode without gradients nn.MultiheadAttention and nn.TransformerEncoderLayer call one operator for the whole
    block (torch._native_multi_head_attention / torch._transformer_encoder_layer_fwd) on this device too. Outputs and attention
    weights against the same modules on ATen CPU, with each kind of mask; the padded batch of a TransformerEncoder stays padded."""
    calls = {"mha": 0, "layer": 0}
    real_mha, real_layer = torch._native_multi_head_attention, torch._transformer_encoder_layer_fwd

    def spy_mha(*a, **k):
        calls["mha"] += a[0].device.type == "vulkan"
        return real_mha(*a, **k)

    def spy_layer(*a, **k):
        calls["layer"] += a[0].device.type == "vulkan"
        return real_layer(*a, **k)

    monkeypatch.setattr(torch, "_native_multi_head_attention", spy_mha)
    monkeypatch.setattr(torch, "_transformer_encoder_layer_fwd", spy_layer)
    g = torch.Generator().manual_seed(9)
    B, T, D, H = 3, 10, 32, 4
    x = torch.randn(B, T, D, generator=g)
    pad = torch.zeros(B, T, dtype=torch.bool)
    pad[0, 7:] = True
    pad[2, 4:] = True
    causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    valid = ~pad

    def close(d, c, tol=2e-5, rows=None):
        d, c = d.cpu().float(), c.float()
        if rows is not None:
            d, c = d[rows], c[rows]
        assert float((d - c).abs().max()) <= tol * (1 + float(c.abs().max())), float((d - c).abs().max())

    torch.manual_seed(0)
    ref = torch.nn.MultiheadAttention(D, H, batch_first=True).eval()
    dev = torch.nn.MultiheadAttention(D, H, batch_first=True)
    dev.load_state_dict(ref.state_dict())
    dev = dev.to(vk).eval()
    xd = x.to(vk)
    with torch.no_grad():
        for kw in ({}, {"key_padding_mask": pad}, {"attn_mask": causal}, {"key_padding_mask": pad, "attn_mask": causal},
                   {"average_attn_weights": False}, {"need_weights": False}, {"need_weights": False, "key_padding_mask": pad}):
            kd = {k: (v.to(vk) if torch.is_tensor(v) else v) for k, v in kw.items()}
            (oc, wc), (od, wd) = ref(x, x, x, **kw), dev(xd, xd, xd, **kd)
            close(od, oc)
            assert (wc is None) == (wd is None)
            if wc is not None:
                close(wd, wc)
    assert calls["mha"] == 7

    for act, norm_first in (("relu", False), ("gelu", True)):
        torch.manual_seed(1)
        make = lambda: torch.nn.TransformerEncoderLayer(D, H, 64, dropout=0.0, activation=act, batch_first=True, norm_first=norm_first)
        ref, dev = make().eval(), make()
        dev.load_state_dict(ref.state_dict())
        dev = dev.to(vk).eval()
        before = calls["layer"]
        with torch.no_grad():
            close(dev(xd), ref(x), 5e-5)
            close(dev(xd, src_key_padding_mask=pad.to(vk)), ref(x, src_key_padding_mask=pad), 5e-5)
            close(dev(xd, src_mask=causal.to(vk)), ref(x, src_mask=causal), 5e-5)
        assert calls["layer"] == before + 3

    torch.manual_seed(2)
    make = lambda: torch.nn.TransformerEncoder(torch.nn.TransformerEncoderLayer(D, H, 64, dropout=0.0, batch_first=True), 2)
    ref, dev = make().eval(), make()
    dev.load_state_dict(ref.state_dict())
    dev = dev.to(vk).eval()
    with torch.no_grad():
        yc, yd = ref(x, src_key_padding_mask=pad), dev(xd, src_key_padding_mask=pad.to(vk))
    close(yd, yc, 1e-4, rows=valid)                       # ATen CPU packs the batch and returns zeros at the padding

    torch.manual_seed(3)
    half = torch.nn.MultiheadAttention(64, 4, batch_first=True).eval()
    dhalf = torch.nn.MultiheadAttention(64, 4, batch_first=True)
    dhalf.load_state_dict(half.state_dict())
    dhalf = dhalf.half().to(vk).eval()
    xh = torch.randn(2, 128, 64, generator=g)
    with torch.no_grad():
        oc = half(xh, xh, xh, need_weights=False)[0]
        od = dhalf(xh.half().to(vk), xh.half().to(vk), xh.half().to(vk), need_weights=False)[0]
    close(od, oc, 1e-2)
