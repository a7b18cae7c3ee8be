"""Generates tests/golden/aten_cpu.npz: ATen-CPU outputs on small seeded inputs.

ATen's CPU kernels are the reference's own CPU path for every op on the hot path (its fallback
is at::native::cpu_fallback, src/api/fallback.cpp:5-9, and its test-suite ground truth,
tests/test_pytorch_ops.py:203-243). The reference ships no golden vectors, so these are the
frozen known answers the numpy oracle is pinned against. Run from the repository root:

    python tests/golden/make_golden.py

The torch version that produced the committed file is stored inside it.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F


def main() -> None:
    torch.manual_seed(1234)
    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}

    def put(name, t):
        # copy: optimizers update tensors in place after they were recorded
        out[name] = t.detach().cpu().numpy().copy() if isinstance(t, torch.Tensor) else np.asarray(t)

    # argmax / argmin with ties and NaN (src/shaders/ops/arg_reduce.slang:49-65)
    x = torch.randn(6, 37)
    x[1, 5] = x[1, 20] = x[1].max() + 1.0          # tie: first wins
    x[2, 30] = float("nan"); x[2, 11] = float("nan")  # first NaN wins
    x[3, :] = 0.5                                   # all equal
    x[4, 0] = float("inf")
    put("arg_x", x)
    put("argmax_d1", torch.argmax(x, 1)); put("argmin_d1", torch.argmin(x, 1))
    put("argmax_d0", torch.argmax(x, 0)); put("argmax_flat", torch.argmax(x))

    # stable sort / topk with ties, NaN and signed zeros (src/shaders/ops/sort.slang:24-49)
    s = torch.randn(5, 50).round(decimals=1)
    s[0, 3] = float("nan"); s[0, 40] = float("nan"); s[1, 7] = 0.0; s[1, 9] = -0.0
    put("sort_x", s)
    for desc in (False, True):
        v, i = torch.sort(s, dim=-1, descending=desc, stable=True)
        put(f"sort_v_desc{int(desc)}", v); put(f"sort_i_desc{int(desc)}", i)

    # GELU (erf) forward / backward (src/shaders/core/dtype.slang:736-744)
    gx = torch.linspace(-6, 6, 97, dtype=torch.float64).requires_grad_()
    gy = F.gelu(gx)
    gg = torch.randn(97, dtype=torch.float64)
    put("gelu_x", gx); put("gelu_y", gy); put("gelu_g", gg)
    put("gelu_gx", torch.autograd.grad(gy, gx, gg)[0])

    # log_softmax + nll_loss (src/api/decompositions.cpp:506-571, src/api/ops/nllloss.cpp:79-174)
    logits = torch.randn(9, 7, dtype=torch.float64, requires_grad=True)
    tgt = torch.tensor([0, 6, 3, -100, 2, 2, 5, -100, 1])
    w = torch.rand(7, dtype=torch.float64) + 0.5
    lp = F.log_softmax(logits, -1)
    put("lsm_x", logits); put("lsm_y", lp); put("nll_t", tgt); put("nll_w", w)
    for red in ("mean", "sum", "none"):
        for wt, tag in ((None, "nw"), (w, "w")):
            loss = F.nll_loss(lp, tgt, weight=wt, reduction=red)
            put(f"nll_{red}_{tag}", loss)
            go = torch.ones_like(loss) if red != "none" else torch.arange(1, 10, dtype=torch.float64)
            put(f"nll_{red}_{tag}_glp", torch.autograd.grad(loss, lp, go, retain_graph=True)[0])
    put("lsm_gx", torch.autograd.grad(lp, logits, torch.randn(9, 7, dtype=torch.float64, generator=torch.Generator().manual_seed(5)))[0])
    put("lsm_g", torch.randn(9, 7, dtype=torch.float64, generator=torch.Generator().manual_seed(5)))
    sm_in = torch.randn(4, 33, dtype=torch.float64)
    put("sm_x", sm_in); put("sm_y", F.softmax(sm_in, -1))

    # AdamW / SGD single and second steps (src/api/ops/optim.cpp:46-86, 195-205)
    p0 = torch.randn(301); g1 = torch.randn(301); g2 = torch.randn(301)
    p = p0.clone().requires_grad_()
    opt = torch.optim.AdamW([p], lr=1e-3, weight_decay=1e-2)
    put("adam_p0", p0); put("adam_g1", g1); put("adam_g2", g2)
    p.grad = g1.clone(); opt.step(); put("adam_p1", p)
    put("adam_m1", opt.state[p]["exp_avg"]); put("adam_v1", opt.state[p]["exp_avg_sq"])
    p.grad = g2.clone(); opt.step(); put("adam_p2", p)
    p = p0.clone().requires_grad_()
    opt = torch.optim.SGD([p], lr=0.1, momentum=0.9)
    p.grad = g1.clone(); opt.step(); put("sgd_p1", p)
    p.grad = g2.clone(); opt.step(); put("sgd_p2", p); put("sgd_buf2", opt.state[p]["momentum_buffer"])

    # batch norm training fwd/bwd (src/shaders/ops/norm.slang:72-191)
    bx = (torch.randn(5, 4, 3, 3, dtype=torch.float64) * 2 + 1).requires_grad_()
    bw = torch.rand(4, dtype=torch.float64) + 0.5; bb = torch.randn(4, dtype=torch.float64)
    rm = torch.zeros(4, dtype=torch.float64); rv = torch.ones(4, dtype=torch.float64)
    by = F.batch_norm(bx, rm, rv, bw.requires_grad_(), bb.requires_grad_(), training=True, momentum=0.1, eps=1e-5)
    bg = torch.randn_like(by)
    gxx, gww, gbb = torch.autograd.grad(by, (bx, bw, bb), bg)
    for k, v in dict(bn_x=bx, bn_w=bw, bn_b=bb, bn_y=by, bn_rm=rm, bn_rv=rv, bn_g=bg, bn_gx=gxx, bn_gw=gww, bn_gb=gbb).items():
        put(k, v)

    # RMSNorm fwd/bwd (src/api/ops/norm.cpp:169-260)
    rx = torch.randn(6, 40, dtype=torch.float64, requires_grad=True)
    rw = (torch.rand(40, dtype=torch.float64) + 0.5).requires_grad_()
    ry = F.rms_norm(rx, (40,), rw, eps=float(torch.finfo(torch.float32).eps))
    rg = torch.randn_like(ry)
    rgx, rgw = torch.autograd.grad(ry, (rx, rw), rg)
    for k, v in dict(rms_x=rx, rms_w=rw, rms_y=ry, rms_g=rg, rms_gx=rgx, rms_gw=rgw).items():
        put(k, v)

    # embedding backward (src/shaders/ops/embedding_backward.slang:36-56)
    table = torch.randn(11, 8, requires_grad=True)
    idx = torch.randint(0, 11, (4, 9))
    eo = F.embedding(idx, table)
    eg = torch.randn_like(eo)
    put("emb_idx", idx); put("emb_g", eg); put("emb_table", table); put("emb_out", eo)
    put("emb_gt", torch.autograd.grad(eo, table, eg)[0])

    # config 1 at reduced size: fp32 mm -> relu -> sum, with an fp64 value beside it
    a = torch.randn(96, 80); b = torch.randn(80, 72)
    put("c1_a", a); put("c1_b", b)
    put("c1_z", (a @ b).relu()); put("c1_s64", (a.double() @ b.double()).relu().sum())

    # config 2 at reduced size: MLP fwd+bwd in fp64 (examples/mlp.py:5-23)
    sizes = (20, 32, 32, 10)
    ws = [torch.randn(sizes[i + 1], sizes[i], dtype=torch.float64) * 0.2 for i in range(3)]
    bs = [torch.randn(sizes[i + 1], dtype=torch.float64) * 0.1 for i in range(3)]
    for t in ws + bs:
        t.requires_grad_()
    mx = torch.randn(16, 20, dtype=torch.float64)
    ml = torch.randint(0, 10, (16,))
    h = mx
    for i in range(3):
        h = F.linear(h, ws[i], bs[i])
        if i < 2:
            h = F.gelu(h)
    loss = F.cross_entropy(h, ml)
    grads = torch.autograd.grad(loss, ws + bs)
    put("mlp_x", mx); put("mlp_labels", ml); put("mlp_loss", loss); put("mlp_logits", h)
    for i in range(3):
        put(f"mlp_w{i}", ws[i]); put(f"mlp_b{i}", bs[i]); put(f"mlp_gw{i}", grads[i]); put(f"mlp_gb{i}", grads[3 + i])

    # conv2d forward and both gradients in float64: stride 1 and 2, padding, odd extents, 1x1 and 3x3 filters
    # (the cases of tests/test_pytorch_ops.py's conv2d entries and of the ResNet blocks)
    conv_cases = {"a": (2, 3, 9, 7, 5, 3, 3, 1, 1), "b": (2, 4, 8, 8, 6, 3, 3, 2, 1), "c": (1, 5, 7, 9, 4, 1, 1, 2, 0),
                  "d": (2, 2, 6, 5, 3, 2, 3, 1, 0), "e": (1, 3, 10, 10, 2, 7, 7, 2, 3)}
    for name, (n, ci, hh, ww, co, kh, kw, st, pd) in conv_cases.items():
        cx = torch.randn(n, ci, hh, ww, dtype=torch.float64, requires_grad=True)
        cw = torch.randn(co, ci, kh, kw, dtype=torch.float64, requires_grad=True)
        cy = F.conv2d(cx, cw, None, stride=st, padding=pd)
        cg = torch.randn_like(cy)
        gx, gw = torch.autograd.grad(cy, (cx, cw), cg)
        put(f"conv_{name}_cfg", np.array([st, pd]))
        put(f"conv_{name}_x", cx); put(f"conv_{name}_w", cw); put(f"conv_{name}_y", cy)
        put(f"conv_{name}_gy", cg); put(f"conv_{name}_gx", gx); put(f"conv_{name}_gw", gw)

    out["torch_version"] = np.array(torch.__version__)
    path = Path(__file__).resolve().parent / "aten_cpu.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes,", len(out), "arrays")


def main_rowops() -> None:
    """tests/golden/aten_cpu_rowops.npz: LayerNorm, GroupNorm, cross-entropy and the scans (a file of its own so that adding
    it left the first file's random stream, and with it every committed value there, untouched)."""
    torch.manual_seed(4321)
    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}

    def put(name, t):
        out[name] = t.detach().cpu().numpy().copy() if isinstance(t, torch.Tensor) else np.asarray(t)

    # layer_norm forward + backward over one and two trailing axes (src/api/ops/norm.cpp:264-325)
    for tag, shape, nd in (("a", (5, 7, 24), 1), ("b", (4, 6, 10), 2)):
        x = torch.randn(*shape, dtype=torch.float64, requires_grad=True)
        w = (torch.rand(shape[-nd:], dtype=torch.float64) + 0.5).requires_grad_()
        b = torch.randn(shape[-nd:], dtype=torch.float64, requires_grad=True)
        y = F.layer_norm(x, shape[-nd:], w, b, 1e-5)
        g = torch.randn_like(y)
        gx, gw, gb = torch.autograd.grad(y, (x, w, b), g)
        for k, v in (("x", x), ("w", w), ("b", b), ("y", y), ("g", g), ("gx", gx), ("gw", gw), ("gb", gb)):
            put(f"ln_{tag}_{k}", v)
        put(f"ln_{tag}_nd", np.array(nd))
    # group_norm forward + backward
    x = torch.randn(3, 12, 5, 4, dtype=torch.float64, requires_grad=True)
    w = (torch.rand(12, dtype=torch.float64) + 0.5).requires_grad_()
    b = torch.randn(12, dtype=torch.float64, requires_grad=True)
    y = F.group_norm(x, 4, w, b, 1e-5)
    g = torch.randn_like(y)
    gx, gw, gb = torch.autograd.grad(y, (x, w, b), g)
    for k, v in (("x", x), ("w", w), ("b", b), ("y", y), ("g", g), ("gx", gx), ("gw", gw), ("gb", gb)):
        put(f"gn_{k}", v)
    # cross_entropy: mean / sum / none, class weights, ignored targets
    logits = torch.randn(11, 9, dtype=torch.float64, requires_grad=True)
    tgt = torch.tensor([0, 8, 3, -100, 2, 2, 5, -100, 1, 7, 4])
    w = torch.rand(9, dtype=torch.float64) + 0.5
    put("ce_x", logits); put("ce_t", tgt); put("ce_w", w)
    for red in ("mean", "sum", "none"):
        for use_w in (0, 1):
            loss = F.cross_entropy(logits, tgt, weight=w if use_w else None, reduction=red)
            go = torch.randn_like(loss)
            gl, = torch.autograd.grad(loss, logits, go)
            put(f"ce_{red}_w{use_w}_loss", loss); put(f"ce_{red}_w{use_w}_go", go); put(f"ce_{red}_w{use_w}_gx", gl)
    # scans
    s = torch.randn(4, 9, 5, dtype=torch.float64)
    put("scan_x", s)
    for d in (0, 1, 2):
        put(f"cumsum_d{d}", torch.cumsum(s, d)); put(f"cumprod_d{d}", torch.cumprod(s, d)); put(f"logcumsumexp_d{d}", torch.logcumsumexp(s, d))
    si = torch.randint(-3, 4, (3, 17))
    put("scan_i", si); put("cumsum_i", torch.cumsum(si, 1)); put("cumprod_i", torch.cumprod(si, 1))
    out["torch_version"] = np.array(torch.__version__)
    path = Path(__file__).resolve().parent / "aten_cpu_rowops.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    import sys

    if "--rowops-only" not in sys.argv:
        main()
    main_rowops()
