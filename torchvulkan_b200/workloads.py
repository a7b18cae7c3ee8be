"""The reference's example training steps written as sequences of tvk C-ABI launches.

``MLPStep`` is the model of examples/mlp.py:5-23 (Linear -> GELU -> ... -> Linear, mean
cross-entropy) with the AdamW step of examples/mlp.py:41, issued in the order PyTorch's eager
autograd issues the ATen ops to a backend (addmm, gelu, ..., _log_softmax, nll_loss_forward,
nll_loss_backward, _log_softmax_backward_data, mm x5, gelu_backward x2, sum.dim x3, then one
fused Adam launch per parameter, or one list launch for all parameters with the step count held in
device memory). Buffers are allocated once; a step allocates nothing, so a whole step can also be
captured once into a CUDA graph and replayed (``capture`` / ``replay``).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from . import cuda_ops as ops


class MLPStep:
    def __init__(self, sizes=(784, 8192, 8192, 10), batch=256, dtype=torch.float16, device="cuda", seed=0,
                 lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, params=None, list_optimizer=False, loss_scale=1.0, fused=False, fuse_forward=None):
        self.sizes, self.batch, self.dtype, self.device = tuple(sizes), batch, dtype, torch.device(device)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.nl = len(sizes) - 1
        if params is None:
            # nn.Linear's default init, generated on the CPU from a fixed seed so that the CPU oracle
            # and the device see the same bits.
            g = torch.Generator().manual_seed(seed)
            ws, bs = [], []
            for i in range(self.nl):
                bound = 1.0 / (sizes[i] ** 0.5)
                ws.append(((torch.rand(sizes[i + 1], sizes[i], generator=g) * 2 - 1) * bound).to(dtype))
                bs.append(((torch.rand(sizes[i + 1], generator=g) * 2 - 1) * bound).to(dtype))
            params = (ws, bs)
        dev = self.device
        self.w = [w.to(dev).contiguous() for w in params[0]]
        self.b = [b.to(dev).contiguous() for b in params[1]]
        self.params = [t for pair in zip(self.w, self.b) for t in pair]
        self.gw = [torch.empty_like(w) for w in self.w]
        self.gb = [torch.empty_like(b) for b in self.b]
        self.grads = [t for pair in zip(self.gw, self.gb) for t in pair]
        self.m = [torch.zeros_like(p) for p in self.params]
        self.v = [torch.zeros_like(p) for p in self.params]
        self.step_count = 0
        # list_optimizer: one tvk_adam_step_multi launch for all parameters, step count in device memory (as
        # torch.optim keeps it for fused optimizers) and advanced on the device: the step is then replayable
        self.list_optimizer = list_optimizer
        # fused: gelu_backward is applied by the epilogue of the input-gradient product (the saved pre-activation is its
        # aux operand; its factors are formed while the product streams the weights, so the launch costs what the plain
        # product costs) wherever that product is long enough to hide them (k >= 1024). fuse_forward also lets the addmm
        # epilogue write gelu(z) next to z (two outputs from one accumulator); measured on B200 that second pass over the
        # accumulator costs more than the separate gelu launch it saves at batch 256, so it is off unless asked for.
        self.fused = fused
        self.fuse_forward = bool(fuse_forward) if fuse_forward is not None else False
        self.step_dev = torch.zeros((), dtype=torch.float32, device=dev)
        self._adam_items = (capi.MultiItem * len(self.params))()
        for i, (p, g, m, v) in enumerate(zip(self.params, self.grads, self.m, self.v)):
            self._adam_items[i].ptr[0], self._adam_items[i].ptr[1] = p.data_ptr(), g.data_ptr()
            self._adam_items[i].ptr[2], self._adam_items[i].ptr[3] = m.data_ptr(), v.data_ptr()
            self._adam_items[i].numel, self._adam_items[i].step = p.numel(), self.step_dev.data_ptr()
        self._step_item = (capi.MultiItem * 1)()
        self._step_item[0].ptr[0], self._step_item[0].numel = self.step_dev.data_ptr(), 1
        self._graph = None
        e = lambda *s: torch.empty(*s, dtype=dtype, device=dev)  # noqa: E731
        self.z = [e(batch, sizes[i + 1]) for i in range(self.nl)]          # pre-activations (last = logits)
        self.h = [e(batch, sizes[i + 1]) for i in range(self.nl - 1)]      # activations
        self.gz = [e(batch, sizes[i + 1]) for i in range(self.nl)]         # grads wrt pre-activations
        self.gh = [e(batch, sizes[i + 1]) for i in range(self.nl - 1)]     # grads wrt activations
        self.logp = e(batch, sizes[-1])
        self.glogp = e(batch, sizes[-1])
        self.lse = torch.empty(batch, dtype=torch.float32, device=dev)       # row log-sum-exp of the logits (fused cross-entropy)
        self.loss = e(())
        self.total_w = e(())
        # gradient of the (scaled) loss with respect to the mean loss: backward runs on loss * loss_scale. fp16 moments of
        # unscaled gradients underflow; with eps scaled by the same factor the AdamW update is the unscaled one exactly.
        self.loss_scale = float(loss_scale)
        self.one = torch.full((), self.loss_scale, dtype=dtype, device=dev)
        self.launches_per_step = 0
        self._descs, self._desc_key = None, None
        self.trace = None   # list of (tag, start_event, end_event) when per-launch timing is on
        # one shared workspace, sized for the largest request of any launch in the step
        self._ws = torch.empty(self._workspace_bytes(), dtype=torch.uint8, device=dev)

    # -- helpers -----------------------------------------------------------------------
    def _gemm_descs(self, x):
        """All GEMMs of one step as (desc, tag); built per call because x may move."""
        d = []
        inp = x

        def supported(desc):
            # a fused form the library cannot run (an operand the tensor-core path cannot address) answers an error
            # here; that product is then issued as the separate operators
            p = C.c_int(0)
            return capi.lib().tvk_gemm_path(C.byref(desc), C.byref(p)) == 0

        self._fused_fwd, self._fused_bwd = [False] * self.nl, [False] * self.nl
        for i in range(self.nl):
            plain = ops.gemm_desc(inp, self.w[i].t(), self.z[i], bias=self.b[i])        # addmm
            if (self.fuse_forward or self.fused) and i < self.nl - 1:
                both = ops.gemm_desc(inp, self.w[i].t(), self.z[i], bias=self.b[i], act="gelu", out2=self.h[i])       # addmm + gelu
                # inside the tensor-core epilogue the second store costs more than the separate gelu launch saves (measured);
                # where the product runs as K slices, the finishing pass stores both for free
                if supported(both) and (self.fuse_forward or ops.gemm_splits(both) > 1):
                    self._fused_fwd[i] = True
                    plain = both
            d.append(plain)
            inp = self.h[i] if i < self.nl - 1 else None
        for i in reversed(range(self.nl)):
            act_in = x if i == 0 else self.h[i - 1]
            d.append(ops.gemm_desc(self.gz[i].t(), act_in, self.gw[i]))                  # wgrad = gz^T @ in
            if i > 0:
                plain = ops.gemm_desc(self.gz[i], self.w[i], self.gh[i - 1])             # dgrad = gz @ W
                # (a product over a classifier's few outputs takes the output-bound small-k kernel, which applies aux in registers)
                if self.fused and (self.sizes[i + 1] >= 1024 or self.sizes[i + 1] <= 16):
                    both = ops.gemm_desc(self.gz[i], self.w[i], self.gz[i - 1], aux=self.z[i - 1], aux_op="gelu_backward")   # mm + gelu_backward
                    self._fused_bwd[i] = supported(both)
                    plain = both if self._fused_bwd[i] else plain
                d.append(plain)
        return d

    def _workspace_bytes(self):
        x = torch.empty(self.batch, self.sizes[0], dtype=self.dtype, device=self.device)
        need = 0
        for d in self._gemm_descs(x):
            n = C.c_uint64(0)
            capi.call("tvk_gemm_workspace_size", C.byref(d), C.byref(n))
            need = max(need, n.value)
        for i in range(self.nl):
            n = C.c_uint64(0)
            capi.call("tvk_reduce_workspace_size", 1, self.batch, self.sizes[i + 1], C.byref(n))
            need = max(need, n.value)
        n = C.c_uint64(0)
        capi.call("tvk_cross_entropy_workspace_size", self.batch, C.byref(n))
        return max(need, n.value, 256)

    def _timed(self, tag, fn):
        """Runs one launch; with `self.trace` set, brackets it with CUDA events on the launch stream."""
        self.launches_per_step += 1
        if self.trace is None:
            fn()
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        self.trace.append((tag, a, b))

    def _gemm(self, d, tag="gemm"):
        tag = f"{tag} m{d.m} n{d.n} k{d.k}"
        self._timed(tag, lambda: capi.call("tvk_gemm", C.byref(d), self._ws.data_ptr(), self._ws.numel(), ops.stream()))

    def _call(self, name, *args, tag=None):
        self._timed(tag or name, lambda: capi.call(name, *args, ops.stream()))

    # -- the step ----------------------------------------------------------------------
    def forward_backward(self, x, labels):
        s = self
        s.launches_per_step = 0
        dtc = ops.dt(x)
        # the descriptors only depend on the buffer addresses: rebuild them when x moves
        if s._desc_key != x.data_ptr():
            s._descs, s._desc_key = s._gemm_descs(x), x.data_ptr()
        descs = s._descs
        k = 0
        for i in range(s.nl):
            s._gemm(descs[k]); k += 1
            if i < s.nl - 1 and not s._fused_fwd[i]:
                s._call("tvk_unary", capi.U_GELU, dtc, s.h[i].data_ptr(), s.z[i].data_ptr(), s.z[i].numel())
        n, c = s.batch, s.sizes[-1]
        if s.fused:
            # cross-entropy as one pass over the logits each way (log_softmax + nll_loss without the table of log-probabilities)
            s._call("tvk_cross_entropy_forward", dtc, s.loss.data_ptr(), s.total_w.data_ptr(), s.lse.data_ptr(), s.z[-1].data_ptr(), labels.data_ptr(),
                    None, n, c, 1, -100, s._ws.data_ptr(), s._ws.numel())
            s._call("tvk_cross_entropy_backward", dtc, s.gz[-1].data_ptr(), s.one.data_ptr(), s.z[-1].data_ptr(), s.lse.data_ptr(), labels.data_ptr(),
                    None, s.total_w.data_ptr(), n, c, 1, -100)
        else:
            s._call("tvk_softmax_forward", 1, dtc, dtc, s.logp.data_ptr(), s.z[-1].data_ptr(), n, c)
            s._call("tvk_nll_loss_forward", dtc, s.loss.data_ptr(), s.total_w.data_ptr(), s.logp.data_ptr(), labels.data_ptr(), None, n, c, 1, -100)
            s._call("tvk_nll_loss_backward", dtc, s.glogp.data_ptr(), s.one.data_ptr(), labels.data_ptr(), None, s.total_w.data_ptr(), n, c, 1, -100)
            s._call("tvk_softmax_backward", 1, dtc, s.gz[-1].data_ptr(), s.glogp.data_ptr(), s.logp.data_ptr(), n, c)
        for i in reversed(range(s.nl)):
            s._gemm(descs[k]); k += 1                                                    # grad W_i
            s._call("tvk_reduce", capi.R_SUM, dtc, dtc, s.gb[i].data_ptr(), s.gz[i].data_ptr(), 1, n, s.sizes[i + 1],
                    s._ws.data_ptr(), s._ws.numel(), tag=f"sum.dim0 {n}x{s.sizes[i + 1]}")  # grad b_i
            if i > 0:
                s._gemm(descs[k]); k += 1                                                # grad h_{i-1} (fused: grad z_{i-1})
                if s._fused_bwd[i]:
                    continue
                s._call("tvk_binary", capi.B_GELU_BACKWARD, dtc, s.gz[i - 1].data_ptr(), s.gh[i - 1].data_ptr(), s.z[i - 1].data_ptr(),
                        0.0, 1.0, s.gz[i - 1].numel())
        return s.loss

    def optimizer_step(self):
        s = self
        s.step_count += 1
        if s.list_optimizer:
            s._call("tvk_foreach_axpby", capi.F32, s._step_item, 1, 1.0, 0.0, 1.0, 0, tag="step += 1")
            s._call("tvk_adam_step_multi", ops.dt(s.params[0]), s._adam_items, len(s.params), s.lr, s.betas[0], s.betas[1], s.eps, s.wd, 0, 1, 0,
                    tag=f"adam_step_multi n{s.num_params()}")
            return
        for p, g, m, v in zip(s.params, s.grads, s.m, s.v):
            s._call("tvk_adam_step", ops.dt(p), p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), s.lr, s.betas[0],
                    s.betas[1], s.eps, s.wd, s.step_count, 1, 0, tag=f"adam_step n{p.numel()}")

    def step(self, x, labels):
        loss = self.forward_backward(x, labels)
        self.optimizer_step()
        return loss

    # -- whole-step replay ---------------------------------------------------------------
    def capture(self, x, labels):
        """Records one step on (x, labels) into a CUDA graph. Needs list_optimizer (a host step count would be frozen
        into the graph) and at least one ordinary step before it (first launches set kernel attributes)."""
        if not self.list_optimizer:
            raise ValueError("capture() needs list_optimizer=True")
        self.trace = None
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step(x, labels)
        self.step_count -= 1          # the capture pass recorded the launches, it did not run them
        self._graph = graph
        return graph

    def replay(self):
        self.step_count += 1
        self._graph.replay()
        return self.loss

    # -- bookkeeping for the bench -------------------------------------------------------
    def gemm_flops(self):
        f = 0
        for i in range(self.nl):
            f += 2 * self.batch * self.sizes[i] * self.sizes[i + 1]          # forward
            f += 2 * self.batch * self.sizes[i] * self.sizes[i + 1]          # wgrad
            if i > 0:
                f += 2 * self.batch * self.sizes[i] * self.sizes[i + 1]      # dgrad
        return f

    def num_params(self):
        return sum(p.numel() for p in self.params)
