"""Batch-sharded bmm across the GPUs of one node: every rank owns a slice of the batches and all ranks
end with the full product.

The reference has no multi-device operator: its `vulkan:i` devices are independent
(src/vulkan/vulkan_context.cpp:626-631) and a user shards by hand. Here device `vulkan:r` is CUDA device
r, one process per GPU (`torch.distributed`), and three ways of completing the output exist:

  "push"       the GEMM epilogue stores every finished tile into all ranks' copies of C (peer-mapped
               pointers over NVLink, `tvk_gemm_desc.peer_c`), so the gather costs no extra pass over C and
               overlaps the tensor-core work tile by tile; one barrier orders the step.
  "copy"       the local batches are cut into chunks; as soon as a chunk is multiplied it is copied into every
               peer's C by the copy engines (one `tvk_memcpy_async` per chunk and peer on side streams, peers'
               buffers mapped as for "push"), which take no SM away from the product of the next chunk.
  "pipelined"  the local batches are cut into chunks; chunk i's NCCL exchange runs on a side stream while
               chunk i+1 is multiplied.
  "allgather"  the whole local GEMM, then one NCCL all-gather: the unfused baseline.

Units are batches: rank r owns `shard_range(batch, r, world)`. Nothing here falls back to another device:
the compute callable defaults to the tcgen05 GEMM of the C-ABI and raises if the library is missing.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

__all__ = ["shard_range", "PeerViews", "ShardedBmm"]


def shard_range(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of batches rank `rank` owns: contiguous, sizes differ by at most one, larger ones first."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside [0, {world})")
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class PeerViews:
    """Addresses, in this process, of the same-shaped buffer of every rank (this rank's own included)."""

    def __init__(self, tensor: torch.Tensor, group=None):
        from . import capi

        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._capi = capi
        mine = capi.IpcHandle()
        capi.call("tvk_ipc_export", tensor.data_ptr(), C.byref(mine))
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(mine), group=group)
        self.ptrs: list[int] = []
        self._opened: list[int] = []
        for r, blob in enumerate(blobs):
            if r == self.rank:
                self.ptrs.append(tensor.data_ptr())
                continue
            handle = capi.IpcHandle.from_buffer_copy(blob)
            p = C.c_void_p()
            capi.call("tvk_ipc_open", C.byref(handle), C.byref(p))
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        self._keepalive = tensor

    def close(self):
        """Unmaps the peers' buffers. Collective: every rank must be done writing before any owner frees."""
        if self._opened:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            for p in self._opened:
                self._capi.call("tvk_ipc_close", p)
            self._opened = []


class ShardedBmm:
    """out_full[b] = a[b] @ b[b] for all `batch` batches, with a_shard/b_shard holding this rank's batches.

    out_full is a [batch, m, n] tensor every rank allocates; after `run()` returns and the stream is synchronised
    every rank's out_full holds the complete product. Work that reads out_full must be issued on the same stream
    before the next `run()`: in "push" mode that next call begins with a rendezvous of all ranks on that stream, so no
    peer overwrites the buffer while a reader of the previous result is still running.
    """

    def __init__(self, out_full: torch.Tensor, mode: str = "push", group=None, chunks: int = 4, compute=None):
        if mode not in ("push", "copy", "pipelined", "allgather"):
            raise ValueError(f"unknown mode {mode!r}")
        self.out, self.mode, self.group = out_full, mode, group
        # without a process group this is the single-device case: one rank that owns every batch
        self.rank, self.world = (dist.get_rank(group), dist.get_world_size(group)) if dist.is_initialized() else (0, 1)
        self.batch = out_full.shape[0]
        self.lo, self.hi = shard_range(self.batch, self.rank, self.world)
        self.mine = out_full[self.lo:self.hi]
        # the same chunk boundaries on every rank: derived from the longest slice, not from this rank's
        self.chunks = max(1, min(chunks, (self.batch + self.world - 1) // self.world))
        self._compute = compute
        self._peers = None
        self._side = None
        self._descs = {}
        self._flag = None
        self._copy_streams = []
        if self.world > 1 and mode in ("push", "copy"):
            self._peers = PeerViews(out_full, group)
            self._flag = torch.zeros(1, device=out_full.device)
        if self.world > 1 and mode == "copy":
            self._copy_streams = [torch.cuda.Stream(device=out_full.device) for _ in range(self.world - 1)]
        if self.world > 1 and mode == "pipelined" and out_full.is_cuda:
            self._side = torch.cuda.Stream(device=out_full.device)

    # ---- local product ---------------------------------------------------------------------------
    def _gemm(self, a, b, out, peer_ptrs=()):
        if self._compute is not None:
            return self._compute(a, b, out)
        from . import capi, cuda_ops as ops

        key = (a.data_ptr(), b.data_ptr(), out.data_ptr(), tuple(peer_ptrs))
        d = self._descs.get(key)
        if d is None:
            d = ops.gemm_desc(a, b, out)
            d.n_peer_c = len(peer_ptrs)
            for i, p in enumerate(peer_ptrs):
                d.peer_c[i] = p
            need = C.c_uint64(0)
            capi.call("tvk_gemm_workspace_size", C.byref(d), C.byref(need))
            ws = torch.empty(need.value, dtype=torch.uint8, device=out.device) if need.value else None
            self._descs[key] = d = (d, ws, need.value)
        desc, ws, nbytes = d
        capi.call("tvk_gemm", C.byref(desc), ops.ptr(ws), nbytes, ops.stream())

    def _exchange(self, lo_off: int, hi_off: int):
        """All ranks exchange local batches [lo_off, hi_off) of their slices (equal slice sizes: one NCCL group of sends/receives)."""
        ops_ = []
        for r in range(self.world):
            if r == self.rank:
                continue
            rlo, rhi = shard_range(self.batch, r, self.world)
            s, e = min(rlo + lo_off, rhi), min(rlo + hi_off, rhi)
            ms, me = min(self.lo + lo_off, self.hi), min(self.lo + hi_off, self.hi)
            if me > ms:
                ops_.append(dist.P2POp(dist.isend, self.out[ms:me], r, group=self.group))
            if e > s:
                ops_.append(dist.P2POp(dist.irecv, self.out[s:e], r, group=self.group))
        if ops_:
            for w in dist.batch_isend_irecv(ops_):
                w.wait()

    # ---- one step ------------------------------------------------------------------------------------
    def run(self, a_shard: torch.Tensor, b_shard: torch.Tensor) -> torch.Tensor:
        nb = self.hi - self.lo
        if self.world == 1:
            if nb:
                self._gemm(a_shard, b_shard, self.mine)
            return self.out
        if self.mode == "push":
            # Peers store into this rank's out_full: no rank may start writing step k+1 while another rank's kernels
            # still read step k's result. The same 4-byte all-reduce, ordered on each rank's stream after whatever
            # consumed out_full there, holds every rank's GEMM back until all ranks have reached this point.
            dist.all_reduce(self._flag, group=self.group)
            if nb:
                esz = self.out.element_size()
                off = self.lo * self.out.stride(0) * esz
                peers = [p + off for r, p in enumerate(self._peers.ptrs) if r != self.rank]
                self._gemm(a_shard, b_shard, self.mine, peers)
            # Stream-ordered rendezvous: a rank leaves it only after every rank's GEMM, and with it every store into
            # this rank's copy, has completed.
            dist.all_reduce(self._flag, group=self.group)
            return self.out
        if self.mode == "copy":
            from . import capi
            dist.all_reduce(self._flag, group=self.group)       # as for "push": nobody still reads the previous result
            main = torch.cuda.current_stream()
            esz = self.out.element_size()
            step = max(1, (nb + self.chunks - 1) // self.chunks) if nb else 1
            for c0 in range(0, nb, step):
                c1 = min(c0 + step, nb)
                self._gemm(a_shard[c0:c1], b_shard[c0:c1], self.mine[c0:c1])
                done = torch.cuda.Event()
                done.record(main)
                off = (self.lo + c0) * self.out.stride(0) * esz
                nbytes = (c1 - c0) * self.out.stride(0) * esz
                # peers in rotated order so that the ranks do not all send to the same GPU first
                for j in range(1, self.world):
                    r = (self.rank + j) % self.world
                    st = self._copy_streams[j - 1]
                    st.wait_event(done)
                    capi.call("tvk_memcpy_async", self._peers.ptrs[r] + off, self.out.data_ptr() + off, nbytes, st.cuda_stream)
            for st in self._copy_streams:
                main.wait_stream(st)
            dist.all_reduce(self._flag, group=self.group)
            return self.out
        if self.mode == "allgather":
            if nb:
                self._gemm(a_shard, b_shard, self.mine)
            if self.batch % self.world == 0:
                dist.all_gather_into_tensor(self.out, self.mine, group=self.group)
            else:
                self._exchange(0, (self.batch + self.world - 1) // self.world)
            return self.out
        # pipelined
        longest = (self.batch + self.world - 1) // self.world
        step = (longest + self.chunks - 1) // self.chunks
        main = torch.cuda.current_stream() if self._side is not None else None
        for c0 in range(0, longest, step):
            c1 = min(c0 + step, longest)
            s, e = min(c0, nb), min(c1, nb)
            if e > s:
                self._gemm(a_shard[s:e], b_shard[s:e], self.mine[s:e])
            if self._side is None:      # host tensors (the CPU tests): no streams, same order of exchanges
                self._exchange(c0, c1)
                continue
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                self._exchange(c0, c1)
        if self._side is not None:
            main.wait_stream(self._side)
        return self.out

    def close(self):
        if self._peers is not None:
            self._peers.close()
            self._peers = None
