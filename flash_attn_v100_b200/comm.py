"""Peer-memory collectives for the tensor-parallel decode step (one process per GPU).

`PeerCollectives` owns this rank's data buffer (plain `cudaMalloc` memory shared with the other
ranks of the node through CUDA IPC handles, exchanged over the `torch.distributed` group) and
launches the library's all-reduce / all-gather kernels on PyTorch's current stream.  The kernels use
plain peer loads and stores over NVLink (no multicast) and can be captured into a CUDA graph, which
NCCL calls in this engine are not.  They stand where the reference calls `dist.all_reduce` and
`dist.all_gather` (flash_attn_llm/parallel/tensor_parallel.py:152-190).

Usage: write the input straight into a view of the buffer (`view()`, e.g. as the `out=` of the
matmul that produces it), call `all_reduce_(view)`, read the result from the same view.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


class _Span:
    """Device memory exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def slice_bounds(n_elems: int, world: int, rank: int):
    """Elements [lo, hi) that rank `rank` reduces in an all-reduce of n_elems (a multiple of 8 * world)."""
    if n_elems % (8 * world) != 0:
        raise ValueError("n_elems must be a multiple of 8 * world")
    per = n_elems // world
    return rank * per, (rank + 1) * per


class PeerCollectives:
    def __init__(self, group, device, data_bytes: int):
        import torch.distributed as dist
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise RuntimeError("peer collectives serve at most 8 ranks of one NVLink domain")
        self.lib = _lib.load()
        self.data_bytes = (int(data_bytes) + 255) // 256 * 256
        d, f, s = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        hd, hf = ctypes.create_string_buffer(64), ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.fa_peer_alloc(self.data_bytes, ctypes.byref(d), ctypes.byref(f), ctypes.byref(s), hd, hf))
        self._own = (d.value, f.value, s.value)
        handles = [None] * self.world
        dist.all_gather_object(handles, (bytes(hd.raw), bytes(hf.raw), self.data_bytes), group=group)
        data, flags, self._opened = [], [], []
        with torch.cuda.device(self.device):
            for r, (bd, bf, nbytes) in enumerate(handles):
                if nbytes != self.data_bytes:
                    raise RuntimeError("all ranks must allocate the same peer buffer size")
                if r == self.rank:
                    data.append(d.value); flags.append(f.value)
                    continue
                pd, pf = ctypes.c_void_p(), ctypes.c_void_p()
                _lib.check(self.lib.fa_peer_open(ctypes.create_string_buffer(bd, 64), ctypes.byref(pd)))
                _lib.check(self.lib.fa_peer_open(ctypes.create_string_buffer(bf, 64), ctypes.byref(pf)))
                self._opened += [pd.value, pf.value]
                data.append(pd.value); flags.append(pf.value)
        self._data = (ctypes.c_void_p * self.world)(*data)
        self._flags = (ctypes.c_void_p * self.world)(*flags)
        self._state = ctypes.c_void_p(s.value)
        self._bytes = torch.as_tensor(_Span(d.value, self.data_bytes), device=self.device)
        dist.barrier(group=group)          # every rank has mapped every buffer before the first collective

    # ---- views of this rank's buffer ---------------------------------------------------
    def view(self, offset_bytes: int, shape, dtype) -> torch.Tensor:
        n = 1
        for x in shape:
            n *= int(x)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset_bytes % 16 != 0 or offset_bytes + nbytes > self.data_bytes:
            raise ValueError("view outside the peer buffer or not 16-byte aligned")
        return self._bytes[offset_bytes:offset_bytes + nbytes].view(dtype).view(*shape)

    def owns(self, t: torch.Tensor) -> bool:
        off = t.data_ptr() - self._own[0]
        return 0 <= off and off + t.numel() * t.element_size() <= self.data_bytes

    def _offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self._own[0]
        if off < 0 or off + t.numel() * t.element_size() > self.data_bytes or not t.is_contiguous():
            raise ValueError("tensor is not a contiguous view of the peer buffer")
        return off

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    # ---- collectives -------------------------------------------------------------------
    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over the ranks of a bf16 view of the buffer (same view on every rank)."""
        if t.dtype != torch.bfloat16:
            raise TypeError("all_reduce_ takes bfloat16")
        _lib.check(self.lib.fa_peer_allreduce_sum_bf16(self._data, self._flags, self._state, self.rank, self.world,
                                                       self._offset_of(t), t.numel(), self._stream()))
        return t

    def all_reduce_add_rmsnorm_(self, part: torch.Tensor, x: torch.Tensor, h: torch.Tensor, weight: torch.Tensor,
                                eps: float) -> torch.Tensor:
        """x += sum over the ranks of `part`; h = rmsnorm(x) * weight — one kernel, x and h identical on every
        rank afterwards.  part, x, h: [rows, cols] bf16 views of the buffer (same views on every rank, rows a
        multiple of the world size); weight [cols] bf16 anywhere on this device.  Bit-identical to
        `all_reduce_(part)` followed by the add + RMS norm kernel."""
        if not (part.dtype == x.dtype == h.dtype == weight.dtype == torch.bfloat16):
            raise TypeError("all_reduce_add_rmsnorm_ takes bfloat16")
        if part.dim() != 2 or part.shape != x.shape or part.shape != h.shape or weight.numel() != part.size(1):
            raise ValueError("part, x and h must be [rows, cols] of one shape and weight [cols]")
        if part.size(0) % self.world != 0:
            raise ValueError("rows must be a multiple of the world size")
        if not weight.is_contiguous() or weight.device != self.device:
            raise ValueError("weight must be contiguous on this rank's device")
        _lib.check(self.lib.fa_peer_allreduce_add_rmsnorm_bf16(
            self._data, self._flags, self._state, self.rank, self.world, self._offset_of(part), self._offset_of(x),
            self._offset_of(h), part.size(0), part.size(1), ctypes.c_void_p(weight.data_ptr()), float(eps),
            self._stream()))
        return h

    def all_gather_into(self, out: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
        """`out` [world, ...] (a view of the buffer) receives `src` of every rank at index rank."""
        nbytes = src.numel() * src.element_size()
        if not src.is_contiguous() or out.numel() * out.element_size() != nbytes * self.world:
            raise ValueError("out must hold world chunks of src's size")
        _lib.check(self.lib.fa_peer_allgather(self._data, self._flags, self._state, self.rank, self.world,
                                              ctypes.c_void_p(src.data_ptr()), self._offset_of(out), nbytes,
                                              self._stream()))
        return out

    def check(self) -> None:
        """Synchronise and raise RuntimeError if a collective gave up waiting for another rank."""
        st = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.fa_peer_status(self._state, self._stream(), ctypes.byref(st)))

    def reset(self) -> None:
        """Recover after a collective gave up waiting (`check()` raised): every rank clears its flags,
        epoch and status between two host barriers.  All ranks must call it, with no collective in flight."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)          # nobody launches a collective any more
        with torch.cuda.device(self.device):
            _lib.check(self.lib.fa_peer_reset(ctypes.c_void_p(self._own[1]), self._state, self._stream()))
        dist.barrier(group=self.group)          # every rank's flags are clean before anyone stamps them again

    def close(self) -> None:
        """Unmap the other ranks' buffers and free this rank's (all ranks, after a barrier)."""
        import torch.distributed as dist
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.fa_peer_close(ctypes.c_void_p(p))
            dist.barrier(group=self.group)
            self._bytes = None
            self.lib.fa_peer_free(*(ctypes.c_void_p(p) for p in self._own))
        self._own = None
