"""One-shot all-reduce over peer memory for the ranks of one node (``ap_allreduce_oneshot``).

The reference runs on one device and has nothing like it.  ``OneShotAllReduce`` owns a rank's
communication buffer, exchanges CUDA IPC handles with the other ranks through the process group
(host side, any backend) and then sums fp16 tensors across ranks with one kernel launch per call:
every rank stores its tensor into an inbox on every rank, publishes a sequence number, waits a
bounded time for the others and adds the inbox slots in rank order (fp32 accumulation), so all
ranks end with identical bits.  Calls can be captured in CUDA graphs.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

import any_precision_ext as _ext


def _lib():
    lib = _ext.load_library()
    if getattr(lib, "_comm_ready", False):
        return lib
    vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.ap_comm_buffer_bytes.restype = sz
    lib.ap_comm_buffer_bytes.argtypes = [sz]
    lib.ap_comm_alloc.restype = i
    lib.ap_comm_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    lib.ap_comm_free.restype = i
    lib.ap_comm_free.argtypes = [vp]
    lib.ap_comm_export.restype = i
    lib.ap_comm_export.argtypes = [vp, ctypes.c_char_p]
    lib.ap_comm_open.restype = i
    lib.ap_comm_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.ap_comm_close.restype = i
    lib.ap_comm_close.argtypes = [vp]
    lib.ap_comm_last_error.restype = ctypes.c_char_p
    lib.ap_allreduce_oneshot.restype = i
    lib.ap_allreduce_oneshot.argtypes = [vp, vp, i, ctypes.POINTER(vp), i, i, sz, vp, vp]
    lib.ap_allreduce_residual_blocks.restype = i
    lib.ap_allreduce_residual_blocks.argtypes = [i, i]
    lib.ap_allreduce_oneshot_collect.restype = i
    lib.ap_allreduce_oneshot_collect.argtypes = [vp, i, i, vp, vp, vp, ctypes.POINTER(vp), i, i, sz, vp, vp]
    lib.ap_allreduce_oneshot_residual.restype = i
    lib.ap_allreduce_oneshot_residual.argtypes = [vp, vp, i, i, vp, vp, vp, ctypes.POINTER(vp), i, i, sz, vp, vp]
    lib._comm_ready = True
    return lib


class OneShotAllReduce:
    """Sum fp16 CUDA tensors over the ranks of ``group`` (all on one node, one GPU each).

    ``max_payload_bytes`` bounds ``tensor.numel() * 2``.  All ranks must construct the object
    together and then issue the same sequence of calls (call by call the same size on every rank;
    consecutive calls may differ in size)."""

    def __init__(self, max_payload_bytes: int, device: torch.device, group=None):
        self.lib = _lib()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.max_payload = int(max_payload_bytes)
        self._mine = ctypes.c_void_p()
        self._opened = []
        with torch.cuda.device(self.device):
            nbytes = self.lib.ap_comm_buffer_bytes(self.max_payload)
            self._check(self.lib.ap_comm_alloc(nbytes, ctypes.byref(self._mine)), "ap_comm_alloc")
            handle = ctypes.create_string_buffer(64)
            self._check(self.lib.ap_comm_export(self._mine, handle), "ap_comm_export")
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self._mine.value)
                else:
                    p = ctypes.c_void_p()
                    self._check(self.lib.ap_comm_open(handles[r], ctypes.byref(p)), f"ap_comm_open(rank {r})")
                    self._opened.append(p)
                    ptrs.append(p.value)
            self._table = (ctypes.c_void_p * self.world)(*ptrs)
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)          # every rank has mapped every buffer before the first call

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {self.lib.ap_strerror(rc).decode()}: {self.lib.ap_comm_last_error().decode()}")

    def __call__(self, tensor: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if tensor.dtype != torch.float16 or not tensor.is_cuda or not tensor.is_contiguous():
            raise TypeError("OneShotAllReduce needs a contiguous float16 CUDA tensor")
        if tensor.device != self.device:
            raise ValueError(f"tensor is on {tensor.device}, the communication buffers are on {self.device}")
        if out is None:
            out = tensor
        elif out.dtype != torch.float16 or not out.is_contiguous() or out.numel() != tensor.numel() \
                or out.device != self.device:
            raise ValueError("out must be a contiguous float16 tensor of the same size on the same device")
        with torch.cuda.device(self.device):
            rc = self.lib.ap_allreduce_oneshot(tensor.data_ptr(), out.data_ptr(), tensor.numel(), self._table,
                                               self.rank, self.world, self.max_payload, self.status.data_ptr(),
                                               torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "ap_allreduce_oneshot")
        return out

    def residual_blocks(self, rows: int, row_len: int) -> int:
        """Entries per row that ``residual`` leaves in ``ssq`` (0: shape not supported)."""
        return self.lib.ap_allreduce_residual_blocks(rows, row_len)

    def residual(self, tensor: torch.Tensor, h: torch.Tensor, norm_weight: torch.Tensor, ssq: torch.Tensor,
                 out: torch.Tensor) -> torch.Tensor:
        """The sum of ``tensor [rows, N]`` over the ranks, added to the residual stream ``h [rows, N]`` in place;
        ``out = h * norm_weight`` (not yet normalised) and ``ssq[rows, residual_blocks(rows, N)]`` the partial sums
        of squares of the new ``h``: the first half of a folded residual add + RMSNorm across a row-parallel
        layer (``ap_allreduce_oneshot_residual``; the second half is ``matmul_kbit(prenorm=)``)."""
        for t in (tensor, h, out, norm_weight):
            if t.dtype != torch.float16 or not t.is_contiguous() or t.device != self.device:
                raise TypeError("OneShotAllReduce.residual needs contiguous float16 tensors on the buffers' device")
        rows, n = tensor.shape
        blocks = self.residual_blocks(rows, n)
        if h.shape != tensor.shape or out.shape != tensor.shape or norm_weight.numel() != n or blocks == 0 or \
                ssq.dtype != torch.float32 or ssq.numel() < rows * blocks or ssq.device != self.device:
            raise ValueError("residual: h and out as tensor, norm_weight [N], ssq fp32 with rows * residual_blocks entries")
        with torch.cuda.device(self.device):
            rc = self.lib.ap_allreduce_oneshot_residual(tensor.data_ptr(), out.data_ptr(), rows, n, h.data_ptr(),
                                                        norm_weight.data_ptr(), ssq.data_ptr(), self._table, self.rank, self.world,
                                                        self.max_payload, self.status.data_ptr(),
                                                        torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "ap_allreduce_oneshot_residual")
        return out

    @property
    def push_target(self):
        """``(peer table, rank, world, max payload)``: what ``matmul_kbit(push=)`` needs to store a row-parallel
        product straight into the ranks' inboxes (``ap_matmul_kbit_push``); ``collect`` must follow."""
        return self._table, self.rank, self.world, self.max_payload

    def collect(self, out: torch.Tensor, h: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                ssq: torch.Tensor | None = None) -> torch.Tensor:
        """The second half of an all-reduce whose partial results ``matmul_kbit(push=)`` has stored in the
        inboxes: ``out [rows, N]`` = the sum over the ranks, or, with ``h``, what ``residual`` leaves (``h``
        updated in place, ``out = h * norm_weight``, ``ssq``)."""
        if out.dim() != 2 or out.dtype != torch.float16 or not out.is_contiguous() or out.device != self.device:
            raise TypeError("collect needs a contiguous float16 [rows, N] tensor on the buffers' device")
        rows, n = out.shape
        if h is not None:
            for t in (h, norm_weight):
                if t is None or t.dtype != torch.float16 or not t.is_contiguous() or t.device != self.device:
                    raise TypeError("collect: h and norm_weight must be contiguous float16 tensors on the buffers' device")
            blocks = self.residual_blocks(rows, n)
            if h.shape != out.shape or norm_weight.numel() != n or blocks == 0 or ssq is None or \
                    ssq.dtype != torch.float32 or ssq.numel() < rows * blocks or ssq.device != self.device:
                raise ValueError("collect: h as out, norm_weight [N], ssq fp32 with rows * residual_blocks entries")
        with torch.cuda.device(self.device):
            rc = self.lib.ap_allreduce_oneshot_collect(out.data_ptr(), rows, n, h.data_ptr() if h is not None else None,
                                                       norm_weight.data_ptr() if h is not None else None,
                                                       ssq.data_ptr() if h is not None else None, self._table, self.rank,
                                                       self.world, self.max_payload, self.status.data_ptr(),
                                                       torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "ap_allreduce_oneshot_collect")
        return out

    def wait_expired(self) -> bool:
        """Synchronises; True if any call so far gave up waiting for a peer (its output is invalid)."""
        return bool(self.status.item())

    def close(self):
        """Unmap the peers' buffers and free this rank's.  All ranks must have finished their calls."""
        if self._mine.value is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.ap_comm_close(p)
            self._opened = []
            if self.world > 1:
                dist.barrier(group=self.group)
            self.lib.ap_comm_free(self._mine)
        self._mine = ctypes.c_void_p()
