"""Tensor-parallel partitioning of any-precision linear layers over the GPUs of one node.

The reference project has no multi-GPU serving path (its model wrapper places the whole model
on one device, any_precision/modules/AnyPrecisionForCausalLM.py:70-80); this module is new.
Correctness is defined against the single-GPU result.

Layout (one process per GPU, ``torch.distributed``):

* column-parallel (q/k/v/gate/up): rank r owns output rows ``[n0, n1)``.  ``qweight[:, n0:n1, :]``
  is used in place as a strided view (the kernels take the plane stride), the tables are sliced.
  Input is the full activation, output is the rank's slice of the features; no communication.
* row-parallel (o/down): rank r owns input columns ``[k0, k1)``.  The packed operand is a plain
  slice of the word axis when the shard starts and ends on 1024-weight group boundaries, otherwise
  it is re-packed (``packing.slice_k``), because the partial group of a shard is laid out with
  its own stride.  Tables are replicated (every rank needs every row's table).  Input is the
  rank's slice of the features, output is a partial sum that is all-reduced (NCCL on GPUs).
"""
from __future__ import annotations

import dataclasses

import torch

import any_precision_ext as _ext
import torch.distributed as dist

from . import packing


def shard_bounds(total: int, world: int, rank: int, multiple: int = 1):
    """Contiguous, near-equal shards whose boundaries are multiples of ``multiple``."""
    if total % multiple:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    units = total // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    size = base + (1 if rank < extra else 0)
    return start * multiple, (start + size) * multiple


@dataclasses.dataclass
class LinearShard:
    style: str                      # "col" or "row"
    qweight: torch.Tensor           # [planes, N_local, K_local/32] (a view for "col")
    luts: dict                      # w_bits -> [N_local, 2**w_bits]
    n_range: tuple
    k_range: tuple
    repacked: bool = False

    @property
    def out_features(self):
        return self.qweight.shape[1]

    @property
    def in_features(self):
        return self.qweight.shape[2] * 32


def shard_linear(qweight: torch.Tensor, luts: dict, style: str, rank: int, world: int) -> LinearShard:
    planes, N, words = qweight.shape
    K = words * 32
    if style == "col":
        n0, n1 = shard_bounds(N, world, rank, 16 if N % (16 * world) == 0 else 1)
        return LinearShard("col", qweight[:, n0:n1, :], {w: l[n0:n1].contiguous() for w, l in luts.items()},
                           (n0, n1), (0, K))
    if style == "row":
        k0, k1 = shard_bounds(K, world, rank, 128 if K % (128 * world) == 0 else 32)
        plain = k0 % 1024 == 0 and (k1 % 1024 == 0 or k1 == K)
        return LinearShard("row", packing.slice_k(qweight, k0, k1), dict(luts), (0, N), (k0, k1), repacked=not plain)
    raise ValueError("style must be 'col' or 'row'")


def shard_forward(x: torch.Tensor, shard: LinearShard, w_bits: int, matmul, group=None, out=None, allreduce=None):
    """One sharded layer.  ``x`` is the full activation for a column-parallel shard and the rank's
    feature slice for a row-parallel shard; the row-parallel result is all-reduced in place, by
    ``allreduce`` (e.g. a ``comm.OneShotAllReduce``) if given, else by the process group's."""
    rows = x.numel() // x.shape[-1]
    sharded_row = shard.style == "row" and dist.is_initialized() and dist.get_world_size(group) > 1
    if sharded_row and allreduce is not None and hasattr(allreduce, "push_target") and rows <= 8 and \
            _ext.gated_supported(x, shard.qweight, shard.luts[w_bits]) and matmul is _ext.matmul_kbit:
        # the decode kernel stores its tiles straight into the ranks' inboxes; the collecting half sums
        matmul(x, shard.qweight, shard.luts[w_bits], w_bits, push=allreduce.push_target)
        if out is None:
            out = torch.empty((*x.shape[:-1], shard.qweight.shape[1]), dtype=torch.float16, device=x.device)
        allreduce.collect(out.view(rows, -1))
        return out
    y = matmul(x, shard.qweight, shard.luts[w_bits], w_bits, out=out) if out is not None else \
        matmul(x, shard.qweight, shard.luts[w_bits], w_bits)
    if sharded_row:
        if allreduce is not None:
            allreduce(y)
        else:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


def stack_column_shards(shards):
    """Stack consecutive column-parallel shards that read the same activation (q/k/v, gate/up) into one
    operand by rows (``packing.concat_rows``): one launch instead of several.  ``shards`` is a list of
    ``(name, LinearShard)``; row-parallel shards and lone column shards pass through."""
    fused, i = [], 0
    while i < len(shards):
        j = i + 1
        while (shards[i][1].style == "col" and j < len(shards) and shards[j][1].style == "col"
               and shards[j][1].in_features == shards[i][1].in_features):
            j += 1
        if j - i > 1:
            q, luts = packing.concat_rows([sh.qweight for _, sh in shards[i:j]], [sh.luts for _, sh in shards[i:j]])
            fused.append(("+".join(n for n, _ in shards[i:j]),
                          LinearShard("col", q, luts, (0, q.shape[1]), shards[i][1].k_range)))
        else:
            fused.append(shards[i])
        i = j
    return fused
