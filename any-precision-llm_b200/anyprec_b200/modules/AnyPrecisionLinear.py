"""``AnyPrecisionLinear``: one linear layer stored once as bitplanes, evaluated at any of
its supported precisions.

Mirrors the module of the same name in the reference project
(any_precision/modules/AnyPrecisionLinear.py:10-78): same constructor arguments, the same
buffer names (``qweight``, ``lut3`` .. ``lut8``, ``bias``) so packed checkpoints load with
``load_state_dict``, and the same ``forward(x, precision=...)``, ``set_precision``,
``prune_precisions`` and ``extra_repr``.  The arithmetic is delegated to
``any_precision_ext.matmul_kbit`` / ``dequant_kbit``, here the sm_100a kernels.
"""
from __future__ import annotations

import torch
import torch.nn as nn

import any_precision_ext as _ext


class AnyPrecisionLinear(nn.Module):
    #: Row count up to which ``forward`` uses the decode kernel (which takes eight rows per pass).
    #: The reference hard-codes 8 (AnyPrecisionLinear.py:60).  Measured on B200 with
    #: examples/measure_crossover.py over the Llama-3-8B layer shapes and w = 3, 4, 8: two passes
    #: (16 rows) still beat dequant_kbit + fp16 GEMM, three passes (24 rows) do not.  On the layers
    #: where the fused prefill kernel is used (below) that kernel already beats the second pass, so
    #: there the decode kernel stops at ``gemv_one_pass_rows``.
    gemv_max_rows = 16
    gemv_one_pass_rows = 8
    #: Above ``gemv_max_rows`` rows.  False: dequant_kbit + torch.matmul, the reference's two-step path
    #: (:61-62).  True: the fused dequantise + tcgen05 GEMM wherever the shape allows (out_features %
    #: 128 == 0, in_features % 128 == 0).  "auto" (default): the fused kernel where it was measured to
    #: win on B200 (examples/measure_crossover.py), the two-step path elsewhere.  The fused kernel
    #: dequantises a block of 128 weight rows once per block of up to 256 activation rows and needs
    #: about one thread block per SM to use the GPU, so it wins on wide layers (out_features >= 12800,
    #: i.e. 100 row blocks) up to 256 activation rows (from 11008 up to 64 rows), and on other large layers (at least 50 M weights),
    #: which it splits along K, up to 128 activation rows.
    fused_prefill = "auto"

    def _use_fused(self, x, rows, w_bits):
        if self.fused_prefill is False or not _ext.gemm_kbit_supported(x, self.qweight):
            return False
        if self.fused_prefill is True:
            return True
        if self.in_features % 256:
            return False
        wide = (self.out_features >= 100 * 128 and rows <= 256) or (self.out_features >= 86 * 128 and rows <= 64)
        # large layers with fewer row blocks (8192 x 8192, 4096 x 14336): the kernel cuts K over several
        # thread blocks per block of rows (split-K)
        big = self.in_features * self.out_features >= 50_000_000 and self.out_features >= 4096 and rows <= 128
        return wide or big

    def _route(self, x, rows, w_bits):
        """'gemv' (matmul_kbit), 'fused' (gemm_kbit) or 'twostep' (dequant_kbit + fp16 GEMM) for this call."""
        if rows <= self.gemv_one_pass_rows:
            return 'gemv'
        if rows <= self.gemv_max_rows:
            return 'fused' if self.fused_prefill == "auto" and self._use_fused(x, rows, w_bits) else 'gemv'
        return 'fused' if self._use_fused(x, rows, w_bits) else 'twostep'

    def __init__(self, in_features, out_features, supported_bits, bias=True, precisions=None, device=None,
                 dtype=None):
        super().__init__()
        _ext.load_library()   # fail at construction if the kernels are missing, like the reference (:14-15)
        if precisions is None:
            precisions = supported_bits
        if not isinstance(precisions, list) or not isinstance(supported_bits, list):
            raise RuntimeError('supported_bits and precisions must be lists of integers.')
        if dtype is not None and dtype != torch.float16:
            raise RuntimeError('Only float16 is supported for now.')
        if in_features % 32 != 0:
            raise RuntimeError('in_features must be a multiple of 32.')
        if any(p not in supported_bits for p in precisions):
            raise RuntimeError('precisions must be a subset of supported_bits.')
        dtype = torch.float16

        self.in_features = in_features
        self.out_features = out_features
        self.supported_bits = supported_bits
        self.precisions = precisions
        self.precision = max(precisions)

        self.register_buffer(
            'qweight',
            torch.empty((max(supported_bits), out_features, in_features // 32), dtype=torch.int32, device=device))
        for bit in supported_bits:
            self.register_buffer(f'lut{bit}', torch.empty((out_features, 2 ** bit), dtype=dtype, device=device))
        if bias:
            self.register_buffer('bias', torch.empty((out_features,), dtype=dtype, device=device))
        else:
            self.bias = None

    def prune_precisions(self):
        """Drop the planes and tables no selected precision needs (reference :48-52)."""
        self.qweight = self.qweight[:max(self.precisions)]
        for bit in self.supported_bits:
            if bit not in self.precisions and hasattr(self, f'lut{bit}'):
                delattr(self, f'lut{bit}')

    def forward(self, x, **kwargs):
        w_bits = kwargs['precision'] if 'precision' in kwargs else self.precision
        lut = self._buffers.get(f'lut{w_bits}')
        if lut is None:
            raise RuntimeError(f'{w_bits}-bit table is not loaded; available: {self.precisions}')
        rows = x.numel() // x.shape[-1]
        path = self._route(x, rows, w_bits)
        if path == 'fused':
            # dequantise inside the tensor-core kernel: the fp16 weight never goes to HBM
            y = _ext.gemm_kbit(x, self.qweight, lut, w_bits)
        elif path == 'twostep':
            # the reference's two-step path (AnyPrecisionLinear.py:61-62)
            weight = _ext.dequant_kbit(self.qweight, lut, w_bits)
            y = torch.matmul(x, weight.T)
        else:
            y = _ext.matmul_kbit(x, self.qweight, lut, w_bits)
        if self.bias is not None:
            y += self.bias
        return y

    @classmethod
    def fuse(cls, layers):
        """One module for layers that read the same input (q/k/v or gate/up): their rows side by
        side, so that a forward is one kernel launch instead of ``len(layers)``.  Rows carry their own
        planes and tables, so nothing is re-packed.  The result has ``split_sizes`` (the layers'
        ``out_features``) and ``forward_split`` returning one view per layer.  The reference's
        ``fuse_layers`` is an unimplemented stub (AnyPrecisionForCausalLM.py:186-190)."""
        from .. import packing
        first = layers[0]
        if any(l.in_features != first.in_features or l.supported_bits != first.supported_bits or
               l.precisions != first.precisions or (l.bias is None) != (first.bias is None) for l in layers):
            raise RuntimeError('layers to fuse must agree in in_features, supported_bits, precisions and bias')
        fused = cls(first.in_features, sum(l.out_features for l in layers), list(first.supported_bits),
                    bias=first.bias is not None, precisions=list(first.precisions), device='meta')
        q, luts = packing.concat_rows([l.qweight for l in layers],
                                      [{b: getattr(l, f'lut{b}') for b in first.supported_bits if hasattr(l, f'lut{b}')}
                                       for l in layers])
        fused.qweight = q
        for b in first.supported_bits:
            if b in luts:
                setattr(fused, f'lut{b}', luts[b])
            elif hasattr(fused, f'lut{b}'):
                delattr(fused, f'lut{b}')
        if first.bias is not None:
            fused.bias = torch.cat([l.bias for l in layers])
        fused.precision = first.precision
        fused.split_sizes = [l.out_features for l in layers]
        return fused

    @classmethod
    def fuse_gated(cls, gate, up):
        """One module for the gate and up projections of a gated MLP, rows stacked tile by tile (of every 16
        rows eight gate rows, then the up rows of the same features: ``packing.interleave_gate_up``), so that
        a decode step gets ``silu(gate) * up`` out of one launch (``forward_gated``).  ``forward`` of the
        result returns the tiled order.  No counterpart in the reference."""
        from .. import packing
        if (gate.in_features, gate.out_features, gate.supported_bits, gate.precisions) != \
                (up.in_features, up.out_features, up.supported_bits, up.precisions) or gate.bias is not None or \
                up.bias is not None:
            raise RuntimeError('gate and up must agree in shape, supported_bits and precisions and have no bias')
        fused = cls(gate.in_features, 2 * gate.out_features, list(gate.supported_bits), bias=False,
                    precisions=list(gate.precisions), device='meta')
        q, luts = packing.interleave_gate_up(
            gate.qweight, up.qweight, {b: getattr(gate, f'lut{b}') for b in gate.supported_bits if hasattr(gate, f'lut{b}')},
            {b: getattr(up, f'lut{b}') for b in up.supported_bits if hasattr(up, f'lut{b}')})
        fused.qweight = q
        for b in gate.supported_bits:
            if b in luts:
                setattr(fused, f'lut{b}', luts[b])
            elif hasattr(fused, f'lut{b}'):
                delattr(fused, f'lut{b}')
        fused.precision = gate.precision
        fused.gated = True
        return fused

    def forward_gated(self, x, out=None, **kwargs):
        """``silu(gate(x)) * up(x)`` of a ``fuse_gated`` module, ``[..., out_features / 2]``: one launch with the
        activation in the kernel's epilogue for up to eight rows of shapes the decode kernel takes, the plain
        product followed by ``ap_silu_mul`` otherwise.  Both round alike (each projection to fp16, the
        activation to fp16, then the product)."""
        if not getattr(self, 'gated', False):
            raise RuntimeError('forward_gated needs a module built by fuse_gated')
        w_bits = kwargs['precision'] if 'precision' in kwargs else self.precision
        lut = self._buffers.get(f'lut{w_bits}')
        if lut is None:
            raise RuntimeError(f'{w_bits}-bit table is not loaded; available: {self.precisions}')
        rows = x.numel() // x.shape[-1]
        if _ext.gated_supported(x, self.qweight, lut):
            return _ext.matmul_kbit(x, self.qweight, lut, w_bits, gated=True, out=out)
        gu = self.forward(x, **kwargs)
        return _ext.silu_mul(gu, tiled=True, out=out)

    def _decode_operands(self, x, kwargs):
        w_bits = kwargs['precision'] if 'precision' in kwargs else self.precision
        lut = self._buffers.get(f'lut{w_bits}')
        if lut is None:
            raise RuntimeError(f'{w_bits}-bit table is not loaded; available: {self.precisions}')
        if self.bias is not None or not _ext.gated_supported(x, self.qweight, lut):
            raise RuntimeError('the fused decoder products need up to eight rows, no bias, and operands the decode kernel takes')
        return w_bits, lut

    def forward_residual(self, x, h, norm_weight, ssq, out=None, **kwargs):
        """``h += self(x)`` in place; returns ``h * norm_weight`` (not yet normalised) and leaves the per-tile
        sums of squares of the new ``h`` in ``ssq``: the first half of a folded residual add + RMSNorm
        (``any_precision_ext.matmul_kbit(residual=)``)."""
        w_bits, lut = self._decode_operands(x, kwargs)
        return _ext.matmul_kbit(x, self.qweight, lut, w_bits, out=out, residual=(h, norm_weight, ssq))

    def forward_push(self, x, allreduce, **kwargs):
        """This rank's partial product of a row-parallel layer, stored by the kernel straight into the all-reduce
        inboxes of all ranks (``comm.OneShotAllReduce``); ``allreduce.collect(...)`` then sums."""
        w_bits, lut = self._decode_operands(x, kwargs)
        return _ext.matmul_kbit(x, self.qweight, lut, w_bits, push=allreduce.push_target)

    def forward_prenorm(self, x, ssq, width, eps, out=None, blocks=None, **kwargs):
        """``self(rmsnorm-scaled x)`` for the ``x`` and ``ssq`` that ``forward_residual`` of the previous layer
        left (``width`` = that layer's ``out_features``); with a ``fuse_gated`` module the result is
        ``silu(gate) * up``."""
        w_bits, lut = self._decode_operands(x, kwargs)
        return _ext.matmul_kbit(x, self.qweight, lut, w_bits, out=out, gated=getattr(self, 'gated', False),
                                prenorm=(ssq, width, eps) if blocks is None else (ssq, width, eps, blocks))

    def forward_split(self, x, **kwargs):
        """``forward`` of a fused module, cut back into the original layers' outputs (views)."""
        return torch.split(self.forward(x, **kwargs), getattr(self, 'split_sizes', [self.out_features]), dim=-1)

    def set_precision(self, precision):
        if precision not in self.precisions:
            raise RuntimeError(f"{self.precisions}-bit precisions are supported but {precision}-bit was specified.")
        self.precision = precision

    def extra_repr(self) -> str:
        return f'in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}'
