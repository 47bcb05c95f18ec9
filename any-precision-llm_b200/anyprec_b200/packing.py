"""The packed bitplane format, written with torch ops so it runs on the device that holds
the codes.

Produces and reads the operand layout of the reference project's packed checkpoints:
``qweight`` int32 ``[P, N, K/32]`` with plane 0 = MSB of the parent code
(any_precision/quantization/pack.py:90-96) and the per-row byte permutation of
pack.py:12-76: word ``t`` of a group of ``E`` words (E = 32, or (K % 1024)/32 in the final
partial group), byte ``j`` from the most significant byte, bit ``e`` from that byte's MSB,
holds the plane bit of weight ``k = group_base + 8*E*j + 8*t + e``.

Used to synthesise operands, to re-pack a K-shard whose length is not a multiple of 1024
(its partial group has a different E than the same weights had in the full row), and by the
tensor-parallel sharding code.
"""
from __future__ import annotations

import functools

import torch


@functools.lru_cache(maxsize=32)
def _element_map_cpu(K: int) -> torch.Tensor:
    if K % 32 != 0 or K <= 0:
        raise ValueError("K must be a positive multiple of 32")
    words, full, tail_e = K // 32, K // 1024, (K % 1024) // 32
    j = torch.arange(4).view(1, 4, 1)
    e = torch.arange(8).view(1, 1, 8)
    parts = []
    if full:
        grp = torch.arange(full).view(full, 1, 1, 1) * 1024
        t = torch.arange(32).view(1, 32, 1, 1)
        parts.append((grp + 256 * j.unsqueeze(0) + 8 * t + e.unsqueeze(0)).reshape(full * 32, 4, 8))
    if tail_e:
        t = torch.arange(tail_e).view(tail_e, 1, 1)
        parts.append(full * 1024 + 8 * tail_e * j + 8 * t + e)
    kmap = torch.cat(parts, dim=0)
    assert kmap.shape == (words, 4, 8)
    return kmap.reshape(-1)


def element_map(K: int, device=None) -> torch.Tensor:
    """int64 ``[K]``: position ``word*32 + 8*j + e`` (MSB-first bit order) -> weight index k."""
    return _element_map_cpu(K).to(device) if device is not None else _element_map_cpu(K)


def _lib():
    import ctypes

    import any_precision_ext
    lib = any_precision_ext.load_library()
    if not getattr(lib, "_pack_ready", False):
        vp, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        lib.ap_pack_codes.restype = i
        lib.ap_pack_codes.argtypes = [vp, vp, i64, i, i, i, vp]
        lib.ap_unpack_codes.restype = i
        lib.ap_unpack_codes.argtypes = [vp, i64, vp, i, i, i, vp]
        lib._pack_ready = True
    return lib


def pack_codes(codes: torch.Tensor, parent_bits: int = 8) -> torch.Tensor:
    """uint8 codes ``[N, K]`` (values < 2**parent_bits) -> int32 ``[parent_bits, N, K/32]``.  On a CUDA tensor
    this is one kernel (``ap_pack_codes``); on the CPU the same map written with torch ops."""
    if codes.dtype != torch.uint8 or codes.dim() != 2:
        raise TypeError("codes must be a uint8 [N, K] tensor")
    N, K = codes.shape
    if codes.is_cuda:
        if K % 32 or K <= 0:
            raise ValueError("K must be a positive multiple of 32")
        codes = codes.contiguous()
        q = torch.empty((parent_bits, N, K // 32), dtype=torch.int32, device=codes.device)
        lib = _lib()
        with torch.cuda.device(codes.device):
            rc = lib.ap_pack_codes(codes.data_ptr(), q.data_ptr(), N * (K // 32), N, K, parent_bits,
                                   torch.cuda.current_stream(codes.device).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"ap_pack_codes: {lib.ap_strerror(rc).decode()}")
        return q
    kmap = element_map(K, codes.device)
    perm = codes[:, kmap].to(torch.int32).view(N, K // 32, 32)     # bit 31 first
    shifts = torch.arange(31, -1, -1, device=codes.device, dtype=torch.int64)
    planes = []
    for p in range(parent_bits):
        bits = ((perm >> (parent_bits - 1 - p)) & 1).to(torch.int64)
        word = (bits << shifts).sum(dim=-1)                           # 0 .. 2**32-1
        word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
        planes.append(word.to(torch.int32))
    return torch.stack(planes, dim=0)


def unpack_codes(qweight: torch.Tensor, w_bits: int) -> torch.Tensor:
    """int32 ``[>=w_bits, N, K/32]`` -> uint8 ``[N, K]`` codes of precision ``w_bits``."""
    if qweight.dtype != torch.int32 or qweight.dim() != 3:
        raise TypeError("qweight must be an int32 [planes, N, K/32] tensor")
    planes, N, words = qweight.shape
    if not 1 <= w_bits <= planes:
        raise ValueError("w_bits out of range")
    K = words * 32
    if qweight.is_cuda and qweight.stride(2) == 1 and qweight.stride(1) == words:
        codes = torch.empty((N, K), dtype=torch.uint8, device=qweight.device)
        lib = _lib()
        with torch.cuda.device(qweight.device):
            rc = lib.ap_unpack_codes(qweight.data_ptr(), qweight.stride(0) if planes > 1 else N * words, codes.data_ptr(),
                                     N, K, w_bits, torch.cuda.current_stream(qweight.device).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"ap_unpack_codes: {lib.ap_strerror(rc).decode()}")
        return codes
    kmap = element_map(K, qweight.device)
    shifts = torch.arange(31, -1, -1, device=qweight.device, dtype=torch.int32)
    codes_perm = torch.zeros((N, K), dtype=torch.int32, device=qweight.device)
    for p in range(w_bits):
        bits = ((qweight[p].unsqueeze(-1) >> shifts) & 1).reshape(N, K)
        codes_perm |= bits << (w_bits - 1 - p)
    codes = torch.empty((N, K), dtype=torch.uint8, device=qweight.device)
    codes[:, kmap] = codes_perm.to(torch.uint8)
    return codes


def slice_k(qweight: torch.Tensor, k0: int, k1: int) -> torch.Tensor:
    """The operand for weights ``[k0, k1)`` of every row, in packed form.

    A plain slice of the word axis when the shard starts on a 1024 boundary and either ends
    on one or runs to the end of the row; otherwise the shard is unpacked and packed again,
    because its partial group is laid out with its own E."""
    planes, N, words = qweight.shape
    K = words * 32
    if not (0 <= k0 < k1 <= K) or k0 % 32 or k1 % 32:
        raise ValueError("shard bounds must be multiples of 32 inside the row")
    if k0 % 1024 == 0 and (k1 % 1024 == 0 or k1 == K):
        return qweight[:, :, k0 // 32:k1 // 32].contiguous()
    codes = unpack_codes(qweight, planes)
    return pack_codes(codes[:, k0:k1].contiguous(), planes)


def concat_rows(qweights, luts):
    """Stack layers that read the same activation (q/k/v, gate/up) into one operand.

    Every row of the packed format carries its own planes and its own table, so layers with the
    same ``in_features`` concatenate along the row axis with no re-packing: ``qweights`` is a list of
    int32 ``[P, N_i, K/32]`` tensors (same ``P`` and ``K``), ``luts`` a list of ``{w_bits: fp16 [N_i,
    2**w_bits]}``.  Returns ``(qweight [P, sum N_i, K/32], {w_bits: lut [sum N_i, 2**w_bits]})``; one
    ``matmul_kbit`` on the result equals the layers' outputs side by side.  The reference leaves this
    fusion as a stub (AnyPrecisionForCausalLM.py:186-190)."""
    planes = {q.shape[0] for q in qweights}
    words = {q.shape[2] for q in qweights}
    if len(planes) != 1 or len(words) != 1:
        raise ValueError("layers must share the number of planes and in_features")
    common = set(luts[0])
    for l in luts[1:]:
        common &= set(l)
    q = torch.cat(list(qweights), dim=1).contiguous()
    return q, {w: torch.cat([l[w] for l in luts], dim=0).contiguous() for w in sorted(common)}


def interleave_gate_up(gate_q: torch.Tensor, up_q: torch.Tensor, gate_luts: dict, up_luts: dict):
    """The operand of ``matmul_kbit(..., gated=True)``: the two projections of a gated MLP stacked tile by
    tile, of every 16 rows the first eight the gate rows ``f .. f+7`` and the last eight the up rows of the
    same features.  Rows carry their own planes and tables, so nothing is re-packed.  Feature count a
    multiple of 8."""
    planes, F, words = gate_q.shape
    if up_q.shape != gate_q.shape or F % 8:
        raise ValueError("gate and up must have the same shape and a row count that is a multiple of 8")
    q = torch.stack([gate_q.reshape(planes, F // 8, 8, words), up_q.reshape(planes, F // 8, 8, words)], dim=2)
    q = q.reshape(planes, 2 * F, words).contiguous()
    luts = {}
    for b in sorted(set(gate_luts) & set(up_luts)):
        g, u = gate_luts[b], up_luts[b]
        luts[b] = torch.stack([g.reshape(F // 8, 8, -1), u.reshape(F // 8, 8, -1)], dim=1).reshape(2 * F, -1).contiguous()
    return q, luts


def random_qweight(planes: int, N: int, K: int, *, device, generator=None) -> torch.Tensor:
    """Bitplanes of i.i.d. uniform parent codes: every bit is a fair coin, so the planes can
    be drawn directly without packing."""
    return torch.randint(-2 ** 31, 2 ** 31, (planes, N, K // 32), dtype=torch.int64, device=device,
                         generator=generator).to(torch.int32)


def random_lut(N: int, bits: int, *, device, generator=None, std: float = 0.02) -> torch.Tensor:
    """fp16 ``[N, 2**bits]``; each row a sorted sample of N(0, std)."""
    c = torch.randn((N, 1 << bits), dtype=torch.float32, device=device, generator=generator) * std
    return torch.sort(c, dim=1).values.to(torch.float16)
