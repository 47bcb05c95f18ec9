"""Host-side pieces that need no GPU: the torch packer against the oracle and the golden
vectors, operand validation in the Python operator API, and the module's bookkeeping."""
import numpy as np
import pytest
import torch

from conftest import make_layer
from oracle import oracle

import any_precision_ext as ext
from anyprec_b200 import AnyPrecisionLinear, packing


def test_torch_packer_matches_reference_packer(golden):
    _, g = golden
    q = packing.pack_codes(torch.from_numpy(g["codes"]))
    assert np.array_equal(q.numpy(), g["qweight"])
    for w in (1, 3, 5, 8):
        assert np.array_equal(packing.unpack_codes(torch.from_numpy(g["qweight"]), w).numpy(), g["codes"] >> (8 - w))


@pytest.mark.parametrize("K,k0,k1", [(4096, 1024, 3072), (4096, 0, 512), (28672 // 4, 3584, 7168), (11008, 10240, 11008),
                                       (11008, 5504, 11008), (2048, 992, 1056)])
def test_k_shard_keeps_the_weights(K, k0, k1):
    codes, _ = make_layer(4, K, seed=K + k0)
    q = packing.pack_codes(torch.from_numpy(codes))
    shard = packing.slice_k(q, k0, k1)
    assert shard.shape == (8, 4, (k1 - k0) // 32)
    assert np.array_equal(oracle.unpack(shard.numpy(), 8), codes[:, k0:k1])


def test_random_operands_have_the_stated_distributions():
    gen = torch.Generator().manual_seed(3)
    q = packing.random_qweight(8, 16, 1024, device="cpu", generator=gen)
    assert q.dtype == torch.int32 and q.shape == (8, 16, 32)
    codes = packing.unpack_codes(q, 8)
    assert 100 < codes.float().mean() < 155          # uniform on [0, 256)
    lut = packing.random_lut(16, 5, device="cpu", generator=gen)
    assert lut.dtype == torch.float16 and lut.shape == (16, 32)
    assert torch.all(lut[:, 1:] >= lut[:, :-1])


def test_operator_api_rejects_bad_operands_without_a_gpu():
    q = torch.zeros((8, 4, 1), dtype=torch.int32)
    lut = torch.zeros((4, 8), dtype=torch.float16)
    x = torch.zeros((1, 32), dtype=torch.float16)
    with pytest.raises(ValueError):      # CPU tensors: there is no CPU path
        ext.dequant_kbit(q, lut, 3)
    with pytest.raises(ValueError):
        ext.matmul_kbit(x, q, lut, 3)
    with pytest.raises(ValueError):
        ext.dequant_kbit(q, lut, 2)
    with pytest.raises(TypeError):
        ext.dequant_kbit(q.to(torch.int64), lut, 3)
    with pytest.raises(TypeError):
        ext.dequant_kbit(q, lut.float(), 3)


def test_module_bookkeeping_matches_the_reference_module():
    m = AnyPrecisionLinear(64, 8, [3, 4, 5, 6, 7, 8], bias=True, precisions=[3, 4, 8])
    assert m.qweight.shape == (8, 8, 2) and m.qweight.dtype == torch.int32
    assert set(k for k, _ in m.named_buffers()) == {"qweight", "bias", *(f"lut{b}" for b in range(3, 9))}
    assert m.lut5.shape == (8, 32) and m.lut5.dtype == torch.float16
    assert m.precision == 8
    m.set_precision(4)
    assert m.precision == 4
    with pytest.raises(RuntimeError):
        m.set_precision(5)
    m.precisions = [3, 4]
    m.prune_precisions()
    assert m.qweight.shape[0] == 4
    assert not hasattr(m, "lut8") and hasattr(m, "lut3")
    assert "in_features=64, out_features=8, bias=True" in repr(m)
    with pytest.raises(RuntimeError):
        AnyPrecisionLinear(64, 8, [3, 4], dtype=torch.float32)
    with pytest.raises(RuntimeError):
        AnyPrecisionLinear(64, 8, [3, 4], precisions=3)
    # packed state dicts load by name
    sd = {"qweight": torch.zeros((4, 8, 2), dtype=torch.int32), "lut3": torch.ones((8, 8), dtype=torch.float16),
          "lut4": torch.ones((8, 16), dtype=torch.float16)}
    m2 = AnyPrecisionLinear(64, 8, [3, 4], bias=False)
    m2.load_state_dict(sd)
    assert m2.bias is None and torch.all(m2.lut3 == 1)


def test_row_concatenation_is_the_layers_side_by_side():
    """q/k/v (or gate/up) stacked along the row axis: the oracle dequantises the stacked operand to
    the layers' weights one under the other, at every precision."""
    parts = [make_layer(n, 1056, seed=40 + n) for n in (16, 4, 12)]
    qs = [packing.pack_codes(torch.from_numpy(c)) for c, _ in parts]
    luts = [{b: torch.from_numpy(l[b]) for b in l} for _, l in parts]
    q, lut = packing.concat_rows(qs, luts)
    assert q.shape == (8, 32, 1056 // 32) and q.is_contiguous()
    for w in (3, 5, 8):
        want = np.concatenate([oracle.dequant(oracle.pack(c), l[w], w) for c, l in parts], axis=0)
        got = oracle.dequant(q.numpy(), lut[w].numpy(), w)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    with pytest.raises(ValueError):
        packing.concat_rows([qs[0], packing.pack_codes(torch.from_numpy(make_layer(4, 1024, seed=1)[0]))], luts[:2])


def test_module_chooses_the_prefill_path_by_the_measured_rule():
    """fused_prefill = "auto": the fused tcgen05 kernel only where it was measured to win (wide layer,
    up to 256 rows; other large layers up to 128 rows); True / False force one path."""
    from anyprec_b200 import AnyPrecisionLinear
    wide = AnyPrecisionLinear(1024, 100 * 128, [3, 8], bias=False, device="cpu")
    narrow = AnyPrecisionLinear(1024, 4096, [3, 8], bias=False, device="cpu")
    x = torch.zeros((64, 1024), dtype=torch.float16)
    assert wide.fused_prefill == "auto"
    assert wide._use_fused(x, 64, 3) and wide._use_fused(x, 256, 6) and wide._use_fused(x, 256, 8)
    assert not wide._use_fused(x, 257, 3)
    assert not narrow._use_fused(x, 64, 3)
    narrow.fused_prefill = True
    assert narrow._use_fused(x, 64, 3)
    wide.fused_prefill = False
    assert not wide._use_fused(x, 64, 3)
    big = AnyPrecisionLinear(8192, 8192, [3], bias=False, device="cpu")              # 67 M weights, 64 row blocks
    xb = torch.zeros((64, 8192), dtype=torch.float16)
    assert big._use_fused(xb, 128, 3) and not big._use_fused(xb, 129, 3)
    # the decode kernel takes up to 8 rows everywhere, up to 16 where the fused kernel is not used
    assert wide._route(x, 8, 3) == "gemv" and narrow._route(x, 16, 3) == "gemv" and narrow._route(x, 17, 3) == "fused"
    assert big._route(xb, 8, 3) == "gemv" and big._route(xb, 9, 3) == "fused" and big._route(xb, 129, 3) == "twostep"
    narrow.fused_prefill = "auto"
    assert narrow._route(x, 16, 3) == "gemv" and narrow._route(x, 17, 3) == "twostep"
    mid = AnyPrecisionLinear(1024, 11008, [3], bias=False, device="cpu")             # 86 row blocks: up to 64 rows
    assert mid._use_fused(x, 64, 3) and not mid._use_fused(x, 65, 3) and mid._route(x, 12, 3) == "fused"
    odd = AnyPrecisionLinear(1024 + 128, 100 * 128, [3], bias=False, device="cpu")   # in_features % 256 != 0
    assert not odd._use_fused(torch.zeros((64, 1152), dtype=torch.float16), 64, 3)


def test_interleave_gate_up_layout():
    from anyprec_b200 import packing
    F, words = 24, 4
    g = torch.arange(3 * F * words, dtype=torch.int32).reshape(3, F, words)
    u = -g - 1
    gl = {3: torch.arange(F * 8, dtype=torch.float16).reshape(F, 8)}
    ul = {3: -gl[3] - 1}
    q, luts = packing.interleave_gate_up(g, u, gl, ul)
    assert q.shape == (3, 2 * F, words) and luts[3].shape == (2 * F, 8)
    for f in range(F):
        row = (f // 8) * 16 + f % 8
        assert torch.equal(q[:, row], g[:, f]) and torch.equal(q[:, row + 8], u[:, f])
        assert torch.equal(luts[3][row], gl[3][f]) and torch.equal(luts[3][row + 8], ul[3][f])
    with pytest.raises(ValueError):
        packing.interleave_gate_up(g[:, :20], u[:, :20], gl, ul)
