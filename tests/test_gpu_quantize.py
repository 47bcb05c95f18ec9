"""The seed + upscale kernel (ap_seed_upscale) against the CPU oracle, bit for bit: on the inputs of the
fixtures that the reference's own routine produced (so also against those), on rows with repeated values,
degenerate rows, every supported row length class, and end to end into a packed layer."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from oracle import seed_upscale as su

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run_kernel(w, s, sb, pb, **kw):
    from anyprec_b200 import quantize
    luts, codes = quantize.seed_and_upscale_layer(torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda(), sb, pb, **kw)
    torch.cuda.synchronize()
    return {b: t.cpu().numpy() for b, t in luts.items()}, codes.cpu().numpy()


def check_against_oracle(w, s, sb, pb, **kw):
    luts, codes = run_kernel(w, s, sb, pb, **kw)
    ref_luts, ref_codes = su.seed_and_upscale_layer(w, s, sb, pb, blocked=True)
    bad = np.nonzero((codes != ref_codes).any(axis=1))[0]
    assert bad.size == 0, f"rows with different codes: {bad[:8]}"
    for b in range(sb, pb + 1):
        assert np.array_equal(luts[b].view(np.uint16), ref_luts[b].view(np.uint16)), f"table {b}"
    return luts, codes


def test_kernel_equals_the_reference_routines_fixture():
    for path in sorted(glob.glob(os.path.join(GOLDEN, "quantizer_*.npz"))):
        g = np.load(path)
        sb, pb = int(g["seed_bit"]), int(g["parent_bit"])
        for i in range(int(g["modules"])):
            luts, codes = run_kernel(g[f"weight{i}"], g[f"sens{i}"], sb, pb)
            assert np.array_equal(codes, g[f"codes{i}"]), (path, i)
            for b in range(sb, pb + 1):
                assert np.array_equal(luts[b].view(np.uint16), g[f"lut{i}_{b}"].view(np.uint16)), (path, i, b)


def layer(rng, N, K, fp16_values=True):
    w = rng.normal(0.0, 0.02, size=(N, K)).astype(np.float32)
    if fp16_values:
        w = w.astype(np.float16).astype(np.float32)         # values repeat, as in a real checkpoint
    w[rng.random((N, K)) < 0.01] = 0.0
    s = (rng.normal(size=(N, K)) ** 2).astype(np.float32)
    return w, s


@pytest.mark.parametrize("N,K", [(5, 32), (7, 96), (6, 1000), (9, 4096), (4, 11008), (3, 28672), (2, 32768)])
def test_kernel_against_oracle(N, K):
    rng = np.random.default_rng(N * 1000 + K)
    w, s = layer(rng, N, K)
    s[0] = 0.0                                               # a row without sample weight
    w[-1, : K // 2] = 0.0                                    # a row that is half zeros
    check_against_oracle(w, s, 3, 8)


@pytest.mark.parametrize("sb,pb", [(3, 3), (4, 6), (1, 8), (8, 8), (2, 5)])
def test_kernel_against_oracle_other_precisions(sb, pb):
    rng = np.random.default_rng(sb * 10 + pb)
    w, s = layer(rng, 6, 2048)
    check_against_oracle(w, s, sb, pb)


def test_more_rows_than_blocks_and_degenerate_rows():
    rng = np.random.default_rng(77)
    w, s = layer(rng, 23, 768)
    w[3] = 0.25                                              # one value
    w[4] = 0.0                                               # nothing but zeros
    w[5] = rng.choice(np.array([-0.03, -0.01, 0.0, 0.02, 0.05], dtype=np.float32), size=768)
    w[6, 1::2] = -0.0
    s[7] = 0.0
    s[8, :700] = 0.0                                         # sample weight on a few values only
    a = check_against_oracle(w, s, 3, 8, blocks=3)           # every block takes several rows in turn
    b = check_against_oracle(w, s, 3, 8)
    assert np.array_equal(a[1], b[1])


def test_quantize_linear_end_to_end():
    """Quantise, pack, and read back through dequant_kbit: W_b[n, k] = lut_b[n, code >> (8 - b)], the weighted
    error falls with every bit, and the module multiplies."""
    import any_precision_ext as ext
    from anyprec_b200 import quantize
    rng = np.random.default_rng(5)
    N, K = 64, 1024
    w, s = layer(rng, N, K, fp16_values=False)
    wt, st = torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda()
    m = quantize.quantize_linear(wt, st)
    luts, codes = quantize.seed_and_upscale_layer(wt, st)
    assert np.array_equal(m.qweight.cpu().numpy(), oracle.pack(codes.cpu().numpy()))
    prev = None
    for b in range(3, 9):
        deq = ext.dequant_kbit(m.qweight, getattr(m, f"lut{b}"), b)
        want = torch.gather(luts[b], 1, (codes >> (8 - b)).long())
        assert torch.equal(deq, want)
        err = su.weighted_error(w, s * (w != 0), luts[b].cpu().numpy(), (codes >> (8 - b)).cpu().numpy())
        assert prev is None or err < prev
        prev = err
    sw = (s * (w != 0)).astype(np.float64)
    assert np.sqrt(prev / float((sw * w.astype(np.float64) ** 2).sum())) < 0.01      # 256 levels per row: weighted rms error
    x = torch.randn(2, K, device="cuda", dtype=torch.float16)
    y = m(x, precision=8)
    ref = x.float() @ deq.float().T
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=2e-3)


def test_save_layer_writes_the_reference_quantisers_file_layout(tmp_path):
    from anyprec_b200 import quantize
    rng = np.random.default_rng(9)
    shapes = {"self_attn.q_proj": (8, 256), "mlp.down_proj": (4, 512)}
    luts_by, codes_by = [], []
    for N, K in shapes.values():
        w, s = layer(rng, N, K)
        luts, codes = quantize.seed_and_upscale_layer(torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda(), 3, 8)
        luts_by.append(luts)
        codes_by.append(codes)
    quantize.save_layer(str(tmp_path), 2, list(shapes), luts_by, codes_by, 3, 8)
    weights = torch.load(tmp_path / "weights" / "l2.pt", weights_only=False)
    for (name, (N, K)), codes in zip(shapes.items(), codes_by):
        assert weights[name].dtype == np.uint8 and weights[name].shape == (N, 1, K)
        assert np.array_equal(weights[name][:, 0], codes.cpu().numpy())
    for b in range(3, 9):
        lut = torch.load(tmp_path / f"lut_{b}" / "l2.pt", weights_only=False)
        for (name, (N, K)), luts in zip(shapes.items(), luts_by):
            assert lut[name].dtype == np.float16 and lut[name].shape == (N, 1, 1 << b)
            assert np.array_equal(lut[name][:, 0], luts[b].cpu().numpy())


def test_refusals():
    from anyprec_b200 import quantize
    w = torch.zeros((2, 64), device="cuda")
    with pytest.raises(ValueError):
        quantize.seed_and_upscale_layer(w, w, 4, 3)
    with pytest.raises(ValueError):
        quantize.seed_and_upscale_layer(w, w[:1])
    with pytest.raises(ValueError):
        quantize.seed_and_upscale_layer(torch.zeros((1, 32800), device="cuda"), torch.zeros((1, 32800), device="cuda"))
    with pytest.raises(ValueError):
        quantize.seed_and_upscale_layer(w.cpu(), w.cpu())
