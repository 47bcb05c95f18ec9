"""matmul_kbit with the gated-MLP epilogue (ap_matmul_kbit_gated): gate and up projections stacked tile by
tile, silu(gate) * up out of one launch.  Checked bit for bit against the plain product of the same operand
followed by ap_silu_mul, and within matmul_kbit's tolerance against the oracle's product of the two
separate layers."""
import numpy as np
import pytest
import torch

from conftest import make_layer
from oracle import oracle

pytestmark = pytest.mark.gpu

# |y - r| <= ATOL + RTOL * |r| against silu(gate) * up of the oracle's fp64-accumulated products: the two
# fp16 roundings before the product and the one after contribute up to 1.5e-3 relative.
RTOL, ATOL = 6e-3, 2e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def build(F, K, seed):
    from anyprec_b200 import packing
    gc, gl = make_layer(F, K, seed=seed)
    uc, ul = make_layer(F, K, seed=seed + 1)
    gq, uq = dev(oracle.pack(gc)), dev(oracle.pack(uc))
    q, luts = packing.interleave_gate_up(gq, uq, {b: dev(t) for b, t in gl.items()}, {b: dev(t) for b, t in ul.items()})
    return (gq, gl), (uq, ul), q, luts


def oracle_gated(x, gate, up, w):
    g = oracle.c_matmul(x, gate[0].cpu().numpy(), gate[1][w], w).astype(np.float64)
    u = oracle.c_matmul(x, up[0].cpu().numpy(), up[1][w], w).astype(np.float64)
    return g / (1.0 + np.exp(-g)) * u


@pytest.mark.parametrize("F,K", [(64, 1024), (344, 4096), (128, 2176), (8, 128)])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_gated_epilogue_equals_product_then_silu_mul(F, K, M):
    import any_precision_ext as ext
    gate, up, q, luts = build(F, K, seed=F + K)
    x = np.random.default_rng(M).normal(size=(M, K)).astype(np.float16)
    xd = dev(x)
    for w in (3, 4, 5, 6, 7, 8):
        for splits in (1, 2, 5):
            y = ext.matmul_kbit(xd, q, luts[w], w, gated=True, splits=splits)
            assert y.shape == (M, F)
            plain = ext.matmul_kbit(xd, q, luts[w], w, splits=splits)
            assert torch.equal(y, ext.silu_mul(plain, tiled=True)), (w, splits)
        ref = oracle_gated(x, gate, up, w)
        err = np.abs(y.cpu().numpy().astype(np.float64) - ref)
        assert (err <= ATOL + RTOL * np.abs(ref)).all(), f"w={w}: max err {err.max():.3e}"


def test_silu_mul_layouts_agree():
    import any_precision_ext as ext
    rng = np.random.default_rng(5)
    rows, F = 5, 72
    g, u = rng.normal(size=(rows, F)).astype(np.float16), rng.normal(size=(rows, F)).astype(np.float16)
    side = dev(np.concatenate([g, u], axis=1))
    tiled = dev(np.stack([g.reshape(rows, F // 8, 8), u.reshape(rows, F // 8, 8)], axis=2).reshape(rows, 2 * F))
    a = ext.silu_mul(side)
    assert torch.equal(a, ext.silu_mul(tiled, tiled=True))
    ref = torch.nn.functional.silu(dev(g).float()).half().float() * dev(u).float()
    assert torch.allclose(a.float(), ref, rtol=2e-3, atol=1e-4)


def test_gated_module_decode_and_prefill_paths():
    """AnyPrecisionLinear.fuse_gated: the one-launch path (up to eight rows) and the product + ap_silu_mul
    path (more rows, i.e. the prompt) against the two separate layers."""
    from anyprec_b200 import AnyPrecisionLinear
    F, K = 256, 2048
    layers = []
    for i in range(2):
        codes, luts = make_layer(F, K, seed=300 + i)
        m = AnyPrecisionLinear(K, F, [3, 4, 8], bias=False, device="cuda")
        m.qweight.copy_(dev(oracle.pack(codes)))
        for b in (3, 4, 8):
            getattr(m, f"lut{b}").copy_(dev(luts[b]))
        layers.append(m)
    fused = AnyPrecisionLinear.fuse_gated(*layers)
    assert fused.out_features == 2 * F and fused.gated
    for rows in (1, 8, 9, 200):
        x = dev(np.random.default_rng(rows).normal(size=(rows, K)).astype(np.float16))
        for w in (3, 8):
            g, u = layers[0](x, precision=w), layers[1](x, precision=w)
            ref = torch.nn.functional.silu(g.float()).half().float() * u.float()
            y = fused.forward_gated(x, precision=w)
            assert y.shape == (rows, F)
            assert torch.allclose(y.float(), ref, rtol=6e-3, atol=2e-3), (rows, w)
    out = torch.empty((3, F), dtype=torch.float16, device="cuda")
    x = dev(np.random.default_rng(0).normal(size=(3, K)).astype(np.float16))
    assert fused.forward_gated(x, out=out) is out and torch.equal(out, fused.forward_gated(x))
    with pytest.raises(RuntimeError):
        layers[0].forward_gated(x)


def test_gated_refuses_what_the_kernel_does_not_take():
    import any_precision_ext as ext
    gate, up, q, luts = build(16, 1024, seed=1)
    x9 = dev(np.zeros((9, 1024), dtype=np.float16))
    with pytest.raises(ValueError):
        ext.matmul_kbit(x9, q, luts[4], 4, gated=True)
    # K not a multiple of 128: only the plain kernel takes it, and that has no gated epilogue
    gate, up, q, luts = build(16, 96, seed=2)
    x = dev(np.ones((1, 96), dtype=np.float16))
    assert not ext.gated_supported(x, q, luts[4])
    with pytest.raises(ValueError):
        ext.matmul_kbit(x, q, luts[4], 4, gated=True)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("splits,H,K1", [(1, 256, 1024), (3, 256, 1024), (2, 384, 11008), (1, 128, 1152)])
def test_residual_and_prenorm_products_fold_add_and_rmsnorm(M, splits, H, K1):
    """h += linear_1(x); z = linear_2(rmsnorm(h) * g) as two launches (ap_matmul_kbit_residual,
    ap_matmul_kbit_prenorm) against the same chain with the add and the norm written out; row lengths with a
    short last group (11008, 1152) and a width that is not a power of two (384) among them."""
    import any_precision_ext as ext
    F = 192
    c1, l1 = make_layer(H, K1, seed=41)
    c2, l2 = make_layer(F, H, seed=42)
    q1, q2 = dev(oracle.pack(c1)), dev(oracle.pack(c2))
    rng = np.random.default_rng(M + splits)
    x = dev(rng.normal(size=(M, K1)).astype(np.float16))
    h0 = dev(rng.normal(size=(M, H)).astype(np.float16))
    g = dev((1.0 + 0.1 * rng.normal(size=H)).astype(np.float16))
    eps = 1e-5
    for w in (3, 4, 6, 8):
        t1, t2 = dev(l1[w]), dev(l2[w])
        # written out
        p = ext.matmul_kbit(x, q1, t1, w, splits=splits)
        h_ref = (h0.float() + p.float()).half()
        r = torch.rsqrt(h_ref.float().pow(2).mean(-1, keepdim=True) + eps)
        y_ref = ((h_ref.float() * r).half().float() * g.float()).half()
        z_ref = ext.matmul_kbit(y_ref, q2, t2, w).float()
        # folded
        h = h0.clone()
        ssq = torch.full((M, H // 16), float("nan"), dtype=torch.float32, device="cuda")
        y = ext.matmul_kbit(x, q1, t1, w, splits=splits, residual=(h, g, ssq))
        assert torch.equal(h, h_ref)                                   # the residual stream itself: bit for bit
        assert torch.equal(y, (h_ref.float() * g.float()).half())
        assert torch.allclose(ssq.sum(-1), h_ref.float().pow(2).sum(-1), rtol=1e-5)
        z = ext.matmul_kbit(y, q2, t2, w, prenorm=(ssq, H, eps)).float()
        err = (z - z_ref).abs()
        assert float((err / z_ref.abs().clamp_min(0.05 * float(z_ref.abs().max()))).max()) < 1e-2, w
        assert float(err.mean()) < 1e-3 * max(1.0, float(z_ref.abs().max()))


def test_gated_prenorm_product():
    import any_precision_ext as ext
    F, K = 128, 512
    gate, up, q, luts = build(F, K, seed=77)
    rng = np.random.default_rng(3)
    M = 4
    hsrc = dev(rng.normal(size=(M, K)).astype(np.float16))                 # plays h * g
    ssq = torch.zeros((M, K // 16), dtype=torch.float32, device="cuda")
    ssq[:, 0] = torch.tensor([K * 4.0, K * 0.25, K * 1.0, K * 9.0])         # root mean squares 2, 0.5, 1, 3
    r = torch.tensor([0.5, 2.0, 1.0, 1.0 / 3.0], device="cuda")[:, None]
    for w in (3, 5, 8):
        y = ext.matmul_kbit(hsrc, q, luts[w], w, gated=True, prenorm=(ssq, K, 0.0)).float()
        plain = ext.matmul_kbit(hsrc, q, luts[w], w).float().view(M, F // 8, 2, 8)
        gs, us = (plain[:, :, 0] * r[:, :, None]).half().float(), (plain[:, :, 1] * r[:, :, None]).half().float()
        ref = (torch.nn.functional.silu(gs).half().float() * us).half().float().reshape(M, F)
        assert torch.allclose(y, ref, rtol=4e-3, atol=1e-4), w
