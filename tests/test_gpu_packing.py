"""The device packer and unpacker (ap_pack_codes / ap_unpack_codes) against the oracle, the committed
output of the reference's packer, and each other; and K-shard re-packing on the device."""
import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_cases())
def test_device_packer_reproduces_the_reference_packers_output(name):
    from anyprec_b200 import packing
    g = load_golden(name)
    codes = torch.from_numpy(g["codes"]).cuda()
    q = packing.pack_codes(codes, 8)
    assert q.dtype == torch.int32 and np.array_equal(q.cpu().numpy(), g["qweight"])
    for w in (3, 5, 8):
        back = packing.unpack_codes(q, w)
        assert np.array_equal(back.cpu().numpy(), g["codes"] >> (8 - w))


@pytest.mark.parametrize("N,K", [(1, 32), (7, 64), (5, 1056), (33, 2048 + 96), (16, 11008), (3, 3584), (257, 4096)])
@pytest.mark.parametrize("P", [3, 5, 8])
def test_device_packer_against_oracle(N, K, P):
    from anyprec_b200 import packing
    rng = np.random.default_rng(N * 131 + K + P)
    codes = rng.integers(0, 1 << P, size=(N, K), dtype=np.uint8)
    q = packing.pack_codes(torch.from_numpy(codes).cuda(), P)
    assert np.array_equal(q.cpu().numpy(), oracle.pack(codes, parent_bits=P))
    assert np.array_equal(packing.unpack_codes(q, P).cpu().numpy(), codes)
    # a row slice of a wider operand (plane stride larger than the slice) unpacks in place
    if N >= 5:
        sl = q[:, 1:4, :]
        assert np.array_equal(packing.unpack_codes(sl, P).cpu().numpy(), codes[1:4])


def test_k_shards_repacked_on_the_device_equal_cpu_repacking():
    from anyprec_b200 import packing
    rng = np.random.default_rng(9)
    N, K = 48, 7168
    codes = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    q_cpu = packing.pack_codes(torch.from_numpy(codes))
    q_gpu = packing.pack_codes(torch.from_numpy(codes).cuda())
    assert torch.equal(q_gpu.cpu(), q_cpu)
    for k0, k1 in ((0, 3584), (3584, 7168), (1024, 4096), (2048, 2048 + 640)):
        shard = packing.slice_k(q_gpu, k0, k1)
        assert shard.is_cuda and torch.equal(shard.cpu(), packing.slice_k(q_cpu, k0, k1))
        assert np.array_equal(shard.cpu().numpy(), oracle.pack(codes[:, k0:k1]))
