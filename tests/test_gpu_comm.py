"""One-shot all-reduce over peer memory (ap_allreduce_oneshot).

With one GPU the rank set is just this process: the kernel still goes through all its steps (store
into the inbox, publish, wait, reduce), on both inbox generations and under CUDA-graph replay.
With two or more GPUs, child processes (one per GPU) sum different tensors and every rank must end
with exactly the bits of an fp32 sum taken in rank order."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


# element counts of consecutive calls: 8 halfs per 16-byte vector, 256 vectors per block
MIXED_COUNTS = (8, 4112, 8192, 8, 65536, 4112, 8, 8200, 4104, 65536, 16, 12304, 8192, 4112)


def test_single_rank_roundtrip_and_graph_replay():
    from anyprec_b200.comm import OneShotAllReduce
    dev = torch.device("cuda", 0)
    ar = OneShotAllReduce(128 * 1024, dev)
    gen = torch.Generator(device=dev).manual_seed(5)
    for n in (8, 4096, 8192, 32768):
        for _ in range(3):                                   # odd count: both generations get used
            x = torch.randn(n, device=dev, generator=gen).to(torch.float16)
            y = ar(x.clone())
            assert torch.equal(y, x)
    # sizes whose block counts change from call to call (1, 2, 2, 1, 16, 2, 1, 64 blocks ...): the inbox
    # generation must follow the call, not the block
    for n in MIXED_COUNTS:
        x = torch.randn(n, device=dev, generator=gen).to(torch.float16)
        assert torch.equal(ar(x.clone()), x), n
    x = torch.randn(8192, device=dev, generator=gen).to(torch.float16)
    out = torch.empty_like(x)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ar(x, out=out)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            ar(x, out=out)
    for _ in range(5):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, x)
    assert not ar.wait_expired()
    with pytest.raises(RuntimeError):
        ar(torch.zeros(128 * 1024, device=dev, dtype=torch.float16))     # 256 KB payload > 128 KB
    # the form that adds the sum to a residual stream: h += x, out = h * g, partial sums of squares of h
    for rows, n in ((1, 512), (3, 4096), (8, 8192), (2, 20000)):
        x = torch.randn((rows, n), device=dev, generator=gen).to(torch.float16)
        h0 = torch.randn((rows, n), device=dev, generator=gen).to(torch.float16)
        gw = (1 + 0.1 * torch.randn(n, device=dev, generator=gen)).to(torch.float16)
        blocks = ar.residual_blocks(rows, n)
        assert blocks == (n // 8 + 255) // 256
        h, out = h0.clone(), torch.empty_like(x)
        ssq = torch.full((rows, blocks), float("nan"), device=dev)
        ar.residual(x, h, gw, ssq, out)
        want_h = (h0.float() + x.float()).half()
        assert torch.equal(h, want_h) and torch.equal(out, (want_h.float() * gw.float()).half())
        assert torch.allclose(ssq.sum(-1), want_h.float().pow(2).sum(-1), rtol=1e-5)
    assert ar.residual_blocks(8, 32768) == 0              # 8 rows x 16 blocks: more blocks than a call may have
    # the product that stores its tiles into the inboxes itself, then the collecting half (plain and residual
    # form), unsplit and split along K, between ordinary calls
    import any_precision_ext as ext
    from anyprec_b200 import packing
    N, K = 512, 2048
    q = packing.random_qweight(8, N, K, device=dev, generator=gen)
    for w in (3, 4, 6, 8):
        lut = packing.random_lut(N, w, device=dev, generator=gen)
        for rows in (1, 3, 8):
            x = torch.randn((rows, K), device=dev, generator=gen).half()
            for splits in (1, 2):
                want = ext.matmul_kbit(x, q, lut, w, splits=splits)
                assert ext.matmul_kbit(x, q, lut, w, splits=splits, push=ar.push_target) is None
                got = ar.collect(torch.empty_like(want))
                assert torch.equal(got, want), (w, rows, splits)
                ar(torch.ones(8, device=dev, dtype=torch.float16))
                h0 = torch.randn((rows, N), device=dev, generator=gen).half()
                gw = (1 + 0.1 * torch.randn(N, device=dev, generator=gen)).half()
                h, y = h0.clone(), torch.empty_like(want)
                ssq = torch.zeros((rows, ar.residual_blocks(rows, N)), device=dev)
                ext.matmul_kbit(x, q, lut, w, splits=splits, push=ar.push_target)
                ar.collect(y, h, gw, ssq)
                want_h = (h0.float() + want.float()).half()
                assert torch.equal(h, want_h) and torch.equal(y, (want_h.float() * gw.float()).half())
                assert torch.allclose(ssq.sum(-1), want_h.float().pow(2).sum(-1), rtol=1e-5)
    assert not ar.wait_expired()
    ar.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from anyprec_b200.comm import OneShotAllReduce
        ar = OneShotAllReduce(128 * 1024, dev)
        ok = True
        for it, n in enumerate((8, 4096, 8192, 8192, 65536, 8192, 1024)):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(100 * it + r)).to(torch.float16) for r in range(world)]
            want = torch.zeros(n, dtype=torch.float32)
            for r in range(world):
                want += xs[r].float()                         # rank order, fp32: what the kernel does
            got = ar(xs[rank].to(dev)).cpu()
            ok = ok and torch.equal(got, want.to(torch.float16))
        # Calls of changing size queued back to back with no host synchronisation in between (a rank can
        # run a call ahead of another): results are compared only after the whole sequence.
        seq = MIXED_COUNTS * 3
        ins, wants = [], []
        for it, n in enumerate(seq):
            xs = [torch.randn(n, generator=torch.Generator().manual_seed(7000 + 10 * it + r)).to(torch.float16)
                  for r in range(world)]
            want = torch.zeros(n, dtype=torch.float32)
            for r in range(world):
                want += xs[r].float()
            ins.append(xs[rank].to(dev))
            wants.append(want.to(torch.float16))
        torch.cuda.synchronize()
        dist.barrier()
        outs = [ar(t, out=torch.empty_like(t)) for t in ins]
        torch.cuda.synchronize()
        for got, want in zip(outs, wants):
            ok = ok and torch.equal(got.cpu(), want)
        # replayed graph: the sequence numbers live on the device
        x = torch.full((8192,), float(rank + 1), device=dev, dtype=torch.float16)
        out = torch.empty_like(x)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            ar(x, out=out)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                ar(x, out=out)
                ar(out, out=out)
        total = world * (world + 1) // 2
        for _ in range(20):
            g.replay()
        torch.cuda.synchronize()
        ok = ok and bool((out == float(total * world)).all())
        # the residual form across ranks, between plain calls of other sizes
        rows, n = 4, 8192
        xs = [torch.randn((rows, n), generator=torch.Generator().manual_seed(900 + r)).to(torch.float16) for r in range(world)]
        h0 = torch.randn((rows, n), generator=torch.Generator().manual_seed(899)).to(torch.float16)
        gw = (1 + 0.1 * torch.randn(n, generator=torch.Generator().manual_seed(898))).to(torch.float16)
        want = torch.zeros((rows, n), dtype=torch.float32)
        for r in range(world):
            want += xs[r].float()
        want_h = (h0.float() + want.half().float()).half()
        h, out = h0.to(dev), torch.empty((rows, n), device=dev, dtype=torch.float16)
        ssq = torch.zeros((rows, ar.residual_blocks(rows, n)), device=dev)
        ar(torch.ones(8, device=dev, dtype=torch.float16))
        ar.residual(xs[rank].to(dev), h, gw.to(dev), ssq, out)
        ar(torch.ones(4112, device=dev, dtype=torch.float16))
        torch.cuda.synchronize()
        ok = ok and torch.equal(h.cpu(), want_h) and torch.equal(out.cpu(), (want_h.float() * gw.float()).half())
        ok = ok and torch.allclose(ssq.sum(-1).cpu(), want_h.float().pow(2).sum(-1), rtol=1e-5)
        # every rank's product pushed from the kernel's epilogue, collected into the same bits as the one-kernel form
        import any_precision_ext as ext
        from anyprec_b200 import packing
        g = torch.Generator(device=dev).manual_seed(50 + rank)
        Nn, Kk = 1024, 1024
        q = packing.random_qweight(8, Nn, Kk, device=dev, generator=g)
        lut = packing.random_lut(Nn, 4, device=dev, generator=g)
        for rows_ in (1, 8):
            xr = torch.randn((rows_, Kk), device=dev, generator=g).half()
            part = ext.matmul_kbit(xr, q, lut, 4)
            want2 = ar(part.clone())
            ext.matmul_kbit(xr, q, lut, 4, push=ar.push_target)
            got2 = ar.collect(torch.empty_like(part))
            torch.cuda.synchronize()
            ok = ok and torch.equal(got2, want2)
        ok = ok and not ar.wait_expired()
        ar.close()
        result[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_on_separate_gpus_agree_bit_for_bit():
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(result.get(r) for r in range(world)), dict(result)
