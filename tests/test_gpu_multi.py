"""Real multi-GPU tests (one process per GPU, NCCL for the bootstrap and the
baseline): the fused exchange over the IPC symmetric heap must give the same
aggregate as the library ``Allgather`` communicator.  Skipped with fewer than
two GPUs."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _token():
    """Rendezvous file of one multi-process test (see tests/_rendezvous.py)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import new_token

    return new_token()


def _entry(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import init_group

    init_group("nccl", rank, world, port, dev)
    try:
        ret[rank] = _body(rank, world, dev)
    finally:
        dist.destroy_process_group()


def _body(rank, world, dev):
    from grace_b200 import grace_from_params
    from grace_b200.ops.exchange import FlatLayout

    out = {}
    cases = [
        ("topk", "residual", {"compress_ratio": 0.01}),
        ("dgc", "dgc", {"compress_ratio": 0.01, "momentum": 0.9}),
        ("qsgd", "none", {"quantum_num": 64}),
        ("signsgd", "none", {}),
        ("efsignsgd", "efsignsgd", {"lr": 0.1}),
        ("fp16", "none", {}),
        ("none", "none", {}),
    ]
    n = 300_007
    for comp, mem, extra in cases:
        fused = grace_from_params({"compressor": comp, "memory": mem, "communicator": "allgather", "world_size": world,
                                   "fused": True, "timeout_ms": 5000, **extra})
        lib = grace_from_params({"compressor": comp, "memory": mem, "communicator": "allgather", "world_size": world,
                                 **extra})
        if comp == "dgc":
            lib.compressor.mode = "exact"
        worst = 0.0
        for step in range(3):
            g = torch.Generator().manual_seed(1000 * step + rank)
            x = (torch.randn(n, generator=g) * 1e-3).to(dev)
            got = fused.step(x.clone(), "w")
            fused.check()
            if comp == "qsgd":
                # stochastic: the library path draws different random numbers; compare against the dense mean
                ref = x.clone()
                dist.all_reduce(ref)
                ref /= world
                err = ((got - ref).norm() / ref.norm()).item()
                worst = max(worst, err)
                continue
            ref = lib.step(x.clone(), "w")
            scale = ref.abs().max().item() + 1e-12
            worst = max(worst, (got - ref).abs().max().item() / scale)
        # all ranks hold identical results
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        out[comp] = (worst, same)
    # small tensors one by one (the single-CTA sparse kernel: one plain launch per tensor and rank, real peers):
    # six steps so that both send slots are reused and the acknowledgements are needed
    for comp, mem, extra in (("topk", "residual", {"compress_ratio": 0.05}),
                             ("dgc", "dgc", {"compress_ratio": 0.01, "momentum": 0.9})):
        fused = grace_from_params({"compressor": comp, "memory": mem, "communicator": "allgather", "world_size": world,
                                   "fused": True, "timeout_ms": 5000, **extra})
        lib = grace_from_params({"compressor": comp, "memory": mem, "communicator": "allgather", "world_size": world,
                                 **extra})
        if comp == "dgc":
            lib.compressor.mode = "exact"
        worst, same = 0.0, True
        for step in range(6):
            for numel in (1, 100, 2048, 8192):
                g = torch.Generator().manual_seed(1000 * step + 10 * rank + numel)
                x = (torch.randn(numel, generator=g) * 1e-3).to(dev)
                got = fused.step(x.clone(), "s%d" % numel)
                ref = lib.step(x.clone(), "s%d" % numel)
                worst = max(worst, (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-12))
                gathered = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(gathered, got)
                same = same and all(torch.equal(gathered[0], t) for t in gathered)
        fused.check()
        out["small_" + comp] = (worst, same)
    # pipelined all-gather mode (encode of chunk c + 1 next to the pull of chunk c) against the phase-by-phase
    # kernel: same random streams, same order of the sums, so the same bits, step after step
    layout = FlatLayout.from_named([("a", 250_000), ("b", 64), ("c", 1_234_567)])
    for comp, extra in (("qsgd", {"quantum_num": 64}), ("natural_cuda", {})):
        pair = [grace_from_params({"compressor": comp, "memory": "residual", "communicator": "allgather",
                                   "world_size": world, "fused": True, "timeout_ms": 5000, "pipeline": mode, **extra})
                for mode in ("force", False)]
        same = True
        for step in range(4):
            g = torch.Generator().manual_seed(31 * step + rank)
            flat = torch.zeros(layout.total, device=dev)
            for o, c in zip(layout.offsets, layout.numels):
                flat[o:o + c] = (torch.randn(c, generator=g) * 1e-3).to(dev)
            a, b = flat.clone(), flat.clone()
            pair[0].step_flat(a, layout)
            pair[1].step_flat(b, layout)
            pair[0].check()
            pair[1].check()
            same = same and torch.equal(a, b)
        plans = [next(iter(c._plans.values())) for c in pair]
        assert plans[0].pipeline is not None and plans[1].pipeline is None
        same = same and torch.equal(plans[0].acc, plans[1].acc)
        out["pipelined_" + comp] = (0.0, same)
    # flat multi-tensor bucket, several steps on one channel (slot reuse, acknowledgements)
    layout = FlatLayout.from_named([("a", 5000), ("b", 64), ("c", 123_457)])
    fused = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                               "world_size": world, "fused": True, "compress_ratio": 0.02})
    for step in range(6):
        g = torch.Generator().manual_seed(77 * step + rank)
        flat = torch.zeros(layout.total, device=dev)
        for o, c in zip(layout.offsets, layout.numels):
            flat[o:o + c] = (torch.randn(c, generator=g) * 1e-3).to(dev)
        fused.step_flat(flat, layout)
    fused.check()
    out["flat_finite"] = bool(torch.isfinite(flat).all())
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_exchange_matches_library_over_real_gpus():
    world = min(torch.cuda.device_count(), 8)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _token()
        procs = [ctx.Process(target=_entry, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(600)
        for p in procs:
            assert p.exitcode == 0, "rank exited with %s" % p.exitcode
        res = dict(ret)
    for rank in range(world):
        r = res[rank]
        for comp, val in r.items():
            if comp == "flat_finite":
                assert val
                continue
            worst, same = val
            assert same, "%s: ranks disagree" % comp
            if comp == "qsgd":
                assert worst < 0.2, (comp, worst)
            else:
                assert worst < 1e-5, (comp, worst)


def _timeout_entry(rank, world, port, ret, pipelined=False):
    sys.path.insert(0, ROOT)
    os.environ.update(NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import init_group

    init_group("nccl", rank, world, port, dev)
    try:
        from grace_b200 import grace_from_params
        from grace_b200.ops.exchange import GraceCommError

        store = dist.distributed_c10d._get_default_store()
        if pipelined:   # the pipelined quantised exchange: its decode tiles wait for the peer's chunk flags
            grc = grace_from_params({"compressor": "qsgd", "memory": "residual", "communicator": "allgather",
                                     "world_size": world, "fused": True, "quantum_num": 64, "timeout_ms": 10000,
                                     "pipeline": "force"})
        else:
            grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                                     "world_size": world, "fused": True, "compress_ratio": 0.01, "timeout_ms": 10000})
        x = torch.randn(100_000, device=dev) * 1e-3
        for _ in range(2):                       # two healthy steps (generous limit: the first launch loads the kernels)
            grc.step(x.clone(), "w")
        grc.check()
        torch.cuda.synchronize()
        dist.barrier()
        for plan in grc._plans.values():         # from here on a wait gives up after half a second
            plan.channel.timeout_ns = int(500e6)
        if rank == 1:
            # leaves between steps: nothing of its own in flight, it just never launches step 3
            store.wait(["rank0_done"])
            ret[rank] = "left"
        else:
            grc.step(x.clone(), "w")             # the peer never publishes: bounded wait expires
            try:
                grc.check()
                ret[rank] = "no error"
            except GraceCommError as e:
                ret[rank] = (e.code, e.detail)
            # the context is still usable
            ret["alive"] = float(torch.ones(8, device=dev).sum())
            store.set("rank0_done", "1")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("pipelined", [False, True])
def test_peer_that_stops_launching_is_reported_as_timeout(pipelined):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _token()
        procs = [ctx.Process(target=_timeout_entry, args=(r, 2, port, ret, pipelined)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            assert p.exitcode == 0, "rank exited with %s" % p.exitcode
        res = dict(ret)
    assert res[1] == "left"
    assert res[0] == (2, 1)          # timeout waiting for peer 1's data
    assert res["alive"] == 8.0


def _ddp_entry(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import init_group

    init_group("nccl", rank, world, port, dev)
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        from grace_b200 import grace_from_params
        from grace_b200.models import resnet20
        from grace_b200.parallel.ddp_hook import register_grace_hook

        torch.manual_seed(0)
        base = resnet20().to(dev)
        ref = resnet20().to(dev)
        ref.load_state_dict(base.state_dict())
        model = DDP(base, device_ids=[rank], bucket_cap_mb=0.25)
        grc = grace_from_params({"compressor": "none", "memory": "none", "communicator": "allreduce",
                                 "world_size": world, "fused": True})
        register_grace_hook(model, grc)
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(8, 3, 32, 32, generator=g).to(dev)
        y = torch.randint(0, 10, (8,), generator=g).to(dev)
        worst = 0.0
        for _ in range(2):
            model.zero_grad(); ref.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            torch.nn.functional.cross_entropy(ref(x), y).backward()
            grc.check()
            for p, q in zip(model.module.parameters(), ref.parameters()):
                expect = q.grad.clone()
                dist.all_reduce(expect)
                expect /= world
                worst = max(worst, ((p.grad - expect).abs().max() / (expect.abs().max() + 1e-12)).item())
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


def test_ddp_comm_hook_with_fused_exchange():
    """DDP buckets go through the fused kernel (dense codec: exact mean)."""
    world = min(max(torch.cuda.device_count(), 1), 2)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _token()
        procs = [ctx.Process(target=_ddp_entry, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            assert p.exitcode == 0, "rank exited with %s" % p.exitcode
        res = dict(ret)
    for r in range(world):
        assert res[r] < 5e-3, res  # two separate cuDNN backward passes agree to ~1e-3 of the largest entry


def _recover_entry(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import init_group

    init_group("nccl", rank, world, port, dev)
    try:
        from grace_b200 import grace_from_params

        store = dist.distributed_c10d._get_default_store()
        grc = grace_from_params({"compressor": "qsgd", "memory": "residual", "communicator": "allgather",
                                 "quantum_num": 64, "world_size": world, "fused": True, "timeout_ms": 10000,
                                 "store": store})
        gen = torch.Generator().manual_seed(rank)
        x = (torch.randn(200_000, generator=gen) * 1e-3).to(dev)
        grc.step(x.clone(), "w")                            # generous limit: the first launch loads the kernels
        grc.check()
        assert grc.agree(timeout_s=60) == []               # a healthy step: nobody votes "failed"
        dist.barrier()
        for plan in grc._plans.values():                    # from here on a wait gives up after 300 ms
            plan.channel.timeout_ns = int(300e6)
        residual_before = next(iter(grc._plans.values())).acc.clone()
        # rank 1 sits this step out (between steps, with nothing of its own in flight): rank 0's wait for its
        # payload expires after 300 ms and is reported; rank 1 itself saw nothing wrong
        if rank == 0:
            grc.step(x.clone(), "w")
        failed = grc.agree(timeout_s=60)                    # every rank learns that rank 0 failed
        grc.recover(timeout_s=60)
        for plan in grc._plans.values():
            plan.channel.timeout_ns = int(10e9)
        if rank == 1:                                       # rank 1's error feedback did not move while it sat out
            assert torch.equal(next(iter(grc._plans.values())).acc, residual_before)
        # after the recovery: a healthy exchange again, identical on both ranks
        out = grc.step(x.clone(), "w")
        grc.check()
        assert grc.agree(timeout_s=60) == []
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        ret[rank] = (failed, bool(torch.equal(gathered[0], gathered[1])), bool(torch.isfinite(out).all()),
                     float(out.abs().max()) > 0)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_failure_is_agreed_on_and_a_healthy_exchange_follows_the_recovery():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _token()
        procs = [ctx.Process(target=_recover_entry, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            assert p.exitcode == 0, "rank exited with %s" % p.exitcode
        res = dict(ret)
    assert res[0] == ([0], True, True, True)
    assert res[1] == ([0], True, True, True)
