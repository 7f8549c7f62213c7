"""Multi-process CPU tests (gloo, 127.0.0.1): the library communicators and the
plumbing configuration (ResNet-20, TopK 1 %, residual memory, all-gather,
world size 2, 20 steps) checked against uncompressed all-reduce training."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _entry(rank, world, port, fn, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = fn(rank, world)
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_entry, args=(r, world, _free_port.port, fn, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            assert p.exitcode == 0, "rank failed with exit code %s" % p.exitcode
        return dict(ret)


@pytest.fixture(autouse=True)
def _port():
    _free_port.port = _free_port()
    yield


def _communicators(rank, world):
    from grace_b200 import grace_from_params

    results = {}
    torch.manual_seed(rank)
    x = torch.randn(1000) * 0.01
    dense = x.clone()
    dist.all_reduce(dense)
    dense /= world
    # dense codecs
    for comp in ("none", "fp16"):
        grc = grace_from_params({"compressor": comp, "memory": "none", "communicator": "allreduce", "world_size": world})
        results[comp] = (grc.step(x.clone(), "w") - dense).abs().max().item()
    # sparse, same-size and variable-size, three transports
    for comp, comm in (("topk", "allgather"), ("topk", "broadcast"), ("threshold", "allgather"),
                       ("dgc", "allgather"), ("randomk", "allreduce"), ("qsgd", "allgather"), ("qsgd", "alltoall"),
                       ("terngrad", "alltoall"), ("natural", "alltoall"), ("signsgd", "allgather"),
                       ("onebit", "allgather"), ("adaq", "allgather"), ("inceptionn", "allgather")):
        mem = "dgc" if comp == "dgc" else "residual"
        grc = grace_from_params({"compressor": comp, "memory": mem, "communicator": comm, "world_size": world,
                                 "compress_ratio": 0.05, "threshold": 0.02, "gradient_clipping": comp == "dgc"})
        out = grc.step(x.clone(), "w")
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        results[comp + "/" + comm] = (bool(torch.isfinite(out).all()), same, out.shape == x.shape)
    # topk allgather equals the hand-computed mean of the per-rank top-k tensors
    grc = grace_from_params({"compressor": "topk", "memory": "none", "communicator": "allgather", "world_size": world,
                             "compress_ratio": 0.1})
    out = grc.step(x.clone(), "t")
    mine = torch.zeros_like(x)
    idx = x.abs().topk(100).indices
    mine[idx] = x[idx]
    dist.all_reduce(mine)
    results["topk_exact"] = (out - mine / world).abs().max().item()
    # powersgd: P and Q averaged over ranks
    grc = grace_from_params({"compressor": "powersgd", "memory": "powersgd", "communicator": "allreduce",
                             "world_size": world, "compress_rank": 2})
    torch.manual_seed(123)  # same Q initialisation on every rank
    m = torch.randn(20, 30)
    out = grc.step(m + rank, "m")
    results["powersgd_shape"] = tuple(out.shape)
    return results


def test_library_communicators_over_gloo():
    res = _run(_communicators, 2)
    for rank in (0, 1):
        r = res[rank]
        assert r["none"] < 1e-7 and r["fp16"] < 1e-4
        assert r["topk_exact"] < 1e-8
        assert r["powersgd_shape"] == (20, 30)
        for key, val in r.items():
            if "/" in key:
                finite, same, shape_ok = val
                assert finite and shape_ok, key
                if not key.startswith(("qsgd", "terngrad", "natural")):
                    assert same, key  # deterministic codecs agree bit for bit across ranks


def _train(rank, world):
    from grace_b200 import grace_from_params
    from grace_b200.models import resnet20

    def run(params):
        torch.manual_seed(0)
        model = resnet20()
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        grc = grace_from_params({**params, "world_size": world})
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for step in range(20):
            x = torch.randn(32, 3, 32, 32, generator=g)
            y = torch.randint(0, 10, (32,), generator=g)
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            for name, p in model.named_parameters():
                p.grad.copy_(grc.step(p.grad, name))
            opt.step()
            losses.append(loss.item())
        return losses

    dense = run({"compressor": "none", "memory": "none", "communicator": "allreduce"})
    topk = run({"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.01})
    return dense, topk


def test_resnet20_topk_tracks_uncompressed_training():
    res = _run(_train, 2)
    dense, topk = res[0]
    assert all(l == l for l in topk)
    # both start from the same loss and neither diverges; compressed training
    # stays within a generous band of the dense run on this 20-step horizon
    assert abs(dense[0] - topk[0]) < 1e-4
    # (random labels with lr 0.1 and momentum 0.9: the loss is noisy in both runs; error feedback
    # releases delayed updates in bursts, hence the wide band)
    assert max(topk) < 2.0 * max(dense) + 4.0
    assert abs(sum(topk[-5:]) / 5 - sum(dense[-5:]) / 5) < 2.5


def _failure_detection(rank, world):
    """A rank that never joins a collective: the others must get an error from a
    short process-group timeout instead of waiting forever (host-side only)."""
    import datetime

    from grace_b200.utils.faults import HeartbeatMonitor

    store = dist.distributed_c10d._get_default_store()
    mon = HeartbeatMonitor(store, rank, world, interval_s=0.05, timeout_s=0.5)
    mon.beat()
    dist.barrier()
    if rank == 1:
        return "left"          # stops beating and never joins the next step
    import time

    time.sleep(1.0)
    mon.beat()
    dead = mon.dead_ranks()
    return dead


def test_heartbeat_detects_a_rank_that_left():
    res = _run(_failure_detection, 2)
    assert res[1] == "left"
    assert res[0] == [1]


def _ddp_hook(rank, world):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from grace_b200 import grace_from_params
    from grace_b200.parallel.ddp_hook import register_grace_hook

    torch.manual_seed(0)
    model = DDP(torch.nn.Sequential(torch.nn.Linear(20, 30), torch.nn.ReLU(), torch.nn.Linear(30, 5)))
    grc = grace_from_params({"compressor": "none", "memory": "none", "communicator": "allreduce", "world_size": world})
    register_grace_hook(model, grc)
    ref = torch.nn.Sequential(torch.nn.Linear(20, 30), torch.nn.ReLU(), torch.nn.Linear(30, 5))
    ref.load_state_dict(model.module.state_dict())
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(8, 20, generator=g)
    model(x).sum().backward()
    ref(x).sum().backward()
    worst = 0.0
    for p, q in zip(model.module.parameters(), ref.parameters()):
        expect = q.grad.clone()
        dist.all_reduce(expect)
        worst = max(worst, (p.grad - expect / world).abs().max().item())
    return worst


def test_ddp_comm_hook_averages_like_allreduce():
    res = _run(_ddp_hook, 2)
    assert res[0] < 1e-6 and res[1] < 1e-6


def _hvd_api(rank, world):
    import grace_b200.parallel.hvd as hvd

    assert hvd.size() == world and hvd.rank() == rank
    t = torch.full((4,), float(rank + 1))
    h = hvd.allreduce_async_(t, average=True)
    assert hvd.synchronize(h) is t and torch.allclose(t, torch.full((4,), (1 + world) * world / 2 / world))
    g = hvd.allgather(torch.arange(rank + 1, dtype=torch.float32))
    model = torch.nn.Linear(3, 2)
    with torch.no_grad():
        model.weight.fill_(float(rank))
    hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    opt = torch.optim.SGD(model.parameters(), lr=0.1 * (rank + 1), momentum=0.9)
    hvd.broadcast_optimizer_state(opt, root_rank=0)
    return g.tolist(), float(model.weight.abs().sum()), opt.param_groups[0]["lr"]


def test_horovod_style_helpers():
    res = _run(_hvd_api, 2)
    for r in (0, 1):
        gathered, wsum, lr = res[r]
        assert gathered == [0.0, 0.0, 1.0] and wsum == 0.0 and abs(lr - 0.1) < 1e-12


def _nvls_fallback(rank, world):
    """``nvls=True`` on CPU ranks: no multicast, so every call lands in the library path and still averages."""
    from grace_b200 import grace_from_params
    from grace_b200.communicator.nvls import NvlsAllreduce

    out = {}
    grc = grace_from_params({"compressor": "none", "memory": "none", "communicator": "allreduce", "world_size": world,
                             "fused": True, "nvls": True, "nvls_min_world": 2})
    out["type"] = isinstance(grc, NvlsAllreduce)
    x = torch.full((1024,), float(rank + 1))
    got = grc.step(x.clone(), "w")
    out["step"] = bool(torch.allclose(got, torch.full_like(got, (world + 1) / 2.0)))
    flat = torch.full((256,), float(rank))
    res = grc.step_flat(flat)                     # no layout: library all-reduce, in place
    out["flat"] = bool(torch.allclose(res, torch.full_like(res, (world - 1) / 2.0))) and res.data_ptr() == flat.data_ptr()
    out["buffer"] = grc.buffer(1024) is None
    out["launches"] = grc.stats()["nvls_launches"]
    # quantised codec with the push option: CPU tensors use the library communicator, the option is inert
    q = grace_from_params({"compressor": "fp16", "memory": "none", "communicator": "allgather", "world_size": world,
                           "fused": True, "nvls": True, "nvls_min_world": 2})
    got = q.step(torch.full((64,), float(rank + 1)), "h")
    out["fp16"] = bool(torch.allclose(got, torch.full_like(got, (world + 1) / 2.0)))
    return out


def test_nvls_options_fall_back_on_cpu_ranks():
    res = _run(_nvls_fallback, world=2)
    for rank in range(2):
        r = res[rank]
        assert r["type"] and r["step"] and r["flat"] and r["buffer"] and r["fp16"], r
        assert r["launches"] == 0


def _hvd_surface(rank, world):
    import grace_b200.parallel.hvd as hvd

    out = {}
    out["sizes"] = (hvd.size(), hvd.rank(), hvd.is_initialized(), hvd.local_size() >= 1, hvd.cross_size() >= 1)
    out["join"] = hvd.join()
    out["bobj"] = hvd.broadcast_object({"lr": 0.1 * (rank + 1)}, root_rank=1)["lr"]
    out["gobj"] = hvd.allgather_object(rank * 10)
    out["metric"] = hvd.metric_average(float(rank))
    hvd.barrier()
    # gradients that bypass grace (op=Sum) travel in fp16 when hvd.Compression.fp16 is given
    torch.manual_seed(0)
    model = torch.nn.Linear(8, 4)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.0), named_parameters=model.named_parameters(),
                                   compression=hvd.Compression.fp16, op=hvd.Sum)
    x = torch.full((2, 8), float(rank + 1))
    model(x).sum().backward()
    opt.step()
    g = model.weight.grad
    out["fp16_wire"] = (g.dtype == torch.float32, bool(torch.allclose(g, torch.full_like(g, 2.0 * sum(range(1, world + 1))))))
    return out


def test_horovod_surface_helpers():
    res = _run(_hvd_surface, world=2)
    for rank in range(2):
        r = res[rank]
        assert r["sizes"] == (2, rank, True, True, True)
        assert r["join"] in (0, 1) and r["join"] == res[0]["join"]
        assert abs(r["bobj"] - 0.2) < 1e-12 and r["gobj"] == [0, 10] and abs(r["metric"] - 0.5) < 1e-12
        assert r["fp16_wire"] == (True, True)


def _num_groups(rank, world):
    """num_groups bypasses GRACE and reduces each group of parameters with ONE all-reduce."""
    from grace_b200.parallel import DistributedOptimizer

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.ReLU(), torch.nn.Linear(5, 4), torch.nn.Linear(4, 2))
    opt = torch.optim.SGD(model.parameters(), lr=0.0)

    class Boom:   # must never be touched when num_groups > 0
        def send_step(self, *a):
            raise AssertionError("GRACE used although num_groups > 0")

    calls = []
    real = dist.all_reduce

    def counting(t, *a, **k):
        calls.append(t.numel())
        return real(t, *a, **k)

    dist.all_reduce = counting
    try:
        d = DistributedOptimizer(opt, grace=Boom(), named_parameters=model.named_parameters(), num_groups=2)
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(7, 6, generator=g)
        model(x).sum().backward()
        local = [p.grad.clone() for p in model.parameters()]
        d.step()
    finally:
        dist.all_reduce = real
    gathered = [None] * world
    dist.all_gather_object(gathered, local)
    mean = [sum(gs) / world for gs in zip(*gathered)]
    for p, m in zip(model.parameters(), mean):
        torch.testing.assert_close(p.grad, m)
    return sorted(calls)


def test_num_groups_reduces_group_wise():
    res = _run(_num_groups, 2)
    total = 6 * 5 + 5 + 5 * 4 + 4 + 4 * 2 + 2
    assert len(res[0]) == 2 and sum(res[0]) == total   # two all-reduces cover all six tensors
    assert res[0] == res[1]


def _agree_and_recover(rank, world):
    """A failure seen by one rank becomes known to all through the store; all recover, then exchange again."""
    from grace_b200 import grace_from_params

    store = dist.distributed_c10d._get_default_store()
    grc = grace_from_params({"compressor": "fp16", "memory": "none", "communicator": "allgather",
                             "world_size": world, "fused": True})
    grc.store = store
    x = torch.full((16,), float(rank + 1))
    first = grc.step(x.clone(), "w")                     # CPU tensors: the library path carries the data
    failed = grc.agree(RuntimeError("injected on the host") if rank == 1 else None, timeout_s=20)
    assert failed == [1], failed
    grc.recover(timeout_s=20)
    assert grc.agree(None, timeout_s=20) == []           # a second vote in the new epoch: all healthy
    again = grc.step(x.clone(), "w2")
    return first.tolist(), again.tolist()


def test_failed_rank_is_agreed_on_and_recovered():
    res = _run(_agree_and_recover, 2)
    assert res[0] == res[1]
    assert res[0][1] == [1.5] * 16    # healthy exchange after the recovery: mean of 1 and 2
