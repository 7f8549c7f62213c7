"""Dense all-reduce through the NVSwitch multicast mapping (``multimem.ld_reduce`` / ``multimem.st``), one
process per GPU.  Every rank records its findings and leaves through a common barrier, so no process exits
while the others still use the multicast object.  Skipped with fewer than two GPUs or without multicast."""
import os
import socket
import sys
import traceback

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


def _guard(res, label, fn, default):
    """Run a rank-local step; on an exception record it and carry on, so that every rank still takes part in
    the collectives that follow (no rank may stop half way while the others wait for it)."""
    try:
        return fn()
    except Exception:  # noqa: BLE001
        res.setdefault("error", "%s: %s" % (label, traceback.format_exc()))
        return default


def _body(rank, world, dev):
    from grace_b200 import grace_from_params

    res = {}
    grc = grace_from_params({"compressor": "none", "memory": "none", "communicator": "allreduce", "world_size": world,
                             "fused": True, "nvls": True, "nvls_min_world": 2, "timeout_ms": 5000})
    n = 1_000_000
    buf = grc.buffer(n)          # collective; returns None on every rank alike when there is no multicast
    if buf is None:
        return {"unavailable": True}
    # 1. a tensor outside the symmetric buffer (staged by the kernel), several exchanges in a row
    worst = 0.0
    for step in range(4):
        g = torch.Generator().manual_seed(31 * step + rank)
        x = torch.randn(n, generator=g).to(dev)
        ref = x.clone()
        dist.all_reduce(ref)
        ref /= world
        got = _guard(res, "staged", lambda: grc.step(x.clone(), "w"), torch.zeros_like(x))
        _guard(res, "check", grc.check, None)
        worst = max(worst, ((got - ref).abs().max() / ref.abs().max()).item())
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        res["same_%d" % step] = all(torch.equal(gathered[0], t) for t in gathered)
    res["staged_err"] = worst
    # 2. gradients that live in the symmetric buffer: reduced in place, no staging
    g = torch.Generator().manual_seed(500 + rank)
    x = torch.randn(n, generator=g).to(dev)
    ref = x.clone()
    dist.all_reduce(ref)
    ref /= world
    buf.copy_(x)
    out = _guard(res, "inplace", lambda: grc.step_flat(buf), buf)
    _guard(res, "check", grc.check, None)
    res["inplace_same_storage"] = out.data_ptr() == buf.data_ptr()
    res["inplace_err"] = ((buf - ref).abs().max() / ref.abs().max()).item()
    # 3. exact arithmetic: rank r contributes (r + 1) everywhere -> mean (W + 1) / 2
    buf.fill_(float(rank + 1))
    _guard(res, "exact", lambda: grc.step_flat(buf), None)
    _guard(res, "check", grc.check, None)
    res["exact"] = bool((buf == (world + 1) / 2.0).all())
    # 4. small tensors take the fallback and still average
    small = torch.full((1000,), float(rank), device=dev)
    got = grc.step(small, "s")
    res["small"] = bool(torch.allclose(got, torch.full_like(got, (world - 1) / 2.0)))
    res["launches"] = grc.stats()["nvls_launches"]
    # 5. optimizer integration: gradients live in the symmetric buffer and are averaged in place
    from grace_b200.optim import FusedSGD
    from grace_b200.parallel import DistributedOptimizer
    from grace_b200.parallel.flat import FlatParams

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 512), torch.nn.ReLU(), torch.nn.Linear(512, 256)).to(dev)
    twin = torch.nn.Sequential(torch.nn.Linear(64, 512), torch.nn.ReLU(), torch.nn.Linear(512, 256)).to(dev)
    twin.load_state_dict(model.state_dict())
    grc.min_numel = 0
    flat = FlatParams(model.named_parameters(), grad_buffer=grc.buffer)
    res["grads_in_symmetric_buffer"] = grc._find(flat.flat_g) is not None
    opt = DistributedOptimizer(FusedSGD(model.parameters(), lr=0.1, momentum=0.9, flat=flat), grace=grc,
                               named_parameters=model.named_parameters(), flat=flat)
    ref_opt = torch.optim.SGD(twin.parameters(), lr=0.1, momentum=0.9)
    before = grc.stats()["nvls_launches"]
    for step in range(2):
        g = torch.Generator().manual_seed(900 + 10 * step + rank)
        x = torch.randn(32, 64, generator=g).to(dev)
        opt.zero_grad()
        model(x).square().mean().backward()
        _guard(res, "optimizer", opt.step, None)
        ref_opt.zero_grad()
        twin(x).square().mean().backward()
        for p in twin.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        ref_opt.step()
    _guard(res, "check", grc.check, None)
    res["optimizer_launches"] = grc.stats()["nvls_launches"] - before
    res["optimizer_err"] = max(((a - b).abs().max() / b.abs().max()).item()
                               for a, b in zip(model.parameters(), twin.parameters()))
    return res


def _push_body(rank, world, dev):
    """Quantised codecs, all-gather mode: the push transport (slots replicated with multimem.st, decode from
    local memory) must give the bits of the pull transport (peers' slots read over NVLink)."""
    from grace_b200 import grace_from_params

    res = {}
    cases = [
        ("qsgd", "residual", {"quantum_num": 64}),
        ("natural", "residual", {}),
        ("terngrad", "none", {}),
        ("efsignsgd", "efsignsgd", {"lr": 0.1}),
        ("signsgd", "none", {}),
        ("onebit", "residual", {}),
        ("u8bit", "none", {}),
        ("fp16", "none", {}),
    ]
    n = 400_003
    for comp, mem, extra in cases:
        base = {"compressor": comp, "memory": mem, "communicator": "allgather", "world_size": world, "fused": True,
                "timeout_ms": 5000, "seed": 11, **extra}
        pull = grace_from_params(dict(base))
        push = grace_from_params(dict(base, nvls=True, nvls_min_world=2))      # collective: allocates the receive area
        same, pushed = True, False
        for step in range(3):
            g = torch.Generator().manual_seed(97 * step + rank)
            x = (torch.randn(n, generator=g) * 1e-3).to(dev)
            a = _guard(res, comp + " pull", lambda: pull.step(x.clone(), "w"), torch.zeros_like(x))
            b = _guard(res, comp + " push", lambda: push.step(x.clone(), "w"), torch.ones_like(x))
            _guard(res, comp + " check", lambda: (pull.check(), push.check()), None)
            same = same and torch.equal(a, b)
        plans = list(push._plans.values())
        pushed = bool(plans) and all(getattr(p, "recv", None) is not None for p in plans)
        res[comp] = (same, pushed)
    return res


def _entry(rank, world, port, ret, body=None):
    sys.path.insert(0, ROOT)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import init_group

    init_group("nccl", rank, world, port, dev)
    try:
        ret[rank] = (body or _body)(rank, world, dev)
    except Exception:  # noqa: BLE001 - reported by the parent; the rank still leaves through the barrier
        ret[rank] = {"error": traceback.format_exc()}
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_multicast_allreduce_matches_library_allreduce():
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
    if all(r.get("unavailable") for r in res.values()):
        pytest.skip("no NVSwitch multicast on this machine")
    for rank in range(world):
        r = res[rank]
        assert "error" not in r, r.get("error")
        assert r["staged_err"] < 1e-6 and r["inplace_err"] < 1e-6, r
        assert all(r["same_%d" % s] for s in range(4)), "ranks disagree"
        assert r["inplace_same_storage"] and r["exact"] and r["small"], r
        assert r["launches"] == 6, r
        assert r["grads_in_symmetric_buffer"] and r["optimizer_launches"] == 2 and r["optimizer_err"] < 1e-5, r


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_push_transport_gives_the_bits_of_the_pull_transport():
    world = min(torch.cuda.device_count(), 8)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _token()
        procs = [ctx.Process(target=_entry, args=(r, world, port, ret, _push_body)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(600)
        for p in procs:
            assert p.exitcode == 0, "rank exited with %s" % p.exitcode
        res = dict(ret)
    for rank in range(world):
        r = res[rank]
        assert "error" not in r, r.get("error")
        if not any(pushed for _, pushed in r.values()):
            pytest.skip("no NVSwitch multicast on this machine")
        for comp, (same, pushed) in r.items():
            assert pushed, "%s: the push transport was not used" % comp
            assert same, "%s: push and pull transports disagree" % comp
