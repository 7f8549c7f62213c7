"""The host engine of the exchange protocol (``csrc/host_exchange.cpp``): CPU ranks over POSIX shared memory.

Ranks are threads of this process (``ThreadWorld``: the native call releases the interpreter lock, so they run
and wait concurrently) or gloo processes.  Checked: every codec against a PyTorch restatement, the error-feedback
identity, slot reuse under a slow peer, both time-outs (a peer that never publishes, a peer that never reads),
recovery with the error-feedback state kept, checkpoint round trip.
"""
import os
import sys
import time

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from grace_b200 import compressor as C_  # noqa: E402
from grace_b200 import memory as M_  # noqa: E402
from grace_b200.communicator.host import HostExchange, ThreadWorld  # noqa: E402
from grace_b200.ops.exchange import GraceCommError  # noqa: E402


def _grads(world, n, steps, scale=1e-3):
    return [[torch.randn(n, generator=torch.Generator().manual_seed(100 * s + r)) * scale for r in range(world)]
            for s in range(steps)]


def _run_ranks(world, make, grads, name="w", timeout_ms=30000.0, hook=None):
    """Every rank steps through ``grads[s][rank]``; returns per-rank lists of outputs and the communicators."""
    tw = ThreadWorld(world)

    def body(view):
        comp, mem = make()
        grc = HostExchange(comp, mem, world, world=view, timeout_ms=timeout_ms)
        outs = []
        for s, per_rank in enumerate(grads):
            if hook is not None:
                hook(view.rank, s)
            outs.append(grc.step(per_rank[view.rank].clone(), name))
        return outs, grc

    res = tw.run(body)
    return [r[0] for r in res], [r[1] for r in res]


def _topk_dense(x, k):
    idx = torch.topk(x.abs(), k, sorted=False).indices
    out = torch.zeros_like(x)
    out[idx] = x[idx]
    return out


@pytest.mark.parametrize("world", [1, 2, 4])
def test_topk_residual_matches_restatement(world):
    n, ratio, steps = 10000, 0.01, 4
    grads = _grads(world, n, steps)
    outs, grcs = _run_ranks(world, lambda: (C_.TopKCompressor(ratio), M_.ResidualMemory()), grads)
    k = max(1, int(n * ratio))
    res = [torch.zeros(n) for _ in range(world)]
    for s in range(steps):
        want = torch.zeros(n)
        for r in range(world):
            acc = res[r] + grads[s][r]
            sent = _topk_dense(acc, k)
            res[r] = acc - sent
            want += sent
        want /= world
        for r in range(world):
            torch.testing.assert_close(outs[r][s], want, rtol=1e-6, atol=1e-9)
    for r in range(world):   # error-feedback state equals the restatement's residual
        torch.testing.assert_close(grcs[r].state_dict()["memory"]["residuals"]["w"], res[r], rtol=1e-6, atol=1e-9)
        assert grcs[r].stats()["compression_ratio"] > 40


def test_topk_ties_pick_lowest_indices():
    x = torch.ones(1000)
    outs, _ = _run_ranks(1, lambda: (C_.TopKCompressor(0.01), M_.NoneMemory()), [[x]])
    assert outs[0][0].nonzero().flatten().tolist() == list(range(10))


def test_threshold_overflow_stays_in_residual():
    n = 4096
    x = torch.full((n,), 0.5)
    tw = ThreadWorld(1)

    def body(view):
        grc = HostExchange(C_.ThresholdCompressor(0.1), M_.ResidualMemory(), 1, world=view, max_ratio=0.25)
        out = grc.step(x.clone(), "t")
        return out, grc.state_dict()["memory"]["residuals"]["t"]

    out, res = tw.run(body)[0]
    assert int((out != 0).sum()) == n // 4            # the slot holds a quarter of the elements
    torch.testing.assert_close(out + res, x)          # what did not fit is kept for the next step


@pytest.mark.parametrize("world", [1, 3])
def test_qsgd_bound_identity_and_unbiasedness(world):
    n, q = 5000, 64
    grads = _grads(world, n, 2)
    outs, grcs = _run_ranks(world, lambda: (C_.QSGDCompressor(q, 128), M_.ResidualMemory()), grads)
    for s in range(2):
        for r in range(1, world):
            assert torch.equal(outs[r][s], outs[0][s])                   # identical on every rank
    # first step: the decode error of an element is below one level of its bucket (norm / q), summed over ranks
    pad = (-n) % 128
    stacked = torch.nn.functional.pad(torch.stack(grads[0]), (0, pad)).view(world, -1, 128)
    level = (stacked.norm(dim=2) / q).sum(0).repeat_interleave(128)[:n]
    err = (outs[0][0] * world - sum(grads[0])).abs()
    assert bool((err <= level * 1.001 + 1e-9).all()), float((err - level).max())
    # error feedback: after two steps, sent_0 + sent_1 + residual = g_0 + g_1 on every rank; summed over the
    # ranks the left side is W * (out_0 + out_1) + sum of the residuals
    res = sum(g.state_dict()["memory"]["residuals"]["w"] for g in grcs)
    torch.testing.assert_close((outs[0][0] + outs[0][1]) * world + res, sum(grads[0]) + sum(grads[1]),
                               rtol=1e-4, atol=1e-7)
    # unbiased over many draws (different tensor names give different Philox keys)
    x = torch.randn(2048, generator=torch.Generator().manual_seed(7)) * 1e-3
    tw = ThreadWorld(1)

    def body(view):
        grc = HostExchange(C_.QSGDCompressor(q, 128), M_.NoneMemory(), 1, world=view)
        return torch.stack([grc.step(x.clone(), "n%d" % i) for i in range(300)]).mean(0)

    mean = tw.run(body)[0]
    one_level = float(x.view(-1, 128).norm(dim=1).max()) / q
    assert float((mean - x).abs().max()) < 4 * 0.5 * one_level / 300 ** 0.5


def test_qsgd_matches_numpy_philox_restatement():
    from grace_b200.communicator.host import _name_seed
    from grace_b200.utils import philox

    n, q = 1024, 64
    x = torch.randn(n, generator=torch.Generator().manual_seed(3)) * 1e-2
    outs, _ = _run_ranks(1, lambda: (C_.QSGDCompressor(q, 128), M_.NoneMemory()), [[x]], name="layer.weight")
    xb = x.view(-1, 128)
    norms = torch.stack([b.pow(2).sum(dtype=torch.float32).sqrt() for b in xb])   # fp32, as the engine sums
    u = torch.from_numpy(philox.uniform(n, _name_seed(0, "layer.weight" + str(n)), 0, 0)).view(-1, 128)
    lf = (q / norms)[:, None] * xb.abs()
    level = torch.floor(lf) + (u < lf - torch.floor(lf)).float()
    want = (norms / q)[:, None] * level * torch.sign(xb)
    diff = (outs[0][0].view(-1, 128) - want).abs()
    # the engine adds squares one after the other, torch in a tree: a norm may differ in its last bit, which moves
    # a decoded value by an ulp and, once in a while, a rounding decision by one level
    one_level = (norms / q)[:, None].expand_as(diff)
    assert float((diff > 1e-7).float().mean()) < 0.01
    assert bool((diff <= one_level * 1.001).all())


@pytest.mark.parametrize("world", [1, 3, 4])
def test_sign_majority_vote(world):
    n = 3000
    grads = _grads(world, n, 2)
    outs, _ = _run_ranks(world, lambda: (C_.SignSGDCompressor(), M_.NoneMemory()), grads)
    for s in range(2):
        votes = sum(torch.where(grads[s][r] >= 0, 1, -1) for r in range(world))
        want = torch.where(votes >= 0, 1.0, -1.0)     # ties go to +1
        for r in range(world):
            assert torch.equal(outs[r][s], want)


def test_signum_momentum_state():
    n, beta = 2000, 0.9
    grads = _grads(2, n, 3)
    outs, grcs = _run_ranks(2, lambda: (C_.SignumCompressor(beta), M_.NoneMemory()), grads)
    m = [None, None]
    for s in range(3):
        for r in range(2):
            m[r] = grads[s][r].clone() if s == 0 else (1 - beta) * grads[s][r] + beta * m[r]
        votes = sum(torch.where(m[r] >= 0, 1, -1) for r in range(2))
        assert torch.equal(outs[0][s], torch.where(votes >= 0, 1.0, -1.0))
    torch.testing.assert_close(grcs[1].state_dict()["compressor"]["momentums"]["w"], m[1])


def test_efsign_scaled_sum_and_memory():
    n, lr, world = 4000, 0.1, 2
    grads = _grads(world, n, 3)
    outs, grcs = _run_ranks(world, lambda: (C_.EFSignSGDCompressor(lr), M_.EFSignSGDMemory(lr)), grads)
    res = [torch.zeros(n) for _ in range(world)]
    for s in range(3):
        want = torch.zeros(n)
        for r in range(world):
            acc = grads[s][r].clone() if s == 0 else res[r] + lr * grads[s][r]
            dec = acc.abs().mean() * torch.where(acc >= 0, 1.0, -1.0)
            res[r] = acc - dec
            want += dec
        torch.testing.assert_close(outs[0][s], want / lr, rtol=1e-5, atol=1e-8)
        assert torch.equal(outs[0][s], outs[1][s])
    torch.testing.assert_close(grcs[0].state_dict()["memory"]["residuals"]["w"], res[0], rtol=1e-5, atol=1e-8)


def test_dense_mean():
    grads = _grads(4, 777, 2)
    outs, _ = _run_ranks(4, lambda: (C_.NoneCompressor(), M_.NoneMemory()), grads)
    for s in range(2):
        torch.testing.assert_close(outs[2][s], sum(grads[s]) / 4, rtol=1e-6, atol=1e-9)


def test_slot_reuse_with_a_slow_peer():
    """Rank 1 lags behind in every step: rank 0 must wait for its acknowledgement before it overwrites a slot,
    and for its data before it decodes; eight steps use each slot four times."""
    n, world, steps = 2048, 2, 8
    grads = _grads(world, n, steps)

    def hook(rank, s):
        if rank == 1:
            time.sleep(0.03)

    outs, _ = _run_ranks(world, lambda: (C_.NoneCompressor(), M_.NoneMemory()), grads, hook=hook)
    for s in range(steps):
        torch.testing.assert_close(outs[0][s], (grads[s][0] + grads[s][1]) / 2, rtol=1e-6, atol=1e-9)
        assert torch.equal(outs[0][s], outs[1][s])


def test_peer_that_never_publishes_times_out_then_recovery():
    """Rank 1 skips the publish of step 1 (host-side injection).  Rank 0's bounded wait gives up and reports the
    peer; after recover() on both ranks the next exchange is healthy and the error feedback went on untouched."""
    from grace_b200.utils.faults import FaultPlan

    n, world = 4096, 2
    grads = _grads(world, n, 3)
    tw = ThreadWorld(world)

    def body(view):
        grc = HostExchange(C_.TopKCompressor(0.05), M_.ResidualMemory(), world, world=view, timeout_ms=300.0)
        grc._faults = FaultPlan("skip_publish", rank=1, step=1)
        out0 = grc.step(grads[0][view.rank].clone(), "w")
        err = None
        t0 = time.time()
        try:
            grc.step(grads[1][view.rank].clone(), "w")
        except GraceCommError as e:
            err = e
        waited = time.time() - t0
        with pytest.raises(GraceCommError):
            grc.check()                        # the channel stays failed until it is reset
        view.barrier()                         # what agree() does through a store among processes
        grc.recover()
        grc._faults = FaultPlan()
        res_before = grc.state_dict()["memory"]["residuals"]["w"].clone()
        out2 = grc.step(grads[2][view.rank].clone(), "w")
        grc.check()
        return out0, err, waited, res_before, out2

    r0, r1 = tw.run(body)
    assert isinstance(r0[1], GraceCommError) and r0[1].code == 2 and r0[1].detail == 1 and r0[1].seq == 2
    assert 0.25 < r0[2] < 20.0
    # rank 1 saw its own flag missing as well (it reads its own slot through the same flags)
    assert isinstance(r1[1], GraceCommError) and r1[1].code == 2
    assert torch.equal(r0[4], r1[4])           # the exchange after the recovery agrees on both ranks
    k = int(n * 0.05)
    want = sum(_topk_dense(rb + g, k) for rb, g in ((r0[3], grads[2][0]), (r1[3], grads[2][1]))) / 2
    torch.testing.assert_close(r0[4], want, rtol=1e-6, atol=1e-9)


def test_peer_that_never_reads_blocks_slot_reuse():
    """send_step twice is fine (two slots); the third needs the peer's acknowledgement of the first."""
    n, world = 512, 2
    tw = ThreadWorld(world)

    def body(view):
        grc = HostExchange(C_.NoneCompressor(), M_.NoneMemory(), world, world=view, timeout_ms=200.0)
        x = torch.ones(n)
        grc.prepare([("w", x)])                # heaps are created by all ranks together
        err = None
        if view.rank == 0:
            grc.send_step(x, "w")
            grc.send_step(x, "w")
            try:
                grc.send_step(x, "w")
            except GraceCommError as e:
                err = e
        view.barrier()
        return err

    e0, _ = tw.run(body)
    assert isinstance(e0, GraceCommError) and e0.code == 3 and e0.detail == 1


def test_split_phase_equals_step_and_checkpoint_round_trip():
    n = 3000
    grads = _grads(1, n, 4)
    tw = ThreadWorld(1)

    def body(view):
        make = lambda: HostExchange(C_.TopKCompressor(0.02), M_.ResidualMemory(0.9, 1.0), 1, world=view)  # noqa: E731
        a, b = make(), make()
        for s in range(2):
            h, ctx = a.send_step(grads[s][0].clone(), "p")
            out_a = a.receive_step(h, ctx)
            out_b = b.step(grads[s][0].clone(), "p")
            assert torch.equal(out_a, out_b)
        c = make()
        c.load_state_dict(a.state_dict())
        for s in range(2, 4):
            assert torch.equal(a.step(grads[s][0].clone(), "p"), c.step(grads[s][0].clone(), "p"))
        for g in (a, b, c):
            g.close()
        return True

    assert tw.run(body) == [True]


def test_unsupported_pairs_use_the_library_path():
    grc = HostExchange(C_.SketchCompressor(64), M_.NoneMemory(), 1)   # quantile sketches have no host codec
    x = torch.randn(100)
    assert not grc.supported(x)
    assert grc.step(x, "t").shape == x.shape


def _gloo_ranks(rank, world):
    from grace_b200 import grace_from_params

    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.02, "world_size": world, "host_protocol": True, "timeout_ms": 20000})
    lib = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.02, "world_size": world})
    worst = 0.0
    for s in range(3):
        g = torch.randn(5000, generator=torch.Generator().manual_seed(10 * s + rank))
        worst = max(worst, float((grc.step(g.clone(), "w") - lib.step(g.clone(), "w")).abs().max()))
    grc.close()
    return worst


def _gloo_failure(rank, world):
    import torch.distributed as dist

    from grace_b200 import grace_from_params
    from grace_b200.utils.faults import FaultPlan

    store = dist.distributed_c10d._get_default_store()
    grc = grace_from_params({"compressor": "efsignsgd", "memory": "efsignsgd", "communicator": "allgather", "lr": 0.1,
                             "world_size": world, "host_protocol": True, "timeout_ms": 400, "store": store})
    grc._faults = FaultPlan("skip_publish", rank=1, step=1)
    g = [torch.randn(3000, generator=torch.Generator().manual_seed(10 * s + rank)) for s in range(3)]
    grc.step(g[0].clone(), "w")
    failed = None
    try:
        grc.step(g[1].clone(), "w")
    except GraceCommError as e:
        failed = e
    bad = grc.agree(failed)                    # every rank learns who failed, through the store
    if bad:
        grc.recover()
    grc._faults = FaultPlan()
    out = grc.step(g[2].clone(), "w")
    grc.check()
    grc.close()
    return (failed.code if failed else 0, bad, float(out.sum()))


def test_gloo_processes_agree_and_recover():
    from test_dist_cpu import _free_port, _run

    _free_port.port = _free_port()
    res = _run(_gloo_failure, world=2)
    assert res[0][0] == 2 and res[0][1] == [0, 1] and res[1][1] == [0, 1], res
    assert res[0][2] == res[1][2]


def test_gloo_processes_match_library_allgather():
    from test_dist_cpu import _free_port, _run

    _free_port.port = _free_port()
    res = _run(_gloo_ranks, world=2)
    assert max(res.values()) < 1e-6, res


def _train_resnet20(rank, world):
    """The plumbing configuration (ResNet-20, TopK 1 %, residual memory, all-gather, two gloo ranks, 20 steps)
    through the host engine and through the library communicator: the same entries travel and the sums are formed
    in the same order, so the two loss curves coincide."""
    from grace_b200 import grace_from_params
    from grace_b200.models import resnet20

    def run(extra):
        torch.manual_seed(0)
        model = resnet20()
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                                 "compress_ratio": 0.01, "world_size": world, **extra})
        if hasattr(grc, "prepare"):
            grc.prepare(list(model.named_parameters()))
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(20):
            x = torch.randn(32, 3, 32, 32, generator=g)
            y = torch.randint(0, 10, (32,), generator=g)
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            for name, p in model.named_parameters():
                p.grad.copy_(grc.step(p.grad, name))
            opt.step()
            losses.append(loss.item())
        if hasattr(grc, "close"):
            grc.close()
        return losses

    return run({}), run({"host_protocol": True, "timeout_ms": 30000})


def test_resnet20_topk_host_engine_tracks_the_library_path():
    from test_dist_cpu import _free_port, _run

    _free_port.port = _free_port()
    res = _run(_train_resnet20, world=2)
    lib, host = res[0]
    assert all(l == l for l in host)
    assert abs(lib[0] - host[0]) < 1e-5
    # identical selections and summation order: the curves agree until rounding differences get amplified
    assert max(abs(a - b) for a, b in zip(lib[:5], host[:5])) < 1e-3
    assert abs(sum(lib[-5:]) / 5 - sum(host[-5:]) / 5) < 1.0


def _optimizer_ranks(rank, world):
    """Horovod-style wrapper over the host engine: hooks call send_step during backward, step() receives."""
    from grace_b200 import grace_from_params
    from grace_b200.parallel import DistributedOptimizer

    def make_model():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(40, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10))

    params = {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.05,
              "world_size": world, "host_protocol": True, "timeout_ms": 30000}
    g = torch.Generator().manual_seed(7 + rank)
    data = [(torch.randn(16, 40, generator=g), torch.randint(0, 10, (16,), generator=g)) for _ in range(5)]

    model = make_model()
    opt = DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05), grace=grace_from_params(dict(params)),
                               named_parameters=model.named_parameters(), always_hook=True)
    for x, y in data:
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()

    ref = make_model()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
    grc = grace_from_params(dict(params))
    grc.prepare(list(ref.named_parameters()))
    for x, y in data:
        ropt.zero_grad()
        torch.nn.functional.cross_entropy(ref(x), y).backward()
        for name, p in ref.named_parameters():
            p.grad.copy_(grc.step(p.grad, name))
        ropt.step()
    return max(float((a - b).abs().max()) for a, b in zip(model.parameters(), ref.parameters()))


def test_distributed_optimizer_over_the_host_engine():
    from test_dist_cpu import _free_port, _run

    _free_port.port = _free_port()
    res = _run(_optimizer_ranks, world=2)
    assert max(res.values()) < 1e-6, res


# ---- the codecs added after the first set: against the Python compressor classes (library path, one rank) ----
def _lib_and_host(params, n, steps=3, scale=1e-3):
    from grace_b200 import grace_from_params

    grads = [torch.randn(n, generator=torch.Generator().manual_seed(11 * s + 1)) * scale for s in range(steps)]
    lib = grace_from_params(dict(params, world_size=1))
    if params["compressor"] == "dgc":
        lib.compressor.mode = "exact"
    want = [lib.step(g.clone(), "w") for g in grads]

    def body(view):
        host = grace_from_params(dict(params, world_size=1, host_protocol=True, host_world=view))
        assert host.supported(grads[0])
        outs = [host.step(g.clone(), "w") for g in grads]
        return outs, host.state_dict()

    got, state = ThreadWorld(1).run(body)[0]
    return want, got, state, lib


@pytest.mark.parametrize("params", [
    {"compressor": "onebit", "memory": "residual", "communicator": "allgather"},
    {"compressor": "fp16", "memory": "residual", "communicator": "allgather"},
    {"compressor": "u8bit", "memory": "residual", "communicator": "allgather"},
    {"compressor": "natural", "memory": "residual", "communicator": "allgather", "deterministic": True},
    {"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "compress_ratio": 0.01, "momentum": 0.9},
], ids=lambda p: p["compressor"] + "+" + p["memory"])
def test_more_codecs_match_the_python_classes(params):
    want, got, state, lib = _lib_and_host(params, 5000)
    for a, b in zip(want, got):
        torch.testing.assert_close(b, a, rtol=1e-6, atol=1e-10)
    if params["memory"] == "dgc":      # checkpoint names of the reference: residuals = u, gradients = v
        torch.testing.assert_close(state["memory"]["residuals"]["w"], lib.memory.residuals["w"].reshape(-1))
        torch.testing.assert_close(state["memory"]["gradients"]["w"], lib.memory.gradients["w"].reshape(-1))
    else:
        # (1-bit: the means are formed in fp64 here and in fp32 there; the residual is a difference of nearly equal
        # numbers, so the comparison is absolute, at rounding level of the 1e-3 sized inputs)
        torch.testing.assert_close(state["memory"]["residuals"]["w"], lib.memory.residuals["w"].reshape(-1),
                                   rtol=1e-6, atol=2e-9)


def test_fp16_conversion_edge_cases():
    x = torch.tensor([0.0, -0.0, 1.0, -2.5, 65504.0, 65520.0, 1e5, -1e5, 6.0e-8, 3.0e-8, 2.0e-8, 1e-4, 0.1,
                      1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, float("inf"), float("-inf")])
    outs, _ = _run_ranks(1, lambda: (C_.FP16Compressor(), M_.NoneMemory()), [[x]])
    assert torch.equal(outs[0][0], x.half().float())


def test_terngrad_and_natural_draw_the_philox_stream():
    from grace_b200.communicator.host import _name_seed
    from grace_b200.utils import philox

    n = 4096
    x = torch.randn(n, generator=torch.Generator().manual_seed(5)) * 1e-2
    u = torch.from_numpy(philox.uniform(n, _name_seed(0, "w" + str(n)), 0, 0))
    # TernGrad: keep with probability |clamp(x)| / s, s = min(max|x|, 2.5 sigma)
    outs, _ = _run_ranks(1, lambda: (C_.TernGradCompressor(), M_.NoneMemory()), [[x]])
    c = 2.5 * x.double().var(unbiased=False).sqrt().float()
    s0 = torch.minimum(x.abs().max(), c)
    want = torch.where(u * s0 < torch.minimum(x.abs(), c), torch.sign(x) * s0, torch.zeros(n))
    mism = (outs[0][0] != want)
    assert float(mism.float().mean()) < 0.002       # sigma in fp64 here and there, but summed in another order
    assert set(torch.unique(outs[0][0] / s0).round().tolist()) <= {-1.0, 0.0, 1.0}
    # natural compression: exponent + 1 with probability mantissa / 2^23
    outs, _ = _run_ranks(1, lambda: (C_.NaturalCompressor(), M_.NoneMemory()), [[x]])
    bits = x.view(torch.int32)
    mant = (bits & 0x7FFFFF).float() * 2.0 ** -23
    low = torch.sign(x) * torch.exp2(torch.floor(torch.log2(x.abs())))
    want = torch.where(u < mant, 2 * low, low)
    assert torch.equal(outs[0][0], want)


@pytest.mark.parametrize("world", [3])
def test_onebit_and_u8bit_average_over_ranks(world):
    n = 3001
    grads = _grads(world, n, 1)
    outs, _ = _run_ranks(world, lambda: (C_.OneBitCompressor(), M_.NoneMemory()), grads)
    want = torch.zeros(n)
    for g in grads[0]:
        neg = g < 0
        want += torch.where(neg, g[neg].mean(), g[~neg].mean())
    torch.testing.assert_close(outs[0][0], want / world, rtol=1e-5, atol=1e-9)
    outs, _ = _run_ranks(world, lambda: (C_.U8bitCompressor(), M_.NoneMemory()), grads)
    comp = C_.U8bitCompressor()
    want = sum(comp.decompress(*comp.compress(g, "w")) for g in grads[0]) / world
    torch.testing.assert_close(outs[1][0], want, rtol=1e-6, atol=1e-10)


def test_step_flat_equals_tensor_by_tensor():
    from grace_b200.ops.exchange import FlatLayout

    world = 2
    layout = FlatLayout.from_named([("a", 700), ("b", 64), ("c", 5001)])
    tw = ThreadWorld(world)

    def body(view):
        make = lambda: HostExchange(C_.TopKCompressor(0.05), M_.ResidualMemory(), world, world=view)  # noqa: E731
        flat_grc, single = make(), make()
        flat_grc.prepare_layouts([layout])
        single.prepare([(n, torch.empty(c)) for n, c in zip(layout.names, layout.numels)])
        worst = 0.0
        for step in range(3):
            flat = torch.zeros(layout.total)
            for i, (o, c) in enumerate(zip(layout.offsets, layout.numels)):
                flat[o:o + c] = torch.randn(c, generator=torch.Generator().manual_seed(100 * step + 10 * view.rank + i))
            want = flat.clone()
            for n, o, c in zip(layout.names, layout.offsets, layout.numels):
                want[o:o + c] = single.step(flat[o:o + c].clone(), n)
            got = flat_grc.step_flat(flat.clone(), layout)
            worst = max(worst, float((got - want).abs().max()))
        return worst

    assert max(tw.run(body)) == 0.0


def test_randomk_positions_from_philox_and_values_only():
    from grace_b200.communicator.host import _name_seed
    from grace_b200.utils import philox

    n, ratio, world = 5000, 0.05, 2
    k = int(n * ratio)
    grads = _grads(world, n, 2)
    outs, grcs = _run_ranks(world, lambda: (C_.RandomKCompressor(ratio), M_.ResidualMemory()), grads, name="fc.weight")
    res = [torch.zeros(n) for _ in range(world)]
    for s in range(2):
        # stream 7 of the tensor's key, entry e uses word e: the same positions on every rank, with replacement
        words = philox.random_words(k, _name_seed(0, "fc.weight"), s, 7)
        pos = torch.from_numpy((words % np.uint32(n)).astype(np.int64))
        want = torch.zeros(n)
        total = torch.zeros(k)
        for r in range(world):
            acc = res[r] + grads[s][r]
            total += acc[pos]
            res[r] = acc.clone()
            res[r][pos] = 0
        want[pos] = total / world                 # a store: a position drawn twice is not counted twice
        for r in range(world):
            torch.testing.assert_close(outs[r][s], want, rtol=1e-6, atol=1e-10)
    assert len(set(pos.tolist())) < k             # the case has repeated positions
    torch.testing.assert_close(grcs[0].state_dict()["memory"]["residuals"]["fc.weight"], res[0], rtol=1e-6, atol=1e-10)
    assert grcs[0].stats()["compression_ratio"] == pytest.approx(1 / ratio, rel=0.01)


def test_general_qsgd_buckets_and_levels():
    """Bucket sizes other than 128 and 128 levels or more (int16 codes): bound, identity and the Philox stream."""
    from grace_b200.communicator.host import _name_seed
    from grace_b200.utils import philox

    n, q, bucket = 1000, 512, 100
    x = torch.randn(n, generator=torch.Generator().manual_seed(9)) * 1e-2
    outs, grcs = _run_ranks(1, lambda: (C_.QSGDCompressor(q, bucket), M_.ResidualMemory()), [[x]])
    xb = x.view(-1, bucket)
    norms = torch.stack([b.pow(2).sum(dtype=torch.float32).sqrt() for b in xb])
    u = torch.from_numpy(philox.uniform(n, _name_seed(0, "w" + str((n + 127) // 128 * 128)), 0, 0)).view(-1, bucket)
    lf = (q / norms)[:, None] * xb.abs()
    want = (norms / q)[:, None] * (torch.floor(lf) + (u < lf - torch.floor(lf)).float()) * torch.sign(xb)
    diff = (outs[0][0].view(-1, bucket) - want).abs()
    assert float((diff > 1e-7).float().mean()) < 0.01
    assert bool((diff <= (norms / q)[:, None] * 1.001).all())
    torch.testing.assert_close(outs[0][0] + grcs[0].state_dict()["memory"]["residuals"]["w"], x, rtol=1e-5, atol=1e-9)


# ---- PowerSGD on the host engine ----
def test_powersgd_matches_the_python_classes_from_the_same_start():
    from grace_b200 import grace_from_params

    shape, name, rank = (48, 5, 8), "conv.weight", 4
    grads = [torch.randn(shape, generator=torch.Generator().manual_seed(3 * s + 1)) for s in range(3)]
    params = {"compressor": "powersgd", "memory": "powersgd", "communicator": "allreduce", "compress_rank": rank,
              "use_memory": True, "world_size": 1}

    def body(view):
        host = grace_from_params(dict(params, host_protocol=True, host_world=view))
        host.prepare([(name, grads[0])])
        q0 = next(iter(host._plans.values())).q.clone()
        outs = [host.step(g.clone(), name) for g in grads]
        bias = host.step(torch.arange(7.0), "conv.bias")          # 1-D tensors travel uncompressed
        return q0, outs, bias, host.state_dict()

    q0, got, bias, state = ThreadWorld(1).run(body)[0]
    lib = grace_from_params(dict(params))
    lib.compressor.q_memory[name] = q0.clone()                     # the same start as the host plan
    for g, out in zip(grads, got):
        want = lib.step(g.clone(), name)
        torch.testing.assert_close(out, want, rtol=2e-4, atol=2e-5)   # Cholesky in fp64 here, Gram-Schmidt in fp32 there
    assert torch.equal(bias, torch.arange(7.0))
    torch.testing.assert_close(state["compressor"]["q_memory"][name], lib.compressor.q_memory[name], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(state["memory"]["residuals"][name].view(shape), lib.memory.residuals[name].view(shape),
                               rtol=2e-3, atol=2e-4)


def test_powersgd_recovers_a_shared_low_rank_mean_over_ranks():
    """Every rank's gradient is A_r B^T with the same B (rank 2 < 4): the mean is in the span PowerSGD can
    represent, so the exchange returns it exactly; the orthogonalisation meets two dependent directions."""
    world, n, m = 3, 40, 64
    B = torch.randn(m, 2, generator=torch.Generator().manual_seed(1))
    A = [torch.randn(n, 2, generator=torch.Generator().manual_seed(10 + r)) for r in range(world)]
    grads = [[A[r] @ B.t() for r in range(world)]]

    def make():
        comp = C_.PowerSGDCompressor(rank=4, use_memory=True, world_size=world)
        return comp, M_.PowerSGDMemory(comp.q_memory, 4)

    outs, grcs = _run_ranks(world, make, grads, name="fc.weight")
    mean = sum(grads[0]) / world
    for r in range(world):
        torch.testing.assert_close(outs[r][0], mean, rtol=1e-3, atol=1e-4)
        assert torch.equal(outs[r][0], outs[0][0])                 # replicas agree bit for bit
    # what a rank could not send stays in its residual: g_r - mean here
    torch.testing.assert_close(grcs[1].state_dict()["memory"]["residuals"]["fc.weight"].view(n, m),
                               grads[0][1] - outs[1][0], rtol=1e-4, atol=1e-5)


def test_powersgd_checkpoint_continues_identically():
    shape = (32, 24)
    grads = [torch.randn(shape, generator=torch.Generator().manual_seed(s)) for s in range(4)]

    def body(view):
        def make():
            comp = C_.PowerSGDCompressor(rank=2, use_memory=True, world_size=1)
            return HostExchange(comp, M_.PowerSGDMemory(comp.q_memory, 2), 1, world=view)

        a = make()
        for g in grads[:2]:
            a.step(g.clone(), "w")
        b = make()
        b.load_state_dict(a.state_dict())
        return all(torch.equal(a.step(g.clone(), "w"), b.step(g.clone(), "w")) for g in grads[2:])

    assert ThreadWorld(1).run(body) == [True]


def test_fused_communicator_with_attached_host_engine_serves_cpu_tensors():
    """``fused`` and ``host_protocol`` together: kernels for CUDA tensors, the host engine for CPU tensors."""
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import FusedExchange

    params = {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.05,
              "world_size": 1}
    grads = [torch.randn(2000, generator=torch.Generator().manual_seed(s)) for s in range(3)]

    def body(view):
        both = grace_from_params(dict(params, fused=True, host_protocol=True, host_world=view))
        alone = grace_from_params(dict(params, host_protocol=True, host_world=view))
        assert isinstance(both, FusedExchange) and isinstance(both._fallback, HostExchange)
        same = all(torch.equal(both.step(g.clone(), "w"), alone.step(g.clone(), "w")) for g in grads)
        both.check()
        state = both.state_dict()
        both.close()
        return same, sorted(state["memory"]["residuals"])

    assert ThreadWorld(1).run(body) == [(True, ["w"])]


# ---- two-phase ("alltoall") mode: compressed reduce-scatter, re-encode, compressed all-gather ----
def _two_phase(world, comp_factory, grads, **kw):
    tw = ThreadWorld(world)

    def body(view):
        grc = HostExchange(comp_factory(), M_.NoneMemory(), world, world=view, mode="alltoall", **kw)
        outs = [grc.step(per_rank[view.rank].clone(), "w") for per_rank in grads]
        assert all(p.two_phase for p in grc._plans.values())
        return outs

    return tw.run(body)


@pytest.mark.parametrize("world", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [1, 127, 129, 1000, 5000])
def test_two_phase_dense_is_the_mean_and_fp16_rounds_twice(world, n):
    grads = _grads(world, n, 3, scale=1.0)
    outs = _two_phase(world, C_.NoneCompressor, grads)
    for s in range(3):
        want = sum(grads[s])                          # ranks are added in order 0..W-1, then scaled
        for r in range(world):
            assert torch.equal(outs[r][s], want * (1.0 / world))
    outs = _two_phase(world, C_.FP16Compressor, grads)
    want = sum(g.half().float() for g in grads[0]).half().float() * (1.0 / world)
    for r in range(world):
        assert torch.equal(outs[r][0], want)


def test_two_phase_natural_deterministic_matches_the_restatement():
    from grace_b200.compressor.natural import natural_decode, natural_encode

    world, n = 3, 4000
    grads = _grads(world, n, 2)

    def det(x):   # deterministic natural compression: the larger power of two when the mantissa is above 1/2
        prob = (x.contiguous().view(torch.int32) & 0x7FFFFF).float() * 2.0 ** -23
        u = torch.where(prob > 0.5, torch.zeros_like(x), torch.ones_like(x))
        return natural_decode(natural_encode(x, u)).view(-1)

    outs = _two_phase(world, lambda: C_.NaturalCompressor(deterministic=True), grads)
    for s in range(2):
        want = det(sum(det(g) for g in grads[s])) / world
        for r in range(world):
            torch.testing.assert_close(outs[r][s], want, rtol=0, atol=0)


def test_two_phase_qsgd_close_to_the_mean_and_identical_on_all_ranks():
    world, n, q = 4, 128 * 40 + 17, 127
    grads = _grads(world, n, 2)
    outs = _two_phase(world, lambda: C_.QSGDCompressor(q, 128), grads)
    for s in range(2):
        mean = sum(grads[s]) / world
        for r in range(1, world):
            assert torch.equal(outs[r][s], outs[0][s])
        err = (outs[0][s] - mean).norm() / mean.norm()
        assert float(err) < 0.25, float(err)          # two lossy steps of 127 levels per 128-element bucket


def test_alltoall_communicator_name_selects_the_two_phase_mode():
    from grace_b200 import grace_from_params

    def body(view):
        grc = grace_from_params({"compressor": "qsgd", "memory": "none", "communicator": "alltoall", "quantum_num": 64,
                                 "world_size": 1, "host_protocol": True, "host_world": view})
        out = grc.step(torch.randn(1000), "w")
        return grc.mode, bool(torch.isfinite(out).all())

    assert ThreadWorld(1).run(body) == [("alltoall", True)]


def test_dgc_gradient_clipping_bound_from_all_ranks():
    """DgcMemory(gradient_clipping=True): clamp to +-sqrt(mean over ranks of sum g^2) before the momentum correction."""
    world, n, ratio, m = 3, 3000, 0.02, 0.9
    k = int(n * ratio)
    grads = _grads(world, n, 3, scale=1.0)
    for s in range(3):                                  # one rank has an outlier above the RMS of the ranks' norms
        grads[s][0][7 + s] = 1000.0
    outs, grcs = _run_ranks(world, lambda: (C_.DgcCompressor(ratio), M_.DgcMemory(m, True, world)), grads)
    u = [torch.zeros(n) for _ in range(world)]
    v = [torch.zeros(n) for _ in range(world)]
    for s in range(3):
        bound = torch.sqrt(sum(g.double().pow(2).sum() for g in grads[s]) / world).float()
        assert any(bool((g.abs() > bound).any()) for g in grads[s])
        want = torch.zeros(n)
        for r in range(world):
            g = torch.maximum(torch.minimum(grads[s][r], bound), -bound)
            u[r] = m * u[r] + g
            v[r] = v[r] + u[r]
            sel = _topk_dense(v[r], k)
            keep = sel == 0
            want += sel
            u[r] = u[r] * keep
            v[r] = v[r] * keep
        for r in range(world):
            torch.testing.assert_close(outs[r][s], want / world, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(grcs[2].state_dict()["memory"]["gradients"]["w"], v[2], rtol=1e-5, atol=1e-7)
