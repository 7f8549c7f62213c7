"""GPU tests of the fused sparse exchange (TopK / DGC / Threshold) against plain
PyTorch fp32 restatements of the same operations."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 31, 32, 33, 127, 128, 129, 2047, 2048, 2049, 6143, 6144, 6145, 100_003, (1 << 20) + 1]


def _dev():
    return torch.device("cuda")


def _rand(n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, generator=g) * 1e-3).to(_dev())


def _dense_topk(x, k):
    _, idx = torch.topk(x.abs(), k, sorted=False)
    out = torch.zeros_like(x)
    out[idx] = x[idx]
    return out


@pytest.mark.parametrize("n", SIZES)
def test_topk_select_matches_torch(n):
    from grace_b200.ops.sparse import topk_select

    x = _rand(n, seed=n)
    for ratio in (0.001, 0.01, 0.3, 1.0):
        k = max(1, int(n * ratio))
        vals, idx = topk_select(x, k)
        assert vals.numel() == k and idx.numel() == k
        idx = idx.long()
        assert idx.unique().numel() == k, "indices must be distinct"
        assert torch.equal(vals, x[idx])
        ref_vals, _ = torch.topk(x.abs(), k)
        got = vals.abs().sort(descending=True).values
        assert torch.equal(got, ref_vals), "selected magnitudes must be exactly the k largest"


def test_topk_select_ties_and_zeros():
    from grace_b200.ops.sparse import topk_select

    x = torch.zeros(5000, device=_dev())
    vals, idx = topk_select(x, 50)
    assert idx.long().unique().numel() == 50 and torch.all(vals == 0)
    x = torch.full((5000,), 0.25, device=_dev())
    x[::7] = -0.25
    vals, idx = topk_select(x, 123)
    assert idx.long().unique().numel() == 123 and torch.all(vals.abs() == 0.25)
    x = torch.zeros(4096, device=_dev())
    x[[5, 77, 4095]] = torch.tensor([3.0, -4.0, 1.0], device=_dev())
    vals, idx = topk_select(x, 2)
    assert sorted(idx.tolist()) == [5, 77]


def test_topk_select_approximate_mode():
    from grace_b200.ops.sparse import topk_select

    x = _rand(300_000, 5)
    k = 3000
    vals, idx = topk_select(x, k, exact=False)
    assert idx.long().unique().numel() == k
    kth = torch.topk(x.abs(), k).values[-1]
    assert vals.abs().min() >= kth * (1 - 2.0 ** -14)


def _world(W, params):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        p = dict(params)
        p.update(world_size=W, fused=True)
        return grace_from_params(p)

    return VirtualWorld(W, make, _dev())


@pytest.mark.parametrize("W", [1, 2, 4])
@pytest.mark.parametrize("n", [1000, 70_001])
def test_topk_residual_exchange_matches_reference_semantics(W, n):
    ratio = 0.01
    k = max(1, int(n * ratio))
    vw = _world(W, {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": ratio})
    residual = [torch.zeros(n, device=_dev()) for _ in range(W)]
    for step in range(3):
        grads = [_rand(n, seed=100 * step + r) for r in range(W)]
        outs = vw.step(grads, "w")
        vw.check()
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            acc = residual[r] + grads[r]
            sel = _dense_topk(acc, k)
            residual[r] = acc - sel
            expect += sel
        expect /= W
        for r in range(W):
            torch.testing.assert_close(outs[r], expect, rtol=1e-6, atol=1e-9)
            plan = next(iter(vw.comms[r]._plans.values()))
            torch.testing.assert_close(plan.acc[:n], residual[r], rtol=0, atol=0)
    # every rank produced bit-identical output
    for r in range(1, W):
        assert torch.equal(outs[0], outs[r])


def test_dgc_momentum_correction_exchange():
    W, n, ratio, m = 2, 50_000, 0.01, 0.9
    k = max(1, int(n * ratio))
    vw = _world(W, {"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "compress_ratio": ratio,
                    "momentum": m})
    u = [torch.zeros(n, device=_dev()) for _ in range(W)]
    v = [torch.zeros(n, device=_dev()) for _ in range(W)]
    for step in range(3):
        grads = [_rand(n, seed=7 * step + r) for r in range(W)]
        outs = vw.step(grads, "w")
        vw.check()
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            u[r] = m * u[r] + grads[r]
            v[r] = v[r] + u[r]
            sel = _dense_topk(v[r], k)
            keep = sel == 0
            expect += sel
            u[r] = u[r] * keep
            v[r] = v[r] * keep
        expect /= W
        torch.testing.assert_close(outs[0], expect, rtol=1e-6, atol=1e-9)
        plan = next(iter(vw.comms[0]._plans.values()))
        torch.testing.assert_close(plan.acc[:n], v[0], rtol=1e-6, atol=1e-9)
        torch.testing.assert_close(plan.u[:n], u[0], rtol=1e-6, atol=1e-9)


def test_threshold_exchange():
    W, n, thr = 2, 40_000, 2e-3
    vw = _world(W, {"compressor": "threshold", "memory": "residual", "communicator": "allgather", "threshold": thr})
    grads = [_rand(n, seed=r + 1) for r in range(W)]
    outs = vw.step(grads, "w")
    vw.check()
    expect = torch.zeros(n, device=_dev())
    for r in range(W):
        t = min(thr, grads[r].max().item())
        expect += torch.where(grads[r].abs() >= t, grads[r], torch.zeros_like(grads[r]))
    torch.testing.assert_close(outs[0], expect / W, rtol=1e-6, atol=1e-9)


def test_flat_multi_segment_topk():
    from grace_b200.ops.exchange import FlatLayout

    W, ratio = 2, 0.05
    numels = [64, 300, 5000, 1, 128, 77_777]
    layout = FlatLayout.from_named([("p%d" % i, n) for i, n in enumerate(numels)])
    vw = _world(W, {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": ratio})
    flats = []
    for r in range(W):
        f = torch.zeros(layout.total, device=_dev())
        for i, (o, n) in enumerate(zip(layout.offsets, layout.numels)):
            f[o:o + n] = _rand(n, seed=10 * r + i)
        flats.append(f)
    ref_in = [f.clone() for f in flats]
    outs = vw.step_flat(flats, layout)
    vw.check()
    expect = torch.zeros(layout.total, device=_dev())
    for r in range(W):
        for o, n in zip(layout.offsets, layout.numels):
            k = max(1, int(n * ratio))
            expect[o:o + n] += _dense_topk(ref_in[r][o:o + n], k)
    torch.testing.assert_close(outs[0], expect / W, rtol=1e-6, atol=1e-9)
    assert torch.equal(outs[0], outs[1])


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A peer that never publishes: the exchange phase must give up after the
    configured limit, leave an error status and keep the context usable."""
    from grace_b200.ops.exchange import GraceCommError, PHASE_COMPRESS, PHASE_EXCHANGE, PHASE_PUBLISH

    W, n = 2, 4096
    vw = _world(W, {"compressor": "topk", "memory": "none", "communicator": "allgather", "compress_ratio": 0.01,
                    "timeout_ms": 50})
    from grace_b200.ops.exchange import FlatLayout

    layout = FlatLayout.single("w", n)
    g = [_rand(n, r) for r in range(W)]
    c0 = vw.comms[0]
    plan0 = c0._plan(layout)
    vw.comms[1]._plan(layout)
    # rank 0 compresses and publishes, rank 1 never does; rank 0 then waits for rank 1
    seq = c0._launch(plan0, g[0], g[0].clone(), PHASE_COMPRESS | PHASE_PUBLISH)
    c0._launch(plan0, g[0], g[0].clone(), PHASE_EXCHANGE, seq=seq)
    with pytest.raises(GraceCommError) as err:
        c0.check()
    assert err.value.code == 2 and err.value.detail == 1
    # the context is still alive
    assert torch.ones(4, device=_dev()).sum().item() == 4


def test_dense_overlap_is_bit_identical_across_ranks():
    """Many indices chosen by three or more ranks: the aggregate must still be
    bit-identical on every rank (lists are applied in rank order)."""
    W, n = 4, 200_000
    vw = _world(W, {"compressor": "topk", "memory": "none", "communicator": "allgather", "compress_ratio": 0.4})
    grads = [_rand(n, seed=900 + r) for r in range(W)]
    outs = vw.step(grads, "w")
    vw.check()
    expect = torch.zeros(n, device=_dev())
    k = int(n * 0.4)
    for r in range(W):  # same order as the kernel: rank 0 first
        expect += _dense_topk(grads[r], k) * (1.0 / W)
    for r in range(W):
        assert torch.equal(outs[r], expect)


@pytest.mark.parametrize("n,ratio", [(3_000_000, 0.001), (500_000, 0.5), (8192, 0.01)])
def test_fast_select_path_large_and_small(n, ratio):
    """Sizes / ratios on both sides of the candidate-list capacity."""
    from grace_b200.ops.sparse import topk_select

    x = _rand(n, seed=n)
    k = max(1, int(n * ratio))
    vals, idx = topk_select(x, k)
    assert idx.long().unique().numel() == k
    assert torch.equal(vals, x[idx.long()])
    assert torch.equal(vals.abs().sort(descending=True).values, torch.topk(x.abs(), k).values)
    heavy = torch.full((300_000,), 0.5, device=_dev())   # every key in one bin: falls back to the full passes
    heavy[:1000] = 2.0
    vals, idx = topk_select(heavy, 5000)
    assert idx.long().unique().numel() == 5000 and (vals == 2.0).sum() == 1000


def test_randomk_same_positions_on_all_ranks_and_mean_of_values():
    W, n, ratio = 3, 50_000, 0.02
    k = int(n * ratio)
    vw = _world(W, {"compressor": "randomk", "memory": "residual", "communicator": "allreduce", "compress_ratio": ratio})
    assert vw.comms[0]._kind == "sparse"
    residual = [torch.zeros(n, device=_dev()) for _ in range(W)]
    prev_idx = None
    for step in range(2):
        grads = [_rand(n, seed=40 * step + r) for r in range(W)]
        outs = vw.step(grads, "w")
        vw.check()
        plans = [next(iter(c._plans.values())) for c in vw.comms]
        seq = plans[0].channel.seq
        idx = [p.channel.slot_view(seq, k, torch.int32, 128 + p.cap * 4).long() for p in plans]
        for r in range(1, W):
            assert torch.equal(idx[0], idx[r]), "every rank must draw the same positions"
        assert idx[0].min() >= 0 and idx[0].max() < n
        if prev_idx is not None:
            assert not torch.equal(prev_idx, idx[0])  # the step is part of the counter
        prev_idx = idx[0].clone()
        expect = torch.zeros(n, device=_dev())
        acc = [residual[r] + grads[r] for r in range(W)]
        expect[idx[0]] = sum(a[idx[0]] for a in acc) / W
        for r in range(W):
            torch.testing.assert_close(outs[r], expect, rtol=1e-6, atol=1e-9)
            res = acc[r].clone()
            res[idx[0]] = 0
            residual[r] = res
            torch.testing.assert_close(plans[r].acc[:n], res, rtol=0, atol=0)


def test_in_place_exchange_without_memory():
    """out aliases the gradient and there is no error-feedback memory."""
    from grace_b200 import grace_from_params

    n, ratio = 30_000, 0.01
    grc = grace_from_params({"compressor": "topk", "memory": "none", "communicator": "allgather", "world_size": 1,
                             "compress_ratio": ratio, "fused": True})
    x = _rand(n, 3)
    expect = _dense_topk(x, int(n * ratio))
    out = grc.step(x, "w")
    grc.check()
    assert out.data_ptr() == x.data_ptr()
    torch.testing.assert_close(out, expect, rtol=0, atol=0)


def test_injected_skip_publish_surfaces_as_timeout_on_the_peer(monkeypatch):
    """GRACE_FAULT makes rank 1 skip its publication at step 1: rank 0 must report a
    bounded-wait timeout for peer 1 (host-side injection, nothing faults on the GPU)."""
    from grace_b200.ops.exchange import GraceCommError

    monkeypatch.setenv("GRACE_FAULT", "skip_publish:rank1:step1")
    W, n = 2, 8192
    vw = _world(W, {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.01,
                    "timeout_ms": 50})
    vw.step([_rand(n, r) for r in range(W)], "w")     # step 0: healthy
    vw.check()
    vw.step([_rand(n, 10 + r) for r in range(W)], "w")  # step 1: rank 1 does not publish
    with pytest.raises(GraceCommError) as err:
        vw.comms[0].check()
    assert err.value.code == 2 and err.value.detail == 1
    for c in vw.comms:  # recovery: clear flags and sequence numbers, then carry on
        try:
            c.check()
        except GraceCommError:
            pass
        c.reset()
    monkeypatch.delenv("GRACE_FAULT")
    for c in vw.comms:
        c._faults.action = ""
    outs = vw.step([_rand(n, 20 + r) for r in range(W)], "w")
    vw.check()
    assert torch.isfinite(outs[0]).all() and torch.equal(outs[0], outs[1])


def test_dgc_with_gradient_clipping_runs_fused():
    from grace_b200 import grace_from_params

    n, ratio = 20_000, 0.01
    grc = grace_from_params({"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "world_size": 1,
                             "compress_ratio": ratio, "momentum": 0.9, "gradient_clipping": True, "fused": True})
    assert grc._kind == "sparse"
    x = _rand(n, 8)
    x[:5] = 1.0          # (with one rank the bound is the tensor's own L2 norm, which no element exceeds)
    bound = x.pow(2).sum().sqrt()
    out = grc.step(x.clone(), "w")
    grc.check()
    clipped = x.clamp(-bound, bound)
    expect = _dense_topk(clipped, int(n * ratio))
    torch.testing.assert_close(out, expect, rtol=1e-6, atol=1e-9)
    assert out.abs().max() <= bound + 1e-6


@pytest.mark.parametrize("W", [1, 2, 4])
@pytest.mark.parametrize("n,ratio", [(200_000, 0.4), (70_001, 0.01), (5000, 0.05)])
def test_tile_bucketed_decode_matches_scatter_decode(monkeypatch, W, n, ratio):
    """The tile-ordered exchange (sender orders its list by 8192-element output tile and publishes a directory;
    receivers build dense tiles in shared memory) must give the bits of the rank-ordered scatter-add, on
    consecutive exchanges of one channel."""
    import grace_b200.ops.exchange as X

    monkeypatch.setattr(X, "TILE_DECODE_DEFAULT", True)
    monkeypatch.setattr(X, "TILE_DECODE_MIN_ELEMS", 0)
    monkeypatch.setattr(X, "TILE_DECODE_MIN_DENSITY", 0.0)
    vw = _world(W, {"compressor": "topk", "memory": "none", "communicator": "allgather", "compress_ratio": ratio})
    k = max(1, int(n * ratio))
    for step in range(3):
        grads = [_rand(n, seed=40 * step + r) for r in range(W)]
        outs = vw.step(grads, "w")
        vw.check()
        plan = next(iter(vw.comms[0]._plans.values()))
        assert plan.tile and plan.channel._tile is not None   # the tile-ordered path really ran
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            expect += _dense_topk(grads[r], k) * (1.0 / W)
        for r in range(W):
            assert torch.equal(outs[r], expect)


def test_tile_bucketed_decode_threshold_and_segments(monkeypatch):
    import grace_b200.ops.exchange as X
    from grace_b200.ops.exchange import FlatLayout

    monkeypatch.setattr(X, "_TILE_ENV", "force")        # threshold exchanges use the tile-ordered path only when forced
    monkeypatch.setattr(X, "TILE_DECODE_DEFAULT", True)
    monkeypatch.setattr(X, "TILE_DECODE_MIN_ELEMS", 0)
    monkeypatch.setattr(X, "TILE_DECODE_MIN_DENSITY", 0.0)
    W = 2
    vw = _world(W, {"compressor": "threshold", "memory": "none", "communicator": "allgather", "threshold": 2e-3})
    names, numels = ["a", "b", "c"], [9000, 130, 20_000]
    lay = FlatLayout(names, numels)
    flats = []
    for r in range(W):
        f = torch.zeros(lay.total, device=_dev())
        for i, (o, m) in enumerate(zip(lay.offsets, numels)):
            f[o : o + m] = _rand(m, seed=7 * r + i)
        flats.append(f)
    outs = vw.step_flat([f.clone() for f in flats], lay)
    vw.check()
    expect = torch.zeros(lay.total, device=_dev())
    for r in range(W):
        expect += torch.where(flats[r].abs() >= 2e-3, flats[r], torch.zeros_like(flats[r])) * (1.0 / W)
    for r in range(W):
        assert torch.equal(outs[r], expect)


@pytest.mark.parametrize("W", [1, 2])
@pytest.mark.parametrize("memory", ["none", "residual"])
def test_topk_over_many_steps_hint_hits_and_misses(W, memory):
    """From its second launch on the kernel counts the previous launch's pivot bin by 24 key bits in its first pass
    (a speed hint for the steady state under error feedback).  Without memory the same gradients are sent three
    times (the hint must hit), then scaled by 64 (it must miss), then sent again; with residual memory sixteen steps
    of similar gradients let the threshold settle.  Every step must select exactly what a dense top-k of the
    accumulator selects, whichever path ran."""
    from grace_b200.ops.exchange import FlatLayout

    ratio = 0.25 if memory == "residual" else 0.01
    numels = [200_000, 4096, 300_003, 130]
    nseg = len(numels)
    layout = FlatLayout.from_named([("p%d" % i, n) for i, n in enumerate(numels)])
    vw = _world(W, {"compressor": "topk", "memory": memory, "communicator": "allgather", "compress_ratio": ratio})
    residual = [torch.zeros(layout.total, device=_dev()) for _ in range(W)]
    steps = 16 if memory == "residual" else 6
    hits = []
    for step in range(steps):
        scale = 64.0 if step == 3 else 1.0
        noise = 0.05 if memory == "residual" else 0.0
        flats = []
        for r in range(W):
            f = torch.zeros(layout.total, device=_dev())
            for i, (o, n) in enumerate(zip(layout.offsets, layout.numels)):
                f[o:o + n] = (_rand(n, seed=10 * r + i) + noise * _rand(n, seed=1000 + 100 * step + 10 * r + i)) * scale
            flats.append(f)
        grads = [f.clone() for f in flats]
        outs = vw.step_flat(flats, layout)
        vw.check()
        expect = torch.zeros(layout.total, device=_dev())
        step_hits = 0
        for r in range(W):
            acc = grads[r] + (residual[r] if memory == "residual" else 0)
            sel = torch.zeros_like(acc)
            for o, n in zip(layout.offsets, layout.numels):
                sel[o:o + n] = _dense_topk(acc[o:o + n], max(1, int(n * ratio)))
            residual[r] = acc - sel
            expect += sel
            plan = next(iter(vw.comms[r]._plans.values()))
            if memory == "residual":
                torch.testing.assert_close(plan.acc[:layout.total], residual[r], rtol=0, atol=0)
            state = plan.channel.sparse_state.view(nseg + 1, -1)
            step_hits += int(state[:nseg, 5].sum())          # SparseState.fine of the launch that just ran
        hits.append(step_hits)
        torch.testing.assert_close(outs[0], expect / W, rtol=1e-6, atol=1e-9)
        for r in range(1, W):
            assert torch.equal(outs[0], outs[r])
    if memory == "none":
        # launch 0 has no hint; 1 and 2 repeat launch 0; 3 is scaled (64 = 6 octaves: another bin); 4 returns (miss), 5 hits
        assert hits == [0, nseg * W, nseg * W, 0, 0, nseg * W], hits
    else:
        assert hits[0] == 0 and sum(hits) > 0, hits
