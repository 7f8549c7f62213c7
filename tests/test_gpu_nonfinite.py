"""Non-finite gradients (NaN, +-Inf) must not derail a fused exchange: the kernels run to their end, report no
error, and what a bad value can spoil is bounded (the element itself for the sparse and sign codecs, its bucket
of 128 for QSGD).  The reference's CUDA quantiser marks such values with a sentinel
(grace_dl/dist/compressor/qsgd_cuda/qsgd_cuda.cu:381-384); its torch compressors propagate them."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _rand(n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, generator=g) * 1e-3).to(_dev())


def _grc(params):
    from grace_b200 import grace_from_params

    p = dict(params)
    p.update(world_size=1, fused=True)
    return grace_from_params(p)


def test_topk_select_puts_nonfinite_values_first():
    from grace_b200.ops.sparse import topk_select

    n, k = 50_000, 10
    x = _rand(n, 1)
    bad = [17, 4096, 49_999]
    x[bad[0]] = float("nan")
    x[bad[1]] = float("inf")
    x[bad[2]] = float("-inf")
    vals, idx = topk_select(x, k)
    torch.cuda.synchronize()
    got = set(idx.tolist())
    assert len(got) == k and set(bad) <= got            # magnitude keys: NaN > Inf > every finite value
    finite = torch.tensor(sorted(got - set(bad)), device=_dev())
    clean = x.clone()
    clean[bad] = 0
    want = torch.topk(clean.abs(), k - 3).values
    assert torch.equal(clean[finite].abs().sort(descending=True).values, want)


def test_sparse_exchange_with_nonfinite_gradient_completes():
    n = 200_000
    x = _rand(n, 2)
    x[123] = float("inf")
    x[77_777] = float("nan")
    grc = _grc({"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.01})
    out = grc.step(x.clone(), "w")
    grc.check()                                          # no time-out, no failed check
    assert out[123] == float("inf") and torch.isnan(out[77_777])
    mask = torch.ones(n, dtype=torch.bool, device=_dev())
    mask[[123, 77_777]] = False
    assert bool(torch.isfinite(out[mask]).all())
    assert int((out[mask] != 0).sum()) == int(n * 0.01) - 2
    out2 = grc.step(_rand(n, 3), "w")                    # the two bad values were sent, not kept: the residual is clean
    grc.check()
    assert bool(torch.isfinite(out2).all())


def test_qsgd_nonfinite_value_spoils_only_its_bucket():
    n = 128 * 100
    x = _rand(n, 4)
    params = {"compressor": "qsgd", "memory": "none", "communicator": "allgather", "quantum_num": 64, "seed": 5}
    clean = _grc(params).step(x.clone(), "w")
    y = x.clone()
    y[128 * 7 + 5] = float("inf")
    grc = _grc(params)
    out = grc.step(y, "w")
    grc.check()
    keep = torch.ones(n, dtype=torch.bool, device=_dev())
    keep[128 * 7:128 * 8] = False
    assert torch.equal(out[keep], clean[keep])           # same name, seed and step: the same random stream
    assert not bool(torch.isfinite(out[128 * 7:128 * 8]).all())


def test_sign_codecs_map_nan_to_minus_one():
    n = 10_000
    x = _rand(n, 6)
    x[5] = float("nan")
    grc = _grc({"compressor": "signsgd", "memory": "none", "communicator": "allgather"})
    out = grc.step(x.clone(), "w")
    grc.check()
    assert bool((out.abs() == 1).all()) and float(out[5]) == -1.0     # "x >= 0" is false for NaN
