"""The fused exchange (``fused=True``) against the UNMODIFIED reference on the GPU.

``tests/ref_gpu_runner.py`` runs, in child processes (one per GPU, NCCL), the reference package installed under
``baseline/_ref`` through its own ``Allgather`` communicator and then this package's fused kernels on the same
inputs: three consecutive steps of TopK, Threshold, fp16, no compression, signSGD, signum, EF-signSGD and DGC
(with the exact k-th magnitude as its threshold on both sides), comparing the aggregated gradients and the
error-feedback state; and 50 training steps of ResNet-20 with TopK 1 %.  One rank always, two ranks when the
machine has two GPUs.  Skipped when the reference is not installed.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _token():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from _rendezvous import new_token

    return new_token()


def _run(world, mode, tmp_path):
    if not os.path.isdir(os.path.join(REF, "grace_dl", "dist")):
        pytest.skip("reference not installed under baseline/_ref")
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    out = str(tmp_path / ("report_%s_%d.json" % (mode, world)))
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT"):
        env.pop(k, None)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_gpu_runner.py"), REF, out, _token(),
                          str(world), mode], cwd="/", env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    return json.load(open(out))


# sparse and sign codecs: the same elements and the same bits; the others: fp32 rounding of differently ordered sums
EXACT = {"topk", "threshold", "signsgd", "none", "fp16"}


@pytest.mark.parametrize("world", [1, 2])
def test_fused_steps_match_the_reference_on_gpu(world, tmp_path):
    rep = _run(world, "cases", tmp_path)
    assert rep["world"] == world and len(rep["ranks"]) == world
    for rank, cases in enumerate(rep["ranks"]):
        for case, r in cases.items():
            where = "%s, rank %d of %d: %s" % (case, rank, world, r)
            if case in EXACT:
                assert r["max_abs_diff"] == 0.0 and r["state_max_abs_diff"] == 0.0, where
            elif case == "signum":
                # the momentum is a fused multiply-add here: a sign may flip where it is ~0
                assert r["mismatching"] <= 1e-4 * r["elements"] and r["state_max_abs_diff"] < 1e-6, where
            else:
                assert r["max_abs_diff"] < 1e-5 and r["state_max_abs_diff"] < 1e-5, where
        assert set(cases) == {"topk", "threshold", "fp16", "none", "signsgd", "signum", "efsignsgd", "dgc_exact"}
        assert cases["dgc_exact"]["state_keys"] == ["gradients", "residuals"]
        assert cases["topk"]["state_keys"] == ["residuals"]


def test_resnet20_topk_loss_curve_tracks_the_reference(tmp_path):
    world = 2 if torch.cuda.device_count() >= 2 else 1
    rep = _run(world, "curves", tmp_path)
    for rank, r in enumerate(rep["ranks"]):
        ref, ours = r["reference"], r["fused"]
        assert len(ref) == len(ours) == 50
        # identical weights, batches and selection rule: the curves start together ...
        for a, b in zip(ours[:5], ref[:5]):
            assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (rank, ours[:5], ref[:5])
        # ... and, rounding differences amplified by 50 SGD steps aside, end together
        tail_o, tail_r = sum(ours[-10:]) / 10, sum(ref[-10:]) / 10
        assert abs(tail_o - tail_r) < 0.25 * max(1.0, tail_r), (rank, tail_o, tail_r)
