"""The checked build of the kernels (``-DGRACE_CHECKED``, loaded with ``GRACE_CHECKED=1``): the small-shape exchanges
run under it with every index / offset check compiled in and report no violation; a launch whose send slot is
declared smaller than what the kernel writes is caught, with the kernel, the source line and the offending offset in
the error, while the access itself is skipped (nothing faults).  Runs in a child process: the variant is chosen when
the extension is first loaded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BODY = r'''
import sys, torch
sys.path.insert(0, %r)
from grace_b200.ops import native
assert native().CHECKED, "the checked variant must be the one loaded"
from grace_b200 import grace_from_params
from grace_b200.communicator.fused import VirtualWorld
from grace_b200.ops import exchange as X
dev = torch.device("cuda")
cases = [dict(compressor="topk", memory="residual", compress_ratio=0.05),
         dict(compressor="dgc", memory="dgc", compress_ratio=0.05, momentum=0.9),
         dict(compressor="qsgd", memory="residual", quantum_num=64),
         dict(compressor="qsgd", memory="residual", quantum_num=300, bucket_size=64),
         dict(compressor="efsignsgd", memory="efsignsgd", lr=0.1),
         dict(compressor="terngrad", memory="none"), dict(compressor="natural", memory="none")]
for W in (1, 4):
    for params in cases:
        for n in (1, 129, 6145, 70001):
            vw = VirtualWorld(W, lambda r: grace_from_params(dict(params, communicator="allgather", world_size=W, fused=True)), dev)
            gen = torch.Generator().manual_seed(n)
            outs = vw.step([torch.randn(n, generator=gen).to(dev) for _ in range(W)], "w")
            vw.check()                                   # raises if any check failed
            assert torch.isfinite(outs[0]).all()
# a slot declared too small: the first store beyond it is recorded and skipped
grc = grace_from_params(dict(compressor="qsgd", memory="none", communicator="allgather", quantum_num=64, world_size=1, fused=True))
x = torch.randn(100000, device=dev)
grc.step(x.clone(), "w")
grc.check()
plan = next(iter(grc._plans.values()))
try:
    X.run_quant(plan.channel, plan.layout, plan.segs, x.clone(), None, None, torch.empty_like(x), codec=plan.codec, quantum=64,
                seed=1, step=1, scale=1.0, slot_bytes=4096)
    plan.channel.check()
    raise SystemExit("the undersized slot was not noticed")
except X.GraceCommError as e:
    assert e.code == 7 and e.kernel == 2 and e.index >= 4096, (e.code, getattr(e, "kernel", None), getattr(e, "index", None))
    print("caught:", e)
print("CHECKED-OK")
'''


def test_checked_build_runs_clean_and_catches_an_undersized_slot():
    env = dict(os.environ, GRACE_CHECKED="1")
    res = subprocess.run([sys.executable, "-c", BODY % ROOT], env=env, capture_output=True, text=True, timeout=420)
    assert res.returncode == 0 and "CHECKED-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
