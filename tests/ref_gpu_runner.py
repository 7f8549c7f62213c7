"""Helper of ``test_gpu_reference_parity.py`` (not a test): on every rank of a small NCCL job, run the UNMODIFIED
reference package from ``baseline/_ref`` on the GPU through its own communicators, then this package's fused
exchange (``fused=True``) on the same inputs, and write what differs to a JSON report.

    python tests/ref_gpu_runner.py <baseline/_ref> <report.json> <rendezvous file> <world> [cases|curves]

``cases``: three consecutive ``grc.step`` calls per deterministic codec (so error-feedback state takes part);
aggregated gradients and residual state are compared.  ``curves``: ResNet-20, TopK 1 % with residual memory, the
reference's own training loop (``examples/dist/CIFAR10-dawndist/core.py:202-208``: ``grc.step`` per parameter after
backward, then the optimizer), 50 steps per arm from the same initial weights on the same synthetic batches.

The reference's package is also called ``grace_dl``: it is imported first, used, and then dropped from
``sys.modules`` before this package is imported.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = {
    "topk": dict(compressor="topk", memory="residual", communicator="allgather", compress_ratio=0.01),
    "threshold": dict(compressor="threshold", memory="residual", communicator="allgather", threshold=2.5),
    "fp16": dict(compressor="fp16", memory="none", communicator="allgather"),
    "none": dict(compressor="none", memory="none", communicator="allgather"),
    "signsgd": dict(compressor="signsgd", memory="none", communicator="allgather"),
    "signum": dict(compressor="signum", memory="none", communicator="allgather", momentum=0.9),
    "efsignsgd": dict(compressor="efsignsgd", memory="efsignsgd", communicator="allgather", lr=0.1),
    "dgc_exact": dict(compressor="dgc", memory="dgc", communicator="allgather", compress_ratio=0.01, momentum=0.9),
}
STEPS = 3
SHAPE = (300, 1001)


def _inputs(case, step, rank, dev):
    import torch

    g = torch.Generator().manual_seed(100003 * sum(case.encode()) + 17 * step + rank)
    return torch.randn(*SHAPE, generator=g).to(dev)


def _drop_grace_dl():
    for mod in [m for m in sys.modules if m == "grace_dl" or m.startswith("grace_dl.")]:
        del sys.modules[mod]


def _reference_objects(ref_root, world):
    """Factory of the reference's communicators; DGC with the exact k-th magnitude as threshold (the reference
    samples 1 % of the elements with a CPU generator; the shim keeps everything else of its compress())."""
    sys.path.insert(0, ref_root)
    import torch
    import grace_dl

    assert os.path.abspath(grace_dl.__file__).startswith(os.path.abspath(ref_root)), grace_dl.__file__
    from grace_dl.dist.communicator.allgather import Allgather
    from grace_dl.dist.compressor.dgc import DgcCompressor
    from grace_dl.dist.helper import grace_from_params
    from grace_dl.dist.memory.dgc import DgcMemory

    class ExactDgc(DgcCompressor):
        def compress(self, tensor, name):
            shape = tensor.size()
            flat = tensor.flatten()
            numel = flat.numel()
            k = max(1, int(numel * self.compress_ratio))
            thr = flat.abs().topk(k, sorted=True)[0][-1]
            mask = flat.abs() >= thr
            indices, = torch.where(mask)
            values = flat[indices]
            return (values, indices), (shape, mask, numel)

    def make(case):
        p = dict(CASES[case], world_size=world)
        if case == "dgc_exact":
            return Allgather(ExactDgc(p["compress_ratio"]), DgcMemory(p["momentum"], False, world), world)
        return grace_from_params(p)

    return make


def _state_of_reference(grc, name):
    out = {}
    for attr in ("residuals", "gradients"):
        d = getattr(grc.memory, attr, None)
        if isinstance(d, dict) and name in d:
            out[attr] = d[name].detach().clone().reshape(-1)
    d = getattr(grc.compressor, "momentums", None)
    if isinstance(d, dict) and name in d:
        out["momentums"] = d[name].detach().clone().reshape(-1)
    return out


def run_cases(ref_root, rank, world, dev):
    import torch

    make_ref = _reference_objects(ref_root, world)
    name = "layer.weight"
    ref_out, ref_state = {}, {}
    for case in CASES:
        grc = make_ref(case)
        ref_out[case] = [grc.step(_inputs(case, s, rank, dev).clone(), name).clone() for s in range(STEPS)]
        ref_state[case] = _state_of_reference(grc, name)
    torch.cuda.synchronize()
    sys.path.remove(ref_root)
    _drop_grace_dl()
    sys.path.insert(0, ROOT)
    from grace_b200 import grace_from_params

    report = {}
    for case in CASES:
        p = dict(CASES[case], world_size=world, fused=True, timeout_ms=5000)
        if case == "dgc_exact":
            p["compressor"] = "dgc"
        grc = grace_from_params(p)
        assert grc.supported(_inputs(case, 0, rank, dev)), case
        worst, mism, total = 0.0, 0, 0
        for s in range(STEPS):
            out = grc.step(_inputs(case, s, rank, dev).clone(), name)
            ref = ref_out[case][s]
            assert out.shape == ref.shape and out.dtype == ref.dtype, (case, out.shape, ref.shape)
            d = (out - ref).abs()
            worst = max(worst, float(d.max()))
            mism += int((d > 0).sum())
            total += d.numel()
        grc.check()
        st = grc.state_dict()
        state_worst = 0.0
        for attr, t in ref_state[case].items():
            src = st["compressor" if attr == "momentums" else "memory"].get(attr, {})
            assert name in src, (case, attr)
            state_worst = max(state_worst, float((src[name].reshape(-1) - t).abs().max()))
        report[case] = {"max_abs_diff": worst, "mismatching": mism, "elements": total, "state_max_abs_diff": state_worst,
                        "state_keys": sorted(ref_state[case])}
    return report


def run_curves(ref_root, rank, world, dev, steps=50):
    import torch
    import torch.nn.functional as F

    sys.path.insert(0, ROOT)
    from grace_b200.models.resnet_cifar import resnet20   # plain torch module; no grace_dl import involved
    sys.path.remove(ROOT)

    torch.manual_seed(0)
    init = resnet20().state_dict()
    gen = torch.Generator().manual_seed(1234 + rank)
    xs = [torch.randn(32, 3, 32, 32, generator=gen).to(dev) for _ in range(4)]
    ys = [torch.randint(0, 10, (32,), generator=gen).to(dev) for _ in range(4)]
    params = dict(compressor="topk", memory="residual", communicator="allgather", compress_ratio=0.01, world_size=world)

    def train(grc):
        model = resnet20().to(dev)
        model.load_state_dict(init)
        opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
        losses = []
        for i in range(steps):
            opt.zero_grad()
            loss = F.cross_entropy(model(xs[i % 4]), ys[i % 4])
            loss.backward()
            for n, p in model.named_parameters():
                p.grad.data.copy_(grc.step(p.grad.data, n).view_as(p.grad))
            opt.step()
            losses.append(float(loss))
        return losses

    torch.backends.cudnn.deterministic = True
    sys.path.insert(0, ref_root)
    from grace_dl.dist.helper import grace_from_params as ref_factory

    ref_losses = train(ref_factory(dict(params)))
    sys.path.remove(ref_root)
    _drop_grace_dl()
    sys.path.insert(0, ROOT)
    from grace_b200 import grace_from_params

    grc = grace_from_params(dict(params, fused=True, timeout_ms=5000))
    our_losses = train(grc)
    grc.check()
    return {"reference": ref_losses, "fused": our_losses}


def _worker(rank, world, ref_root, out_path, port, mode):
    import torch
    import torch.distributed as dist

    import datetime

    os.environ.update(NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # rendezvous through a file (``port`` is its path): no TCP port to lose a race for
    dist.init_process_group("nccl", init_method="file://" + port, rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=180))
    try:
        report = run_cases(ref_root, rank, world, dev) if mode == "cases" else run_curves(ref_root, rank, world, dev)
        gathered = [None] * world
        dist.all_gather_object(gathered, report)
        if rank == 0:
            with open(out_path, "w") as f:
                json.dump({"world": world, "ranks": gathered}, f)
    finally:
        dist.destroy_process_group()


def main():
    ref_root, out_path, port, world = sys.argv[1], sys.argv[2], sys.argv[3], int(sys.argv[4])
    mode = sys.argv[5] if len(sys.argv) > 5 else "cases"
    if ROOT in sys.path:
        sys.path.remove(ROOT)
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, ref_root, out_path, port, mode), nprocs=world, join=True)


if __name__ == "__main__":
    main()
