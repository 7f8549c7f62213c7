"""Helper of ``test_reference_parity_cpu.py`` (not a test): runs the UNMODIFIED reference package found under
``baseline/_ref`` on CPU (gloo, world size 1) for a fixed set of inputs and saves what it returns.  Runs in its own
process because the reference's package is also called ``grace_dl``.

    python tests/ref_oracle_runner.py <baseline/_ref> <out.pt>
"""
import os
import sys


def inputs(case, step, shape=(40, 25)):
    import torch

    g = torch.Generator().manual_seed(1000 * sum(case.encode()) + step)
    return torch.randn(*shape, generator=g)


CASES = {
    "topk": dict(compressor="topk", memory="residual", communicator="allgather", compress_ratio=0.05),
    "threshold": dict(compressor="threshold", memory="residual", communicator="allgather", threshold=1.2),
    "fp16": dict(compressor="fp16", memory="none", communicator="allreduce"),
    "none": dict(compressor="none", memory="none", communicator="allreduce"),
    "signsgd": dict(compressor="signsgd", memory="none", communicator="allgather"),
    "efsignsgd": dict(compressor="efsignsgd", memory="efsignsgd", communicator="allgather", lr=0.1),
    "signum": dict(compressor="signum", memory="none", communicator="allgather", momentum=0.9),
    "randomk": dict(compressor="randomk", memory="residual", communicator="allgather", compress_ratio=0.1),
    # stochastic codecs: both sides draw from torch's global generator, seeded alike before every step
    "qsgd": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=64),
    "terngrad": dict(compressor="terngrad", memory="residual", communicator="allgather"),
    "dgc": dict(compressor="dgc", memory="residual", communicator="allgather", compress_ratio=0.05),
    "dgc_momentum": dict(compressor="dgc", memory="dgc", communicator="allgather", compress_ratio=0.05, momentum=0.9,
                         gradient_clipping=False),
}
STEPS = 3


def pipeline(grc, x, name):
    """What ``Communicator.step`` does around the collective, for one rank: compensate, compress, update the
    memory, decompress the own payload, aggregate (a list of one) and average.  Uses only the compressor and
    memory objects, so it runs where a communicator could not (the reference's variable-size all-gather calls
    ``.cuda()``)."""
    import torch

    comp, mem = grc.compressor, grc.memory
    torch.manual_seed(4242)
    t = mem.compensate(x, name)
    payload, ctx = comp.compress(t, name)
    mem.update(t, name, comp, payload, ctx)
    out = comp.aggregate([comp.decompress(payload, ctx)])
    return out / 1 if comp.average else out


DIST_CASES = ["topk", "fp16", "none", "signsgd", "efsignsgd", "signum", "randomk", "qsgd", "terngrad"]


def dist_inputs(case, step, rank, shape=(40, 25)):
    import torch

    g = torch.Generator().manual_seed(1000 * sum(case.encode()) + 10 * step + rank + 5)
    return torch.randn(*shape, generator=g)


def dist_steps(grace_from_params, rank, world):
    """``grc.step`` through the real communicator (same-size payloads only: they run on gloo) on every rank."""
    import torch

    out = {}
    for case in DIST_CASES:
        grc = grace_from_params(dict(CASES[case], world_size=world))
        res = []
        for step in range(STEPS):
            torch.manual_seed(77 + rank)
            res.append(grc.step(dist_inputs(case, step, rank).clone(), "layer.weight").clone())
        out[case] = res
    return out


def _dist_worker(rank, world, ref_root, out_path, port):
    sys.path.insert(0, ref_root)
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from grace_dl.dist.helper import grace_from_params

    out = dist_steps(grace_from_params, rank, world)
    if rank == 0:
        torch.save(out, out_path)
    dist.barrier()
    dist.destroy_process_group()


def main():
    if len(sys.argv) > 4 and int(sys.argv[4]) > 1:
        import torch.multiprocessing as mp

        world = int(sys.argv[4])
        mp.spawn(_dist_worker, args=(world, sys.argv[1], sys.argv[2], int(sys.argv[3])), nprocs=world, join=True)
        return
    ref_root, out_path = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref_root)
    import torch
    import torch.distributed as dist

    import grace_dl

    assert os.path.abspath(grace_dl.__file__).startswith(os.path.abspath(ref_root)), grace_dl.__file__
    from grace_dl.dist.helper import grace_from_params
    from grace_dl.dist.compressor.powersgd import orthogonalize

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", sys.argv[3] if len(sys.argv) > 3 else "29577")
    dist.init_process_group("gloo", rank=0, world_size=1)
    out = {}
    for case, params in CASES.items():
        grc = grace_from_params(dict(params, world_size=1))
        res = []
        for step in range(STEPS):
            res.append(pipeline(grc, inputs(case, step).clone(), "layer.weight").clone())
        out[case] = res
    m = inputs("orth", 0, (64, 4)).clone()
    orthogonalize(m)
    out["orthogonalize"] = [m]
    torch.save(out, out_path)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
