"""Factory, base-class contract, import paths, checkpointing, optimizer wrapper."""
import warnings

import pytest
import torch

import grace_b200
from grace_b200 import grace_from_params


def test_reference_import_paths():
    from grace_dl.dist import Communicator, Compressor, Memory  # noqa: F401
    from grace_dl.dist.communicator.all_to_all import AllToAll  # noqa: F401
    from grace_dl.dist.communicator.allgather import Allgather
    from grace_dl.dist.communicator.allreduce import Allreduce  # noqa: F401
    from grace_dl.dist.communicator.broadcast import Broadcast  # noqa: F401
    from grace_dl.dist.compressor.natural import NaturalCompressor_CUDA  # noqa: F401
    from grace_dl.dist.compressor.qsgd import QSGDCompressor_CUDA  # noqa: F401
    from grace_dl.dist.compressor.topk import TopKCompressor
    from grace_dl.dist.helper import grace_from_params as g2
    from grace_dl.dist.memory.residual import ResidualMemory
    from grace_dl.torch.optimizer import DistributedOptimizer  # noqa: F401
    from grace_dl.torch.helper import grace_from_params as g3  # noqa: F401

    grc = Allgather(TopKCompressor(0.3), ResidualMemory(), 1)
    out = grc.step(torch.randn(4, 5), "w")
    assert out.shape == (4, 5)
    assert g2 is grace_from_params
    # the TensorFlow tree's module names resolve to the PyTorch implementations (TensorFlow itself is not used)
    from grace_dl.tensorflow.communicator.allgather import Allgather as TfAllgather
    from grace_dl.tensorflow.compressor.inceptionn import INCEPTIONNCompressor  # noqa: F401
    from grace_dl.tensorflow.compressor.packing import decode_byte, encode_byte  # noqa: F401
    from grace_dl.tensorflow.compressor.u8bit import U8bitCompressor
    from grace_dl.tensorflow.helper import grace_from_params as g4
    from grace_dl.tensorflow.memory.residual import ResidualMemory as TfResidual

    assert TfAllgather is Allgather and g4 is grace_from_params
    out = TfAllgather(U8bitCompressor(), TfResidual(), 1).step(torch.randn(300), "u")
    assert out.shape == (300,)


COMPRESSORS = ["dgc", "efsignsgd", "fp16", "natural", "natural_cuda", "none", "onebit", "powersgd", "qsgd",
               "qsgd_cuda", "randomk", "signsgd", "signum", "terngrad", "threshold", "topk", "u8bit", "adaq",
               "inceptionn", "sketch"]


@pytest.mark.parametrize("name", COMPRESSORS)
def test_factory_builds_every_compressor(name):
    mem = {"dgc": "dgc", "efsignsgd": "efsignsgd", "powersgd": "powersgd"}.get(name, "residual")
    comm = "allreduce" if name in ("none", "fp16", "randomk", "powersgd") else "allgather"
    grc = grace_from_params({"compressor": name, "memory": mem, "communicator": comm, "world_size": 1})
    x = torch.randn(6, 50) * 0.01
    for _ in range(2):
        out = grc.step(x.clone(), "w")
    assert out.shape == x.shape and torch.isfinite(out).all()
    assert grc.stats()["steps"] == 2


def test_factory_defaults_and_errors():
    grc = grace_from_params({"world_size": 2})
    assert type(grc).__name__ == "Allreduce" and type(grc.compressor).__name__ == "NoneCompressor"
    assert type(grc.memory).__name__ == "NoneMemory" and grc.world_size == 2
    assert grace_from_params({"compressor": "topk", "world_size": 1}).compressor.compress_ratio == 0.3
    q = grace_from_params({"compressor": "qsgd", "world_size": 1}).compressor
    assert q.quantum_num == 127 and q.bucket_size == 128
    assert grace_from_params({"compressor": "signum", "world_size": 1}).compressor.momentum == 0.9
    assert grace_from_params({"compressor": "threshold", "world_size": 1}).compressor.threshold == 0.01
    assert grace_from_params({"compressor": "efsignsgd", "world_size": 1}).compressor.learning_rate == 0.1
    p = grace_from_params({"compressor": "powersgd", "memory": "powersgd", "compress_rank": 4, "world_size": 3})
    assert p.compressor.rank == 4 and p.compressor.world_size == 3 and p.memory.compress_rank == 4
    b = grace_from_params({"compressor": "topk", "communicator": "broadcast", "world_size": 1})
    assert b.rank == 0
    for bad in ({"compressor": "nope"}, {"memory": "nope"}, {"communicator": "nope"}):
        with pytest.raises(NotImplementedError):
            grace_from_params({"world_size": 1, **bad})
    with pytest.raises(KeyError):
        grace_from_params({"compressor": "topk"})


def test_send_receive_split_matches_step():
    a = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather", "world_size": 1})
    b = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather", "world_size": 1})
    for i in range(3):
        x = torch.randn(200)
        h, ctx = a.send_step(x, "w")
        torch.testing.assert_close(a.receive_step(h, ctx), b.step(x, "w"))


def test_state_dict_roundtrip_resumes_identically():
    def make():
        return grace_from_params({"compressor": "signum", "memory": "residual", "communicator": "allgather",
                                  "world_size": 1})

    a = make()
    xs = [torch.randn(300) for _ in range(4)]
    a.step(xs[0], "w"); a.step(xs[1], "w")
    state = a.state_dict()
    assert set(state) >= {"compressor", "memory", "world_size"}
    assert "residuals" in state["memory"] and "momentums" in state["compressor"]
    b = make()
    b.load_state_dict(state)
    torch.testing.assert_close(a.step(xs[2], "w"), b.step(xs[2], "w"))
    torch.testing.assert_close(a.memory.residuals["w"], b.memory.residuals["w"])
    c = grace_from_params({"compressor": "signum", "memory": "residual", "communicator": "allgather", "world_size": 2})
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        c.load_state_dict(state)
    assert w and not c.memory.residuals


def test_checkpoint_files(tmp_path):
    from grace_b200.utils.checkpoint import load_checkpoint, save_checkpoint

    model = torch.nn.Linear(8, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather", "world_size": 1})
    for n, p in model.named_parameters():
        grc.step(torch.randn_like(p), n)
    save_checkpoint(str(tmp_path), model=model, optimizer=opt, grace=grc, rank=0, step=7)
    assert (tmp_path / "grace_rank0.pt").exists() and (tmp_path / "model.pt").exists()
    grc2 = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather", "world_size": 1})
    meta = load_checkpoint(str(tmp_path), model=model, optimizer=opt, grace=grc2, rank=0)
    assert meta["step"] == 7
    for n in grc.memory.residuals:
        torch.testing.assert_close(grc.memory.residuals[n], grc2.memory.residuals[n])


# ---------------------------------------------------------------- optimizer wrapper
class _FakeGrace:
    def __init__(self):
        self.sent, self.received = [], 0

    def send_step(self, tensor, name):
        self.sent.append(name)
        return ("h", tensor * 2), name

    def receive_step(self, handle, ctx):
        self.received += 1
        return handle[1]


def _wrapped(passes=1, fake=None, named=True):
    from grace_b200.parallel import DistributedOptimizer

    model = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    opt = torch.optim.SGD(model.parameters(), lr=0.0, momentum=0.9)
    fake = fake or _FakeGrace()
    d = DistributedOptimizer(opt, grace=fake, named_parameters=model.named_parameters() if named else None,
                             backward_passes_per_step=passes, always_hook=True)
    return model, d, fake


def test_distributed_optimizer_contract():
    model, d, fake = _wrapped()
    assert isinstance(d, torch.optim.SGD) and type(d).__name__ == "SGD"
    model(torch.randn(5, 4)).sum().backward()
    assert sorted(fake.sent) == sorted(n for n, _ in model.named_parameters())
    with pytest.raises(AssertionError):
        d.zero_grad()  # exchanges in flight
    grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    d.step()
    assert fake.received == 4
    for n, p in model.named_parameters():
        torch.testing.assert_close(p.grad, grads[n] * 2)  # grad replaced by the exchanged tensor
    d.zero_grad()
    # synchronize + skip_synchronize, and the warning on a redundant synchronize
    model(torch.randn(5, 4)).sum().backward()
    d.synchronize()
    with d.skip_synchronize():
        d.step()
    model(torch.randn(5, 4)).sum().backward()
    d.synchronize()
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        d.step()
    assert any("skip_synchronize" in str(x.message) for x in w)


def test_distributed_optimizer_accumulation_and_validation():
    from grace_b200.parallel import DistributedOptimizer

    model, d, fake = _wrapped(passes=2)
    model(torch.randn(5, 4)).sum().backward()
    assert fake.sent == []  # first pass only accumulates
    model(torch.randn(5, 4)).sum().backward()
    assert len(fake.sent) == 4
    d.step()
    d.set_backward_passes_per_step(1)
    d.zero_grad()
    model(torch.randn(5, 4)).sum().backward()
    assert len(fake.sent) == 8
    d.load_state_dict(d.state_dict())  # resets in-flight handles
    d.zero_grad()
    _, d2, fake2 = _wrapped(named=False)
    assert sorted(d2._parameter_names.values())[0].startswith("allreduce.noname.")
    m = torch.nn.Linear(2, 2)
    o = torch.optim.SGD(m.parameters(), lr=0.1)
    with pytest.raises(ValueError):
        DistributedOptimizer(o, grace=fake, named_parameters=[("a", m.weight), ("a", m.bias)])
    with pytest.raises(ValueError):
        DistributedOptimizer(o, grace=fake, named_parameters=[("a", m.weight)])
    with pytest.raises(ValueError):
        DistributedOptimizer(o, grace=fake, named_parameters=["a", "b"])


def test_missing_hooks_are_launched_at_synchronize():
    model, d, fake = _wrapped()
    model[0](torch.randn(5, 4)).sum().backward()  # second layer never gets a gradient hook call
    d.step()
    assert len(fake.sent) == 4


def test_wrapper_keeps_the_wrapped_optimizers_own_attributes():
    from grace_b200.optim import FusedSGD
    from grace_b200.parallel import DistributedOptimizer

    m = torch.nn.Linear(3, 2)
    opt = FusedSGD(m.parameters(), lr=0.1, momentum=0.9)
    opt.grad_scale = 0.5
    marker = object()
    opt.flat = marker
    d = DistributedOptimizer(opt, grace=_FakeGrace(), named_parameters=m.named_parameters(), always_hook=True)
    assert d.flat is marker and d.grad_scale == 0.5 and d.param_groups[0]["lr"] == 0.1


def test_metrics_helpers(tmp_path):
    import json

    from grace_b200.utils.metrics import DeviceTimer, JsonlLogger, TableLogger, ThroughputMeter

    with DeviceTimer("cpu") as t:
        sum(range(1000))
    assert t.ms >= 0
    m = ThroughputMeter()
    m.update(256, 100.0); m.update(256, 100.0)
    assert abs(m.rate() - 2560.0) < 1e-6
    log = JsonlLogger(str(tmp_path / "log.jsonl"))
    log.log(step=1, loss=0.5)
    rec = json.loads(open(tmp_path / "log.jsonl").read().splitlines()[0])
    assert rec["step"] == 1 and rec["rank"] == 0
    text = TableLogger().append({"epoch": 1, "loss": 0.25})
    assert "epoch" in text and "0.2500" in text
    grc = grace_from_params({"compressor": "topk", "memory": "none", "communicator": "allgather", "world_size": 1,
                             "compress_ratio": 0.1})
    grc.step(torch.randn(1000), "w")
    s = grc.stats()
    assert s["steps"] == 1 and 4.9 < s["compression_ratio"] < 5.1


def test_tile_ordered_exchange_rule_is_a_pure_function_of_layout_capacity_and_world():
    """Every rank must size its send slot alike, so the rule may only look at (elements, capacity, world, mode)."""
    import grace_b200.ops.exchange as X

    n = 256 << 20
    k = n // 100
    assert X.tile_decode_wanted(n, k, 8, X.SPARSE_TOPK)          # 8 lists of 1 %: dense tiles win
    assert not X.tile_decode_wanted(n, k, 1, X.SPARSE_TOPK)      # one list: scattered adds win
    assert not X.tile_decode_wanted(n, n // 1000, 8, X.SPARSE_TOPK)
    assert not X.tile_decode_wanted(1 << 20, 1 << 14, 8, X.SPARSE_TOPK)   # fits the L2 cache
    assert not X.tile_decode_wanted(n, k, 8, X.SPARSE_RANDOMK)   # random-k sends no indices at all
    assert not X.tile_decode_wanted(n, n // 4, 8, X.SPARSE_THRESHOLD)   # capacity is a bound there, not a density


def test_nvls_option_falls_back_cleanly_without_multicast():
    from grace_b200 import grace_from_params
    from grace_b200.communicator.nvls import NvlsAllreduce

    grc = grace_from_params({"compressor": "none", "memory": "none", "communicator": "allreduce", "world_size": 1,
                             "fused": True, "nvls": True})
    assert isinstance(grc, NvlsAllreduce)
    x = torch.arange(8.0)
    assert torch.equal(grc.step(x.clone(), "w"), x)
    assert grc.buffer(1024) is None and grc.stats()["nvls_launches"] == 0
    h, ctx = grc.send_step(x.clone(), "w")
    assert torch.equal(grc.receive_step(h, ctx), x)
    # the option is ignored for compressors that are not the identity
    other = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                               "world_size": 1, "compress_ratio": 0.5, "fused": True, "nvls": True})
    assert not isinstance(other, NvlsAllreduce)


def test_native_module_loads_without_a_gpu_and_sizes_its_slots():
    """The extension links no driver library, so its host-side helpers work on a machine without a GPU."""
    from grace_b200.ops import native

    C = native()
    cap, total = 4096, 1 << 20
    plain = C.sparse_slot_bytes(cap)
    tiled = C.sparse_slot_bytes(cap, total)
    tiles = total // 8192
    assert plain == 128 + 8 * cap
    # tile-ordered layout: a second (value, index) list and a directory of tiles + 1 offsets, 16-byte granular
    assert tiled == plain + 8 * cap + (tiles + 1 + 3) // 4 * 16
    q8 = C.quant_slot_bytes(0, total, 1)          # codec 0 = QSGD: 1 byte per element + one norm per 128
    assert q8 >= 128 + total + total // 128 * 4 and q8 % 256 == 0
    assert C.MAX_WORLD == 16


def test_timeline_records_every_exchange_as_chrome_trace(tmp_path):
    import json

    import grace_b200.parallel.hvd as hvd
    from grace_b200 import grace_from_params
    from grace_b200.utils import timeline

    path = str(tmp_path / "trace.json")
    assert timeline.active() is None and hvd.stop_timeline() is None
    hvd.start_timeline(path)                      # same entry points as horovod.torch
    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.1, "world_size": 1})
    for step in range(3):
        grc.step(torch.randn(1000), "layer.weight")
    timeline.active().instant("epoch", index=0)
    assert hvd.stop_timeline() == path and timeline.active() is None
    trace = json.load(open(path))
    xs = [e for e in trace["traceEvents"] if e.get("ph") == "X"]
    assert len(xs) == 3 and all(e["name"] == "layer.weight" and e["cat"] == "Allgather" for e in xs)
    assert all(e["args"]["numel"] == 1000 and e["args"]["payload_bytes"] == 100 * 8 and e["dur"] >= 0 for e in xs)
    assert xs[0]["ts"] <= xs[1]["ts"] <= xs[2]["ts"]
    assert any(e.get("ph") == "i" and e["name"] == "epoch" for e in trace["traceEvents"])
    grc.step(torch.randn(10), "untraced")          # no active timeline: nothing is recorded, nothing breaks


def test_threshold_flavours_of_the_two_import_paths():
    """``grace_dl.dist``: ``|x| >= min(thr, max(x))``; ``grace_dl.torch`` (Horovod flavour): ``|x| > thr``."""
    from grace_b200.communicator.fused import FusedExchange
    from grace_b200.memory.none import NoneMemory
    from grace_dl.dist.compressor.threshold import ThresholdCompressor as DistThreshold
    from grace_dl.torch.compressor.threshold import ThresholdCompressor as TorchThreshold

    x = torch.tensor([0.5, -1.0, 2.0, 1.0])
    assert DistThreshold(1.0).compress(x, "a")[0][1].tolist() == [1, 2, 3]
    assert TorchThreshold(1.0).compress(x, "a")[0][1].tolist() == [2]
    assert DistThreshold(5.0).compress(x, "a")[0][1].tolist() == [2]      # capped at the largest element
    assert TorchThreshold(5.0).compress(x, "a")[0][1].tolist() == []
    # the fused kernel implements the dist rule only: the strict flavour is left to the library path
    assert FusedExchange(DistThreshold(1.0), NoneMemory(), 1)._kind == "sparse"
    assert FusedExchange(TorchThreshold(1.0), NoneMemory(), 1)._kind == "sparse"   # the kernel has both rules


def test_bindings_reject_inconsistent_arguments_before_any_launch():
    """Argument checks of the launch bindings run on the host, ahead of every CUDA call."""
    from grace_b200.ops import native

    C = native()
    heaps = [4096]
    with pytest.raises(ValueError):     # push transport needs both addresses of the receive area
        C.quant_exchange(16, 0, 0, 16, 16, 1, 128, 0, 64, 0, 0, 1.0, 1.0, 0.0, 1.0, 1.0, 0, 0, 16, 16, 16, 7, 0, 1, 1,
                         10 ** 9, heaps, 0, 128, 256, 1, 0, 0, 0, 16, 0, 256, 0, 0, 0, 4096, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):     # total must be a multiple of 128
        C.quant_exchange(16, 0, 0, 16, 16, 1, 100, 0, 64, 0, 0, 1.0, 1.0, 0.0, 1.0, 1.0, 0, 0, 16, 16, 16, 7, 0, 1, 1,
                         10 ** 9, heaps, 0, 128, 256, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 4096, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):     # rank outside the world
        C.quant_exchange(16, 0, 0, 16, 16, 1, 128, 0, 64, 0, 0, 1.0, 1.0, 0.0, 1.0, 1.0, 0, 0, 16, 16, 16, 7, 3, 1, 1,
                         10 ** 9, heaps, 0, 128, 256, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 4096, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):     # gradient element type: 0 fp32, 1 bf16, 2 fp16
        C.quant_exchange(16, 0, 0, 16, 16, 1, 128, 0, 64, 0, 0, 1.0, 1.0, 0.0, 1.0, 1.0, 0, 0, 16, 16, 16, 7, 0, 1, 1,
                         10 ** 9, heaps, 0, 128, 256, 1, 0, 0, 0, 0, 0, 0, 5, 0, 0, 4096, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):     # dense all-reduce: 16-byte aligned pointers only
        C.dense_allreduce(8, 16, 16, 16, 128, 1.0, 16, 16, 0, 0, 1, 1, 10 ** 9, heaps, 0, 128, 1, 0)


def test_pipeline_plan_covers_the_buffer_with_whole_chunks():
    from grace_b200.ops.exchange import CODEC, pipeline_plan

    assert pipeline_plan(1 << 20, 4, CODEC["qsgd"]) is None            # too small to pay
    assert pipeline_plan(256 << 20, 1, CODEC["qsgd"]) is None          # nobody to overlap with
    assert pipeline_plan(256 << 20, 4, CODEC["efsign"]) is None
    for total in (32 << 20, (336 << 20) + 128 * 77, 256 << 20, 1 << 30):
        chunks, per_chunk, item = pipeline_plan(total, 8, CODEC["natural"])
        items = -(-total // item)
        assert item % 8192 == 0 and 2 <= chunks <= 16
        assert (chunks - 1) * per_chunk < items <= chunks * per_chunk
    chunks, per_chunk, item = pipeline_plan(300_032, 1, CODEC["qsgd"], force=True)
    assert (chunks - 1) * per_chunk < -(-300_032 // item) <= chunks * per_chunk
