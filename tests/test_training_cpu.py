"""Training-loop helpers (schedule, batched augmentations, manual-loop epoch) on CPU."""
import torch

from grace_b200 import grace_from_params
from grace_b200.utils.training import PiecewiseLinear, cutout, evaluate, random_crop, random_flip, train_epoch


def test_piecewise_linear_schedule_matches_the_dawn_shape():
    sched = PiecewiseLinear([0, 5, 24], [0.0, 0.4, 0.0])
    assert sched(0) == 0.0 and abs(sched(5) - 0.4) < 1e-12 and sched(24) == 0.0 and sched(30) == 0.0
    assert abs(sched(2.5) - 0.2) < 1e-12 and abs(sched(14.5) - 0.2) < 1e-12
    assert sched(-1) == 0.0


def test_batched_augmentations_are_reproducible_and_shape_preserving():
    x = torch.arange(2 * 3 * 8 * 8, dtype=torch.float32).view(2, 3, 8, 8) + 1.0
    g1, g2 = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
    a = cutout(random_flip(random_crop(x, 8, 2, g1), g1), 3, g1)
    b = cutout(random_flip(random_crop(x, 8, 2, g2), g2), 3, g2)
    assert a.shape == x.shape and torch.equal(a, b)
    # cutout zeroes exactly one 3 x 3 square per image (inputs are strictly positive)
    holes = (cutout(x, 3, torch.Generator().manual_seed(1)) == 0).sum(dim=(1, 2, 3))
    assert holes.tolist() == [27, 27]
    # a crop with pad 0 of the full size is the identity; a flip either mirrors or keeps each image
    assert torch.equal(random_crop(x, 8, 0, torch.Generator().manual_seed(0)), x)
    f = random_flip(x, torch.Generator().manual_seed(5))
    assert all(torch.equal(f[i], x[i]) or torch.equal(f[i], x[i].flip(-1)) for i in range(2))
    # every cropped window is a window of the reflected-padded image: values stay within the input's range
    c = random_crop(x, 8, 2, torch.Generator().manual_seed(9))
    assert c.min() >= x.min() and c.max() <= x.max()


def test_train_epoch_runs_the_manual_grace_loop_and_learns():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(3 * 4 * 4, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.25, "world_size": 1})
    opt = torch.optim.SGD(model.parameters(), lr=0.0, momentum=0.9, nesterov=True)
    g = torch.Generator().manual_seed(1)
    proto = torch.randn(4, 3, 4, 4, generator=g)
    y = torch.randint(0, 4, (256,), generator=g)
    x = proto[y] + 0.1 * torch.randn(256, 3, 4, 4, generator=g)
    data = [(x[i : i + 32], y[i : i + 32]) for i in range(0, 256, 32)]
    sched = PiecewiseLinear([0, 1, 6], [0.0, 0.1, 0.0])
    first = last = None
    step = 0
    for epoch in range(6):
        out = train_epoch(model, data, opt, grace=grc, lr_schedule=sched, step0=step, steps_per_epoch=len(data))
        step += out["steps"]
        first = out if first is None else first
        last = out
    assert out["steps"] == len(data) and last["loss"] < 0.5 * first["loss"]
    assert grc.stats()["steps"] == 6 * len(data) * 4          # four parameter tensors per step
    assert evaluate(model, data)["acc"] > 0.9


def test_model_diagram_is_valid_dot_with_residual_joins():
    from grace_b200.models import resnet9
    from grace_b200.utils.diagram import model_to_dot

    dot = model_to_dot(resnet9(), torch.zeros(1, 3, 32, 32), "resnet9")
    assert dot.startswith("digraph resnet9 {") and dot.rstrip().endswith("}")
    assert dot.count("{") == dot.count("}") == 1
    assert '"input" -> ' in dot and '-> "output"' in dot
    assert "Conv2d" in dot and "(1, 10)" in dot
    # every edge endpoint is a declared node
    import re

    declared = set(re.findall(r'^  "([^"]+)" \[', dot, flags=re.M))
    for src, dst in re.findall(r'^  "([^"]+)" -> "([^"]+)";', dot, flags=re.M):
        assert src in declared and dst in declared
