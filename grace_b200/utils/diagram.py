"""Network diagram as Graphviz DOT text.

The reference's example draws its ResNet from the dict-of-layers graph it trains with and keeps the picture in
the tree (``examples/dist/CIFAR10-dawndist/core.py:242-305`` via pydot, result ``net.svg``).  Models here are
ordinary ``nn.Module`` trees, so the diagram is derived from a traced forward pass: every leaf module becomes a
node labelled with its type, parameter count and output shape, edges follow the order in which tensors flow
between leaves (residual additions show up as nodes with two incoming edges).  Needs no Graphviz to produce
the text; render with ``dot -Tsvg net.dot -o net.svg`` where Graphviz is installed.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


def model_to_dot(model: torch.nn.Module, example_input: torch.Tensor, name: str = "net") -> str:
    from torch.overrides import TorchFunctionMode

    leaves = {m: n for n, m in model.named_modules() if len(list(m.children())) == 0}
    producer: Dict[int, str] = {id(example_input): "input"}
    nodes: List[Tuple[str, str]] = [("input", "input\\n%s" % (tuple(example_input.shape),))]
    edges: List[Tuple[str, str]] = []
    keep = []            # intermediate tensors stay alive during the trace so that ids are never reused
    depth = [0]          # > 0 while a leaf module runs: its internal torch calls are not part of the picture
    joins = [0]

    def tensors_in(obj):
        if torch.is_tensor(obj):
            yield obj
        elif isinstance(obj, (list, tuple)):
            for o in obj:
                yield from tensors_in(o)
        elif isinstance(obj, dict):
            for o in obj.values():
                yield from tensors_in(o)

    class Trace(TorchFunctionMode):
        def __torch_function__(self, func, types, args=(), kwargs=None):
            out = func(*args, **(kwargs or {}))
            if depth[0] == 0 and torch.is_tensor(out):
                srcs = []
                for t in tensors_in((args, kwargs or {})):
                    s = producer.get(id(t))
                    if s is not None and s not in srcs:
                        srcs.append(s)
                if len(srcs) == 1:                       # view / pooling / scaling between modules: transparent
                    producer[id(out)] = srcs[0]
                    keep.append(out)
                elif len(srcs) > 1:                      # a join, e.g. the residual addition
                    joins[0] += 1
                    node = "%s_%d" % (getattr(func, "__name__", "op"), joins[0])
                    nodes.append((node, "%s\\n%s" % (getattr(func, "__name__", "op"), tuple(out.shape))))
                    for s in srcs:
                        edges.append((s, node))
                    producer[id(out)] = node
                    keep.append(out)
            return out

    def pre_hook(mod, inputs):
        depth[0] += 1

    def hook(mod, inputs, output):
        depth[0] -= 1
        node = leaves[mod]
        nparams = sum(p.numel() for p in mod.parameters(recurse=False))
        label = "%s\\n%s" % (node, type(mod).__name__)
        if nparams:
            label += "\\n%d params" % nparams
        if torch.is_tensor(output):
            label += "\\n%s" % (tuple(output.shape),)
        nodes.append((node, label))
        for t in tensors_in(inputs):
            s = producer.get(id(t))
            if s is not None:
                edges.append((s, node))
        for t in tensors_in(output):
            producer[id(t)] = node
            keep.append(t)

    hooks = []
    for m in leaves:
        hooks.append(m.register_forward_pre_hook(pre_hook))
        hooks.append(m.register_forward_hook(hook))
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad(), Trace():
            out = model(example_input)
    finally:
        for h in hooks:
            h.remove()
        model.train(was_training)
    lines = ["digraph %s {" % name, "  rankdir=TB;", '  node [shape=box, fontname="Helvetica", fontsize=10];']
    seen = set()
    for node, label in nodes:
        if node in seen:
            continue
        seen.add(node)
        lines.append('  "%s" [label="%s"];' % (node, label))
    for s, d in dict.fromkeys(edges):
        lines.append('  "%s" -> "%s";' % (s, d))
    if torch.is_tensor(out) and id(out) in producer:
        lines.append('  "output" [label="output\\n%s"];' % (tuple(out.shape),))
        lines.append('  "%s" -> "output";' % producer[id(out)])
    lines.append("}")
    return "\n".join(lines) + "\n"
