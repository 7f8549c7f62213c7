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
    leaves = {m: n for n, m in model.named_modules() if len(list(m.children())) == 0}
    producer: Dict[int, str] = {id(example_input): "input"}
    nodes: List[Tuple[str, str]] = [("input", "input\\n%s" % (tuple(example_input.shape),))]
    edges: List[Tuple[str, str]] = []
    hooks = []

    def hook(mod, inputs, output):
        node = leaves[mod]
        srcs = []
        for t in inputs:
            if torch.is_tensor(t):
                srcs.append(producer.get(id(t), None))
        nparams = sum(p.numel() for p in mod.parameters(recurse=False))
        label = "%s\\n%s" % (node, type(mod).__name__)
        if nparams:
            label += "\\n%d params" % nparams
        if torch.is_tensor(output):
            label += "\\n%s" % (tuple(output.shape),)
            producer[id(output)] = node
        nodes.append((node, label))
        for s in srcs:
            edges.append((s if s is not None else "(op)", node))

    for m in leaves:
        hooks.append(m.register_forward_hook(hook))
    was_training = model.training
    model.eval()
    keep = []  # keep intermediate tensors alive so that ids stay unique during the trace

    def keeper(mod, inputs, output):
        keep.append(output)

    for m in leaves:
        hooks.append(m.register_forward_hook(keeper))
    try:
        with torch.no_grad():
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
    if any(s == "(op)" for s, _ in edges):
        lines.append('  "(op)" [label="tensor op\\n(add / view / ...)", shape=ellipse];')
    for s, d in edges:
        lines.append('  "%s" -> "%s";' % (s, d))
    if torch.is_tensor(out) and id(out) in producer:
        lines.append('  "output" [label="output\\n%s"];' % (tuple(out.shape),))
        lines.append('  "%s" -> "output";' % producer[id(out)])
    lines.append("}")
    return "\n".join(lines) + "\n"
