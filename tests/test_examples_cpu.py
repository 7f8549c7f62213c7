"""The example scripts run end to end on CPU (single process, and two gloo ranks through torch.distributed.run)."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run(args, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    res = subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return res.stdout


def _torchrun(script, extra=(), nproc=2):
    return ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
            "--master-port", str(_free_port()), script] + list(extra)


def test_manual_loop_example_single_process():
    out = _run(["examples/dist_resnet_manual_loop.py", "--steps", "3", "--batch", "8"])
    assert "loss" in out.lower()


def test_manual_loop_example_host_protocol_two_gloo_ranks():
    out = _run(_torchrun("examples/dist_resnet_manual_loop.py", ["--steps", "6", "--batch", "8", "--host-protocol"]))
    assert "loss" in out.lower() and "compression_ratio" in out


def test_cifar10_fast_example_two_gloo_ranks():
    out = _run(_torchrun("examples/cifar10_fast_dawn.py", ["--epochs", "1", "--train-size", "256", "--test-size", "64",
                                                            "--batch", "64", "--peak-epoch", "0.5", "--compressor", "topk",
                                                            "--memory", "residual", "--communicator", "allgather",
                                                            "--compress-ratio", "0.05"]))
    assert "test acc" in out


def test_distributed_optimizer_example_single_process():
    _run(["examples/distributed_optimizer_mnist.py"])


def test_ddp_hook_example_two_gloo_ranks():
    _run(_torchrun("examples/ddp_hook_example.py"))


def test_native_ops_demo_checks_pass():
    out = _run(["examples/native_ops_demo.py"])
    assert "equals torch.topk: True" in out and "within one level: True" in out
