"""Process-group rendezvous for the multi-process tests: through a file, not a TCP port.

A port found free by bind-and-close can be taken by anything (an outgoing connection of another process, a
lingering socket of the previous test) before rank 0 listens on it, and the other ranks then wait out the store's
ten-minute connect timeout.  A fresh file has no such race; the short process-group timeout bounds what is left.
"""
import datetime
import os
import tempfile


def new_token() -> str:
    fd, path = tempfile.mkstemp(prefix="grace_rdzv_")
    os.close(fd)
    os.unlink(path)            # the FileStore wants to create it
    return path


def init_group(backend: str, rank: int, world: int, token: str, device=None, timeout_s: float = 180.0):
    import torch.distributed as dist

    kw = {"device_id": device} if device is not None else {}
    dist.init_process_group(backend, init_method="file://" + token, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
