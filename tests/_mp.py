"""Spawns `world` processes that form a process group and run a top-level function."""
import os
import tempfile

import torch.multiprocessing as mp


def _entry(rank, fn, world, backend, initfile, args):
    import torch
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if backend == "nccl":
        torch.cuda.set_device(rank)
        dist.init_process_group(
            backend, init_method=f"file://{initfile}", rank=rank, world_size=world, device_id=torch.device("cuda", rank)
        )
    else:
        torch.set_num_threads(2)
        dist.init_process_group(backend, init_method=f"file://{initfile}", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def run_ranks(fn, world, *args, backend="gloo"):
    """Raises if any rank raises."""
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_entry, args=(fn, world, backend, os.path.join(d, "init"), args), nprocs=world, join=True)
