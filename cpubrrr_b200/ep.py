"""Expert-parallel set-up over torch.distributed: one process per GPU, experts sharded by index.

torch.distributed is only the plumbing (exchange of the 64-byte IPC handles and a barrier); the
per-layer exchange itself happens inside the library's kernels over peer memory."""
import ctypes as C

import numpy as np

from ._lib import check, lib
from .engine import Engine


def expert_range(n_expert, rank, world):
    """Experts [first, first + count) held by `rank` (contiguous blocks, the layout the kernels assume)."""
    if world < 1 or world > 8 or n_expert % world or not 0 <= rank < world:
        raise ValueError(f"cannot shard {n_expert} experts over {world} ranks (rank {rank})")
    per = n_expert // world
    return rank * per, per


def gather_handles(handle, rank, world, dist=None, device=None):
    """All-gather of fixed-size byte strings in rank order.  dist: torch.distributed (already
    initialised) or None for a single rank; device: where the tensors live (CUDA for NCCL)."""
    if world == 1:
        return handle
    import torch
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
    out = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(out, mine)
    return b"".join(bytes(t.cpu().tolist()) for t in out)


def _finish(h, rank, world, dist, device):
    L = lib()
    buf = C.create_string_buffer(64)
    check(L.brrr_model_ep_handle(h, buf), "brrr_model_ep_handle")
    handles = gather_handles(buf.raw, rank, world, dist, device)
    if world > 1:
        dist.barrier()                      # every rank has opened: the first step may wait for the peers
    check(L.brrr_model_ep_attach(h, handles), "brrr_model_ep_attach")
    return Engine(h.value)


def open_synth_ep(cfg, seed, rank, world, device=0, dist=None, torch_device=None):
    """Seeded synthetic model, this rank's experts only; collective over all ranks."""
    expert_range(cfg.n_expert, rank, world)
    h = C.c_void_p()
    check(lib().brrr_model_open_synth_ep(C.byref(cfg), seed, device, rank, world, C.byref(h)), "brrr_model_open_synth_ep")
    return _finish(h, rank, world, dist, torch_device)


def open_ep(data_dir, blob_path, rank, world, device=0, dist=None, torch_device=None):
    h = C.c_void_p()
    check(lib().brrr_model_open_ep(str(data_dir).encode(), str(blob_path).encode(), device, rank, world, C.byref(h)), "brrr_model_open_ep")
    return _finish(h, rank, world, dist, torch_device)
