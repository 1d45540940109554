"""Tensor-parallel plumbing: torch.distributed carries the NCCL unique id and the
IPC handles between the ranks; the data path (all-reduce of partial sums, logits
all-gather) runs inside libtorchburn_b200.so."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import ALLGATHER_FN, check, lib


def init_tensor_parallel(decoder, dist, device=None, fused: bool = True) -> None:
    """Joins `decoder` (created with tp_size = dist.get_world_size(), tp_rank =
    dist.get_rank()) to its communicator.  Collective over the default process group.

    dist: the torch.distributed module with an initialised process group ("nccl" on
    GPUs).  fused=False keeps every all-reduce on ncclAllReduce."""
    import torch

    rank, world = dist.get_rank(), dist.get_world_size()
    on_gpu = dist.get_backend() == "nccl"
    dev = device if (on_gpu and device is not None) else (torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu"))
    uid = np.zeros(128, np.uint8)
    if rank == 0:
        check(lib().tb_tp_unique_id(uid.ctypes.data))
    t = torch.from_numpy(uid).to(dev)
    dist.broadcast(t, src=0)
    uid = t.cpu().numpy().copy()

    def allgather(_user, send, recv, nbytes):
        try:
            mine = torch.from_numpy(np.ctypeslib.as_array(C.cast(send, C.POINTER(C.c_uint8)), (nbytes,)).copy()).to(dev)
            outs = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(outs, mine)
            flat = torch.cat(outs).cpu().numpy()
            C.memmove(recv, flat.ctypes.data, nbytes * world)
            return 0
        except Exception:  # reported through the C ABI as TB_ERR_NCCL
            return 1

    cb = ALLGATHER_FN(allgather) if fused else C.cast(None, ALLGATHER_FN)
    check(lib().tb_decoder_tp_init(decoder.handle, uid.ctypes.data, cb, None))
    decoder._tp_callback = cb  # keep alive
