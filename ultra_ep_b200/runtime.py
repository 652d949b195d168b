"""Process-wide runtime bootstrap: which EP group this process serves and how large its
NVLink domain is. Replaces the reference's NVSHMEM bootstrap (ultra_ep/runtime.py:12-60 of the
reference): torch.distributed is used for the handle exchange only, nothing else."""

from __future__ import annotations

import os

import torch.distributed as dist

from .native import load
from .util import print_rank_0

_group = None
_nvl_domain_size = None


def init_runtime(group: dist.ProcessGroup) -> int:
    """Idempotent per process; returns the NVLink-domain size. All EP managers of a process
    must share one group."""
    global _group, _nvl_domain_size
    _C = load()
    if _C.is_runtime_initialized():
        assert group == _group, "All EP buffers should share the same process group"
        return _nvl_domain_size

    detected = _C.IpcManager().detect_accessible_ranks(group)
    override = os.getenv("MAX_NUM_NVL_PEERS")
    if override is not None:
        peers = int(override)
        if peers != detected:
            print_rank_0(f"[WARN] MAX_NUM_NVL_PEERS={peers} differs from detected value {detected}. "
                         "Using environment variable.")
    else:
        peers = detected
    world = dist.get_world_size(group)
    if peers < world:
        raise RuntimeError(
            f"the EP group has {world} ranks but only {peers} share this rank's NVLink domain; groups spanning "
            "several NVLink domains are not supported by this library")
    peers = world

    def exchange(blob: bytes):
        parts = [None] * world
        dist.all_gather_object(parts, blob, group)
        return parts

    _C.set_handle_exchange(exchange)
    _C.init_runtime(dist.get_rank(group), world, peers, b"")
    _group, _nvl_domain_size = group, peers
    return peers


def shutdown_runtime() -> None:
    """Forget the group (tests that build several groups in one process call this)."""
    global _group, _nvl_domain_size
    load().shutdown_runtime()
    _group = _nvl_domain_size = None
