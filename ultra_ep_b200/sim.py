"""Simulated expert-parallel group: all N ranks of a group hosted on ONE device.

The C-ABI manager runs the same kernels as in the one-rank-per-process case, once for all
hosted ranks (one launch each); "peers" are buffers on the same device, so weight_sync and the
Wgrad reduce are bounded by HBM here, not by NVLink. Used for single-GPU parity tests and for
the single-GPU leg of the benchmark.
"""

from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import capi

_TYPESTR = {torch.int32: "<i4", torch.uint8: "|u1", torch.float32: "<f4"}


class _DeviceView:
    """Minimal __cuda_array_interface__ carrier so torch can wrap memory the library owns."""

    def __init__(self, ptr: int, shape, strides_elems, dtype: torch.dtype):
        item = torch.empty((), dtype=dtype).element_size()
        self.__cuda_array_interface__ = {
            "shape": tuple(int(s) for s in shape),
            "typestr": _TYPESTR[dtype],
            "data": (int(ptr), False),
            "version": 3,
            "strides": tuple(int(s) * item for s in strides_elems),
        }


def wrap_device_memory(ptr: int, shape, strides_elems, dtype: torch.dtype, device) -> torch.Tensor:
    """torch view (no copy, no ownership) of library-owned device memory."""
    if any(int(s) == 0 for s in shape) or ptr == 0:
        return torch.empty(tuple(int(s) for s in shape), dtype=dtype, device=device)
    return torch.as_tensor(_DeviceView(ptr, shape, strides_elems, dtype), device=device)


_BUF_DTYPE = {
    capi.BUF_P2L: torch.int32, capi.BUF_L2P: torch.int32, capi.BUF_LCNTS: torch.int32, capi.BUF_QUOTA: torch.int32,
    capi.BUF_QUOTA_PREFIX: torch.int32, capi.BUF_RANK_QUOTA_PREFIX: torch.int32, capi.BUF_GLOBAL_LOADS: torch.int32,
    capi.BUF_LOADS_PER_RANK: torch.int32, capi.BUF_REPLICA_WEIGHT: torch.uint8, capi.BUF_REPLICA_FC1_WEIGHT: torch.uint8,
    capi.BUF_REPLICA_FC2_WEIGHT: torch.uint8, capi.BUF_REPLICA_SCALE: torch.uint8, capi.BUF_REPLICA_FC1_SCALE: torch.uint8,
    capi.BUF_REPLICA_FC2_SCALE: torch.uint8, capi.BUF_REPLICA_GRAD: torch.float32,
    capi.BUF_REPLICA_FC1_GRAD: torch.float32, capi.BUF_REPLICA_FC2_GRAD: torch.float32,
    capi.BUF_PHYSICAL_LOADS: torch.int32,
}


def manager_buffer(handle, local_rank: int, buffer_id: int, device) -> torch.Tensor:
    L = capi.lib()
    p, nd = C.c_void_p(), C.c_int()
    shape, stride = (C.c_int64 * 3)(), (C.c_int64 * 3)()
    capi.check(L.uep_manager_buffer(handle, local_rank, buffer_id, C.byref(p), C.byref(nd), shape, stride),
               "uep_manager_buffer")
    n = nd.value
    return wrap_device_memory(p.value or 0, list(shape)[:n], list(stride)[:n], _BUF_DTYPE[buffer_id], device)


def make_config(num_ranks: int, masters: int, redundant: int, num_layers: int = 1, *, fc1_numel: int = 0,
                fc2_numel: int = 0, weight_elem_bytes: int = 2, scale_elem_bytes: int = 1, fc1_scale_numel: int = 0,
                fc2_scale_numel: int = 0, is_train: bool = True, rank: int = 0, sim: bool = False,
                solver: Optional[capi.SolverParams] = None, grad_reduce_num_sms: int = 42,
                weight_sync_num_sms: int = 0, wait_timeout_ms: int = 0, plan_mode: int = 0,
                relay_min_replicas: int = 4) -> capi.Config:
    cfg = capi.Config()
    cfg.num_ranks = num_ranks
    cfg.nvl_ranks = num_ranks
    cfg.rank = rank
    cfg.sim_ranks = num_ranks if sim else 0
    cfg.num_layers = num_layers
    cfg.num_local_master_experts = masters
    cfg.num_local_redundant_experts = redundant
    cfg.expert_fc1_numel = fc1_numel
    cfg.expert_fc2_numel = fc2_numel
    cfg.weight_data_element_bytes = weight_elem_bytes
    cfg.weight_scale_element_bytes = scale_elem_bytes
    cfg.expert_fc1_weight_scale_numel = fc1_scale_numel
    cfg.expert_fc2_weight_scale_numel = fc2_scale_numel
    cfg.grad_element_bytes = 4
    cfg.is_train = int(is_train)
    cfg.legacy_placement = 0
    cfg.solver = solver or capi.SolverParams.defaults()
    cfg.quota_kernel_stage = 1
    cfg.grad_reduce_num_sms = grad_reduce_num_sms
    cfg.grad_reduce_deterministic = 1
    cfg.weight_sync_plan_mode = plan_mode
    cfg.weight_sync_relay_min_replicas = relay_min_replicas
    cfg.weight_sync_relay_max_relays = 8
    cfg.weight_sync_relay_min_fanout_gain = 2
    cfg.weight_sync_num_sms = weight_sync_num_sms
    cfg.wait_timeout_ms = wait_timeout_ms
    return cfg


class SimGroup:
    """All ranks of one EP group on the current CUDA device, driven through the C ABI."""

    PLAN_BUFFERS = {"p2l": capi.BUF_P2L, "l2p": capi.BUF_L2P, "lcnts": capi.BUF_LCNTS, "quota": capi.BUF_QUOTA,
                    "quota_prefix": capi.BUF_QUOTA_PREFIX, "rank_quota_prefix": capi.BUF_RANK_QUOTA_PREFIX}

    def __init__(self, cfg: capi.Config):
        if not torch.cuda.is_available():
            raise capi.UepError("a CUDA device is required; there is no CPU implementation of this library")
        self.lib = capi.lib()
        self.cfg = cfg
        self.N = cfg.num_ranks
        self.M = cfg.num_local_master_experts
        self.R = cfg.num_local_redundant_experts
        self.L = self.N * self.M
        self.P = self.N * (self.M + self.R)
        self.device = torch.device("cuda", torch.cuda.current_device())
        h = C.c_void_p()
        capi.check(self.lib.uep_manager_create(C.byref(cfg), C.byref(h)), "uep_manager_create")
        self.handle = h
        self._connect()
        self.nlocal = self.lib.uep_manager_num_local(self.handle)
        self._keep = []  # pointer tables of the latest calls (must outlive the launches)

    def _connect(self):
        assert self.cfg.sim_ranks == self.cfg.num_ranks
        capi.check(self.lib.uep_manager_connect(self.handle, None), "uep_manager_connect")

    # -- buffers ---------------------------------------------------------------------
    def buffer(self, rank: int, buffer_id: int) -> torch.Tensor:
        return manager_buffer(self.handle, rank, buffer_id, self.device)

    def plan(self, rank: int, layer: int) -> dict:
        return {k: self.buffer(rank, b)[layer] for k, b in self.PLAN_BUFFERS.items()}

    # -- operations ------------------------------------------------------------------
    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def update_placement(self, layer: int, inputs: Sequence[torch.Tensor]):
        """inputs[r]: bool [T,L] routing map, or int32/int64 [T,K] ids, of rank r."""
        x0 = inputs[0]
        kind = 0 if x0.dtype == torch.bool else (1 if x0.dtype == torch.int32 else 2)
        ptrs = capi.ptr_array([x.data_ptr() for x in inputs])
        Ts = capi.int_array([int(x.shape[0]) for x in inputs])
        capi.check(self.lib.uep_update_placement(self.handle, layer, kind, ptrs, Ts, int(x0.shape[1]), self._stream()),
                   "uep_update_placement")

    def pointer_tables(self, tensors_per_rank: Sequence[Sequence[torch.Tensor]]) -> List[torch.Tensor]:
        """int64 device tables of raw addresses, one per rank (what construct_local_master_ptr_pool builds)."""
        return [torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=self.device)
                for ts in tensors_per_rank]

    def weight_sync(self, layer: int, fc1_tables, fc2_tables, fc1_scale_tables=None, fc2_scale_tables=None,
                    async_finish: bool = False):
        args = [capi.ptr_array([t.data_ptr() for t in tabs]) if tabs is not None else None
                for tabs in (fc1_tables, fc2_tables, fc1_scale_tables, fc2_scale_tables)]
        self._keep = [fc1_tables, fc2_tables, fc1_scale_tables, fc2_scale_tables]
        done = C.c_void_p()
        capi.check(self.lib.uep_weight_sync(self.handle, layer, args[0], args[1], args[2], args[3], None,
                                            int(async_finish), self._stream(), C.byref(done)), "uep_weight_sync")
        return done if async_finish else None

    def grad_reduce(self, layer: int, fc1_grad_tables, fc2_grad_tables, async_finish: bool = False):
        a = capi.ptr_array([t.data_ptr() for t in fc1_grad_tables])
        b = capi.ptr_array([t.data_ptr() for t in fc2_grad_tables])
        self._keep = [fc1_grad_tables, fc2_grad_tables]
        done = C.c_void_p()
        capi.check(self.lib.uep_grad_reduce(self.handle, layer, a, b, None, int(async_finish), self._stream(),
                                            C.byref(done)), "uep_grad_reduce")
        return done if async_finish else None

    def wait_event(self, ev):
        capi.check(self.lib.uep_event_stream_wait(ev, self._stream()), "uep_event_stream_wait")
        self.lib.uep_event_destroy(ev)

    def reroute_sparse(self, layer: int, ids: Sequence[torch.Tensor], out: Optional[Sequence[torch.Tensor]] = None):
        out = [torch.empty_like(x) for x in ids] if out is None else out
        kind = 1 if ids[0].dtype == torch.int32 else 2
        capi.check(self.lib.uep_reroute_sparse(
            self.handle, layer, kind, capi.ptr_array([x.data_ptr() for x in ids]),
            capi.ptr_array([x.data_ptr() for x in out]), capi.int_array([int(x.shape[0]) for x in ids]),
            int(ids[0].shape[1]), self._stream()), "uep_reroute_sparse")
        return out

    def reroute_dense(self, layer: int, maps: Sequence[torch.Tensor], probs: Sequence[torch.Tensor], out=None):
        """out: optional (out_probs, out_maps) lists to write into instead of allocating."""
        if out is None:
            out_maps = [torch.empty((m.shape[0], self.P), dtype=torch.bool, device=self.device) for m in maps]
            out_probs = [torch.empty((m.shape[0], self.P), dtype=torch.float32, device=self.device) for m in maps]
        else:
            out_probs, out_maps = out
        capi.check(self.lib.uep_reroute_dense_forward(
            self.handle, layer, capi.ptr_array([x.data_ptr() for x in maps]),
            capi.ptr_array([x.data_ptr() for x in probs]), capi.ptr_array([x.data_ptr() for x in out_maps]),
            capi.ptr_array([x.data_ptr() for x in out_probs]), capi.int_array([int(x.shape[0]) for x in maps]),
            self._stream()), "uep_reroute_dense_forward")
        return out_probs, out_maps

    def reroute_dense_backward(self, layer: int, grads, maps, expanded_maps):
        outs = [torch.empty((m.shape[0], self.L), dtype=torch.float32, device=self.device) for m in maps]
        capi.check(self.lib.uep_reroute_dense_backward(
            self.handle, layer, capi.ptr_array([x.data_ptr() for x in grads]),
            capi.ptr_array([x.data_ptr() for x in maps]), capi.ptr_array([x.data_ptr() for x in expanded_maps]),
            capi.ptr_array([x.data_ptr() for x in outs]), capi.int_array([int(x.shape[0]) for x in maps]), self.P,
            self._stream()), "uep_reroute_dense_backward")
        return outs

    def status(self, rank: int = 0):
        code, detail = C.c_int(), C.c_int()
        self.lib.uep_poll_status(self.handle, rank, C.byref(code), C.byref(detail))
        return code.value, detail.value

    def check_status(self):
        for r in range(self.nlocal):
            code, detail = self.status(r)
            if code != 0:
                raise capi.UepError(f"rank {r}: device status {code} ({capi.DEV_STATUS_NAMES.get(code, '?')}), "
                                    f"detail {detail}")

    def comm_stream(self) -> torch.cuda.Stream:
        return torch.cuda.ExternalStream(self.lib.uep_manager_comm_stream(self.handle), device=self.device)

    def destroy(self):
        if self.handle:
            capi.check(self.lib.uep_manager_destroy(self.handle), "uep_manager_destroy")
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class IpcGroup(SimGroup):
    """One rank of a multi-process group (one process per GPU). The 64-byte cudaIpc handles of
    the peer-visible arenas are all-gathered through the given torch.distributed group, which is
    the only thing that group is used for. Per-call lists have one element: this rank's tensor."""

    def __init__(self, cfg: capi.Config, group=None):
        import torch.distributed as dist

        self._dist = dist
        self._pg = group
        assert cfg.sim_ranks == 0
        super().__init__(cfg)

    def _connect(self):
        dist = self._dist
        handle = torch.zeros(capi.IPC_HANDLE_BYTES, dtype=torch.uint8)
        capi.check(self.lib.uep_manager_export_handle(self.handle, handle.data_ptr()), "uep_manager_export_handle")
        world = dist.get_world_size(self._pg)
        backend = dist.get_backend(self._pg)
        send = handle.to(self.device) if backend == "nccl" else handle
        gathered = [torch.empty_like(send) for _ in range(world)]
        dist.all_gather(gathered, send, group=self._pg)
        blob = torch.stack([g.cpu() for g in gathered]).contiguous()
        capi.check(self.lib.uep_manager_connect(self.handle, blob.data_ptr()), "uep_manager_connect")
        dist.barrier(group=self._pg)  # every rank has mapped every arena before the first kernel

    def destroy(self):
        if self.handle:
            torch.cuda.synchronize()
            self._dist.barrier(group=self._pg)  # nobody unmaps while a peer may still write
            super().destroy()
