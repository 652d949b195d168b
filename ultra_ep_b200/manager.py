"""`Manager`: the per-EP-group object a framework's MoE layer talks to.

Drop-in for the reference's ultra_ep.Manager (ultra_ep/manager.py:18-770 of the reference): same
constructor arguments, methods, properties, buffer attributes and virtual-layer arithmetic.
Differences: the expert-load trace (ULTRA_EP_LOAD_PROFILING) is recorded when the plan is made,
from the per-slot loads the plan kernel writes itself, instead of by a separate kernel at reroute
time (same trace files); its viewer is not part of this library; legacy_placement=True runs its counts-only greedy
solver as a kernel (same results as the reference's host-side solver, no host round trip).
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .config import load_tuning_from_env
from .event import EventHandle
from .native import load
from .profiling import ExpertLoadProfiler, load_profile_config
from .reroute import _DenseRerouteFunction
from .runtime import init_runtime
from .util import check_dtype, dtype_element_size


class Manager:
    def __init__(
        self,
        group: dist.ProcessGroup,
        num_layers: int,
        num_local_master_experts: int,
        num_local_redundant_experts: int,
        expert_fc1_numel: int,
        expert_fc2_numel: int,
        is_train: bool = True,
        explicitly_destroy: bool = False,
        max_microbatches: int = 1,
        legacy_placement: bool = False,
        weight_data_dtype: torch.dtype = torch.bfloat16,
        weight_scale_dtype: torch.dtype = torch.float32,
        expert_fc1_weight_scale_numel: int = 0,
        expert_fc2_weight_scale_numel: int = 0,
        grad_dtype: torch.dtype = torch.float32,
    ):
        if legacy_placement and load_profile_config().enabled:
            raise AssertionError("UltraEP load profiling is only supported by quota placement; "
                                 "disable ULTRA_EP_LOAD_PROFILING or legacy_placement.")
        _C = load()
        self.nvl_domain_size = init_runtime(group)
        self.group = group
        self.id = id(group)
        self.device = torch.cuda.current_device()
        self.rank = group.rank()
        self.num_ranks = group.size()

        self.num_layers = num_layers
        self.num_local_master_experts = num_local_master_experts
        self.num_local_redundant_experts = num_local_redundant_experts
        self.expert_fc1_numel = expert_fc1_numel
        self.expert_fc2_numel = expert_fc2_numel
        self.expert_total_numel = expert_fc1_numel + expert_fc2_numel
        self.expert_fc1_weight_scale_numel = expert_fc1_weight_scale_numel
        self.expert_fc2_weight_scale_numel = expert_fc2_weight_scale_numel
        self.expert_weight_scale_total_numel = expert_fc1_weight_scale_numel + expert_fc2_weight_scale_numel
        self.weight_data_dtype = check_dtype("weight_data_dtype", weight_data_dtype)
        self.weight_scale_dtype = check_dtype("weight_scale_dtype", weight_scale_dtype)
        self.grad_dtype = check_dtype("grad_dtype", grad_dtype)
        if self.grad_dtype is not torch.float32:
            raise ValueError("UltraEP currently supports only fp32 gradients")
        self.weight_data_element_bytes = dtype_element_size(self.weight_data_dtype)
        self.weight_scale_element_bytes = dtype_element_size(self.weight_scale_dtype)
        self.grad_element_bytes = dtype_element_size(self.grad_dtype)
        self.num_local_physical_experts = num_local_master_experts + num_local_redundant_experts
        self.num_global_physical_experts = self.num_local_physical_experts * self.num_ranks
        self.num_global_logical_experts = num_local_master_experts * self.num_ranks
        self.is_train = is_train

        # Several microbatches of one layer can be in flight under pipeline parallelism: every
        # (real layer, microbatch slot) pair owns a "virtual layer" with its own plan storage.
        self.max_microbatches = max(1, max_microbatches)
        self.real_num_alloc_layers = num_layers + 3  # room for 1-based layer ids
        self.num_alloc_layers = self.real_num_alloc_layers * self.max_microbatches
        n = self.real_num_alloc_layers
        self.local_master_fc1_weight_ptr_pool = [None] * n
        self.local_master_fc2_weight_ptr_pool = [None] * n
        self.local_master_fc1_weight_scale_ptr_pool = [None] * n
        self.local_master_fc2_weight_scale_ptr_pool = [None] * n
        self.local_master_fc1_grad_ptr_pool = [None] * n
        self.local_master_fc2_grad_ptr_pool = [None] * n
        self._mb_counters = [0] * n

        tuning = load_tuning_from_env()
        self.grad_reduce_num_sms = tuning.grad_reduce_num_sms
        self.grad_reduce_deterministic = tuning.grad_reduce_deterministic
        self.explicitly_destroy = explicitly_destroy
        self.legacy_placement = legacy_placement
        self.quota_kernel_stage = tuning.quota_kernel_stage
        self.quota_reroute_interleave = tuning.quota_reroute_interleave
        plan_mode, plan_mode_id = tuning.weight_sync_plan_mode, tuning.weight_sync_plan_mode_id
        # The reference forces the direct fan-out when the NVLink domain has at most 8 ranks, because its relay is a
        # second stage with its own launches. Here relaying is scatter + replica-to-replica forward inside the one
        # copy kernel and the adaptive mode only relays what relieves the busiest sender of the layer's plan, so the
        # default (adaptive) stays adaptive at any domain size.
        self.weight_sync_plan_mode = plan_mode
        self.weight_sync_relay_min_replicas = tuning.weight_sync_relay_min_replicas
        self.weight_sync_relay_max_relays = tuning.weight_sync_relay_max_relays
        self.weight_sync_relay_min_fanout_gain = tuning.weight_sync_relay_min_fanout_gain
        self.reroute_mode = "round_robin" if legacy_placement else "quota"
        self.runtime = _C.Manager(
            self.num_alloc_layers, num_local_master_experts, num_local_redundant_experts, expert_fc1_numel,
            expert_fc2_numel, self.weight_data_element_bytes, self.weight_scale_element_bytes,
            expert_fc1_weight_scale_numel, expert_fc2_weight_scale_numel, self.grad_element_bytes, is_train,
            explicitly_destroy, legacy_placement, tuning.balance_threshold, tuning.quota_locality_aware,
            tuning.quota_min_tokens_per_replica, tuning.quota_allow_zero_master_quota, tuning.quota_oracle_eps,
            tuning.quota_kernel_stage, tuning.quota_reroute_interleave, self.grad_reduce_num_sms,
            self.grad_reduce_deterministic, plan_mode_id, tuning.weight_sync_relay_min_replicas,
            tuning.weight_sync_relay_max_relays, tuning.weight_sync_relay_min_fanout_gain)
        assert self.runtime.is_available()

        rt = self.runtime
        self._physical_to_logical_map = rt.get_physical_to_logical_map_tensor()
        self._logical_to_physical_map = rt.get_logical_to_physical_map_tensor()
        self._logical_replica_counts = rt.get_logical_replica_counts_tensor()
        self._logical_instance_quota = rt.get_logical_instance_quota_tensor()
        self._logical_instance_quota_prefix = rt.get_logical_instance_quota_prefix_tensor()
        self._rank_quota_prefix = rt.get_rank_quota_prefix_tensor()

        R = num_local_redundant_experts
        # Full buffers keep one contiguous row per replica slot; the fc1 / fc2 tensors are strided
        # views into them (each row contiguous, rows at the full-expert stride).
        self.local_replica_weight_buffer = (
            rt.get_local_replica_weight_buffer_tensor().view(self.weight_data_dtype).view(R, self.expert_total_numel))
        self.local_replica_fc1_weight_buffer = (
            rt.get_local_replica_fc1_weight_buffer_tensor().view(self.weight_data_dtype).view(R, expert_fc1_numel))
        self.local_replica_fc2_weight_buffer = (
            rt.get_local_replica_fc2_weight_buffer_tensor().view(self.weight_data_dtype).view(R, expert_fc2_numel))
        self.local_replica_weight_scale_buffer_raw = rt.get_local_replica_weight_scale_buffer_tensor()
        raw1 = rt.get_local_replica_fc1_weight_scale_buffer_tensor()
        raw2 = rt.get_local_replica_fc2_weight_scale_buffer_tensor()
        if self.expert_weight_scale_total_numel > 0:
            self.local_replica_fc1_weight_scale_buffer = raw1.view(self.weight_scale_dtype).view(
                R, expert_fc1_weight_scale_numel)
            self.local_replica_fc2_weight_scale_buffer = raw2.view(self.weight_scale_dtype).view(
                R, expert_fc2_weight_scale_numel)
        else:
            self.local_replica_fc1_weight_scale_buffer = torch.empty((R, 0), dtype=self.weight_scale_dtype,
                                                                     device=raw1.device)
            self.local_replica_fc2_weight_scale_buffer = torch.empty((R, 0), dtype=self.weight_scale_dtype,
                                                                     device=raw2.device)
        if self.is_train:
            self.local_replica_grad_buffer = rt.get_local_replica_grad_buffer_tensor()
            self.local_replica_fc1_grad_buffer = rt.get_local_replica_fc1_grad_buffer_tensor()
            self.local_replica_fc2_grad_buffer = rt.get_local_replica_fc2_grad_buffer_tensor()
        else:
            self.local_replica_grad_buffer = None
            self.local_replica_fc1_grad_buffer = None
            self.local_replica_fc2_grad_buffer = None
        self.check_tensors_blob_from_cpp()
        self._physical_expert_loads = rt.get_physical_expert_loads_tensor()
        self._load_profiler = ExpertLoadProfiler(
            config=load_profile_config(),
            group_rank=self.rank,
            global_rank=dist.get_rank() if dist.is_initialized() else self.rank,
            metadata={
                "ep_group_id": f"{self.id:x}", "ep_rank": self.rank, "ep_size": self.num_ranks,
                "num_layers": self.num_layers, "max_microbatches": self.max_microbatches,
                "num_local_master_experts": self.num_local_master_experts,
                "num_local_redundant_experts": self.num_local_redundant_experts,
                "num_local_physical_experts": self.num_local_physical_experts,
                "num_global_logical_experts": self.num_global_logical_experts,
                "num_global_physical_experts": self.num_global_physical_experts,
                "nvl_domain_size": self.nvl_domain_size, "placement_mode": self.reroute_mode,
            },
            num_logical=self.num_global_logical_experts, num_physical=self.num_global_physical_experts)

    # -- plan maps (device resident, all virtual layers) -----------------------------------
    @property
    def physical_to_logical_map(self) -> torch.Tensor:
        return self._physical_to_logical_map

    @property
    def logical_to_physical_map(self) -> torch.Tensor:
        return self._logical_to_physical_map

    @property
    def logical_replica_counts(self) -> torch.Tensor:
        return self._logical_replica_counts

    @property
    def logical_instance_quota(self) -> torch.Tensor:
        return self._logical_instance_quota

    @property
    def logical_instance_quota_prefix(self) -> torch.Tensor:
        return self._logical_instance_quota_prefix

    @property
    def rank_quota_prefix(self) -> torch.Tensor:
        return self._rank_quota_prefix

    def get_quota_tensor(self, layer_id: int) -> torch.Tensor:
        return self._logical_instance_quota[layer_id]

    def get_quota_prefix_tensor(self, layer_id: int) -> torch.Tensor:
        return self._logical_instance_quota_prefix[layer_id]

    def get_rank_quota_prefix_tensor(self, layer_id: int) -> torch.Tensor:
        return self._rank_quota_prefix[layer_id]

    def destroy(self):
        assert self.explicitly_destroy
        self._teardown()

    def _teardown(self) -> bool:
        """Collective release of the native resources: every rank first finishes its own work and then
        waits for all the others, because the peers hold mappings of this rank's arena and their kernels store
        into it; only then is it freed. Returns False (and frees nothing) when the barrier cannot be made, e.g.
        because the process group is gone: the native layer then keeps the arena until the process exits rather
        than free memory a peer may still write."""
        if self.runtime is None:
            return True
        try:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dist.barrier(group=self.group)  # no peer may still be writing into this rank's slots
        except Exception as e:  # group destroyed, interpreter shutting down, ...
            print(f"UltraEP: manager teardown without a group barrier ({type(e).__name__}); the peer-visible "
                  "memory is kept until the process exits", flush=True)
            abandon = getattr(self.runtime, "abandon", None)
            if abandon is not None:
                abandon()
            self.runtime = None
            return False
        self._load_profiler.close()
        self.runtime.destroy()
        self.runtime = None
        return True

    def __del__(self):
        # explicitly_destroy=False: the same ordered release when the last reference goes (every rank drops its
        # manager at the same point of the program, as with the reference's destructor-side barrier)
        try:
            if getattr(self, "runtime", None) is not None and not self.explicitly_destroy:
                self._teardown()
        except Exception:
            pass

    # -- virtual layers --------------------------------------------------------------------
    def allocate_microbatch_slot(self, real_layer_id: int) -> int:
        """Next virtual layer id of a real layer: real * max_microbatches + (counter mod max_microbatches)."""
        assert real_layer_id < self.real_num_alloc_layers
        slot = self._mb_counters[real_layer_id] % self.max_microbatches
        self._mb_counters[real_layer_id] += 1
        return real_layer_id * self.max_microbatches + slot

    def _real_layer_id(self, virtual_layer_id: int) -> int:
        return virtual_layer_id // self.max_microbatches

    # -- master pointer pools ----------------------------------------------------------------
    def construct_local_master_ptr_pool(
        self,
        layer_id: int,
        fc1_weights: List[torch.Tensor],
        fc2_weights: List[torch.Tensor],
        fc1_grads: Optional[List[torch.Tensor]] = None,
        fc2_grads: Optional[List[torch.Tensor]] = None,
        fc1_weight_scales: Optional[List[torch.Tensor]] = None,
        fc2_weight_scales: Optional[List[torch.Tensor]] = None,
    ):
        M = self.num_local_master_experts
        assert layer_id < self.real_num_alloc_layers
        assert len(fc1_weights) == M and len(fc2_weights) == M
        device = torch.device("cuda", self.device)

        def table(tensors, dtype):
            for t in tensors:
                assert t.dtype == dtype, f"Expected weight/grad dtype {dtype}, got {t.dtype}"
            return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device).contiguous()

        self.local_master_fc1_weight_ptr_pool[layer_id] = table(fc1_weights, self.weight_data_dtype)
        self.local_master_fc2_weight_ptr_pool[layer_id] = table(fc2_weights, self.weight_data_dtype)
        if self.expert_weight_scale_total_numel > 0:
            if fc1_weight_scales is None or fc2_weight_scales is None:
                raise AssertionError("Weight scale tensors are required when scale numel is non-zero")
            assert len(fc1_weight_scales) == M and len(fc2_weight_scales) == M
            self.local_master_fc1_weight_scale_ptr_pool[layer_id] = table(fc1_weight_scales, self.weight_scale_dtype)
            self.local_master_fc2_weight_scale_ptr_pool[layer_id] = table(fc2_weight_scales, self.weight_scale_dtype)
        else:
            empty = torch.empty(0, dtype=torch.int64, device=device)
            self.local_master_fc1_weight_scale_ptr_pool[layer_id] = empty
            self.local_master_fc2_weight_scale_ptr_pool[layer_id] = empty
        if self.is_train:
            assert fc1_grads is not None and fc2_grads is not None, "Grad tensors required in training mode"
            assert len(fc1_grads) == M and len(fc2_grads) == M
            self.local_master_fc1_grad_ptr_pool[layer_id] = table(fc1_grads, self.grad_dtype)
            self.local_master_fc2_grad_ptr_pool[layer_id] = table(fc2_grads, self.grad_dtype)

    # -- hot path --------------------------------------------------------------------------
    def grad_reduce(self, layer_id: int, previous_event: Optional[EventHandle] = None, async_finish: bool = False):
        """Sum replica gradients into the masters (fp32, fixed order) and zero the replicas.
        `layer_id` is the virtual id; pointer pools are looked up by the real layer."""
        assert layer_id < self.num_alloc_layers
        real = self._real_layer_id(layer_id)
        assert self.local_master_fc1_grad_ptr_pool[real] is not None and self.local_master_fc2_grad_ptr_pool[real] is not None
        event = self.runtime.grad_reduce(layer_id, self.local_master_fc1_grad_ptr_pool[real],
                                         self.local_master_fc2_grad_ptr_pool[real],
                                         getattr(previous_event, "event", None), async_finish)
        return EventHandle(event)

    def weight_sync(self, layer_id: int, previous_event: Optional[EventHandle] = None, async_finish: bool = False):
        """Push every replicated local master into its peers' replica slots, using the plan stored
        under the virtual layer id. Returns an EventHandle (its event is None when synchronous)."""
        assert layer_id < self.num_alloc_layers
        real = self._real_layer_id(layer_id)
        assert (self.local_master_fc1_weight_ptr_pool[real] is not None
                and self.local_master_fc2_weight_ptr_pool[real] is not None
                and self.local_master_fc1_weight_scale_ptr_pool[real] is not None
                and self.local_master_fc2_weight_scale_ptr_pool[real] is not None)
        with torch.cuda.nvtx.range(f"Launch weight_sync (layer {layer_id})"):
            event = self.runtime.weight_sync(
                layer_id, self.local_master_fc1_weight_ptr_pool[real], self.local_master_fc2_weight_ptr_pool[real],
                self.local_master_fc1_weight_scale_ptr_pool[real], self.local_master_fc2_weight_scale_ptr_pool[real],
                getattr(previous_event, "event", None), async_finish)
        return EventHandle(event)

    def set_weight_sync_plan_mode(self, plan_mode: str):
        key = plan_mode.lower().replace("_", "")
        ids = {"direct": 0, "adaptive": 1, "adaptiverelay": 1, "forcerelay": 2}
        if key not in ids:
            raise ValueError("plan_mode must be one of: direct, adaptive_relay, force_relay")
        self.weight_sync_plan_mode = key
        self.runtime.set_weight_sync_plan_mode(ids[key])

    def set_grad_reduce_deterministic(self, deterministic: bool):
        self.grad_reduce_deterministic = bool(deterministic)
        self.runtime.set_grad_reduce_deterministic(self.grad_reduce_deterministic, self.grad_reduce_num_sms)

    def update_placement(self, layer_id: int, routing_map: torch.Tensor, verify_reduced_loads: bool = False):
        """New replication plan of one virtual layer from this microbatch's routing.
        routing_map: bool [tokens, logical experts]. Collective; every rank derives the same plan."""
        assert layer_id < self.num_alloc_layers
        with torch.cuda.nvtx.range(f"Update placement (layer {layer_id})"):
            self.runtime.update_placement(layer_id, routing_map)
        self._record_loads(layer_id)
        if verify_reduced_loads:
            loads = routing_map.sum(dim=0, dtype=torch.int32)
            dist.all_reduce(loads, group=self.group)
            assert torch.equal(loads, self.runtime.get_global_logical_expert_loads_tensor())

    def update_placement_sparse(self, layer_id: int, topk_ids: torch.Tensor):
        """Same from top-k ids [tokens, k] (int64, or int32); runs on the communication stream."""
        assert layer_id < self.num_alloc_layers
        self.runtime.update_placement_sparse(layer_id, topk_ids)
        if self._load_profiler.enabled:
            with torch.cuda.stream(self.get_comm_stream()):
                self._record_loads(layer_id)

    def _record_loads(self, layer_id: int):
        """Expert-load trace: loads before balancing (logical) and after it (physical slots)."""
        if self._load_profiler.enabled:
            self._load_profiler.record(layer_id, self._real_layer_id(layer_id),
                                       self.runtime.get_global_logical_expert_loads_tensor(),
                                       self._physical_expert_loads[layer_id])

    def _profile_physical_loads_from_quota(self, layer_id: int, fused: bool = True) -> torch.Tensor:
        """Tokens per physical slot under the layer's plan: int32 [physical experts]. The plan kernel
        writes this vector itself; `fused` is accepted for compatibility and has no effect."""
        return self._physical_expert_loads[layer_id]

    def reroute(self, layer_id: int, probs: torch.Tensor, routing_map: torch.Tensor, backend: str = "cuda"):
        """Expand [tokens, logical] probabilities and routing map to [tokens, physical] under this
        rank's quota split of the layer's plan. Differentiable with respect to probs."""
        if backend != "cuda":
            raise ValueError("Only backend='cuda' is supported; CPU reroute has been removed")
        if self.is_train and probs.requires_grad:
            return _DenseRerouteFunction.apply(probs, routing_map, self.runtime, layer_id)
        with torch.cuda.nvtx.range(f"Dense reroute forward (layer {layer_id})"):
            return self.runtime.dense_reroute_forward(layer_id, probs, routing_map)

    def reroute_sparse(self, layer_id: int, topk_ids: torch.Tensor):
        """In place: logical ids [tokens, k] -> physical ids (deterministic, row-major ordinals)."""
        assert layer_id < self.num_alloc_layers
        self.runtime.reroute_sparse(layer_id, topk_ids)

    def check_status(self):
        """Raise if a kernel of this manager reported an error (e.g. a peer wait ran out)."""
        code, detail = self.runtime.poll_status()
        if code != 0:
            raise RuntimeError(f"UltraEP device status {code} (detail {detail})")

    def get_comm_stream(self) -> torch.Stream:
        ts = self.runtime.get_comm_stream()
        return torch.cuda.Stream(stream_id=ts.stream_id, device_index=ts.device_index, device_type=ts.device_type)

    # -- layout checks of what the native layer hands out --------------------------------------
    def check_tensors_blob_from_cpp(self):
        dev = torch.device("cuda", self.device)
        A, L, P, N, R = (self.num_alloc_layers, self.num_global_logical_experts, self.num_global_physical_experts,
                         self.num_ranks, self.num_local_redundant_experts)
        expect = {
            "_physical_to_logical_map": (A, P), "_logical_to_physical_map": (A, L, N), "_logical_replica_counts": (A, L),
            "_logical_instance_quota": (A, L, N), "_logical_instance_quota_prefix": (A, L, N),
            "_rank_quota_prefix": (A, L, N),
        }
        for name, shape in expect.items():
            t = getattr(self, name)
            assert t.device == dev and t.dtype == torch.int32 and tuple(t.shape) == shape, name
        weights = {
            "local_replica_weight_buffer": self.expert_total_numel,
            "local_replica_fc1_weight_buffer": self.expert_fc1_numel,
            "local_replica_fc2_weight_buffer": self.expert_fc2_numel,
        }
        for name, cols in weights.items():
            t = getattr(self, name)
            assert t.device == dev and t.dtype == self.weight_data_dtype and tuple(t.shape) == (R, cols), name
        raw = self.local_replica_weight_scale_buffer_raw
        assert raw.device == dev and raw.dtype == torch.uint8
        for name, cols in (("local_replica_fc1_weight_scale_buffer", self.expert_fc1_weight_scale_numel),
                           ("local_replica_fc2_weight_scale_buffer", self.expert_fc2_weight_scale_numel)):
            t = getattr(self, name)
            assert t.device == dev and t.dtype == self.weight_scale_dtype and tuple(t.shape) == (R, cols), name
        if self.is_train:
            for name, cols in (("local_replica_grad_buffer", self.expert_total_numel),
                               ("local_replica_fc1_grad_buffer", self.expert_fc1_numel),
                               ("local_replica_fc2_grad_buffer", self.expert_fc2_numel)):
                t = getattr(self, name)
                assert t.device == dev and t.dtype == self.grad_dtype and tuple(t.shape) == (R, cols), name
