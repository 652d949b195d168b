"""Expert-load trace: per recorded microbatch, the token count of every logical expert before
balancing and of every physical slot after it.

Same switches, file names and file contents as the reference's profiler
(ultra_ep/profiling.py:25-344 of the reference: ULTRA_EP_LOAD_PROFILING, ULTRA_EP_LOAD_PROFILE_DIR,
ULTRA_EP_LOAD_PROFILE_FLUSH_INTERVAL, ULTRA_EP_LOAD_PROFILE_RECORD_INTERVAL; schema
"ultra_ep_trace_v1": `<trace>.manifest.json` and `<trace>.chunkNNNNNN.npz` with the arrays
metadata, layers, virtual_layers, microbatches, pre_logical_loads, post_physical_loads), so the
reference's viewer reads these traces unchanged.

The mechanism is different. The reference stages the logical loads when the plan is made, runs a
separate kernel over the plan when the tokens are rerouted, and pairs the two copies afterwards.
Here the plan kernel itself writes the per-slot loads next to the plan, so both vectors exist as
soon as update_placement has been issued: one record is two asynchronous copies into a slot of a
pinned ring, closed by one event, and there is nothing to pair. A full ring drops the record
(counted in the manifest) instead of stalling the step.
"""

from __future__ import annotations

import atexit
import json
import queue
import threading
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .util import read_bool_env, read_int_env, read_str_env

SCHEMA = "ultra_ep_trace_v1"
WRITER_GROUP_RANK = 0
RING_SLOTS = 16


@dataclass(frozen=True)
class LoadProfileConfig:
    enabled: bool
    output_dir: Path
    flush_interval: int
    record_interval: int


def load_profile_config() -> LoadProfileConfig:
    flush_interval = read_int_env("ULTRA_EP_LOAD_PROFILE_FLUSH_INTERVAL", 128)
    record_interval = read_int_env("ULTRA_EP_LOAD_PROFILE_RECORD_INTERVAL", 1)
    if flush_interval <= 0:
        raise ValueError("ULTRA_EP_LOAD_PROFILE_FLUSH_INTERVAL must be positive")
    if record_interval <= 0:
        raise ValueError("ULTRA_EP_LOAD_PROFILE_RECORD_INTERVAL must be positive")
    return LoadProfileConfig(
        enabled=read_bool_env("ULTRA_EP_LOAD_PROFILING", False),
        output_dir=Path(read_str_env("ULTRA_EP_LOAD_PROFILE_DIR", "ultra_ep_traces")),
        flush_interval=flush_interval,
        record_interval=record_interval,
    )


class _Ready:
    """Stand-in for a CUDA event when the source tensors live on the host (tests)."""

    def query(self) -> bool:
        return True

    def synchronize(self) -> None:
        return None


class ExpertLoadProfiler:
    """Writes the trace on the group's rank 0; a no-op everywhere else and when switched off."""

    def __init__(self, config: LoadProfileConfig, group_rank: int, global_rank: int, metadata: Dict[str, Any],
                 num_logical: int, num_physical: int):
        self.config = config
        self.enabled = bool(config.enabled) and group_rank == WRITER_GROUP_RANK
        self.metadata = dict(metadata)
        self.trace_id = ""
        self.dropped = 0
        self.chunks_written = 0
        self._closed = False
        self._seen: Dict[int, int] = {}  # real layer -> microbatches seen so far
        if not self.enabled:
            return
        stamp = int(time.time() * 1000)
        self.trace_id = f"epg{metadata['ep_group_id']}_gr{group_rank}_r{global_rank}_{stamp}"
        self.metadata.update({
            "trace_id": self.trace_id, "schema": SCHEMA, "created_unix": time.time(),
            "writer_group_rank": WRITER_GROUP_RANK, "max_pending_records": RING_SLOTS,
            "record_interval": config.record_interval, "flush_interval": config.flush_interval,
        })
        pin = torch.cuda.is_available()
        self._pre = torch.empty((RING_SLOTS, num_logical), dtype=torch.int32, pin_memory=pin)
        self._post = torch.empty((RING_SLOTS, num_physical), dtype=torch.int32, pin_memory=pin)
        self._slot_event: List[Any] = [None] * RING_SLOTS
        self._slot_info: List[Optional[tuple]] = [None] * RING_SLOTS
        self._head = 0   # oldest slot in flight
        self._count = 0  # slots in flight
        self._rows: List[tuple] = []  # harvested (real layer, virtual layer, microbatch, pre, post)
        config.output_dir.mkdir(parents=True, exist_ok=True)
        self._jobs: "queue.Queue" = queue.Queue()
        self._writer_error: Optional[BaseException] = None
        self._writer = threading.Thread(target=self._write_loop, name="ultra_ep_load_profile", daemon=True)
        self._writer.start()
        self._write_manifest()
        atexit.register(self.close)

    # -- recording -----------------------------------------------------------------------------
    def record(self, virtual_layer: int, real_layer: int, pre_logical_loads: torch.Tensor,
               post_physical_loads: torch.Tensor) -> None:
        """Queue one record. The copies are issued on the current stream of the tensors' device,
        behind the kernel that produced them; nothing waits."""
        if not self.enabled or self._closed or self._capturing():
            return
        microbatch = self._seen.get(real_layer, 0)
        self._seen[real_layer] = microbatch + 1
        if microbatch % self.config.record_interval != 0:
            return
        self._harvest()
        if self._count == RING_SLOTS:
            self.dropped += 1
            return
        slot = (self._head + self._count) % RING_SLOTS
        self._pre[slot].copy_(pre_logical_loads.detach().reshape(-1), non_blocking=True)
        self._post[slot].copy_(post_physical_loads.detach().reshape(-1), non_blocking=True)
        if pre_logical_loads.is_cuda:
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(pre_logical_loads.device))
        else:
            event = _Ready()
        self._slot_event[slot] = event
        self._slot_info[slot] = (real_layer, virtual_layer, microbatch)
        self._count += 1

    @staticmethod
    def _capturing() -> bool:
        if not torch.cuda.is_available():
            return False
        try:
            return bool(torch.cuda.is_current_stream_capturing())
        except RuntimeError:
            return False

    def _harvest(self, wait: bool = False) -> None:
        """Move finished ring slots (oldest first, so records stay in issue order) to the row list."""
        while self._count > 0:
            event = self._slot_event[self._head]
            if wait:
                event.synchronize()
            elif not event.query():
                break
            real_layer, virtual_layer, microbatch = self._slot_info[self._head]
            self._rows.append((real_layer, virtual_layer, microbatch, self._pre[self._head].numpy().copy(),
                               self._post[self._head].numpy().copy()))
            self._head = (self._head + 1) % RING_SLOTS
            self._count -= 1
        if len(self._rows) >= self.config.flush_interval or (wait and self._rows):
            self._submit_chunk()
        self._raise_writer_error()

    # -- writing -------------------------------------------------------------------------------
    def _submit_chunk(self) -> None:
        rows, self._rows = self._rows, []
        self._jobs.put((self.chunks_written, self.dropped, rows))
        self.chunks_written += 1

    def _write_loop(self) -> None:
        while True:
            job = self._jobs.get()
            if job is None:
                return
            try:
                self._write_chunk(*job)
            except BaseException as exc:  # surfaced on the recording thread
                self._writer_error = exc

    def _write_chunk(self, chunk_id: int, dropped: int, rows: List[tuple]) -> None:
        meta = dict(self.metadata, chunk_id=chunk_id, records=len(rows), dropped_records=dropped)
        path = self.config.output_dir / f"{self.trace_id}.chunk{chunk_id:06d}.npz"
        tmp = path.with_suffix(".npz.tmp")
        with tmp.open("wb") as handle:
            np.savez(
                handle,
                metadata=np.asarray(json.dumps(meta, separators=(",", ":"))),
                layers=np.asarray([r[0] for r in rows], dtype=np.int32),
                virtual_layers=np.asarray([r[1] for r in rows], dtype=np.int32),
                microbatches=np.asarray([r[2] for r in rows], dtype=np.int64),
                pre_logical_loads=np.stack([r[3] for r in rows]).astype(np.int32, copy=False),
                post_physical_loads=np.stack([r[4] for r in rows]).astype(np.int32, copy=False),
            )
        tmp.replace(path)

    def _write_manifest(self) -> None:
        manifest = dict(self.metadata, chunks=self.chunks_written, dropped_records=self.dropped)
        path = self.config.output_dir / f"{self.trace_id}.manifest.json"
        tmp = path.with_suffix(".json.tmp")
        tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True))
        tmp.replace(path)

    def _raise_writer_error(self) -> None:
        if self._writer_error is not None:
            exc, self._writer_error = self._writer_error, None
            raise RuntimeError("expert-load trace writer failed") from exc

    def close(self) -> None:
        if self._closed or not self.enabled:
            self._closed = True
            return
        self._closed = True
        self._harvest(wait=True)
        self._jobs.put(None)
        self._writer.join()
        self._raise_writer_error()
        self._write_manifest()
        # Release the pinned ring now, while the CUDA context is alive: torch's pinned-memory pool
        # records an event when such a tensor is freed, which fails once the interpreter is shutting
        # down. Nothing may keep this object (and the ring) alive until then.
        self._pre = self._post = None
        self._slot_event = []
        atexit.unregister(self.close)
