"""CPU-only tests: the library loads and exports every declared symbol, the configuration layer
keeps the reference's variable names / defaults / validation, virtual-layer arithmetic, and the
two-rank bootstrap (gloo) that carries the arena handles between processes."""

import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(native_lib):
    from ultra_ep_b200 import capi

    assert capi.MISSING == []
    header = open(os.path.join(ROOT, "include", "uep_b200.h")).read()
    declared = set(re.findall(r"\b(uep_[a-z0-9_]+)\s*\(", header))
    declared -= {"uep_status"}
    for name in sorted(declared):
        assert hasattr(native_lib, name), f"{name} is declared in include/uep_b200.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature in ultra_ep_b200/capi.py"
    assert native_lib.uep_version().startswith(b"uep_b200")


def test_no_compute_without_gpu_but_clean_errors(native_lib):
    """Argument validation happens on the host and never needs a device."""
    import ctypes as C

    from ultra_ep_b200 import capi

    prm = capi.SolverParams.defaults()
    assert native_lib.uep_solve_placement(None, None, None, None, None, None, None, None, 8, 8, 8, 2, 8, C.byref(prm),
                                          0, None, None) == -1
    assert b"null argument" in native_lib.uep_last_error()
    assert native_lib.uep_manager_create(None, None) == -1
    assert native_lib.uep_reroute_scratch_elems(8192, 8, 128) == 32 * 128 + 4
    assert native_lib.uep_reroute_scratch_elems(8192, 0, 128) == 128 * 128 + 4


def test_tuning_defaults_and_validation(monkeypatch):
    from ultra_ep_b200.config import load_tuning_from_env

    for k in list(os.environ):
        if k.startswith("ULTRA_EP_"):
            monkeypatch.delenv(k)
    t = load_tuning_from_env()
    assert (t.balance_threshold, t.quota_locality_aware, t.quota_min_tokens_per_replica) == (1.0, True, 1024)
    assert (t.quota_allow_zero_master_quota, t.quota_oracle_eps, t.quota_kernel_stage) == (False, 0.01, 1)
    assert (t.quota_reroute_interleave, t.grad_reduce_num_sms, t.grad_reduce_deterministic) == (True, 42, True)
    assert (t.weight_sync_plan_mode, t.weight_sync_plan_mode_id) == ("adaptive", 1)
    assert (t.weight_sync_relay_min_replicas, t.weight_sync_relay_max_relays, t.weight_sync_relay_min_fanout_gain) == (4, 8, 2)
    monkeypatch.setenv("ULTRA_EP_GRAD_REDUCE_NUM_SMS", "41")
    with pytest.raises(ValueError):
        load_tuning_from_env()
    monkeypatch.setenv("ULTRA_EP_GRAD_REDUCE_NUM_SMS", "64")
    monkeypatch.setenv("ULTRA_EP_WEIGHT_SYNC_PLAN_MODE", "Force_Relay")
    monkeypatch.setenv("ULTRA_EP_QUOTA_LOCALITY_AWARE", "off")
    monkeypatch.setenv("ULTRA_EP_QUOTA_ORACLE_EPS", " 0.05 ")
    t = load_tuning_from_env()
    assert t.grad_reduce_num_sms == 64 and t.weight_sync_plan_mode_id == 2 and t.quota_locality_aware is False
    assert t.quota_oracle_eps == 0.05
    monkeypatch.setenv("ULTRA_EP_QUOTA_KERNEL_STAGE", "2")
    with pytest.raises(ValueError):
        load_tuning_from_env()
    monkeypatch.setenv("ULTRA_EP_QUOTA_KERNEL_STAGE", "1")
    monkeypatch.setenv("ULTRA_EP_QUOTA_REROUTE_INTERLEAVE", "maybe")
    with pytest.raises(ValueError):
        load_tuning_from_env()


def test_microbatch_slot_arithmetic():
    from ultra_ep_b200.manager import Manager

    m = Manager.__new__(Manager)
    m.max_microbatches = 4
    m.real_num_alloc_layers = 5
    m._mb_counters = [0] * 5
    assert [m.allocate_microbatch_slot(2) for _ in range(6)] == [8, 9, 10, 11, 8, 9]
    assert m.allocate_microbatch_slot(0) == 0
    assert m._real_layer_id(11) == 2
    with pytest.raises(AssertionError):
        m.allocate_microbatch_slot(5)


WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["UEP_ROOT"])
import torch.distributed as dist
dist.init_process_group("gloo")
from ultra_ep_b200 import runtime
from ultra_ep_b200.native import load
C = load()
captured = {}
orig = C.set_handle_exchange
def spy(fn):
    captured["fn"] = fn
    orig(fn)
C.set_handle_exchange = spy
peers = runtime.init_runtime(dist.group.WORLD)
assert peers == 2 and C.is_runtime_initialized()
assert runtime.init_runtime(dist.group.WORLD) == 2           # idempotent
rank = dist.get_rank()
blob = bytes([rank]) * 64
parts = captured["fn"](blob)
assert [p[0] for p in parts] == [0, 1] and all(len(p) == 64 for p in parts)
# a Manager cannot be built without a CUDA device: the error must be loud, not a fallback
try:
    C.Manager(1, 2, 1, 16, 16, 2, 1, 0, 0, 4, True, True)
    raise SystemExit("Manager construction without a GPU must fail")
except RuntimeError as e:
    assert "CUDA" in str(e) or "cuda" in str(e), str(e)
runtime.shutdown_runtime()
assert not C.is_runtime_initialized()
dist.barrier()
open(os.path.join(os.environ["UEP_OUT"], f"ok{rank}"), "w").write("ok")
'''


def test_two_rank_bootstrap_over_gloo(tmp_path, native_lib):
    from ultra_ep_b200 import build

    build.build_ext()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, UEP_ROOT=ROOT, UEP_OUT=str(tmp_path), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29631", str(script)], env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_expert_load_trace_files(tmp_path, monkeypatch):
    """The load trace writes the reference's file layout: a manifest and .npz chunks with the
    arrays its viewer reads; record_interval thins the records, flush_interval cuts chunks."""
    import json

    import numpy as np
    import torch

    from ultra_ep_b200 import profiling

    monkeypatch.setenv("ULTRA_EP_LOAD_PROFILING", "1")
    monkeypatch.setenv("ULTRA_EP_LOAD_PROFILE_DIR", str(tmp_path))
    monkeypatch.setenv("ULTRA_EP_LOAD_PROFILE_FLUSH_INTERVAL", "4")
    monkeypatch.setenv("ULTRA_EP_LOAD_PROFILE_RECORD_INTERVAL", "2")
    cfg = profiling.load_profile_config()
    assert cfg.enabled and cfg.flush_interval == 4 and cfg.record_interval == 2
    L, P = 6, 8
    meta = {"ep_group_id": "abc", "ep_rank": 0, "ep_size": 2}
    prof = profiling.ExpertLoadProfiler(cfg, group_rank=0, global_rank=0, metadata=meta, num_logical=L, num_physical=P)
    other = profiling.ExpertLoadProfiler(cfg, group_rank=1, global_rank=1, metadata=meta, num_logical=L, num_physical=P)
    assert prof.enabled and not other.enabled
    sent = []
    for mb in range(12):  # two real layers, alternating; every second microbatch of each is kept
        real = mb % 2
        pre = torch.arange(L, dtype=torch.int32) + mb
        post = torch.arange(P, dtype=torch.int32) * 2 + mb
        prof.record(virtual_layer=real * 3 + 1, real_layer=real, pre_logical_loads=pre, post_physical_loads=post)
        other.record(real * 3 + 1, real, pre, post)
        if (mb // 2) % 2 == 0:
            sent.append((real, real * 3 + 1, mb // 2, pre.numpy(), post.numpy()))
    prof.close()
    prof.close()  # idempotent
    manifest = json.loads(next(tmp_path.glob("*.manifest.json")).read_text())
    assert manifest["schema"] == "ultra_ep_trace_v1" and manifest["chunks"] == 2 and manifest["dropped_records"] == 0
    chunks = sorted(tmp_path.glob("*.chunk*.npz"))
    assert len(chunks) == 2 and not list(tmp_path.glob("*.tmp"))
    rows = []
    for path in chunks:
        z = np.load(path)
        assert set(z.files) == {"metadata", "layers", "virtual_layers", "microbatches", "pre_logical_loads",
                                "post_physical_loads"}
        assert json.loads(str(z["metadata"]))["trace_id"] == manifest["trace_id"]
        assert z["pre_logical_loads"].dtype == np.int32 and z["pre_logical_loads"].shape[1] == L
        assert z["post_physical_loads"].shape[1] == P
        for i in range(len(z["layers"])):
            rows.append((int(z["layers"][i]), int(z["virtual_layers"][i]), int(z["microbatches"][i]),
                         z["pre_logical_loads"][i], z["post_physical_loads"][i]))
    assert len(rows) == len(sent) == 6
    for got, exp in zip(rows, sent):
        assert got[:3] == exp[:3] and np.array_equal(got[3], exp[3]) and np.array_equal(got[4], exp[4])


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs without a GPU (the CPU restatement on host threads) and prints one JSON
    line with the keys the harness reads."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--cpu-budget-s", "1", "--no-ref", "--config", "cfg1_plan_reroute"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "us_per_layer_plan_sync_reroute" and d["unit"] == "us/layer"
    assert d["higher_is_better"] is False and d["value"] > 0 and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


TEARDOWN_WORKER = r'''
import os, sys, time
sys.path.insert(0, os.environ["UEP_ROOT"])
import torch.distributed as dist
dist.init_process_group("gloo")
from ultra_ep_b200.manager import Manager

rank = dist.get_rank()
out = os.environ["UEP_OUT"]


class FakeRuntime:  # stands in for the native manager: records WHEN the arena would be freed
    def destroy(self):
        open(os.path.join(out, f"freed{rank}"), "w").write(repr(time.time()))


class FakeProfiler:
    def close(self):
        pass


mgr = Manager.__new__(Manager)  # the constructor needs a GPU; teardown ordering does not
mgr.runtime, mgr.group, mgr.explicitly_destroy, mgr._load_profiler = FakeRuntime(), dist.group.WORLD, False, FakeProfiler()
dist.barrier()
if rank == 1:
    time.sleep(1.5)  # rank 1 is still "computing": its kernels may still store into rank 0's arena
open(os.path.join(out, f"entered{rank}"), "w").write(repr(time.time()))
del mgr  # explicitly_destroy=False: releasing the last reference runs the ordered teardown
assert os.path.exists(os.path.join(out, f"freed{rank}"))

# without a usable group nothing is freed: the native layer is told to keep the memory
class Abandoned(FakeRuntime):
    abandoned = False
    def abandon(self):
        Abandoned.abandoned = True
    def destroy(self):
        raise SystemExit("freed peer-visible memory without a barrier")
m2 = Manager.__new__(Manager)
m2.runtime, m2.group, m2.explicitly_destroy, m2._load_profiler = Abandoned(), "not a process group", False, FakeProfiler()
assert m2._teardown() is False and Abandoned.abandoned and m2.runtime is None
dist.barrier()
dist.destroy_process_group()
'''


def test_teardown_waits_for_every_rank_over_gloo(tmp_path):
    """A rank's peer-visible arena is freed only after EVERY rank of the group has entered teardown (the peers'
    kernels store into it), also on the implicit path (explicitly_destroy=False, last reference dropped); and
    when no barrier can be made, nothing is freed."""
    script = tmp_path / "teardown_worker.py"
    script.write_text(TEARDOWN_WORKER)
    env = dict(os.environ, UEP_ROOT=ROOT, UEP_OUT=str(tmp_path), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29633", str(script)], env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    t = {name: float((tmp_path / name).read_text()) for name in ("entered0", "entered1", "freed0", "freed1")}
    assert t["freed0"] >= t["entered1"] and t["freed1"] >= t["entered0"]
    assert t["freed0"] - t["entered0"] > 1.0  # rank 0 really waited for the late rank
