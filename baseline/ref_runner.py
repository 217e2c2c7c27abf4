"""Reference arm of bench.py: runs the UNMODIFIED files of huangs0/mintccl from ``baseline/_ref`` through
their own public functions (``allgather(buff)``, ``broadcast(buff, root)``, ``reduce(buff, root)``), with
the mpi4py stand-in of ``baseline/mpi_shim`` as control plane.  Nothing of mintccl_b200 is on this path.

What can be measured is limited by the reference itself:
  * it needs at least two ranks (its ring search returns no ring for one device);
  * broadcast and reduce hard-code a two-rank ring (4_broadcast.py:86, 5_reduce.py:106);
  * reduce-scatter does not run as shipped (7_reducescatter.py:107) and all-reduce does not exist;
  * on eight GPUs it deadlocks by its own account (README.md:62-63) and its waits are unbounded, so it is
    not launched there at all: a hung kernel on a shared GPU is not an acceptable outcome.
Every run is guarded by a watchdog that ends the process if a call does not return.
"""
from __future__ import annotations

import importlib.util
import json
import os
import shutil
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
WATCHDOG_S = 90


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _load(name: str, filename: str):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, filename))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(a) -> None:
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if not os.path.isdir(REF) or not os.path.exists(os.path.join(REF, "6_allgather.py")):
        return _unavailable("baseline/_ref is missing (copy the reference's files there; it has no installer)")
    if world < 2:
        return _unavailable("the reference's collectives need at least two ranks (its ring search finds no ring for one device)")
    if world > 4:
        return _unavailable("not launched on more than 4 GPUs: the reference documents a deadlock on 8-GPU machines "
                            "(README.md:62-63) and its waits are unbounded (protocol.py:115,127,177)")
    import torch
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")

    done = threading.Event()

    def watchdog():
        if not done.wait(WATCHDOG_S):
            _unavailable(f"a reference call did not return within {WATCHDOG_S} s (unbounded spin in its kernel); process ended")
            os._exit(0)

    threading.Thread(target=watchdog, daemon=True).start()
    sys.path.insert(0, os.path.join(HERE, "mpi_shim"))
    sys.path.insert(0, REF)
    work = tempfile.mkdtemp(prefix="mintccl_ref_")
    os.chdir(work)  # the reference caches topo.json in the working directory
    os.environ.pop("MINTCCL_TEST_MODE", None)
    try:
        torch.cuda.set_device(local)
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("gloo", rank=rank, world_size=world)
        import common  # noqa: F401  (reference module)
        common.set_gpu(local)
        numel = a.size // 2
        results, errors = {}, {}
        plans = [("allgather", "6_allgather.py")]
        if world == 2:
            plans += [("broadcast", "4_broadcast.py"), ("reduce", "5_reduce.py")]
        for name, fname in plans:
            try:
                mod = _load("ref_" + name, fname)
                if name == "allgather":
                    buff = torch.zeros((world, numel // world), dtype=torch.float16)
                    buff[rank].normal_()
                    call = lambda: mod.allgather(buff)  # noqa: E731
                elif name == "broadcast":
                    buff = torch.randn(numel, dtype=torch.float32).to(torch.float16)
                    call = lambda: mod.broadcast(buff, 0)  # noqa: E731
                else:
                    buff = torch.randn(numel, dtype=torch.float32).to(torch.float16)
                    call = lambda: mod.reduce(buff, 0)  # noqa: E731
                for _ in range(max(1, a.warmup)):
                    call()
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                e0.record()
                for _ in range(a.steps):
                    call()
                e1.record()
                torch.cuda.synchronize()
                wall_ms = (time.perf_counter() - t0) * 1e3 / a.steps
                dist.barrier()
                ms = torch.tensor([e0.elapsed_time(e1) / a.steps, wall_ms], dtype=torch.float64)
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                results[name] = (float(ms[0]), float(ms[1]))
            except Exception as e:  # noqa: BLE001
                errors[name] = f"{type(e).__name__}: {e}"[:300]
        done.set()
        if rank == 0:
            fac = {"allgather": (world - 1) / world, "broadcast": 1.0, "reduce": 1.0}
            if not results:
                return _unavailable("every reference collective failed: " + json.dumps(errors))
            busbw = {k: round(fac[k] * a.size / (v[0] * 1e-3) / 1e9, 3) for k, v in results.items()}
            tot_ms = sum(v[0] for v in results.values())
            value = world * sum(fac[k] * a.size for k in results) / (tot_ms * 1e-3) / 1e9
            print(json.dumps({
                "impl": "reference", "metric": "aggregate bus GB/s over the collectives the reference can run: " + "+".join(results),
                "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": a.steps, "warmup": max(1, a.warmup),
                "ms_per_step": round(tot_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp16", "data": "synthetic", "covers": sorted(results), "not_runnable": errors,
                "busbw_GBps": busbw, "ms": {k: round(v[0], 4) for k, v in results.items()},
                "wall_ms": {k: round(v[1], 4) for k, v in results.items()},
                "config": {"model": "reference collectives through their own API (each call re-allocates its staging "
                                    "buffer and re-exchanges IPC handles, as the reference does)", "message_bytes": a.size,
                           "parallelism": f"collective x{world}"},
                "note": "reduce-scatter and all-reduce do not exist / do not run in the reference; broadcast and reduce only on 2 ranks",
            }), flush=True)
    except Exception as e:  # noqa: BLE001
        done.set()
        _unavailable(f"reference failed to start: {type(e).__name__}: {e}"[:400])
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
