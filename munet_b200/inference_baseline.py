"""Replay of the reference's inference benchmark protocol (tools/inference_baseline.cpp) on the
B200 executor: the same three-layer MLP (matmul+bias, ReLU, matmul+bias, ReLU, matmul+bias with
uniform(-1/sqrt(fan_in), 1/sqrt(fan_in)) parameters), the same phases (cold load, compile with
warm-up runs, steady single runs, steady batch runs) and the same JSON report keys, so numbers from
`munet_inference_baseline` and from this tool can be laid side by side.

    python -m munet_b200.inference_baseline [--dtype float32|bfloat16] [--batch 32] [--input-dim 256]
        [--hidden-dim 512] [--output-dim 128] [--warmup-runs 5] [--single-run-iters 50]
        [--batch-run-inputs 4] [--batch-run-iters 20] [--prepared-input-cache-entries 8]
        [--prepared-input-cache-max-bytes 67108864] [--preallocate-batch-inputs 0|1]

Inputs are host tensors, as in the reference tool: every run includes the host-to-device copy of
its input (or a prepared-input cache hit when `--preallocate-batch-inputs 1`) and the copy of the
result back to the host.
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

import munet_b200 as mb
from munet_b200.inference import Engine


def _flag(v: str) -> bool:
    return v.lower() in ("1", "true", "yes", "on")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--input-dim", type=int, default=256)
    ap.add_argument("--hidden-dim", type=int, default=512)
    ap.add_argument("--output-dim", type=int, default=128)
    ap.add_argument("--warmup-runs", type=int, default=5)
    ap.add_argument("--single-run-iters", type=int, default=50)
    ap.add_argument("--batch-run-inputs", type=int, default=4)
    ap.add_argument("--batch-run-iters", type=int, default=20)
    ap.add_argument("--lean-mode", default="0")
    ap.add_argument("--prepared-input-cache-entries", type=int, default=8)
    ap.add_argument("--prepared-input-cache-max-bytes", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--preallocate-batch-inputs", default="0")
    a = ap.parse_args()
    if a.device != "cuda":
        raise SystemExit("munet_b200 runs on a CUDA device (sm_100) only")
    dtype = mb.F32 if a.dtype == "float32" else mb.BF16
    rng = np.random.default_rng(0)

    def uni(shape, fan_in):
        lim = 1.0 / np.sqrt(fan_in)
        return rng.uniform(-lim, lim, shape).astype(np.float32)

    dims = [a.input_dim, a.hidden_dim, a.hidden_dim, a.output_dim]
    layers, tensors = [], {}
    for i in range(3):
        layers.append({"type": "Linear", "in_features": dims[i], "out_features": dims[i + 1], "bias": True})
        tensors[f"{len(layers) - 1}.weight"] = uni((dims[i], dims[i + 1]), dims[i])
        tensors[f"{len(layers) - 1}.bias"] = uni((dims[i + 1],), dims[i + 1])
        if i < 2:
            layers.append({"type": "ReLU"})
    cfg = {"type": "Sequential", "layers": layers}

    def host_input():
        x = torch.from_numpy(rng.standard_normal((a.batch, a.input_dim)).astype(np.float32))
        return x if dtype == mb.F32 else x.bfloat16()

    eng = Engine(compute_dtype=dtype)
    eng.set_lean_mode(_flag(a.lean_mode))
    eng.set_prepared_input_cache_entries(a.prepared_input_cache_entries)
    eng.set_prepared_input_cache_max_bytes(a.prepared_input_cache_max_bytes)
    t0 = time.perf_counter()
    eng.load(cfg, tensors)
    load_wall_ms = (time.perf_counter() - t0) * 1e3
    load_stats = eng.engine_stats
    x0 = host_input()
    t0 = time.perf_counter()
    eng.compile((a.batch, a.input_dim))
    forward0 = time.perf_counter()
    for _ in range(max(a.warmup_runs, 0)):
        eng.run(x0)
    warm_ms = (time.perf_counter() - forward0) * 1e3
    compile_stats = eng.engine_stats
    compile_ms = (time.perf_counter() - t0) * 1e3

    single_wall = single_run = single_prep = single_fwd = 0.0
    for _ in range(a.single_run_iters):
        x = host_input()
        t0 = time.perf_counter()
        eng.run(x)
        single_wall += (time.perf_counter() - t0) * 1e3
        st = eng.engine_stats
        single_run += st["last_run_ms"]
        single_prep += st["last_prepare_input_ms"]
        single_fwd += st["last_forward_ms"]

    batch_wall = 0.0
    for _ in range(a.batch_run_iters):
        inputs = [host_input() for _ in range(a.batch_run_inputs)]
        if _flag(a.preallocate_batch_inputs):
            eng.prepare_batch(inputs)
        outs = []
        t0 = time.perf_counter()
        eng.run_batch_into(inputs, outs)
        batch_wall += (time.perf_counter() - t0) * 1e3

    final = eng.engine_stats
    plan = eng.stats()
    n1, nb = max(a.single_run_iters, 1), max(a.batch_run_iters, 1)
    report = {
        "device": "cuda:0", "dtype": a.dtype, "build_profile_hint": "sm_100a tcgen05",
        "lean_mode": _flag(a.lean_mode),
        "memory_policy": {"prepared_input_cache_entries": a.prepared_input_cache_entries,
                          "prepared_input_cache_max_bytes": a.prepared_input_cache_max_bytes,
                          "preallocate_batch_inputs": _flag(a.preallocate_batch_inputs)},
        "shape_contract": {"compiled_input_shape": compile_stats["compiled_input_shape"],
                           "compiled_output_shape": compile_stats["compiled_output_shape"]},
        "cold_load": {"wall_ms": load_wall_ms, "to_device_ms": load_stats["load_to_device_ms"], "eval_ms": 0.0},
        "compile": {"compile_ms": compile_ms, "prepare_input_ms": 0.0,
                    "forward_ms": compile_stats["compile_ms"], "warmup_ms": warm_ms},
        "steady_single_run": {"iters": a.single_run_iters, "avg_wall_ms": single_wall / n1,
                              "avg_engine_run_ms": single_run / n1, "avg_prepare_input_ms": single_prep / n1,
                              "avg_forward_ms": single_fwd / n1, "avg_output_validation_ms": 0.0},
        "steady_batch_run": {"iters": a.batch_run_iters, "inputs_per_iter": a.batch_run_inputs,
                             "avg_wall_ms": batch_wall / nb,
                             "avg_per_input_wall_ms": batch_wall / (nb * max(a.batch_run_inputs, 1))},
        "memory_bytes": {"engine_current": plan["arena_bytes"] + plan["weight_bytes"],
                         "engine_peak": plan["arena_bytes"] + plan["weight_bytes"],
                         "prepared_input_cache_entries": final["prepared_input_cache_entries"],
                         "prepared_input_cache_bytes": final["prepared_input_cache_bytes"],
                         "prepared_input_cache_hits": final["prepared_input_cache_hits"],
                         "prepared_input_cache_misses": final["prepared_input_cache_misses"],
                         "prepared_input_cache_evictions": final["prepared_input_cache_evictions"],
                         "profiler_current": 0, "profiler_peak": 0},
    }
    print(json.dumps(report, indent=2))


if __name__ == "__main__":
    main()
