"""Throughput of the smaller reference workloads through the executor, one JSON line each:

    python -m munet_b200.config_bench [mlp] [linear_sweep] [cnn] [gpt_s]   (default: all)

* ``mlp``          784-512-512-10 MLP, fp32, batch 256 (+ argmax)
* ``linear_sweep`` Y = GELU(X.W + b) for n = 1024..8192, fp32 and bf16
* ``cnn``          3x(conv3x3 + ReLU + pool) + Linear on [512,3,32,32], fp32
* ``gpt_s``        6-layer d512 decoder, vocab 8192, seq 256, batch 32, bf16

Inputs are seeded synthetic tensors already resident on the device; time is CUDA events over
``--reps`` engine runs after three warm-up runs. ``work`` is the algorithmic FLOP count of one
forward; ``frac`` compares it with the measured bf16 tensor peak passed in ``--peak-tflops``
(for fp32 rows this is only a common yardstick: fp32 runs on the CUDA cores, bit-exact with the
reference's accumulation order, not on tensor cores).
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

import munet_b200 as mb
from munet_b200.inference import Engine, gpt_decoder_config, gpt_param_shapes


def _time(eng, x, reps):
    stream = torch.cuda.current_stream()
    lib = mb.lib()

    def run():
        rc = lib.mu_engine_run(eng._h, x.data_ptr(), 0, None, 0, None, 0, stream.cuda_stream)
        if rc:
            raise mb.MuNetError(rc, lib.mu_engine_last_error(eng._h).decode())
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    eng.ctx.check()
    return e0.elapsed_time(e1) / reps


def _emit(name, ms, flops, units, unit_name, peak, **extra):
    print(json.dumps({"config": name, "ms": round(ms, 4), unit_name + "_per_s": units / ms * 1e3,
                      "work_gflop": flops / 1e9, "tflops": flops / ms / 1e9,
                      "frac_of_bf16_peak": flops / ms / 1e9 / peak, **extra}), flush=True)


def _normal(rng, shape, std, dtype):
    a = (rng.standard_normal(shape) * std).astype(np.float32)
    t = torch.from_numpy(a).cuda()
    return t.bfloat16() if dtype == mb.BF16 else t


def mlp(a):
    rng = np.random.default_rng(1001)
    sizes = [784, 512, 512, 10]
    layers, tensors = [], {}
    for i in range(3):
        layers.append({"type": "Linear", "in_features": sizes[i], "out_features": sizes[i + 1], "bias": True})
        tensors[f"{len(layers) - 1}.weight"] = _normal(rng, (sizes[i], sizes[i + 1]), (2 / sizes[i]) ** 0.5, mb.F32)
        tensors[f"{len(layers) - 1}.bias"] = torch.zeros(sizes[i + 1], device="cuda")
        if i < 2:
            layers.append({"type": "ReLU"})
    eng = Engine(compute_dtype=mb.F32, argmax=True)
    eng.load({"type": "Sequential", "layers": layers}, tensors).compile((256, 784))
    x = torch.from_numpy(np.random.default_rng(2001).random((256, 784), dtype=np.float32)).cuda()
    ms = _time(eng, x, a.reps)
    fl = 2 * 256 * (784 * 512 + 512 * 512 + 512 * 10)
    _emit("mlp fp32 B256", ms, fl, 256, "samples", a.peak_tflops, launches=eng.stats()["n_launches"])


def linear_sweep(a):
    for dtype, dn in ((mb.BF16, "bf16"), (mb.F32, "fp32")):
        for n in (1024, 2048, 4096, 8192):
            rng = np.random.default_rng(1002 + n)
            tensors = {"0.weight": _normal(rng, (n, n), n ** -0.5, dtype), "0.bias": _normal(rng, (n,), 0.02, dtype)}
            cfg = {"type": "Sequential", "layers": [
                {"type": "Linear", "in_features": n, "out_features": n, "bias": True}, {"type": "GELU"}]}
            eng = Engine(compute_dtype=dtype)
            eng.load(cfg, tensors).compile((n, n))
            x = _normal(np.random.default_rng(2002 + n), (n, n), 1.0, dtype)
            reps = a.reps if (dtype == mb.BF16 or n <= 4096) else max(1, a.reps // 4)
            ms = _time(eng, x, reps)
            _emit(f"linear+gelu {dn} n={n}", ms, 2.0 * n ** 3, n, "rows", a.peak_tflops,
                  launches=eng.stats()["n_launches"])
            eng.close()
            del eng, x, tensors
            torch.cuda.empty_cache()


def cnn(a):
    rng = np.random.default_rng(1003)
    layers, tensors = [], {}
    chans = [3, 64, 128, 256]
    for i in range(3):
        ic, oc = chans[i], chans[i + 1]
        layers.append({"type": "Conv2d", "in_channels": ic, "out_channels": oc, "kernel_size": 3,
                       "stride": 1, "padding": 1})
        tensors[f"{len(layers) - 1}.weight"] = _normal(rng, (oc, ic, 3, 3), (2 / (ic * 9)) ** 0.5, mb.F32)
        tensors[f"{len(layers) - 1}.bias"] = torch.zeros(oc, device="cuda")
        layers.append({"type": "ReLU"})
        layers.append({"type": "MaxPool2d", "kernel_size": 2, "stride": 2, "padding": 0} if i < 2
                      else {"type": "GlobalAvgPool2d"})
    layers.append({"type": "Flatten"})
    layers.append({"type": "Linear", "in_features": 256, "out_features": 10, "bias": True})
    tensors[f"{len(layers) - 1}.weight"] = _normal(rng, (256, 10), (2 / 256) ** 0.5, mb.F32)
    tensors[f"{len(layers) - 1}.bias"] = torch.zeros(10, device="cuda")
    eng = Engine(compute_dtype=mb.F32, argmax=True)
    eng.load({"type": "Sequential", "layers": layers}, tensors).compile((512, 3, 32, 32))
    x = torch.from_numpy(np.random.default_rng(2003).random((512, 3, 32, 32), dtype=np.float32)).cuda()
    ms = _time(eng, x, a.reps)
    fl = 2.0 * 512 * (32 * 32 * 64 * 27 + 16 * 16 * 128 * 576 + 8 * 8 * 256 * 1152 + 256 * 10)
    _emit("cnn fp32 B512", ms, fl, 512, "images", a.peak_tflops, launches=eng.stats()["n_launches"])


def gpt_s(a):
    L, d, H, V, T, B = 6, 512, 8, 8192, 256, 32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1004)
    tensors = {}
    for name, shape in gpt_param_shapes(V, T, d, L).items():
        if ".ln" in name or name.startswith("ln_f"):
            t = torch.ones(*shape, device="cuda") if name.endswith("weight") else torch.zeros(*shape, device="cuda")
        elif name.endswith("bias"):
            t = torch.zeros(*shape, device="cuda")
        else:
            t = torch.randn(*shape, device="cuda", generator=gen) * 0.02
        tensors[name] = t.bfloat16()
    eng = Engine(compute_dtype=mb.BF16, argmax=True)
    eng.load(gpt_decoder_config(V, T, d, H, L), tensors).compile((B, T), mb.I32)
    ids = torch.randint(0, V, (B, T), dtype=torch.int32, device="cuda")
    ms = _time(eng, ids, a.reps)
    tok = B * T
    fl = tok * (L * (2 * 4 * d * d + 2 * 8 * d * d) + 2 * d * V) + L * B * H * 2 * T * T * (d // H)
    _emit("gpt_s bf16 B32 T256", ms, fl, tok, "tokens", a.peak_tflops, launches=eng.stats()["n_launches"],
          attention_flops="causal-useful")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="*", default=["mlp", "linear_sweep", "cnn", "gpt_s"])
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--peak-tflops", type=float, default=1651.0)
    a = ap.parse_args()
    for w in a.which:
        {"mlp": mlp, "linear_sweep": linear_sweep, "cnn": cnn, "gpt_s": gpt_s}[w](a)


if __name__ == "__main__":
    main()
