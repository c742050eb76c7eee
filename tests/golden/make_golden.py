"""Regenerates tests/golden/reference_outputs.npz: outputs of the UNMODIFIED reference CPU core
(oracle/_ref/libmunet_ref.so, built by `make -C oracle ref` where the reference checkout is
present) on small seeded inputs, stored together with those inputs.

    python tests/golden/make_golden.py

The fixture lets the checker restatement (oracle/oracle.c) and the GPU kernels be compared with the
reference's own results on machines that have neither the reference checkout nor its built library.
bfloat16 tensors are stored as their uint16 bit patterns.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oracle import BF16, F32  # noqa: E402


def rnd(rng, shape, dtype, scale=1.0):
    a = (rng.standard_normal(shape) * scale).astype(np.float32)
    return a if dtype == F32 else oracle.to_bf16(a)


def main():
    R = oracle.ref()
    out = {}
    for dtype, tag in ((F32, "f32"), (BF16, "bf16")):
        rng = np.random.default_rng(4242)
        x, w, b = rnd(rng, (19, 40), dtype), rnd(rng, (40, 24), dtype, 0.2), rnd(rng, (24,), dtype, 0.1)
        out[f"linear.{tag}.x"], out[f"linear.{tag}.w"], out[f"linear.{tag}.b"] = x, w, b
        for act in ("none", "relu", "gelu", "sigmoid", "tanh"):
            out[f"linear.{tag}.{act}.y"] = R.linear(x, w, b, dtype, act)
        u, v = rnd(rng, (300,), dtype, 3.0), rnd(rng, (300,), dtype)
        out[f"add.{tag}.a"], out[f"add.{tag}.b"], out[f"add.{tag}.y"] = u, v, R.add(u, v, dtype)
        z = rnd(rng, (13, 72), dtype, 2.0)
        g, bb = rnd(rng, (72,), dtype), rnd(rng, (72,), dtype)
        out[f"norm.{tag}.x"], out[f"norm.{tag}.g"], out[f"norm.{tag}.b"] = z, g, bb
        out[f"norm.{tag}.layer_norm"] = R.layer_norm(z, g, bb, dtype)
        out[f"norm.{tag}.softmax"] = R.softmax(z, dtype)
        out[f"norm.{tag}.rms_norm"] = R.rms_norm(z, g, dtype)
        out[f"norm.{tag}.leaky_relu"] = R.leaky_relu(z.reshape(-1), 0.1, dtype)
        B, T, E, H = 2, 12, 32, 4
        xm = rnd(rng, (B, T, E), dtype)
        ps = [rnd(rng, s, dtype, 0.2) for s in ((E, E), (E,)) * 4]
        out[f"mha.{tag}.x"] = xm
        for i, p in enumerate(ps):
            out[f"mha.{tag}.p{i}"] = p
        for causal in (0, 1):
            out[f"mha.{tag}.causal{causal}.y"] = R.mha(xm, ps, H, bool(causal), dtype)
        V, d, Hh, L, Tt = 50, 32, 2, 2, 9
        from tests.test_oracle_vs_ref import gpt_params
        gp = gpt_params(np.random.default_rng(7), V, Tt, d, L, dtype, std=0.1)
        ids = np.random.default_rng(8).integers(0, V, (2, Tt)).astype(np.int32)
        out[f"gpt.{tag}.ids"] = ids
        for i, p in enumerate(gp):
            out[f"gpt.{tag}.p{i:02d}"] = p
        out[f"gpt.{tag}.logits"] = R.gpt_forward(ids, gp, V, d, Hh, L, dtype)
    rng = np.random.default_rng(99)
    xc = rng.random((2, 3, 9, 8), dtype=np.float32)
    wc = (rng.standard_normal((5, 3, 3, 3)) * 0.3).astype(np.float32)
    bc = (rng.standard_normal(5) * 0.1).astype(np.float32)
    out["conv.x"], out["conv.w"], out["conv.b"] = xc, wc, bc
    yc = R.conv2d(xc, wc, bc, 1, 1)
    out["conv.y"], out["conv.pool"], out["conv.gap"] = yc, R.max_pool2d(np.maximum(yc, 0)), R.global_avg_pool(yc)
    mean, var = rng.standard_normal(5).astype(np.float32), (rng.random(5) + 0.2).astype(np.float32)
    g5, b5 = rng.standard_normal(5).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    out["bn.g"], out["bn.b"], out["bn.mean"], out["bn.var"] = g5, b5, mean, var
    out["bn.y"] = R.batch_norm_eval(yc, g5, b5, mean, var, F32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"{path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
