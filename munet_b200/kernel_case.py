"""Run ONE kernel of the library on one shape: for timing a kernel in isolation and as
the command to put under a profiler.

    python -m munet_b200.kernel_case linear  M K N [--act gelu] [--no-bias] [--residual] [--reps 5]
    python -m munet_b200.kernel_case attention B H T D [--kmode 0|1] [--non-causal] [--reps 5]
    python -m munet_b200.kernel_case layer_norm ROWS COLS [--reps 5]
    python -m munet_b200.kernel_case softmax ROWS COLS [--reps 5]
    python -m munet_b200.kernel_case argmax ROWS COLS [--reps 5]
    python -m munet_b200.kernel_case eltwise ROWS COLS [--act gelu] [--residual] [--reps 5]

Operands are random bf16 tensors (torch is used for allocation and CUDA events only).
Prints mean milliseconds over ``--reps`` launches after two warm-up launches, with the
algorithmic TFLOP/s or GB/s of the shape.
"""
from __future__ import annotations

import argparse

import torch

import munet_b200 as mb


def timed(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["linear", "attention", "layer_norm", "softmax", "argmax", "eltwise"])
    ap.add_argument("dims", type=int, nargs="+")
    ap.add_argument("--act", default="none")
    ap.add_argument("--no-bias", action="store_true")
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--kmode", type=int, default=0)
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--reps", type=int, default=5)
    a = ap.parse_args()
    ctx = mb.Context(0)
    bf = dict(dtype=torch.bfloat16, device="cuda")
    if a.kernel == "linear":
        M, K, N = a.dims
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(K, N, device="cuda") / K ** 0.5).bfloat16()
        y = torch.empty(M, N, **bf)
        bias = None if a.no_bias else torch.zeros(N, **bf)
        res = torch.randn(M, N, device="cuda").bfloat16() if a.residual else None
        ms = timed(lambda: ctx.linear(x, w, bias, y, M, K, N, mb.BF16, act=a.act, residual=res), a.reps)
        print(f"linear {M}x{K}x{N} act={a.act} bias={bias is not None} residual={a.residual}: "
              f"{ms:.4f} ms  {2 * M * K * N / ms / 1e9:.1f} TFLOP/s")
    elif a.kernel == "attention":
        B, H, T, D = a.dims
        q, k, v = (torch.randn(B * H * T, D, device="cuda").bfloat16() for _ in range(3))
        out = torch.empty(B * T, H * D, **bf)
        nbytes = ctx.attention_workspace_bytes(B, H, T, D, mb.BF16)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        causal = not a.non_causal
        ms = timed(lambda: ctx.attention(q, k, v, out, B, H, T, D, causal, a.kmode, mb.BF16, ws,
                                         nbytes), a.reps)
        fl = (2.0 if causal else 4.0) * B * H * T * T * D
        print(f"attention B{B} H{H} T{T} D{D} kmode={a.kmode} causal={causal}: {ms:.4f} ms  "
              f"{fl / ms / 1e9:.1f} TFLOP/s ({'causal-useful' if causal else 'full'})")
    elif a.kernel == "argmax":
        rows, cols = a.dims
        x = torch.randn(rows, cols, device="cuda").bfloat16()
        idx = torch.empty(rows, dtype=torch.int32, device="cuda")
        ms = timed(lambda: ctx.argmax(x, idx, rows, cols, mb.BF16), a.reps)
        print(f"argmax {rows}x{cols}: {ms:.4f} ms  {(rows * cols * 2 + rows * 4) / ms / 1e6:.0f} GB/s")
    elif a.kernel == "eltwise":
        rows, cols = a.dims
        x = torch.randn(rows, cols, device="cuda").bfloat16()
        y = torch.empty_like(x)
        bias = torch.zeros(cols, **bf)
        res = torch.randn(rows, cols, device="cuda").bfloat16() if a.residual else None
        ms = timed(lambda: ctx.eltwise(x, y, rows * cols, mb.BF16, act=a.act, bias=bias, cols=cols,
                                       residual=res), a.reps)
        nb = (3 if a.residual else 2) * rows * cols * 2
        print(f"eltwise {rows}x{cols} act={a.act} residual={a.residual}: {ms:.4f} ms  {nb / ms / 1e6:.0f} GB/s")
    else:
        rows, cols = a.dims
        x = torch.randn(rows, cols, device="cuda").bfloat16()
        y = torch.empty_like(x)
        if a.kernel == "layer_norm":
            g, b = torch.ones(cols, **bf), torch.zeros(cols, **bf)
            ms = timed(lambda: ctx.layer_norm(x, g, b, y, rows, cols, mb.BF16), a.reps)
        else:
            ms = timed(lambda: ctx.softmax(x, y, rows, cols, mb.BF16), a.reps)
        print(f"{a.kernel} {rows}x{cols}: {ms:.4f} ms  {2 * rows * cols * 2 / ms / 1e6:.0f} GB/s")
    ctx.check()


if __name__ == "__main__":
    main()
