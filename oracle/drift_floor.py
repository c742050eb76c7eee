"""TEST INFRASTRUCTURE ONLY: how far do two valid evaluation orders of the same bf16 decoder
drift apart with depth?  CPU only, no kernel in the loop.

The C restatement runs the decoder once with the reference's arithmetic (variant 0: double
accumulation, normalised probabilities rounded to bf16) and again with the pieces a tensor-core
kernel changes (variant 1: float accumulation in every contraction; variant 2: online-softmax
order, i.e. unnormalised probabilities rounded to bf16; variant 3: both).  The differences are
reported in the units the parity tests use:

    worst/bound  max over elements of |a-b| / (2e-2*|b| + 2e-2*rms(b))   (must be <= 1 to pass)
    rel-inf      max|a-b| / max|b|
    rel-rms      rms(a-b) / rms(b)

    python -m oracle.drift_floor [--tokens 48] [--layers 6 24] [--small]
"""
from __future__ import annotations

import argparse
import time

import numpy as np

import oracle
from oracle import BF16


def decoder_weights(rng, V, T, d, L):
    def w(*s):
        return oracle.to_bf16((rng.standard_normal(s) * 0.02).astype(np.float32))
    one, zero = oracle.to_bf16(np.ones(d, np.float32)), oracle.to_bf16(np.zeros(d, np.float32))

    def z(n):
        return oracle.to_bf16(np.zeros(n, np.float32))
    ps = [w(V, d), w(T, d)]
    for _ in range(L):
        ps += [one, zero]
        for _ in range(4):
            ps += [w(d, d), z(d)]
        ps += [one, zero, w(d, 4 * d), z(4 * d), w(4 * d, d), z(d)]
    ps += [one, zero, w(d, V), z(V)]
    return ps


def metrics(got, want, rtol=2e-2):
    g = oracle.from_bf16(got).astype(np.float64)
    w = oracle.from_bf16(want).astype(np.float64)
    rms = float(np.sqrt(np.mean(w * w)))
    err = np.abs(g - w)
    worst = float((err / (rtol * np.abs(w) + rtol * rms)).max())
    return worst, float(err.max() / np.abs(w).max()), float(np.sqrt(np.mean(err ** 2)) / rms)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=48)
    ap.add_argument("--layers", type=int, nargs="+", default=[6, 24])
    ap.add_argument("--small", action="store_true", help="d512 h8 V8192 instead of d2048 h16 V32000")
    ap.add_argument("--seeds", type=int, default=1)
    args = ap.parse_args()
    V, d, H = (8192, 512, 8) if args.small else (32000, 2048, 16)
    T = args.tokens
    P = oracle.port()
    names = {1: "float accumulation", 2: "unnormalised-P rounding", 3: "both"}
    print(f"decoder d{d} h{H} V{V}, {T} tokens of one sequence, weights N(0,0.02), math K addressing")
    print("| layers | seed | variant | worst/bound | rel-inf | rel-rms |")
    print("|---|---|---|---|---|---|")
    for L in args.layers:
        for seed in range(args.seeds):
            rng = np.random.default_rng(1005 + seed)
            ps = decoder_weights(rng, V, T, d, L)
            ids = np.random.default_rng(2005 + seed).integers(0, V, (1, T)).astype(np.int32)
            P.set_variant(0)
            t0 = time.time()
            want = P.gpt_forward(ids, ps, V, d, H, L, BF16, kmode=oracle.K_MATH)
            for var in (1, 2, 3):
                P.set_variant(var)
                got = P.gpt_forward(ids, ps, V, d, H, L, BF16, kmode=oracle.K_MATH)
                P.set_variant(0)
                worst, rel_inf, rel_rms = metrics(got, want)
                print(f"| {L} | {seed} | {names[var]} | {worst:.2f} | {rel_inf:.4f} | {rel_rms:.4f} |",
                      flush=True)
            print(f"<!-- {L} layers seed {seed}: {time.time() - t0:.0f} s -->", flush=True)


if __name__ == "__main__":
    main()
