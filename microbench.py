"""Micro-benchmarks of single kernels of libpom_b200 (CUDA-event timing, optional cuBLAS comparison).

    python microbench.py gemm --m 32768 --n 2304 --k 1152 [--a-mn] [--b-mn] [--accumulate] [--mode 0|1|2]
    python microbench.py ctx|gate|gate_bwd --b 32 --tokens 1024 --d 1152 --expand 2 --degree 2 [--rope 0|1|2]
    python microbench.py agg_bwd|agg_fwd|select --b 32 --tokens 1024 --p 2304 --degree 2 [--causal] [--rope 0|1|2]

Each run prints one line with the average launch time and the achieved TFLOP/s or GB/s; the commands that
were profiled with ncu are of this form.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from pom_b200 import _abi, ops  # noqa: E402


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _rope_spec(kind: int, n: int, p: int, dev):
    if kind == 0:
        return None
    from pom_b200.pom_rope import precompute_freqs_1d, precompute_freqs_2d

    if kind == 1:
        c, s = precompute_freqs_1d(p, n)
        pos = torch.arange(n, device=dev)
        return ops.RopeSpec(_abi.ROPE_1D, c.to(dev), s.to(dev), pos, steps=(ops.rope_pos_info(pos)[0][2], -1))
    side = int(n ** 0.5)
    rc, rs, cc, cs = precompute_freqs_2d(p, side, side)
    idx = torch.arange(n, device=dev)
    hw = torch.stack([idx // side, idx % side], 1).contiguous()
    steps = tuple(s for _, _, s in ops.rope_pos_info(hw))
    return ops.RopeSpec(_abi.ROPE_2D, rc.to(dev), rs.to(dev), hw, cc.to(dev), cs.to(dev), steps=steps)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["gemm", "ctx", "gate", "gate_bwd", "agg_fwd", "agg_bwd", "select", "select_bwd"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=1152)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--b", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--d", type=int, default=1152)
    ap.add_argument("--p", type=int, default=2304)
    ap.add_argument("--expand", type=int, default=2)
    ap.add_argument("--degree", type=int, default=2)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--rope", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul on the same operands")
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    _abi.check(_abi.lib().pom_set_gemm_mode(a.mode), "pom_set_gemm_mode")
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g).bfloat16()

    if a.what == "gemm":
        A = rnd(a.k, a.m) if a.a_mn else rnd(a.m, a.k)
        B = rnd(a.k, a.n) if a.b_mn else rnd(a.n, a.k)
        out = torch.zeros(a.m, a.n, device=dev) if a.accumulate else torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: ops.gemm(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=out, accumulate=a.accumulate), a.iters)
        fl = 2.0 * a.m * a.n * a.k
        line = f"gemm m={a.m} n={a.n} k={a.k} a_mn={a.a_mn} b_mn={a.b_mn} acc={a.accumulate} mode={a.mode}: {ms:.4f} ms {fl / ms / 1e9:.0f} TFLOP/s"
        if a.cublas:
            Am, Bm = (A.t() if a.a_mn else A), (B.t() if a.b_mn else B)
            ms2 = _time(lambda: torch.matmul(Am, Bm.t()), a.iters)
            line += f" | cuBLAS {ms2:.4f} ms {fl / ms2 / 1e9:.0f} TFLOP/s"
        print(line)
    elif a.what in ("ctx", "gate", "gate_bwd"):
        P = a.expand * a.d
        x = rnd(a.b, a.tokens, a.d)
        fl = 2.0 * a.b * a.tokens * a.d * P
        rope = _rope_spec(a.rope, a.tokens, P, dev)
        # --causal: the token-causal forms of the three phases (running sums per 32-token group in the epilogue)
        causal = None
        if a.causal and a.what != "ctx":
            pre = rnd(a.b, a.tokens, P)
            carry = torch.randn(a.b, ops.token_groups(a.tokens), P, device=dev, generator=g)
            causal = (pre, carry, 0)
        if a.what == "ctx":
            w = rnd(P, a.d) * 0.03
            coeff = torch.randn(P, a.degree, device=dev, generator=g) * 0.1
            ms = _time(lambda: ops.ctx_gemm(x, w, coeff, rope=rope, causal=a.causal), a.iters)
        elif a.what == "gate":
            w = rnd(P, a.d) * 0.03
            bias = torch.zeros(P, device=dev)
            h = torch.randn(a.b, P, device=dev, generator=g)
            ms = _time(lambda: ops.gate_gemm(x, w, bias, h, rope=rope, causal=causal), a.iters)
        else:
            wo = rnd(a.d, P) * 0.03
            wot = wo.t().contiguous()
            bias = torch.zeros(P, device=dev)
            h = torch.randn(a.b, P, device=dev, generator=g)
            z = rnd(a.b, a.tokens, P)
            G = torch.empty(a.b * a.tokens, 2 * P, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: ops.gate_bwd_gemm(x, wo, bias, h, z, G[:, P:], rope=rope, w_o_t=wot, causal=causal),
                       a.iters)
        print(f"{a.what} b={a.b} tokens={a.tokens} d={a.d} p={P} degree={a.degree} rope={a.rope} causal={a.causal} mode={a.mode}: {ms:.4f} ms {fl / ms / 1e9:.0f} TFLOP/s")
    else:
        P = a.p
        x = rnd(a.b, a.tokens, P) * 0.5
        coeff = torch.randn(P, a.degree, device=dev, generator=g) * 0.1
        rope = _rope_spec(a.rope, a.tokens, P, dev)
        elems = a.b * a.tokens * P
        if a.what == "agg_fwd":
            ms = _time(lambda: ops.poly_agg_fwd(x, coeff, causal=a.causal, rope=rope), a.iters)
            nbytes = elems * 2 * (2 if a.causal else 1) + (elems * 2 if a.causal else 0)
        elif a.what == "agg_bwd":
            dx = torch.empty_like(x)
            if a.causal:
                dout = rnd(a.b, a.tokens, P)
                ms = _time(lambda: ops.poly_agg_bwd(x, coeff, dx_out=dx, dout=dout, causal=True, rope=rope), a.iters)
                nbytes = elems * 2 * 4
            else:
                dH = torch.randn(a.b, P, device=dev, generator=g)
                ms = _time(lambda: ops.poly_agg_bwd(x, coeff, dx_out=dx, dH=dH, scale=1.0 / a.tokens, rope=rope), a.iters)
                nbytes = elems * 2 * 2
        else:
            bias = torch.zeros(P, device=dev)
            h = rnd(a.b, a.tokens, P) if a.causal else torch.randn(a.b, P, device=dev, generator=g)
            if a.what == "select":
                ms = _time(lambda: ops.select_fwd(x, bias, h, rope=rope), a.iters)
                nbytes = elems * 2 * (3 if a.causal else 2)
            else:
                dsh = rnd(a.b, a.tokens, P)
                dz = torch.empty_like(x)
                ms = _time(lambda: ops.select_bwd(dsh, x, bias, h, dz, rope=rope), a.iters)
                nbytes = elems * 2 * (5 if a.causal else 3)
        print(f"{a.what} b={a.b} tokens={a.tokens} p={P} degree={a.degree} causal={a.causal} rope={a.rope}: "
              f"{ms:.4f} ms {nbytes / ms / 1e6:.0f} GB/s (algorithmic bytes {nbytes / 1e6:.0f} MB)")
    st = _abi.read_status(dev)
    if st:
        raise SystemExit(f"device status {st}: a bounded wait expired")


if __name__ == "__main__":
    main()
