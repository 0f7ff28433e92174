"""Times ONE kernel class of the attention path in isolation (CUDA events around the C-ABI `*_core` entry)
and prints its roofline line.  Sized by flags so the same command serves as a small profiler target:

    python kernel_bench.py --kernel la_decode  --seqs 128
    python kernel_bench.py --kernel fa_decode  --seqs 128 --ctx 1280 --kv fp16
    python kernel_bench.py --kernel fa_prefill --seqs 16  --ctx 1024
    python kernel_bench.py --kernel la_prefill --seqs 10  --ctx 1024

Inputs are synthetic (unit-RMS q/k, N(0, 0.6) v, decays as in the model) and stay larger than L2 for the
decode kernels by rotating over `--layers` independent caches.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured (burst)"
    return 6650.0, 1590.0, "fallback"


def time_ms(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def measure(kernel: str, seqs: int = 128, ctx: int = 1024, kv: str = "fp16", layers: int = 4, iters: int = 20, warmup: int = 3,
            serial: bool = False) -> dict:
    """Times `iters` back-to-back launches of one kernel class on the current device and returns its roofline record."""
    args = argparse.Namespace(kernel=kernel, seqs=seqs, ctx=ctx, kv=kv, layers=layers, iters=iters, warmup=warmup, serial=serial)
    ops = entry.load_ops()
    g = torch.Generator(device="cuda").manual_seed(1)
    hbm, tfl, src = peaks()
    n, L = args.seqs, args.ctx
    out = dict(kernel=args.kernel, seqs=n, ctx=L)

    if args.kernel == "la_decode":
        la = ops.LinearAttention(ops.PROJ_FP16, max_batch=n, max_prefill_rows=64)
        la.set_weights(entry.load_package().synth.la_weights(3))
        st = ops.LinearAttnState(args.layers, n)
        mixed = torch.randn((n, 8224), device="cuda", generator=g) * 0.6
        slots = torch.arange(n, dtype=torch.int32, device="cuda")
        state = {"l": 0}

        def fn():
            la.decode_core(mixed, st, state["l"] % args.layers, slots)
            state["l"] += 1
        ms = time_ms(fn, args.iters, args.warmup)
        byts = n * (2 * 16 * 128 * 128 * 4 + 2 * 3 * 6144 * 4 + 8224 * 4 + 2048 * 4)
        out.update(ms=ms, achieved=byts / ms / 1e6, unit="GB/s", peak=hbm, bound="hbm")
    elif args.kernel == "fa_decode":
        fp16 = args.kv == "fp16"
        fa = ops.FullAttention(ops.PROJ_FP16, max_batch=n, max_prefill_rows=64)
        kv = ops.KVCache(args.layers, n, max(L, 64), ops.KV_FP16 if fp16 else ops.KV_INT8)
        slots = [kv.allocate_sequence(L) for _ in range(n)]
        for layer in range(args.layers):
            for s0 in range(0, n, 16):        # fill the caches 16 sequences at a time
                m = min(16, n - s0)
                k = torch.randn((m * L, 512), device="cuda", generator=g)
                v = torch.randn((m * L, 512), device="cuda", generator=g) * 0.6
                kv.append(layer, slots[s0:s0 + m], [L] * m, k, v)
        q = torch.randn((n, 8, 256), device="cuda", generator=g)
        d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
        state = {"l": 0}

        def fn():
            fa.decode_core(q, kv, state["l"] % args.layers, d_slots)
            state["l"] += 1
        ms = time_ms(fn, args.iters, args.warmup)
        per_tok = 2 * 2 * 256 * (2 if fp16 else 1) + (0 if fp16 else 16)
        byts = n * (per_tok * L + 8 * 256 * (4 + 4))
        out.update(ms=ms, achieved=byts / ms / 1e6, unit="GB/s", peak=hbm, bound="hbm", kv=args.kv,
                   note="time includes the fp32->fp16 query conversion launch of the core entry")
        assert kv.device_status() == 0
    elif args.kernel == "fa_prefill":
        rows = n * L
        fa = ops.FullAttention(ops.PROJ_FP16, max_batch=4, max_prefill_rows=rows)
        q = torch.randn((rows, 8, 256), device="cuda", generator=g)
        k = torch.randn((rows, 2, 256), device="cuda", generator=g)
        v = torch.randn((rows, 2, 256), device="cuda", generator=g) * 0.6
        ms = time_ms(lambda: fa.prefill_core(q, k, v, [L] * n, use_tensor_cores=not args.serial), args.iters, args.warmup)
        flops = n * 2.0 * (2 * 8 * 256) * L * (L + 1) / 2
        out.update(ms=ms, achieved=flops / ms / 1e9, unit="TFLOP/s", peak=tfl, bound="tensor",
                   note="time includes three fp32->fp16 conversion launches and a status read of the core entry")
    else:
        rows = n * L
        la = ops.LinearAttention(ops.PROJ_FP16, max_batch=4, max_prefill_rows=rows)
        st = ops.LinearAttnState(1, n)
        q = torch.randn((rows, 16, 128), device="cuda", generator=g)
        q = q / q.norm(dim=-1, keepdim=True) / 128 ** 0.5
        k = torch.randn((rows, 16, 128), device="cuda", generator=g)
        k = k / k.norm(dim=-1, keepdim=True)
        v = torch.randn((rows, 16, 128), device="cuda", generator=g) * 0.6
        gl = -torch.exp(torch.rand((rows, 16), device="cuda", generator=g) * 5.0 - 4.0)
        beta = torch.rand((rows, 16), device="cuda", generator=g)
        ms = time_ms(lambda: la.prefill_core(q, k, v, gl, beta, st, 0, list(range(n)), [L] * n, use_tensor_cores=not args.serial),
                     args.iters, args.warmup)
        chunks = -(-L // 64)
        flops = n * 16 * chunks * (5 * 2 * 64 * 64 * 128 + 3 * 2 * 64 * 128 * 128 + 64 ** 3 / 3)
        out.update(ms=ms, achieved=flops / ms / 1e9, unit="TFLOP/s", peak=tfl, bound="tensor",
                   note="time includes two fp32->fp16 conversion launches and a status read of the core entry")
    out["frac"] = out["achieved"] / out["peak"]
    out["peak_source"] = src
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=["la_decode", "fa_decode", "fa_prefill", "la_prefill"])
    ap.add_argument("--seqs", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--kv", default="fp16", choices=["fp16", "int8"])
    ap.add_argument("--layers", type=int, default=4, help="independent caches to rotate over (decode kernels)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--serial", action="store_true", help="la_prefill / fa_prefill: run the plain cross-check kernel instead")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    print(json.dumps(measure(a.kernel, a.seqs, a.ctx, a.kv, a.layers, a.iters, a.warmup, a.serial)))


if __name__ == "__main__":
    main()
