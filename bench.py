"""Benchmark of the attention hot path inside the Qwen3.5-0.8B-shaped hybrid stack.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

One "step" = one whole job on one batch: prefill 1024 tokens then greedy-decode 512 tokens for 128
sequences per GPU (24 layers = 6 x [3 Gated DeltaNet + 1 gated full attention], INT8-quantised
weights, FP16 paged KV cache), synthetic token ids, random-init weights.  Sequences are partitioned
across ranks (one process per GPU, model replicated, no collective on the data path), so N GPUs run
N x 128 sequences: weak scaling.  The same line also carries `strong`: one batch of 128 sequences
partitioned s mod N over the ranks (128 / N per GPU).  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "E2E tok/s, bs128 pp1024/tg512, 1-8 B200; attn % of HBM/TC roofline"
UNIT = "tok/s"
NUM_LAYERS, INTER, VOCAB = 24, 3584, 248320

# Algorithmic bytes / flops per launch of the kernels the roofline object can describe.
def algo_la_decode_bytes(n_seqs: int) -> float:
    # per (sequence, layer, step): 2 MiB of fp32 state (read + write), conv cache 3*6144*4 B read + written,
    # projection row 8224*4 B read, 2048 outputs (bf16) written
    return n_seqs * (2 * 16 * 128 * 128 * 4 + 2 * 3 * 6144 * 4 + 8224 * 4 + 2048 * 2)


def algo_fa_decode_bytes(n_seqs: int, ctx_len: float, fp16: bool) -> float:
    # per (sequence, layer, step) at cache length L: K and V rows (+ scales for INT8) read once for all 8 q heads,
    # q (fp16) + gate (fp16) read, output (bf16) written
    per_tok = 2 * 2 * 256 * (2 if fp16 else 1) + (0 if fp16 else 2 * 2 * 4)
    return n_seqs * (per_tok * ctx_len + 8 * 256 * (2 + 2 + 2))


def algo_fa_prefill_flops(n_seqs: int, length: int) -> float:
    return n_seqs * 2.0 * (2 * 8 * 256) * length * (length + 1) / 2      # causal QK^T + PV


def algo_la_prefill_flops(n_seqs: int, length: int) -> float:
    # chunk-64 gated delta rule, per (chunk, head): five 64x64x128 products (K K^T, Q K^T, T K, T V, A V_new), three
    # 64x128x128 products (W S, Q S, K^T V_new) and the triangular solve: 11.6 MFLOP
    per_chunk_head = 5 * 2 * 64 * 64 * 128 + 3 * 2 * 64 * 128 * 128 + 64 ** 3 / 3
    return n_seqs * 16 * (-(-length // 64)) * per_chunk_head


def ncu_traffic(kernel: str, scale: float):
    """DRAM bytes (read + write) of one launch of `kernel` from the committed ncu summary of its small case
    (profiles/<kernel>_kernel_small_case.md, last captured launch), scaled by `scale` = units of a bench launch /
    units of the captured launch.  None if the summary is missing."""
    path = os.path.join(ROOT, "profiles", f"{kernel}_kernel_small_case.md")
    if not os.path.exists(path):
        return None
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total, seen = 0.0, 0
    for line in open(path):
        cells = [c.strip() for c in line.split("|")]
        if len(cells) >= 4 and cells[1] in ("`dram__bytes_read.sum`", "`dram__bytes_write.sum`") and cells[3] in unit:
            total += float(cells[2].replace(",", "")) * unit[cells[3]]
            seen += 1
    return total * scale if seen == 2 else None


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU classes (oracle/_ref) or the C restatement, on the host cores
# ------------------------------------------------------------------------------------------------------
class CpuArm:
    """The reference's CPU path for the same job on the host cores: each thread drives ONE sequence through the
    24-layer CPU stack (reference FullAttention / LinearAttention / MLP classes from oracle/_ref when present,
    else the C restatement) for a bounded number of tokens, greedy."""

    def __init__(self, prompt_tokens: int, gen_tokens: int, threads: int, seed: int = 1234):
        import psutil
        from oracle import cpu_oracle as O, cpu_stack
        synth = entry.load_package().synth
        O.build()
        self.use_ref = O.have_ref()
        self.P, self.G = prompt_tokens, gen_tokens
        weights = cpu_stack.make_stack_weights(synth, seed, NUM_LAYERS, INTER, VOCAB, int8=False)   # the CPU classes take fp32 weights
        qw = dict(layers=weights["layers"], embed=weights["embed"], final_norm=weights["final_norm"])
        per_seq_gb = 2.1 if self.use_ref else 0.1            # the reference classes copy their weights per object
        free_gb = psutil.virtual_memory().available / 2**30
        self.threads = max(1, min(threads, int((free_gb - 8) / per_seq_gb)))
        self.make = lambda: [cpu_stack.OracleStackSequence(qw, self.P + self.G + 1, kv_mode=0, use_ref=self.use_ref)
                             for _ in range(self.threads)]
        self.toks = synth.rng(seed, "cpu.tokens").integers(0, VOCAB, (self.threads, self.P))
        self.sample = (f"{self.threads} sequences (one per host thread) x ({self.P} prompt + {self.G} generated tokens) through the "
                       f"24-layer stack, context <= {self.P + self.G} tokens; fp32 weights, fp32 KV")
        self.kind = "reference" if self.use_ref else "port"

    def step(self) -> float:
        """One bounded sample; returns tokens/s over all threads (fresh caches every call)."""
        seqs = self.make()

        def work(i):
            logits = None
            for t in range(self.P):
                _, logits = seqs[i].forward_token(int(self.toks[i, t]), want_logits=(t == self.P - 1))
            tok = int(np.argmax(logits))
            for _ in range(self.G):
                _, logits = seqs[i].forward_token(tok)
                tok = int(np.argmax(logits))

        t0 = time.time()
        ths = [threading.Thread(target=work, args=(i,)) for i in range(self.threads)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        self.seconds = time.time() - t0
        return self.threads * (self.P + self.G) / self.seconds


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm(args.cpu_prompt, args.cpu_gen, os.cpu_count() or 1)
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        v = arm.step()
        if i >= args.warmup:
            vals.append(v); secs.append(arm.seconds)
    v = statistics.mean(vals)
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=statistics.mean(secs) * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
                data="synthetic", impl="reference", config=workload_config(args),
                cpu_baseline=dict(value=v, unit=UNIT, cores=arm.threads, kind=arm.kind, sample=arm.sample),
                e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


def workload_config(args) -> dict:
    return dict(workload="24-layer hybrid stack (18 Gated DeltaNet + 6 gated full attention, FFN 3584, vocab 248320, tied "
                         "embeddings), fp16 weights carrying INT8 per-output-channel quantised values, FP16 paged KV, greedy decode",
                batch_per_gpu=args.batch, prompt_len=args.prompt, gen_len=args.gen,
                parallelism=f"replica per GPU, sequences partitioned ({args.batch} per GPU)",
                l2="inputs larger than L2: each decode step streams 4.8 GB of DeltaNet state and the KV cache")


# ------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------
def prefill_chunk_seqs(args) -> int:
    """Activation scratch sized so the whole batch's prompt goes through each layer in one pass."""
    return -(-args.batch * args.prompt // (args.prompt + args.gen))


def build_stack(ops, synth, args, seed=1234):
    st = ops.HybridStack(num_layers=NUM_LAYERS, intermediate_size=INTER, vocab_size=VOCAB, max_seqs=args.batch,
                         max_seq_len=args.prompt + args.gen, prefill_chunk_seqs=prefill_chunk_seqs(args),
                         kv_dtype=ops.KV_FP16, int8_weights=True)
    for i in range(NUM_LAYERS):
        lw = dict(input_norm=np.zeros(1024, np.float32), post_norm=np.zeros(1024, np.float32))
        ffn = synth.ffn_weights(seed, f"L{i}")
        fa = synth.fa_weights(seed, f"L{i}.fa") if synth.is_full_attention_layer(i) else None
        la = None if fa is not None else synth.la_weights(seed, f"L{i}.la")
        st.set_layer_weights(i, lw, ffn, fa=fa, la=la)
    st.init_embedding_random(seed, 0.02, np.zeros(1024, np.float32))
    return st


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--gen", type=int, default=512)
    ap.add_argument("--cpu-prompt", type=int, default=24)
    ap.add_argument("--cpu-gen", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import importlib
    import torch
    import torch.distributed as dist
    entry.load_package()
    replica = importlib.import_module(entry.PKG_NAME + ".replica")
    rank, world, local = replica.env_rank()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    if world > 1:
        replica.init("nccl", local)
    ops = entry.load_ops()
    synth = entry.load_package().synth
    peaks = read_peaks()

    st = build_stack(ops, synth, args)
    B, P, G = args.batch, args.prompt, args.gen
    stream = torch.cuda.Stream()
    h_tokens = torch.from_numpy(synth.rng(77 + rank, "bench.tokens").integers(0, VOCAB, (B, P)).astype(np.int32)).pin_memory()
    d_tokens = h_tokens.cuda()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def job_device():
        """Whole job with inputs resident in HBM: reset, prefill, G captured decode steps."""
        st.reset_cache()
        first = st.forward_batch_prefill(d_tokens)
        st.set_tokens(first)
        st.launch_decode(G)          # G captured decode steps; the cache ends at P + G tokens

    h_ring = [torch.empty(B, dtype=torch.int32).pin_memory() for _ in range(2)]
    ring_ev = [torch.cuda.Event() for _ in range(2)]
    e2e_check = [0]

    def job_e2e():
        """Same job through the public API with host buffers: prompt ids H2D, generated ids D2H every step.  The ids of
        step i are read on the host while step i + 1 runs (two pinned buffers, one event each), as a serving loop that
        streams tokens out would do; every step's ids do reach the host inside the timed region."""
        cur = torch.cuda.current_stream()
        st.reset_cache()
        dev = h_tokens.to("cuda", non_blocking=True)
        first = st.forward_batch_prefill(dev)
        st.set_tokens(first)
        h_ring[0].copy_(first, non_blocking=True)
        ring_ev[0].record(cur)
        for i in range(1, G + 1):
            st.launch_decode(1)
            h_ring[i & 1].copy_(st.get_tokens(B), non_blocking=True)
            ring_ev[i & 1].record(cur)
            ring_ev[(i - 1) & 1].synchronize()                  # the previous step's ids are on the host now
            e2e_check[0] ^= int(h_ring[(i - 1) & 1][0])
        ring_ev[G & 1].synchronize()
        e2e_check[0] ^= int(h_ring[G & 1][0])

    with torch.cuda.stream(stream):
        # one eager pass warms cuBLAS heuristics and kernel attributes, then the decode step is captured once
        st.reset_cache()
        first = st.forward_batch_prefill(d_tokens)
        st.forward_batch_decode(first)
        stream.synchronize()
        status = st.device_status()
        assert status == 0, f"device status {status} after the first eager step: a kernel gave up on a bounded wait"
        st.set_tokens(first)
        st.capture_decode(B)
        for _ in range(args.warmup):
            job_device()
        stream.synchronize()
        barrier()
        clocks = ClockSampler(local)
        if rank == 0:
            clocks.start()
        ops.launch_count(reset=True)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            job_device()
        ev1.record(stream)
        stream.synchronize()
        barrier()
        launches = ops.launch_count(reset=True)
        clk = clocks.stop() if rank == 0 else {}
        ms_total = ev0.elapsed_time(ev1)
        status = st.device_status()
        assert status == 0, f"device status {status} after the timed region"

        # end-to-end arm (host buffers, copies inside the timed region)
        job_e2e()
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record(stream)
        for _ in range(args.steps):
            job_e2e()
        ev3.record(stream)
        stream.synchronize()
        barrier()
        ms_e2e = ev2.elapsed_time(ev3)

        # per-kernel device times (rank 0): the prefill kernels in an eager pass (milliseconds each, launch gaps do not
        # matter), the decode kernels inside a captured decode step with event-record nodes around them, so that an
        # event pair sees exactly one kernel and no CPU launch gap.  The decode attention kernel is read twice: in the
        # first steps after the prompt (cache length P + 2) and in the middle of the job (P + G / 2).
        prof, phases, timing, fa_mid = {}, {}, "", None
        if rank == 0:
            st.reset_cache()
            ops.profile_reset(); ops.profile_enable(True)
            first = st.forward_batch_prefill(d_tokens)
            stream.synchronize()
            for name in ("fa_prefill", "la_prefill", "kv_append"):
                prof[name] = ops.profile_read(name)
            ops.profile_reset()
            st.set_tokens(first)
            st.capture_decode(B)                       # the captured attention kernels carry time-stamp slots
            ops.profile_enable(False)

            def read_steps(k):
                acc = dict(fa_decode=[0.0, 0], la_decode=[0.0, 0])
                stream.synchronize()
                for name in acc:                       # a read arms the slots again: drop what earlier replays left
                    ops.profile_read(name)
                for _ in range(k):
                    st.launch_decode(1)
                    stream.synchronize()
                    for name in acc:
                        ms, cnt = ops.profile_read(name)
                        acc[name][0] += ms; acc[name][1] += cnt
                return {k2: tuple(v) for k2, v in acc.items()}
            early = read_steps(max(1, min(4, G // 4)))
            timing = "in-kernel time stamps (first CTA past its dependency wait .. last CTA done) inside the captured decode step, programmatic dependent launch on"
            if early["la_decode"][1] == 0 or early["fa_decode"][1] == 0:
                raise RuntimeError("the stamped decode step returned no times")
            prof.update(early)
            if G // 2 - 6 > 0:
                st.launch_decode(G // 2 - 6)
                fa_mid = read_steps(4)["fa_decode"]
            st.capture_decode(B)                       # back to the plain graph before the events go away
            ops.profile_reset()
            # where the job time goes: prefill pass vs captured decode steps
            job_device()
            ea, eb, ec = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            st.reset_cache()
            ea.record(stream)
            first = st.forward_batch_prefill(d_tokens)
            st.set_tokens(first)
            eb.record(stream)
            st.launch_decode(G)
            ec.record(stream)
            stream.synchronize()
            phases = dict(prefill_ms=ea.elapsed_time(eb), decode_step_ms=eb.elapsed_time(ec) / G)

        # The contract's split of ONE batch: sequence s belongs to rank s mod N, so every rank runs B / N sequences of
        # the same job (its own pages, states and captured step).  Timed like the headline: max over ranks.
        strong = None
        if world > 1:
            mine = list(replica.partition(B, world, rank))
            ns = len(mine)
            d_tok_s = d_tokens[:ns].contiguous()

            def job_strong():
                st.reset_cache()
                f = st.forward_batch_prefill(d_tok_s)
                st.set_tokens(f)
                st.launch_decode(G)
            st.reset_cache()
            f = st.forward_batch_prefill(d_tok_s)
            st.set_tokens(f)
            st.capture_decode(ns)
            job_strong()
            stream.synchronize()
            barrier()
            es = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            es[0].record(stream)
            job_strong()
            es[1].record(stream)
            stream.synchronize()
            barrier()
            st.reset_cache()
            es[2].record(stream)
            f = st.forward_batch_prefill(d_tok_s)
            st.set_tokens(f)
            es[3].record(stream)
            stream.synchronize()
            strong = [es[0].elapsed_time(es[1]), es[2].elapsed_time(es[3]), float(ns)]

    # NCCL: the only collective of the run, and only on the counters (max of the times, sum of the tokens)
    tokens_per_job = B * (P + G)
    mx = [ms_total, ms_e2e] + (strong[:2] if strong else [])
    sm = [float(tokens_per_job * args.steps)] + ([strong[2]] if strong else [])
    mx, sm = replica.reduce_counters(mx, sm, "cuda")
    ms_total, ms_e2e, tokens_all = mx[0], mx[1], sm[0]
    value = replica.job_throughput(tokens_all, ms_total)
    e2e_value = replica.job_throughput(tokens_all, ms_e2e)

    if rank == 0:
        chunks = -(-B // max(1, (prefill_chunk_seqs(args) * (P + G)) // P))
        per = {k: (v[0] / max(v[1], 1)) for k, v in prof.items()}       # ms per launch
        # share of one whole job spent in each kernel class (launch counts of a full job x measured ms per launch)
        job_ms = dict(la_decode=per["la_decode"] * 18 * G, fa_decode=per["fa_decode"] * 6 * G,
                      fa_prefill=prof["fa_prefill"][0], la_prefill=prof["la_prefill"][0])
        ctx_avg = P + 2.5                                                # cache length the first timed decode launches saw
        seqs_per_chunk = B / max(chunks, 1)
        roof = dict(
            la_decode=dict(bound="hbm", achieved=algo_la_decode_bytes(B) / (per["la_decode"] * 1e-3) / 1e9, peak=peaks["hbm_gbs"], unit="GB/s"),
            fa_decode=dict(bound="hbm", achieved=algo_fa_decode_bytes(B, ctx_avg, True) / (per["fa_decode"] * 1e-3) / 1e9, peak=peaks["hbm_gbs"], unit="GB/s"),
            fa_prefill=dict(bound="tensor", achieved=algo_fa_prefill_flops(seqs_per_chunk, P) / (per["fa_prefill"] * 1e-3) / 1e12, peak=peaks["tflops_sustained"], unit="TFLOP/s"),
            la_prefill=dict(bound="tensor", achieved=algo_la_prefill_flops(seqs_per_chunk, P) / (per["la_prefill"] * 1e-3) / 1e12, peak=peaks["tflops_sustained"], unit="TFLOP/s"),
        )
        # units of one bench launch / units of the launch captured under ncu (kernel_bench.py commands in profiles/):
        # la_decode 128 sequences; fa_decode 128 sequences x 1280 cached tokens; fa_prefill 16 and la_prefill 18 sequences x 1024
        traffic_scale = dict(la_decode=B / 128.0, fa_decode=(B / 128.0) * (ctx_avg / 1280.0), fa_prefill=seqs_per_chunk * P / (16.0 * 1024),
                             la_prefill=seqs_per_chunk * P / (18.0 * 1024))
        for k, r in roof.items():
            r.update(kernel=k, frac=r["achieved"] / r["peak"], ms_per_launch=per[k], timing=(timing if k.endswith("decode") else "eager launches"), job_ms=job_ms[k],
                     ctx_len=(ctx_avg if k == "fa_decode" else None),
                     traffic=ncu_traffic(k, traffic_scale[k]), traffic_source="ncu capture of the small case in profiles/, scaled by the units one bench launch processes",
                     peak_source=peaks["source"])
        # The same two decode kernels timed as back-to-back launches on caches of their own (no event pair per launch, no
        # neighbours): what the kernel itself does, next to what it does inside the step.
        if fa_mid and fa_mid[1]:
            ms_mid, ctx_mid = fa_mid[0] / fa_mid[1], P + G // 2
            a_mid = algo_fa_decode_bytes(B, ctx_mid, True) / (ms_mid * 1e-3) / 1e9
            roof["fa_decode"]["mid_job"] = dict(ctx_len=ctx_mid, ms_per_launch=ms_mid, achieved=a_mid, frac=a_mid / peaks["hbm_gbs"], timing=timing)
        extra = []
        try:
            import kernel_bench as kb
            with torch.cuda.stream(stream):
                iso = dict(la_decode=kb.measure("la_decode", seqs=B, layers=4, iters=40),
                           fa_decode=kb.measure("fa_decode", seqs=B, ctx=P + G // 2, kv="fp16", layers=2, iters=40))
                i8 = kb.measure("fa_decode", seqs=B, ctx=P + G // 2, kv="int8", layers=2, iters=40)
            for k, m in iso.items():
                roof[k]["isolated"] = dict(ms_per_launch=m["ms"], achieved=m["achieved"], frac=m["frac"], ctx_len=m.get("ctx"),
                                           note="back-to-back launches through the core entry" + ("; includes its query-conversion launch" if k == "fa_decode" else ""))
            extra.append(dict(kernel="fa_decode_int8", bound="hbm", achieved=i8["achieved"], peak=peaks["hbm_gbs"], unit="GB/s", frac=i8["achieved"] / peaks["hbm_gbs"],
                              ms_per_launch=i8["ms"], ctx_len=P + G // 2, timing="back-to-back launches through the core entry on an INT8 cache "
                              "(includes its query-conversion launch); the job itself runs the FP16 cache",
                              traffic=ncu_traffic("fa_decode_int8", (B / 128.0) * ((P + G // 2) / 1280.0)),
                              traffic_source="ncu capture of the small case in profiles/, scaled by the units one bench launch processes", peak_source=peaks["source"]))
        except Exception as e:          # the job's own numbers stand without it
            roof["la_decode"]["isolated"] = dict(error=str(e)[:200])
        dominant = max(job_ms, key=job_ms.get)
        cpu = None
        if not args.no_cpu_baseline:
            arm = CpuArm(args.cpu_prompt, args.cpu_gen, os.cpu_count() or 1)
            cpu = dict(value=arm.step(), unit=UNIT, cores=arm.threads, kind=arm.kind, sample=arm.sample)
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_total / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="fp16",
                    data="synthetic", config=workload_config(args), clocks=clk,
                    e2e=dict(value=e2e_value, unit=UNIT, h2d_bytes_per_step=B * P * 4, d2h_bytes_per_step=B * G * 4),
                    gpu_launches=launches, phases=phases, roofline=roof[dominant], roofline_other=[roof[k] for k in roof if k != dominant] + extra,
                    cpu_baseline=cpu)
        if strong:
            ms_job, ms_pre, nseq = mx[2], mx[3], sm[1]
            line["strong"] = dict(scaling="strong", sequences_total=int(nseq), sequences_per_gpu=int(nseq) // world, tok_s=nseq * (P + G) / (ms_job * 1e-3),
                                  ms_per_job=ms_job, prefill_ms=ms_pre, decode_step_ms=(ms_job - ms_pre) / G,
                                  note="one batch of %d sequences partitioned s mod N; max over ranks; speed-up = tok_s / the N = 1 line's value" % int(nseq))
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
