"""GPU: gated full attention — whole-layer parity with the CPU reference semantics (prefill then
decode, INT8 / FP16 KV), the decode and prefill attention cores against a float64 restatement, and
the tensor-core prefill kernel against the plain SIMT kernel at full length."""
import os

import numpy as np
import pytest

from conftest import allclose_report

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL, RTOL = 2e-3, 1e-2      # max-abs 2e-3 / rel 1e-2 on outputs for fp16/bf16 compute


def _run_layer(ops, torch, w, x, n_prefill, kv_dtype, proj):
    T = x.shape[0]
    fa = ops.FullAttention(proj, max_batch=4, max_prefill_rows=max(256, n_prefill))
    fa.set_weights(w)
    kv = ops.KVCache(1, 4, T + 64, kv_dtype)
    slot = kv.allocate_sequence(T)
    xt = torch.from_numpy(x).cuda()
    outs = [fa.forward_batch_prefill(xt[:n_prefill].contiguous(), kv, 0, [slot], [n_prefill])]
    d_slots = torch.tensor([slot], dtype=torch.int32, device="cuda")
    for t in range(n_prefill, T):
        outs.append(fa.forward(xt[t:t + 1].contiguous(), kv, 0, d_slots))
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert kv.length(0, slot) == T
    return torch.cat(outs).cpu().numpy(), kv, slot


@pytest.mark.parametrize("kv_dtype,kv_mode", [(0, 1), (1, 2)])
def test_layer_prefill128_decode16_fp32_projections(ops, cuda, oracle, synth, kv_dtype, kv_mode):
    """Workload: batch 1, prefill 128 tokens then 16 decode steps, fp32 projections."""
    w = synth.fa_weights(31)
    x = synth.hidden_states(31, "cfg0.x", 144)
    ref = oracle.OracleFullAttention(w, 144, kv_mode=kv_mode)
    want = ref.forward_sequence(x)
    got, kv, slot = _run_layer(ops, cuda, w, x, 128, kv_dtype, ops.PROJ_FP32)
    ok, msg = allclose_report(got, want, ATOL, RTOL)
    assert ok, msg
    if kv_dtype == ops.KV_INT8:
        # codes may differ by one step where the fp32 projection rounds differently; scales track closely
        kc, vc, ks, vs = [t.cpu().numpy() for t in kv.export(0, slot)]
        assert np.abs(kc.reshape(144, 512).astype(int) - ref.k_codes[:144].astype(int)).max() <= 1
        assert np.abs(vc.reshape(144, 512).astype(int) - ref.v_codes[:144].astype(int)).max() <= 1
        assert (kc.reshape(144, 512) != ref.k_codes[:144]).mean() < 0.01
        np.testing.assert_allclose(ks, ref.k_scale[:144], rtol=1e-5)
        np.testing.assert_allclose(vs, ref.v_scale[:144], rtol=1e-5)


def test_layer_against_reference_fixture(ops, cuda, synth):
    """The committed outputs of the reference's own qwen::FullAttention (fp32 cache) on 24 tokens."""
    g = np.load(os.path.join(GOLD, "fa_ref_seed101_t24.npz"))
    seed, T = int(g["seed"]), int(g["tokens"])
    w = synth.fa_weights(seed)
    x = synth.hidden_states(seed, "golden.fa.x", T)
    got, _, _ = _run_layer(ops, cuda, w, x, 20, ops.KV_FP16, ops.PROJ_FP32)
    ok, msg = allclose_report(got, g["y"], ATOL, RTOL)
    assert ok, msg


@pytest.mark.parametrize("kv_dtype,kv_mode", [(0, 1), (1, 2)])
def test_layer_prefill128_decode16_fp16_projections(ops, cuda, oracle, synth, kv_dtype, kv_mode, capsys):
    """The same workload in the precision the benchmark runs: fp16 weights and activations in the projections, fp32
    accumulation.  Held to the same bound as the fp32 mode; the measured error is printed."""
    w = synth.fa_weights(32)
    x = synth.hidden_states(32, "cfg0.fp16.x", 144)
    want = oracle.OracleFullAttention(w, 144, kv_mode=kv_mode).forward_sequence(x)
    got, _, _ = _run_layer(ops, cuda, w, x, 128, kv_dtype, ops.PROJ_FP16)
    ok, msg = allclose_report(got, want, ATOL, RTOL)
    with capsys.disabled():
        print(f"\n[fa fp16 projections, kv_dtype {kv_dtype}] {msg}")
    assert ok, msg


@pytest.mark.parametrize("proj", [0, 1])
def test_int8_decode_512_steps_after_prompt_1024(ops, cuda, oracle, synth, proj, capsys):
    """The INT8-cache decode workload at its stated length on a sub-batch the CPU checker can follow: 4 sequences,
    prompt 1024 then 512 single-token steps (512 quantise-on-append + decode-attention launches per sequence, caches
    growing from 1025 to 1536 tokens across page boundaries), fp32 and fp16 projections.  Outputs of the prompt pass
    and of every step against the oracle; lengths, codes and scales at the end."""
    import threading
    torch = cuda
    n, P, G = 4, 1024, 512
    w = synth.fa_weights(34)
    xs = [synth.hidden_states(34, f"cfg2.{i}", P + G) for i in range(n)]
    want = [None] * n
    refs = [oracle.OracleFullAttention(w, P + G, kv_mode=1) for _ in range(n)]

    def run_ref(i):
        want[i] = refs[i].forward_sequence(xs[i])
    ths = [threading.Thread(target=run_ref, args=(i,)) for i in range(n)]
    [t.start() for t in ths]
    fa = ops.FullAttention(proj, max_batch=n, max_prefill_rows=n * P)
    fa.set_weights(w)
    kv = ops.KVCache(1, n, P + G, ops.KV_INT8)
    slots = [kv.allocate_sequence(P + G) for _ in range(n)]
    xt = [torch.from_numpy(x).cuda() for x in xs]
    y0 = fa.forward_batch_prefill(torch.cat([x[:P] for x in xt]), kv, 0, slots, [P] * n).cpu().numpy()
    d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    steps = []
    for t in range(P, P + G):
        steps.append(fa.forward(torch.stack([x[t] for x in xt]), kv, 0, d_slots))
    got_steps = torch.stack(steps).cpu().numpy()                 # [G, n, 1024]
    assert kv.device_status() == 0
    [t.join() for t in ths]
    worst = ""
    for i in range(n):
        got = np.concatenate([y0[i * P:(i + 1) * P], got_steps[:, i]])
        ok, msg = allclose_report(got, want[i], ATOL, RTOL)
        worst = msg
        assert ok, f"sequence {i}: {msg}"
        assert kv.length(0, slots[i]) == P + G
        kc, vc, ks, vs = [t.cpu().numpy() for t in kv.export(0, slots[i])]
        # the codes follow the projection's rounding (bit-exactness on identical fp32 K/V is tested in test_gpu_kv.py)
        assert np.abs(kc.reshape(P + G, 512).astype(int) - refs[i].k_codes.astype(int)).max() <= 1
        assert np.abs(vc.reshape(P + G, 512).astype(int) - refs[i].v_codes.astype(int)).max() <= 1
        np.testing.assert_allclose(ks, refs[i].k_scale, rtol=2e-3 if proj else 1e-5)
        np.testing.assert_allclose(vs, refs[i].v_scale, rtol=2e-3 if proj else 1e-5)
    with capsys.disabled():
        print(f"\n[fa int8 decode 1024 + 512, proj {proj}] {worst}")


def test_prefill_ragged_batch_and_continuation(ops, cuda, oracle, synth):
    """Three sequences of different lengths in one call, then a second prefill call that continues
    two of them (cache not empty), each compared with its own token-serial reference."""
    torch = cuda
    w = synth.fa_weights(33)
    lens1, lens2 = [5, 130, 64], [70, 0, 3]
    xs = [synth.hidden_states(33, f"rag.{i}", lens1[i] + lens2[i]) for i in range(3)]
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=4, max_prefill_rows=512)
    fa.set_weights(w)
    kv = ops.KVCache(1, 4, 256, ops.KV_INT8)
    slots = [kv.allocate_sequence(0) for _ in range(3)]
    x1 = torch.from_numpy(np.concatenate([xs[i][:lens1[i]] for i in range(3)])).cuda()
    y1 = fa.forward_batch_prefill(x1, kv, 0, slots, lens1).cpu().numpy()
    x2 = torch.from_numpy(np.concatenate([xs[i][lens1[i]:] for i in range(3)])).cuda()
    y2 = fa.forward_batch_prefill(x2, kv, 0, slots, lens2).cpu().numpy()
    assert kv.device_status() == 0
    o1 = o2 = 0
    for i in range(3):
        want = oracle.OracleFullAttention(w, 256, kv_mode=1).forward_sequence(xs[i])
        got = np.concatenate([y1[o1:o1 + lens1[i]], y2[o2:o2 + lens2[i]]])
        o1 += lens1[i]; o2 += lens2[i]
        ok, msg = allclose_report(got, want, ATOL, RTOL)
        assert ok, f"sequence {i}: {msg}"
        assert kv.length(0, slots[i]) == lens1[i] + lens2[i]


def _attention_f64(q, k, v):
    """softmax(q k^T / 16) v for one kv group: q [heads, 256], k/v [L, 256] (float64)."""
    s = (q @ k.T) / 16.0
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(axis=1, keepdims=True)) @ v


@pytest.mark.parametrize("kv_dtype", [0, 1])
@pytest.mark.parametrize("lengths", [[1, 63, 64, 65], [130, 1025, 384, 7]])
def test_decode_core_against_float64(ops, cuda, oracle, synth, kv_dtype, lengths):
    torch = cuda
    n = len(lengths)
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=8, max_prefill_rows=64)
    kv = ops.KVCache(1, 8, 1536, kv_dtype)
    slots = [kv.allocate_sequence(0) for _ in range(n)]
    ks = [synth.normal(41, f"dc.k.{i}.{L}", (L, 512), 1.0) for i, L in enumerate(lengths)]
    vs = [synth.normal(41, f"dc.v.{i}.{L}", (L, 512), 0.6) for i, L in enumerate(lengths)]
    kv.append(0, slots, lengths, torch.from_numpy(np.concatenate(ks)).cuda(), torch.from_numpy(np.concatenate(vs)).cuda())
    q = synth.normal(41, "dc.q", (n, 8, 256), 1.0)
    out = fa.decode_core(torch.from_numpy(q).cuda(), kv, 0, torch.tensor(slots, dtype=torch.int32, device="cuda")).cpu().numpy()
    assert kv.device_status() == 0
    qh = q.astype(np.float16).astype(np.float64)
    for i, L in enumerate(lengths):
        if kv_dtype == ops.KV_INT8:
            kc, ksc = oracle.quantize_rows(ks[i].reshape(L, 2, 256)); vc, vsc = oracle.quantize_rows(vs[i].reshape(L, 2, 256))
            kd = kc.astype(np.float64) * ksc[..., None]; vd = vc.astype(np.float64) * vsc[..., None]
        else:
            kd = ks[i].reshape(L, 2, 256).astype(np.float16).astype(np.float64)
            vd = vs[i].reshape(L, 2, 256).astype(np.float16).astype(np.float64)
        for g in range(2):
            want = _attention_f64(qh[i, 4 * g:4 * g + 4], kd[:, g], vd[:, g])
            err = np.abs(out[i, 4 * g:4 * g + 4] - want).max()
            assert err <= 2e-3, f"seq {i} (L={L}) group {g}: max abs err {err:.3e}"


@pytest.mark.parametrize("kv_dtype", [0, 1])
def test_decode_core_full_batch_against_float64(ops, cuda, kv_dtype):
    """The decode configuration at full size: 128 sequences with ragged caches of 1025 .. 1536 tokens (INT8 and FP16),
    one decode step, every sequence checked against a float64 softmax over the exported cache contents (so the check
    does not depend on the append path, which has its own bit-exact tests).  At this size every consumer warp of the
    persistent kernel works through several (sequence, kv head) pairs and most pairs are split between warps."""
    torch = cuda
    n = 128
    g = torch.Generator(device="cuda").manual_seed(43)
    lengths = (1025 + torch.randint(0, 512, (n,), generator=g, device="cuda")).tolist()
    lengths[0], lengths[1], lengths[2] = 1025, 1536, 1088
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=n, max_prefill_rows=64)
    kv = ops.KVCache(1, n, 1536, kv_dtype)
    slots = [kv.allocate_sequence(0) for _ in range(n)]
    for s0 in range(0, n, 16):
        cnt = lengths[s0:s0 + 16]
        k = torch.randn((sum(cnt), 512), device="cuda", generator=g)
        v = torch.randn((sum(cnt), 512), device="cuda", generator=g) * 0.6
        kv.append(0, slots[s0:s0 + 16], cnt, k, v)
    q = torch.randn((n, 8, 256), device="cuda", generator=g)
    out = fa.decode_core(q, kv, 0, torch.tensor(slots, dtype=torch.int32, device="cuda"))
    assert kv.device_status() == 0
    q64 = q.half().double()
    worst = 0.0
    for i in range(n):
        kc, vc, ksc, vsc = kv.export(0, slots[i])
        kd, vd = kc.double(), vc.double()
        if ksc is not None:
            kd, vd = kd * ksc.double()[..., None], vd * vsc.double()[..., None]
        assert kd.shape[0] == lengths[i]
        for grp in range(2):
            sc = q64[i, 4 * grp:4 * grp + 4] @ kd[:, grp].T / 16.0
            p = torch.softmax(sc, dim=1)
            want = p @ vd[:, grp]
            worst = max(worst, float((out[i, 4 * grp:4 * grp + 4].double() - want).abs().max()))
    assert worst <= 2e-3, f"max abs err {worst:.3e}"


@pytest.mark.parametrize("counts", [[1], [64], [65, 128], [200, 3, 129]])
def test_prefill_core_against_float64(ops, cuda, synth, counts):
    torch = cuda
    rows = sum(counts)
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=4, max_prefill_rows=512)
    q = synth.normal(42, f"pc.q.{rows}", (rows, 8, 256), 1.0)
    k = synth.normal(42, f"pc.k.{rows}", (rows, 2, 256), 1.0)
    v = synth.normal(42, f"pc.v.{rows}", (rows, 2, 256), 0.6)
    args = [torch.from_numpy(a).cuda() for a in (q, k, v)]
    out_tc = fa.prefill_core(*args, counts, use_tensor_cores=True).cpu().numpy()
    out_simt = fa.prefill_core(*args, counts, use_tensor_cores=False).cpu().numpy()
    q64, k64, v64 = [a.astype(np.float16).astype(np.float64) for a in (q, k, v)]
    r0 = 0
    for c in counts:
        for t in range(c):
            for g in range(2):
                want = _attention_f64(q64[r0 + t, 4 * g:4 * g + 4], k64[r0:r0 + t + 1, g], v64[r0:r0 + t + 1, g])
                for name, out in (("tcgen05", out_tc), ("simt", out_simt)):
                    err = np.abs(out[r0 + t, 4 * g:4 * g + 4] - want).max()
                    assert err <= 2e-3, f"{name}: row {r0 + t} group {g}: max abs err {err:.3e}"
        r0 += c


def test_prefill_core_full_length_tensor_core_vs_simt(ops, cuda, synth):
    """Two sequences of 1024 tokens: the tcgen05 kernel against the SIMT kernel (size-independent check)."""
    torch = cuda
    counts = [1024, 1024]
    rows = sum(counts)
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=4, max_prefill_rows=rows)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((rows, 8, 256), device="cuda", generator=g)
    k = torch.randn((rows, 2, 256), device="cuda", generator=g)
    v = torch.randn((rows, 2, 256), device="cuda", generator=g) * 0.6
    a = fa.prefill_core(q, k, v, counts, use_tensor_cores=True)
    b = fa.prefill_core(q, k, v, counts, use_tensor_cores=False)
    err = (a - b).abs().max().item()
    assert err <= 2e-3, f"max abs diff {err:.3e}"
    # causality: output rows of the first sequence do not depend on the second sequence's inputs
    k2 = k.clone(); k2[1024:] += 1.0
    c = fa.prefill_core(q, k2, v, counts, use_tensor_cores=True)
    assert torch.equal(a[:1024], c[:1024])


def test_errors(ops, cuda, synth):
    torch = cuda
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=64)
    kv = ops.KVCache(1, 2, 256, ops.KV_INT8)
    s = kv.allocate_sequence(8)
    x = torch.zeros((4, 1024), device="cuda")
    with pytest.raises(ops.B200AttnError) as e:       # weights not set -> the reference throws runtime_error
        fa.forward_batch_prefill(x, kv, 0, [s], [4])
    assert e.value.status == ops.ERR_NOT_READY and "weights not set" in str(e.value)
    fa.set_weights(synth.fa_weights(1))
    with pytest.raises(ops.InvalidArgument):
        fa.forward_batch_prefill(torch.zeros((100, 1024), device="cuda"), kv, 0, [s], [100])   # > max_prefill_rows
    with pytest.raises(ops.InvalidArgument):
        fa.forward(torch.zeros((3, 1024), device="cuda"), kv, 0, torch.zeros(3, dtype=torch.int32, device="cuda"))
