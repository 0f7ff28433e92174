"""GPU: Gated DeltaNet — whole-layer parity with the CPU reference semantics (sequence pass and
recurrent decode, outputs and final state), the recurrence cores against each other, state
import/export in the reference's layouts."""
import os

import numpy as np
import pytest

from conftest import allclose_report

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL, RTOL, STATE_REL = 2e-3, 1e-2, 1e-3


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def test_layer_prefill1024_outputs_and_final_state(ops, cuda, oracle, synth):
    """Workload: batch 1, 1024 tokens, zero initial state, fp32 projections; compare outputs and final state."""
    torch = cuda
    w = synth.la_weights(51)
    x = synth.hidden_states(51, "cfg1.x", 1024)
    ref = oracle.OracleLinearAttention(w)
    want = ref.forward_sequence(x)
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=1024)
    la.set_weights(w)
    st = ops.LinearAttnState(1, 2)
    got = la.forward_batch(torch.from_numpy(x).cuda(), st, 0, [1], [1024]).cpu().numpy()
    ok, msg = allclose_report(got, want, ATOL, RTOL)
    assert ok, msg
    rec, conv = st.export_state(0, 1)
    assert _rel(rec.cpu().numpy(), ref.recurrent) <= STATE_REL
    np.testing.assert_allclose(conv.cpu().numpy(), ref.conv_state, rtol=1e-4, atol=1e-5)


def test_layer_against_reference_fixture(ops, cuda, synth):
    torch = cuda
    g = np.load(os.path.join(GOLD, "la_ref_seed202_t24.npz"))
    seed, T = int(g["seed"]), int(g["tokens"])
    w = synth.la_weights(seed)
    x = synth.hidden_states(seed, "golden.la.x", T)
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=64)
    la.set_weights(w)
    st = ops.LinearAttnState(1, 1)
    xt = torch.from_numpy(x).cuda()
    d_slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = [la.forward_batch(xt[:20].contiguous(), st, 0, [0], [20])]
    for t in range(20, T):
        got.append(la.forward(xt[t:t + 1].contiguous(), st, 0, d_slots))
    got = torch.cat(got).cpu().numpy()
    ok, msg = allclose_report(got, g["y"], ATOL, RTOL)
    assert ok, msg
    rec, conv = st.export_state(0, 0)
    assert _rel(rec.cpu().numpy()[g["recurrent_heads"]], g["recurrent"]) <= STATE_REL
    np.testing.assert_allclose(conv.cpu().numpy(), g["conv"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("kernel,occ", [("classic", ""), ("classic", "512"), ("stream", ""), ("prefetch", "")])
def test_decode_from_seeded_state(ops, cuda, oracle, synth, monkeypatch, kernel, occ):
    """Recurrent decode: 4 sequences, state ~ N(0, 0.05) and a warm conv cache imported in the
    reference's layouts, 24 single-token steps; outputs every step, state at the end.  Every form of the decode
    kernel: one CTA per unit with 256 threads or 512 threads, the persistent one with a TMA state ring, and the
    persistent one that prefetches the next state by TMA; the library reads the variables per call."""
    monkeypatch.setenv("B200ATTN_LA_DECODE", kernel)
    monkeypatch.setenv("B200ATTN_LA_DECODE_OCC", occ)
    torch = cuda
    w = synth.la_weights(52)
    n, steps = 4, 24
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=n, max_prefill_rows=64)
    la.set_weights(w)
    st = ops.LinearAttnState(2, n)
    refs = []
    for i in range(n):
        r = oracle.OracleLinearAttention(w)
        r.recurrent[:] = synth.normal(52, f"state.{i}", (16, 128, 128), 0.05)
        r.conv_state[:] = synth.normal(52, f"conv.{i}", (6144, 3), 0.5)
        st.import_state(1, i, torch.from_numpy(r.recurrent).cuda(), torch.from_numpy(r.conv_state).cuda())
        refs.append(r)
    # import/export round trip is exact
    rec, conv = st.export_state(1, 2)
    np.testing.assert_array_equal(rec.cpu().numpy(), refs[2].recurrent)
    np.testing.assert_array_equal(conv.cpu().numpy(), refs[2].conv_state)
    d_slots = torch.arange(n, dtype=torch.int32, device="cuda")
    for t in range(steps):
        x = synth.hidden_states(52, f"step.{t}", n)
        got = la.forward(torch.from_numpy(x).cuda(), st, 1, d_slots).cpu().numpy()
        want = np.stack([refs[i].forward(x[i]) for i in range(n)])
        ok, msg = allclose_report(got, want, ATOL, RTOL)
        assert ok, f"step {t}: {msg}"
    for i in range(n):
        rec, conv = st.export_state(1, i)
        assert _rel(rec.cpu().numpy(), refs[i].recurrent) <= STATE_REL
        np.testing.assert_allclose(conv.cpu().numpy(), refs[i].conv_state, rtol=1e-4, atol=1e-5)
    rec0, _ = st.export_state(0, 0)          # the other layer was never touched
    assert not rec0.any()


def test_decode_full_batch_against_oracle(ops, cuda, oracle, synth):
    """The recurrent-decode configuration at full batch: 128 sequences (2048 (sequence, head) units, several waves of
    CTAs) with seeded states and conv caches, two single-token steps through the whole layer, every sequence against
    the CPU oracle; states of a sample of sequences at the end."""
    torch = cuda
    w = synth.la_weights(58)
    n, steps = 128, 2
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=n, max_prefill_rows=64)
    la.set_weights(w)
    st = ops.LinearAttnState(1, n)
    refs = []
    for i in range(n):
        r = oracle.OracleLinearAttention(w)
        r.recurrent[:] = synth.normal(58, f"state.{i}", (16, 128, 128), 0.05)
        r.conv_state[:] = synth.normal(58, f"conv.{i}", (6144, 3), 0.5)
        st.import_state(0, i, torch.from_numpy(r.recurrent).cuda(), torch.from_numpy(r.conv_state).cuda())
        refs.append(r)
    d_slots = torch.arange(n, dtype=torch.int32, device="cuda")
    for t in range(steps):
        x = synth.hidden_states(58, f"step.{t}", n)
        got = la.forward(torch.from_numpy(x).cuda(), st, 0, d_slots).cpu().numpy()
        want = np.stack([refs[i].forward(x[i]) for i in range(n)])
        ok, msg = allclose_report(got, want, ATOL, RTOL)
        assert ok, f"step {t}: {msg}"
    for i in (0, 1, 63, 64, 127):
        rec, conv = st.export_state(0, i)
        assert _rel(rec.cpu().numpy(), refs[i].recurrent) <= STATE_REL
        np.testing.assert_allclose(conv.cpu().numpy(), refs[i].conv_state, rtol=1e-4, atol=1e-5)
    assert la.device_status() == 0


def test_persistent_decode_kernels_equal_classic_kernel(ops, cuda, synth, monkeypatch):
    """72 sequences x 16 heads = 1152 units on 148 (state ring) or 444 (prefetch) persistent CTAs: every CTA walks
    several units (stage reuse, write-back, refill).  They do the same arithmetic in the same order as the 256-thread
    one-CTA-per-unit kernel, so outputs, recurrent states and conv states must be identical bit for bit.  One slot is
    out of range and must be skipped."""
    torch = cuda
    n, steps = 72, 3
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=n, max_prefill_rows=64)
    la.set_weights(synth.la_weights(57))
    g = torch.Generator(device="cuda").manual_seed(57)
    results = {}
    monkeypatch.setenv("B200ATTN_LA_DECODE_OCC", "3")     # 256 threads, 16 state rows per warp, as in the persistent kernel
    for kernel in ("classic", "stream", "prefetch"):
        monkeypatch.setenv("B200ATTN_LA_DECODE", kernel)
        st = ops.LinearAttnState(1, n)
        g.manual_seed(57)
        for i in range(0, n, 9):
            st.import_state(0, i, torch.randn((16, 128, 128), device="cuda", generator=g) * 0.05,
                            torch.randn((6144, 3), device="cuda", generator=g) * 0.5)
        slots = torch.arange(n, dtype=torch.int32, device="cuda")
        slots[5] = -1
        outs = []
        for t in range(steps):
            mixed = torch.randn((n, 8224), device="cuda", generator=g) * 0.6
            outs.append(la.decode_core(mixed, st, 0, slots).clone())
        states = [st.export_state(0, i) for i in (0, 5, 9, 36, 71)]
        results[kernel] = (outs, states)
        assert la.device_status() == 0
    keep = torch.ones(n, dtype=torch.bool, device="cuda")
    keep[5] = False                          # the skipped sequence's output rows are not written by any kernel
    for other in ("stream", "prefetch"):
        for a, b in zip(results["classic"][0], results[other][0]):
            assert torch.equal(a[keep], b[keep]), other
        for (ra, ca), (rb, cb) in zip(results["classic"][1], results[other][1]):
            assert torch.equal(ra, rb) and torch.equal(ca, cb), other
        assert not results[other][1][1][0].any()     # slot 5's state was never touched


def test_ragged_batch_and_continuation(ops, cuda, oracle, synth):
    torch = cuda
    w = synth.la_weights(53)
    lens1, lens2 = [2, 70, 64], [1, 0, 67]
    xs = [synth.hidden_states(53, f"rag.{i}", lens1[i] + lens2[i]) for i in range(3)]
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=4, max_prefill_rows=256)
    la.set_weights(w)
    st = ops.LinearAttnState(1, 4)
    slots = [3, 0, 2]
    y1 = la.forward_batch(torch.from_numpy(np.concatenate([xs[i][:lens1[i]] for i in range(3)])).cuda(), st, 0, slots, lens1).cpu().numpy()
    y2 = la.forward_batch(torch.from_numpy(np.concatenate([xs[i][lens1[i]:] for i in range(3)])).cuda(), st, 0, slots, lens2).cpu().numpy()
    o1 = o2 = 0
    for i in range(3):
        ref = oracle.OracleLinearAttention(w)
        want = ref.forward_sequence(xs[i])
        got = np.concatenate([y1[o1:o1 + lens1[i]], y2[o2:o2 + lens2[i]]])
        o1 += lens1[i]; o2 += lens2[i]
        ok, msg = allclose_report(got, want, ATOL, RTOL)
        assert ok, f"sequence {i}: {msg}"
        rec, conv = st.export_state(0, slots[i])
        assert _rel(rec.cpu().numpy(), ref.recurrent) <= STATE_REL
        np.testing.assert_allclose(conv.cpu().numpy(), ref.conv_state, rtol=1e-4, atol=1e-5)


def test_recurrence_cores_agree_and_match_oracle(ops, cuda, oracle, synth):
    """Core kernels on oracle-produced q, k, v, g, beta: the chunked tensor-core path and the
    token-serial path against the reference recurrence (outputs before the gated norm, final state)."""
    torch = cuda
    w = synth.la_weights(54)
    T = 200
    x = synth.hidden_states(54, "core.x", T)
    ref = oracle.OracleLinearAttention(w)
    taps = []
    for t in range(T):
        d = {}
        ref.forward(x[t], d)
        taps.append(d)
    q = np.stack([d["q"] for d in taps]).reshape(T, 16, 128)
    k = np.stack([d["k"] for d in taps]).reshape(T, 16, 128)
    v = np.stack([d["v"] for d in taps]).reshape(T, 16, 128)
    g = np.stack([d["g"] for d in taps]); beta = np.stack([d["beta"] for d in taps])
    core = np.stack([d["core"] for d in taps]).reshape(T, 16, 128)
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=256)
    args = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, k, v, g, beta)]
    for use_tc in (False, True):
        st = ops.LinearAttnState(1, 1)
        out = la.prefill_core(*args, st, 0, [0], [T], use_tensor_cores=use_tc).cpu().numpy()
        err = np.abs(out - core)
        assert np.all(err <= 1e-4 + 2e-3 * np.abs(core)), f"tensor_cores={use_tc}: max abs err {err.max():.3e}"
        rec, _ = st.export_state(0, 0)
        assert _rel(rec.cpu().numpy(), ref.recurrent) <= STATE_REL, f"tensor_cores={use_tc}"


@pytest.mark.parametrize("counts", [[1], [63], [64], [65], [129, 1, 300]])
def test_chunked_kernel_equals_serial_kernel_from_a_nonzero_state(ops, cuda, synth, counts):
    """Tensor-core chunked recurrence against the token-serial fp32 kernel on random inputs (decays spanning
    e^-10 .. 1 per step), starting from a random state, in two consecutive calls."""
    torch = cuda
    n = len(counts)
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=4, max_prefill_rows=1024)
    outs, states = [], []
    for use_tc in (False, True):
        st = ops.LinearAttnState(1, 4)
        for i in range(n):
            st.import_state(0, i, torch.from_numpy(synth.normal(55, f"s0.{i}", (16, 128, 128), 0.05)).cuda(), None)
        res = []
        for call in range(2):
            rows = sum(counts)
            q = synth.normal(55, f"q.{call}.{rows}", (rows, 16, 128)); q /= np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(128)
            k = synth.normal(55, f"k.{call}.{rows}", (rows, 16, 128)); k /= np.linalg.norm(k, axis=-1, keepdims=True)
            v = synth.normal(55, f"v.{call}.{rows}", (rows, 16, 128), 0.5)
            g = -np.exp(synth.rng(55, f"g.{call}.{rows}").uniform(-6.0, 2.3, (rows, 16))).astype(np.float32)
            beta = synth.rng(55, f"b.{call}.{rows}").uniform(0.0, 1.0, (rows, 16)).astype(np.float32)
            args = [torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda() for a in (q, k, v, g, beta)]
            res.append(la.prefill_core(*args, st, 0, list(range(n)), counts, use_tensor_cores=use_tc).cpu().numpy())
        outs.append(np.concatenate(res))
        states.append([st.export_state(0, i)[0].cpu().numpy() for i in range(n)])
    err = np.abs(outs[0] - outs[1])
    assert np.all(err <= 1e-4 + 2e-3 * np.abs(outs[0])), f"outputs: max abs err {err.max():.3e}"
    for i in range(n):
        assert _rel(states[1][i], states[0][i]) <= STATE_REL, f"state of sequence {i}: rel {_rel(states[1][i], states[0][i]):.3e}"


def test_errors(ops, cuda, synth):
    torch = cuda
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=64)
    st = ops.LinearAttnState(1, 2)
    x = torch.zeros((4, 1024), device="cuda")
    with pytest.raises(ops.B200AttnError) as e:
        la.forward_batch(x, st, 0, [0], [4])
    assert e.value.status == ops.ERR_NOT_READY and "weights not set" in str(e.value)
    la.set_weights(synth.la_weights(1))
    with pytest.raises(ops.InvalidArgument):
        la.forward_batch(x, st, 0, [5], [4])         # slot out of range
    with pytest.raises(ops.InvalidArgument):
        la.forward_batch(x, st, 2, [0], [4])         # layer out of range
    with pytest.raises(ops.InvalidArgument):
        st.export_state(0, 9)
