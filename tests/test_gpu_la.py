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


def test_layer_prefill1024_fp16_projections(ops, cuda, oracle, synth, capsys):
    """The same workload in the precision the benchmark runs (fp16 weights and activations in the projections, fp32
    accumulation), held to the same bounds; the measured errors are printed."""
    torch = cuda
    w = synth.la_weights(56)
    x = synth.hidden_states(56, "cfg1.fp16.x", 1024)
    ref = oracle.OracleLinearAttention(w)
    want = ref.forward_sequence(x)
    la = ops.LinearAttention(ops.PROJ_FP16, max_batch=2, max_prefill_rows=1024)
    la.set_weights(w)
    st = ops.LinearAttnState(1, 2)
    got = la.forward_batch(torch.from_numpy(x).cuda(), st, 0, [0], [1024]).cpu().numpy()
    ok, msg = allclose_report(got, want, ATOL, RTOL)
    rec, conv = st.export_state(0, 0)
    rel = _rel(rec.cpu().numpy(), ref.recurrent)
    with capsys.disabled():
        print(f"\n[la fp16 projections, 1024 tokens] {msg}; state rel {rel:.3e}")
    assert ok, msg
    assert rel <= STATE_REL
    assert la.device_status() == 0


@pytest.mark.parametrize("proj", [0, 1])
def test_recurrent_decode_512_steps_three_layers(ops, cuda, oracle, synth, proj, capsys):
    """The recurrent-decode workload at its stated length on a sub-batch the CPU checker can follow: 2 sequences x 3
    DeltaNet layers, states ~ N(0, 0.05), conv caches warm, 512 single-token steps per layer; outputs every step and
    the final states, fp32 and fp16 projections."""
    import threading
    torch = cuda
    n, layers, steps = 2, 3, 512
    ws = [synth.la_weights(60, f"cfg3.L{l}") for l in range(layers)]
    las = []
    for l in range(layers):
        la = ops.LinearAttention(proj, max_batch=n, max_prefill_rows=64)
        la.set_weights(ws[l])
        las.append(la)
    st = ops.LinearAttnState(layers, n)
    xs = synth.normal(60, "cfg3.x", (steps, layers, n, 1024), 1.0)
    refs, want = {}, {}
    for l in range(layers):
        for i in range(n):
            r = oracle.OracleLinearAttention(ws[l])
            r.recurrent[:] = synth.normal(60, f"state.{l}.{i}", (16, 128, 128), 0.05)
            r.conv_state[:] = synth.normal(60, f"conv.{l}.{i}", (6144, 3), 0.5)
            st.import_state(l, i, torch.from_numpy(r.recurrent).cuda(), torch.from_numpy(r.conv_state).cuda())
            refs[l, i] = r

    def run_ref(l, i):
        want[l, i] = np.stack([refs[l, i].forward(xs[t, l, i]) for t in range(steps)])
    ths = [threading.Thread(target=run_ref, args=k) for k in refs]
    [t.start() for t in ths]
    d_slots = torch.arange(n, dtype=torch.int32, device="cuda")
    xd = torch.from_numpy(xs).cuda()
    got = torch.stack([torch.stack([las[l].forward(xd[t, l].contiguous(), st, l, d_slots) for l in range(layers)]) for t in range(steps)])
    got = got.cpu().numpy()                                      # [steps, layers, n, 1024]
    [t.join() for t in ths]
    worst_rel, last = 0.0, ""
    for (l, i), r in refs.items():
        ok, msg = allclose_report(got[:, l, i], want[l, i], ATOL, RTOL)
        last = msg
        assert ok, f"layer {l} sequence {i}: {msg}"
        rec, conv = st.export_state(l, i)
        rel = _rel(rec.cpu().numpy(), r.recurrent)
        worst_rel = max(worst_rel, rel)
        assert rel <= STATE_REL, f"layer {l} sequence {i}: state rel {rel:.3e}"
        np.testing.assert_allclose(conv.cpu().numpy(), r.conv_state, rtol=1e-3 if proj else 1e-4, atol=1e-3 if proj else 1e-5)
    with capsys.disabled():
        print(f"\n[la decode 512 steps x 3 layers, proj {proj}] {last}; worst state rel {worst_rel:.3e}")


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


def test_decode_from_seeded_state(ops, cuda, oracle, synth):
    """Recurrent decode: 4 sequences, state ~ N(0, 0.05) and a warm conv cache imported in the
    reference's layouts, 24 single-token steps; outputs every step, state at the end."""
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


def test_decode_core_back_to_back_on_one_layer(ops, cuda, oracle, synth):
    """The core entry called eight times in a row on one layer and one stream with nothing in between (token by token,
    two sequences = 32 CTAs, far less than one wave): launch k + 1 must see the state launch k wrote.  Outputs and the
    final state against the CPU oracle's recurrence fed with the same projected rows."""
    torch = cuda
    w = synth.la_weights(59)
    n, steps = 2, 8
    la = ops.LinearAttention(ops.PROJ_FP32, max_batch=n, max_prefill_rows=64)
    la.set_weights(w)
    st = ops.LinearAttnState(1, n)
    refs = [oracle.OracleLinearAttention(w) for _ in range(n)]
    for i, r in enumerate(refs):
        r.recurrent[:] = synth.normal(59, f"state.{i}", (16, 128, 128), 0.05)
        r.conv_state[:] = synth.normal(59, f"conv.{i}", (6144, 3), 0.5)
        st.import_state(0, i, torch.from_numpy(r.recurrent).cuda(), torch.from_numpy(r.conv_state).cuda())
    d_slots = torch.arange(n, dtype=torch.int32, device="cuda")
    xs = [synth.hidden_states(59, f"b2b.{t}", n) for t in range(steps)]
    w_in = np.concatenate([w["w_qkv"], w["w_z"], w["w_a"], w["w_b"]]).astype(np.float64)
    mixed = [torch.from_numpy((x.astype(np.float64) @ w_in.T).astype(np.float32)).cuda() for x in xs]
    torch.cuda.synchronize()
    outs = [la.decode_core(m, st, 0, d_slots) for m in mixed]        # eight launches queued back to back
    torch.cuda.synchronize()
    for t in range(steps):
        for i in range(n):
            tap = {}
            refs[i].forward(xs[t][i], tap)
            core = tap["core"].reshape(16, 128).astype(np.float64)
            z = (xs[t][i].astype(np.float64) @ w["w_z"].astype(np.float64).T).reshape(16, 128)
            want = core / np.sqrt((core ** 2).mean(axis=1, keepdims=True) + 1e-6) * w["norm_w"][None, :] * (z / (1.0 + np.exp(-z)))
            ok, msg = allclose_report(outs[t][i].cpu().numpy().reshape(16, 128), want, ATOL, RTOL)
            assert ok, f"step {t} sequence {i}: {msg}"
    for i in range(n):
        rec, conv = st.export_state(0, i)
        assert _rel(rec.cpu().numpy(), refs[i].recurrent) <= STATE_REL, f"sequence {i}"
        np.testing.assert_allclose(conv.cpu().numpy(), refs[i].conv_state, rtol=1e-4, atol=1e-5)


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
