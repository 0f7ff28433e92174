"""GPU: the hybrid stack (4 layers = 3 DeltaNet + 1 full attention, small FFN and vocabulary so the CPU
checker finishes in seconds) — prefill hidden states and greedy tokens against the CPU composition,
eager decode against the graph-captured decode step."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

L, INTER, VOCAB = 4, 256, 512


def _build(ops, synth, weights, max_seqs=4, max_seq_len=128, kv_dtype=1):
    st = ops.HybridStack(num_layers=L, intermediate_size=INTER, vocab_size=VOCAB, max_seqs=max_seqs,
                         max_seq_len=max_seq_len, prefill_chunk_seqs=2, kv_dtype=kv_dtype, int8_weights=True)
    for i, lw in enumerate(weights["layers"]):
        st.set_layer_weights(i, lw, lw["ffn"], fa=lw.get("fa"), la=lw.get("la"))
    st.set_embedding(weights["embed"], weights["final_norm"])
    return st


@pytest.fixture(params=["cublas", "inproj", "tc", "fused"])
def decode_gemm(request, monkeypatch):
    """Every implementation of the decode-step projections: cuBLAS + separate SwiGLU / argmax kernels, cuBLAS with only
    the input projection of each attention layer on the tcgen05 kernel, the tcgen05
    skinny GEMM with fused epilogues, and the persistent per-layer chain kernel (projections and norms between two
    attention kernels in one cooperative launch).  The library reads the variable on every call."""
    monkeypatch.setenv("B200ATTN_DECODE_GEMM", request.param)
    return request.param


def test_prefill_and_decode_against_cpu_composition(ops, cuda, oracle, synth, decode_gemm):
    torch = cuda
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 61, L, INTER, VOCAB, int8=True)
    qw = cpu_stack.quantized_view(weights)
    n, T, D = 3, 48, 4            # 144 prefill rows: the many-row form of the norm kernel is on the path
    tokens = synth.rng(61, "tokens").integers(0, VOCAB, (n, T)).astype(np.int32)
    st = _build(ops, synth, weights)
    nxt, hid = st.forward_batch_prefill(torch.from_numpy(tokens).cuda(), want_hidden=True)
    nxt, hid = nxt.cpu().numpy(), hid.cpu().numpy()
    seqs = [cpu_stack.OracleStackSequence(qw, T + D + 1, kv_mode=2) for _ in range(n)]
    for i in range(n):
        for t in range(T):
            hn, logits = seqs[i].forward_token(int(tokens[i, t]), want_logits=(t == T - 1))
        cos = float(hn @ hid[i] / (np.linalg.norm(hn) * np.linalg.norm(hid[i])))
        assert cos > 0.999, f"sequence {i}: cosine {cos:.5f}"
        assert np.abs(hid[i] - hn).max() < 0.08, f"sequence {i}: max abs err {np.abs(hid[i] - hn).max():.3e}"
        # greedy token: the GPU's pick must be (near-)maximal under the CPU logits
        assert logits[nxt[i]] >= logits.max() - 0.05 * (logits.max() - logits.mean())
    # decode steps fed with the GPU's own tokens on both sides
    cur = torch.from_numpy(nxt).cuda()
    for d in range(D):
        fed = cur.cpu().numpy()
        cur = st.forward_batch_decode(cur)
        got = cur.cpu().numpy()
        for i in range(n):
            _, logits = seqs[i].forward_token(int(fed[i]))
            assert logits[got[i]] >= logits.max() - 0.05 * (logits.max() - logits.mean()), f"step {d} seq {i}"


def test_graph_replay_equals_eager_decode(ops, cuda, synth, decode_gemm):
    torch = cuda
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 62, L, INTER, VOCAB, int8=True)
    n, T, D = 4, 70, 6
    tokens = torch.from_numpy(synth.rng(62, "tokens").integers(0, VOCAB, (n, T)).astype(np.int32)).cuda()
    st = _build(ops, synth, weights)
    first = st.forward_batch_prefill(tokens)
    cur, eager = first.clone(), []
    for _ in range(D):
        cur = st.forward_batch_decode(cur)
        eager.append(cur.clone())
    st.reset_cache()
    again = st.forward_batch_prefill(tokens)
    assert torch.equal(again, first)                  # reset + prefill is reproducible
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        st.set_tokens(again)
        ops.launch_count(reset=True)
        st.capture_decode(n)
        assert ops.launch_count() == 0                # capture runs nothing
        replayed = []
        for _ in range(D):
            st.launch_decode(1)
            replayed.append(st.get_tokens(n))
        side.synchronize()
        assert ops.launch_count() > D * 10             # every replay counts its kernel nodes (17 per step in the fused mode)
    for a, b in zip(eager, replayed):
        assert torch.equal(a, b)
    assert st.device_status() == 0


def test_plain_stream_order_gives_the_same_tokens(ops, cuda, synth, monkeypatch):
    """The decode kernels are launched as programmatic dependents (they may start while their predecessor drains and
    wait before touching its results).  With the attribute switched off every launch waits for the previous one to
    finish; both must produce identical tokens, eagerly and from the captured graph."""
    torch = cuda
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 63, L, INTER, VOCAB, int8=True)
    n, T, D = 4, 50, 5
    tokens = torch.from_numpy(synth.rng(63, "tokens").integers(0, VOCAB, (n, T)).astype(np.int32)).cuda()
    runs = {}
    for pdl in ("1", "0"):
        monkeypatch.setenv("B200ATTN_PDL", pdl)
        st = _build(ops, synth, weights)
        cur = st.forward_batch_prefill(tokens)
        eager = [cur.clone()]
        for _ in range(D):
            cur = st.forward_batch_decode(cur)
            eager.append(cur.clone())
        st.reset_cache()
        first = st.forward_batch_prefill(tokens)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            st.set_tokens(first)
            st.capture_decode(n)
            replay = []
            for _ in range(D):
                st.launch_decode(1)
                replay.append(st.get_tokens(n))
            side.synchronize()
        for a, b in zip(eager[1:], replay):
            assert torch.equal(a, b)
        assert st.device_status() == 0
        runs[pdl] = eager
    for a, b in zip(runs["1"], runs["0"]):
        assert torch.equal(a, b)


def test_decode_after_a_prefill_that_fills_the_working_buffers(ops, cuda, oracle, synth):
    """The operators of one stack overlay their working buffers on one area.  A prefill that uses (nearly) every row of
    it must leave nothing behind that the decode step depends on: the split counters and status words live outside it.
    Four pages of context per sequence make the decode attention combine several partials per head."""
    torch = cuda
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 65, L, INTER, VOCAB, int8=True)
    qw = cpu_stack.quantized_view(weights)
    n, T, D = 2, 250, 4
    tokens_np = synth.rng(65, "tokens").integers(0, VOCAB, (n, T)).astype(np.int32)
    st = _build(ops, synth, weights, max_seqs=n, max_seq_len=256)      # 2 x 256 rows of working space, 500 used
    cur = st.forward_batch_prefill(torch.from_numpy(tokens_np).cuda())
    picks = [cur.cpu().numpy()]
    for _ in range(D):
        cur = st.forward_batch_decode(cur)
        picks.append(cur.cpu().numpy())
    assert st.device_status() == 0
    for i in range(n):
        seq = cpu_stack.OracleStackSequence(qw, T + D + 1, kv_mode=2)
        for t in range(T):
            _, logits = seq.forward_token(int(tokens_np[i, t]), want_logits=(t == T - 1))
        for d in range(D + 1):
            assert logits[picks[d][i]] >= logits.max() - 0.05 * (logits.max() - logits.mean()), f"seq {i} step {d}"
            if d < D:
                _, logits = seq.forward_token(int(picks[d][i]))


@pytest.mark.parametrize("branches", ["2", "3"])
def test_decode_branches_against_single_chain_and_cpu(ops, cuda, oracle, synth, monkeypatch, branches):
    """B200ATTN_DECODE_BRANCHES cuts the step's sequences into groups that walk the layers on streams of their own.  The
    groups' GEMMs have fewer rows than the single chain's, so the library may sum in another order: tokens are compared
    with the single chain by agreement on the first step (identical inputs), exactly between eager launches and the
    captured graph, and against the CPU composition for one sequence of every group."""
    torch = cuda
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 64, L, INTER, VOCAB, int8=True)
    qw = cpu_stack.quantized_view(weights)
    n, T, D = 48, 24, 3
    tokens_np = synth.rng(64, "tokens").integers(0, VOCAB, (n, T)).astype(np.int32)
    tokens = torch.from_numpy(tokens_np).cuda()
    st = _build(ops, synth, weights, max_seqs=n, max_seq_len=64)

    def eager_run():
        st.reset_cache()
        cur = st.forward_batch_prefill(tokens)
        out = [cur.clone()]
        for _ in range(D):
            cur = st.forward_batch_decode(cur)
            out.append(cur.clone())
        return out

    monkeypatch.setenv("B200ATTN_DECODE_BRANCHES", "1")
    single = eager_run()
    monkeypatch.setenv("B200ATTN_DECODE_BRANCHES", branches)
    ops.launch_count(reset=True)
    split = eager_run()
    assert torch.equal(single[0], split[0])                       # prefill does not branch
    agree = (single[1] == split[1]).float().mean().item()
    assert agree >= 0.9, f"first decode step: {agree:.2f} of the tokens agree with the single chain"
    st.reset_cache()
    first = st.forward_batch_prefill(tokens)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        st.set_tokens(first)
        st.capture_decode(n)
        for d in range(D):
            st.launch_decode(1)
            assert torch.equal(st.get_tokens(n), split[d + 1]), f"replayed step {d}"
        side.synchronize()
    assert st.device_status() == 0
    # one sequence of each group (and the last one) against the CPU composition, fed with the GPU's own tokens
    picks = [s.cpu().numpy() for s in split]
    for i in sorted({0, n // 2, n - 1}):
        seq = cpu_stack.OracleStackSequence(qw, T + D + 1, kv_mode=2)
        for t in range(T):
            _, logits = seq.forward_token(int(tokens_np[i, t]), want_logits=(t == T - 1))
        for d in range(D + 1):
            assert logits[picks[d][i]] >= logits.max() - 0.05 * (logits.max() - logits.mean()), f"seq {i} step {d}"
            if d < D:
                _, logits = seq.forward_token(int(picks[d][i]))


def test_stack_errors(ops, cuda, synth):
    torch = cuda
    st = ops.HybridStack(num_layers=L, intermediate_size=INTER, vocab_size=VOCAB, max_seqs=2, max_seq_len=64,
                         prefill_chunk_seqs=1)
    toks = torch.zeros((1, 8), dtype=torch.int32, device="cuda")
    with pytest.raises(ops.B200AttnError) as e:
        st.forward_batch_prefill(toks)
    assert e.value.status == ops.ERR_NOT_READY
    with pytest.raises(ops.B200AttnError):
        st.launch_decode(1)                            # nothing captured
    with pytest.raises(ops.InvalidArgument):
        st.set_layer_weights(99, dict(input_norm=np.zeros(1024), post_norm=np.zeros(1024)),
                             dict(gate=np.zeros((INTER, 1024)), up=np.zeros((INTER, 1024)), down=np.zeros((1024, INTER))))
