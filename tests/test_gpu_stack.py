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


@pytest.fixture(params=["cublas", "tc"])
def decode_gemm(request, monkeypatch):
    """Both implementations of the decode-step projections: cuBLAS + separate norm / SwiGLU kernels, and the fused step
    on the tcgen05 skinny GEMMs (norm scale and SwiGLU in the epilogues, residual add through a cluster reduction).
    The library reads the variable when a stack is created."""
    monkeypatch.setenv("B200ATTN_DECODE_GEMM", request.param)
    return request.param


def test_prefill_and_decode_against_cpu_composition(ops, cuda, oracle, synth, decode_gemm):
    torch = cuda
    from oracle import cpu_stack
    # RMSNorm weights away from zero: the stack folds (1 + w) into the matrices behind each norm
    weights = cpu_stack.make_stack_weights(synth, 61, L, INTER, VOCAB, int8=True, norm_std=0.1)
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
    side.wait_stream(torch.cuda.current_stream())
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
        assert ops.launch_count() > D * 10             # every replay counts its kernel nodes
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
        side.wait_stream(torch.cuda.current_stream())      # the prefill is asynchronous on the stream it was given
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


def _quantized_fp16(torch, w):
    """code * scale of the per-output-channel INT8 quantiser (scale = absmax / 127, round half away from zero), rounded
    to fp16: the weights the stack's GEMMs read, computed independently on the GPU."""
    amax = w.abs().amax(dim=1, keepdim=True)
    scale = amax / 127.0
    scale = torch.where(scale > 1e-8, scale, torch.ones_like(scale))
    x = (w / scale).double()                                          # the +0.5 below is exact in float64
    code = torch.clamp(torch.sign(x) * torch.floor(x.abs() + 0.5), -127, 127).float()
    return (code * scale).half()


def test_real_shapes_ffn_3584_and_lm_head_248320(ops, cuda, oracle, synth, decode_gemm, monkeypatch):
    """The FFN (intermediate 3584) and the tied LM head (248 320 rows) at the shapes of the model, 128 sequences: one
    DeltaNet layer + FFN + final norm + LM head.  (a) The final hidden state of a one-token prefill against the CPU
    composition.  (b) The greedy token of the prefill against a float64 product of the returned hidden state (rounded
    to fp16, as the kernel reads it) with the quantised embedding matrix: the pick must be the float64 argmax or within
    1e-4 of it.  (c) The decode step (skinny GEMM with 970 column tiles and the cross-CTA 64-bit atomicMax argmax, or the
    library GEMM + argmax kernel) against the many-row path: the token the decode step picks for position 1 equals the
    token a two-token prefill picks, up to near-ties judged by float64 logits of that prefill's hidden state."""
    torch = cuda
    from oracle import cpu_stack
    n, INTER_R, VOCAB_R = 128, 3584, 248320
    weights = cpu_stack.make_stack_weights(synth, 66, 1, INTER_R, 8, int8=True)        # layer weights; the vocabulary comes next
    g = torch.Generator(device="cuda").manual_seed(66)
    embed = torch.randn((VOCAB_R, 1024), device="cuda", generator=g) * 0.02
    st = ops.HybridStack(num_layers=1, intermediate_size=INTER_R, vocab_size=VOCAB_R, max_seqs=n, max_seq_len=64,
                         prefill_chunk_seqs=8, kv_dtype=1, int8_weights=True)
    lw = weights["layers"][0]
    st.set_layer_weights(0, lw, lw["ffn"], la=lw["la"])
    st.set_embedding(embed.cpu().numpy(), weights["final_norm"])
    wq = _quantized_fp16(torch, embed).double()
    tokens = torch.randint(0, VOCAB_R, (n, 2), device="cuda", generator=g, dtype=torch.int32)
    first = tokens[:, :1].contiguous()
    nxt, hid = st.forward_batch_prefill(first, want_hidden=True)
    # (a) hidden state of 8 of the sequences against the CPU composition
    qw = cpu_stack.quantized_view(weights)
    emb_rows = wq.float()
    for i in range(0, n, 16):
        qw["embed"] = {int(first[i, 0]): emb_rows[int(first[i, 0])].cpu().numpy()}
        seq = cpu_stack.OracleStackSequence(qw, 4, kv_mode=2)
        hn, _ = seq.forward_token(int(first[i, 0]), want_logits=False)
        err = np.abs(hid[i].cpu().numpy() - hn)
        # one operator + FFN + three norms: twice as many fp16 roundings in a row as a single operator, whose own bound
        # is 2e-3 + 1e-2 |ref| (tests/test_gpu_la.py); the final norm rescales the sum to unit RMS
        assert np.all(err <= 4e-3 + 1e-2 * np.abs(hn)), f"sequence {i}: hidden max abs err {err.max():.3e}"
    # (b) LM head + argmax of the prefill path
    def check_pick(hidden, picked, what):
        logits = hidden.half().double() @ wq.T                       # [n, vocab] float64
        best = logits.max(dim=1).values
        mine = logits.gather(1, picked.long().view(-1, 1)).view(-1)
        gap = (best - mine).max().item()
        assert gap <= 1e-4, f"{what}: picked logit is {gap:.3e} below the float64 maximum"
        return logits
    check_pick(hid, nxt, "prefill")
    # (c) decode step for position 1 against a two-token prefill
    got = st.forward_batch_decode(tokens[:, 1].contiguous())
    assert st.device_status() == 0
    st.reset_cache()
    nxt2, hid2 = st.forward_batch_prefill(tokens, want_hidden=True)
    logits2 = hid2.half().double() @ wq.T
    best = logits2.max(dim=1).values
    mine = logits2.gather(1, got.long().view(-1, 1)).view(-1)
    agree = (got == nxt2).float().mean().item()
    assert agree >= 0.95, f"decode step and prefill pick the same token for {agree:.2f} of the sequences"
    assert (best - mine).max().item() <= 2e-2, f"decode pick is {(best - mine).max().item():.3e} below the maximum of the prefill's logits"
    assert st.device_status() == 0


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
