"""GPU: continuous batching on the hybrid stack — requests of different lengths flow through four rows (admission into
freed rows between captured decode steps, the last row moving into a retired row's place); every request must produce
the tokens it produces when it runs alone, and the pools must be empty again at the end."""
import importlib

import numpy as np
import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu
L, INTER, VOCAB = 4, 256, 512


def test_requests_keep_their_tokens_while_rows_change_hands(ops, cuda, synth):
    torch = cuda
    from oracle import cpu_stack
    batching = importlib.import_module(entry.PKG_NAME + ".batching")
    weights = cpu_stack.make_stack_weights(synth, 67, L, INTER, VOCAB, int8=True, norm_std=0.05)
    st = ops.HybridStack(num_layers=L, intermediate_size=INTER, vocab_size=VOCAB, max_seqs=4, max_seq_len=192,
                         prefill_chunk_seqs=2, kv_dtype=ops.KV_FP16, int8_weights=True)
    for i, lw in enumerate(weights["layers"]):
        st.set_layer_weights(i, lw, lw["ffn"], fa=lw.get("fa"), la=lw.get("la"))
    st.set_embedding(weights["embed"], weights["final_norm"])
    rng = synth.rng(67, "requests")
    specs = [(70, 12), (5, 30), (130, 3), (64, 1), (33, 20), (9, 25), (100, 8)]       # (prompt tokens, tokens to generate)
    prompts = [torch.from_numpy(rng.integers(0, VOCAB, p).astype(np.int32)).cuda() for p, _ in specs]

    # every request alone, plain mode
    alone = []
    for prompt, (_, n_new) in zip(prompts, specs):
        st.reset_cache()
        cur = st.forward_batch_prefill(prompt.view(1, -1).contiguous())
        toks = [int(cur[0])]
        for _ in range(n_new - 1):
            cur = st.forward_batch_decode(cur)
            toks.append(int(cur[0]))
        alone.append(toks)
    torch.cuda.synchronize()

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        cb = batching.ContinuousBatcher(batching.StackBackend(st, ops), max_rows=4)
        for rid, (prompt, (_, n_new)) in enumerate(zip(prompts, specs)):
            cb.submit(batching.Request(rid, prompt, n_new))
        done = cb.run()
        side.synchronize()
    assert sorted(r.rid for r in done) == list(range(len(specs)))
    for r in done:
        assert r.tokens == alone[r.rid], f"request {r.rid}: {r.tokens} != {alone[r.rid]}"
    assert cb.steps < sum(n for _, n in specs)                      # sequences shared steps
    n_active, slots = st.rows()
    assert n_active == 0 and all(s == -1 for s in slots)
    assert st.device_status() == 0
    # the plain mode works again after a reset
    st.reset_cache()
    cur = st.forward_batch_prefill(prompts[0].view(1, -1).contiguous())
    assert int(cur[0]) == alone[0][0]


def test_admission_errors(ops, cuda, synth):
    torch = cuda
    st = ops.HybridStack(num_layers=L, intermediate_size=INTER, vocab_size=VOCAB, max_seqs=2, max_seq_len=64, prefill_chunk_seqs=1)
    p = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.B200AttnError):
        st.admit(p, 16)                                   # weights not set
    from oracle import cpu_stack
    weights = cpu_stack.make_stack_weights(synth, 68, L, INTER, VOCAB, int8=True)
    for i, lw in enumerate(weights["layers"]):
        st.set_layer_weights(i, lw, lw["ffn"], fa=lw.get("fa"), la=lw.get("la"))
    st.set_embedding(weights["embed"], weights["final_norm"])
    with pytest.raises(ops.InvalidArgument):
        st.admit(p, 16)                                   # not in batching mode
    st.begin_batching()
    with pytest.raises(ops.InvalidArgument):
        st.admit(p, 4)                                    # reserve smaller than the prompt
    with pytest.raises(ops.InvalidArgument):
        st.admit(p, 65)                                   # beyond max_seq_len
    assert st.admit(p, 16) == 0 and st.admit(p, 64) == 1
    with pytest.raises(ops.B200AttnError) as e:
        st.admit(p, 16)                                   # no row left
    assert e.value.status == ops.ERR_NOMEM
    with pytest.raises(ops.InvalidArgument):
        st.retire(2)
    with pytest.raises(ops.InvalidArgument):
        st.forward_batch_prefill(p.view(1, -1))           # plain prefill is refused while batching
    st.retire(0)
    n, slots = st.rows()
    assert n == 1 and slots[0] == 1 and slots[1] == -1    # the second sequence moved into row 0
