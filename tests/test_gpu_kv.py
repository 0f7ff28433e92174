"""GPU: paged KV cache — quantise-on-append is bit-exact against the oracle's quantiser on the same
fp32 K/V rows (ragged batches, page-boundary crossings, repeated appends), FP16 storage is the IEEE
round-to-nearest conversion, and the page bookkeeping behaves like the reference's allocator."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _kv_rows(oracle, synth, seed, tokens):
    """fp32 K (normalised + rotated) and raw V rows as the reference computes them."""
    w = synth.fa_weights(seed)
    x = synth.hidden_states(seed, "kv.rows", tokens)
    o = oracle.OracleFullAttention(w, tokens, kv_mode=0)
    o.forward_sequence(x)
    return o.k_cache[:tokens].copy(), o.v_cache[:tokens].copy()


def test_int8_append_bit_exact_ragged(ops, cuda, oracle, synth):
    torch = cuda
    counts = [1, 63, 64, 65, 130, 7]
    k, v = _kv_rows(oracle, synth, 21, max(counts) + 70)
    kv = ops.KVCache(2, 8, 512, ops.KV_INT8)
    slots = [kv.allocate_sequence(0) for _ in counts]
    # first append: ragged batch, each sequence takes rows [0, c)
    rows_k = np.concatenate([k[:c] for c in counts])
    rows_v = np.concatenate([v[:c] for c in counts])
    kv.append(1, slots, counts, torch.from_numpy(rows_k).cuda(), torch.from_numpy(rows_v).cuda())
    # second append continues each sequence mid-page: rows [c, c + 70)
    rows_k2 = np.concatenate([k[c:c + 70] for c in counts])
    rows_v2 = np.concatenate([v[c:c + 70] for c in counts])
    kv.append(1, slots, [70] * len(counts), torch.from_numpy(rows_k2).cuda(), torch.from_numpy(rows_v2).cuda())
    assert kv.device_status() == 0
    for s, c in zip(slots, counts):
        n = c + 70
        assert kv.length(1, s) == n and kv.length(0, s) == 0
        kc, vc, ks, vs = [t.cpu().numpy() for t in kv.export(1, s)]
        want_kc, want_ks = oracle.quantize_rows(k[:n].reshape(n, 2, 256))
        want_vc, want_vs = oracle.quantize_rows(v[:n].reshape(n, 2, 256))
        np.testing.assert_array_equal(kc, want_kc)
        np.testing.assert_array_equal(vc, want_vc)
        np.testing.assert_array_equal(ks.view(np.uint32), want_ks.view(np.uint32))   # scales bit for bit
        np.testing.assert_array_equal(vs.view(np.uint32), want_vs.view(np.uint32))


def test_int8_append_edge_rows(ops, cuda, oracle):
    torch = cuda
    rows = np.zeros((5, 512), np.float32)
    rows[1, :] = 1e-7                       # absmax/127 below 1e-8 -> scale 1.0, codes 0
    rows[2, 0], rows[2, 1], rows[2, 2] = 127.0, 0.5, -2.5     # ties: roundf goes away from zero
    rows[3, :256] = np.linspace(-3, 3, 256)
    rows[4, 256:] = -np.linspace(0, 9, 256)
    kv = ops.KVCache(1, 2, 64, ops.KV_INT8)
    s = kv.allocate_sequence(5)
    kv.append(0, [s], [5], torch.from_numpy(rows).cuda(), torch.from_numpy(rows[::-1].copy()).cuda())
    kc, vc, ks, vs = [t.cpu().numpy() for t in kv.export(0, s)]
    wk, wks = oracle.quantize_rows(rows.reshape(5, 2, 256))
    wv, wvs = oracle.quantize_rows(rows[::-1].reshape(5, 2, 256))
    np.testing.assert_array_equal(kc, wk)
    np.testing.assert_array_equal(ks, wks)
    np.testing.assert_array_equal(vc, wv)
    np.testing.assert_array_equal(vs, wvs)
    assert kc[2, 0, 0] == 127 and kc[2, 0, 1] == 1 and kc[2, 0, 2] == -3


def test_fp16_append_is_ieee_rounding(ops, cuda, oracle, synth):
    torch = cuda
    k, v = _kv_rows(oracle, synth, 22, 100)
    kv = ops.KVCache(1, 2, 128, ops.KV_FP16)
    s = kv.allocate_sequence(100)
    kv.append(0, [s], [100], torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    kc, vc, ks, vs = kv.export(0, s)
    assert ks is None and vs is None
    np.testing.assert_array_equal(kc.cpu().numpy().reshape(100, 512), k.astype(np.float16))
    np.testing.assert_array_equal(vc.cpu().numpy().reshape(100, 512), v.astype(np.float16))


def test_page_bookkeeping(ops, cuda):
    kv = ops.KVCache(1, 4, 256, ops.KV_INT8, num_pages=6)
    assert kv.pages() == (6, 0)
    a = kv.allocate_sequence(65)           # 2 pages
    b = kv.allocate_sequence(0)
    assert kv.pages() == (6, 2)
    kv.reserve(b, 256)                     # 4 pages -> pool full
    assert kv.pages() == (6, 6)
    c = kv.allocate_sequence(0)
    with pytest.raises(ops.B200AttnError) as e:
        kv.reserve(c, 1)                   # exhausted pool
    assert e.value.status == ops.ERR_NOMEM
    with pytest.raises(ops.B200AttnError):
        kv.reserve(a, 257)                 # beyond the block-table width
    kv.release_sequence(b)
    assert kv.pages() == (6, 2)
    kv.reserve(c, 64)
    assert kv.pages() == (6, 3)
    with pytest.raises(ops.InvalidArgument):
        kv.release_sequence(b)             # already released
    with pytest.raises(ops.InvalidArgument):
        kv.length(0, 99)


def test_shrink_sequence_truncates_and_returns_pages(ops, cuda, oracle, synth):
    """PagedKVCache::shrink_sequence semantics (one page is always kept, a longer length is a no-op), and the cache
    content after a shrink + re-append equals a cache that was filled that way from the start (INT8 codes bit-exact)."""
    torch = cuda
    kv = ops.KVCache(2, 2, 512, ops.KV_INT8, num_pages=16)
    s = kv.allocate_sequence(0)
    k = torch.from_numpy(synth.normal(71, "k", (200, 512), 1.0)).cuda()
    v = torch.from_numpy(synth.normal(71, "v", (200, 512), 0.6)).cuda()
    for layer in range(2):
        kv.append(layer, [s], [200], k, v)
    assert kv.pages() == (16, 4) and kv.length(0, s) == 200 and kv.length(1, s) == 200
    kv.shrink_sequence(s, 300)                      # not shorter: nothing happens
    assert kv.pages() == (16, 4) and kv.length(0, s) == 200
    kv.shrink_sequence(s, 70)                       # 2 pages stay
    assert kv.pages() == (16, 2) and kv.length(0, s) == 70 and kv.length(1, s) == 70
    kv.append(0, [s], [30], k[100:130], v[100:130])  # positions 70..99 again, with other rows
    assert kv.length(0, s) == 100 and kv.length(1, s) == 70
    got = kv.export(0, s)
    ref = ops.KVCache(1, 1, 512, ops.KV_INT8, num_pages=4)
    r = ref.allocate_sequence(0)
    ref.append(0, [r], [70], k[:70], v[:70])
    ref.append(0, [r], [30], k[100:130], v[100:130])
    want = ref.export(0, r)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    kv.shrink_sequence(s, 0)
    assert kv.pages() == (16, 1) and kv.length(0, s) == 0
    with pytest.raises(ops.InvalidArgument):
        kv.shrink_sequence(s, -1)
    with pytest.raises(ops.InvalidArgument):
        kv.shrink_sequence(1 - s, 0)               # the other slot was never allocated
    assert kv.device_status() == 0


def test_append_rejects_bad_batches(ops, cuda):
    torch = cuda
    kv = ops.KVCache(1, 2, 64, ops.KV_INT8)
    s = kv.allocate_sequence(8)
    z = torch.zeros((4, 512), device="cuda")
    with pytest.raises(ops.InvalidArgument):
        kv.append(0, [s, s], [2, 2], z, z)            # same slot twice
    with pytest.raises(ops.InvalidArgument):
        kv.append(3, [s], [4], z, z)                  # layer out of range
    with pytest.raises(ops.InvalidArgument):
        kv.append(0, [1], [4], z, z)                  # slot never allocated
    kv.append(0, [s], [0], z, z)                      # empty append is a no-op
    assert kv.length(0, s) == 0
    kv.clear()
    assert kv.length(0, s) == 0


def test_bookkeeping_after_decode_on_a_side_stream(ops, cuda, synth):
    """Decode steps advance the cache lengths on the device, on whatever stream the caller uses.  After steps on a
    non-blocking side stream (which the legacy default stream does not wait for), the length query, a follow-up
    prefill-append and a shrink must see the advanced lengths without any manual synchronisation in between."""
    torch = cuda
    w = synth.fa_weights(72)
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=256)   # a continuation stages its whole context
    fa.set_weights(w)
    kv = ops.KVCache(1, 2, 256, ops.KV_INT8)
    slots = [kv.allocate_sequence(200) for _ in range(2)]        # decode steps cannot grow a sequence: pages are reserved up front
    x = torch.from_numpy(synth.hidden_states(72, "side.x", 2 * 40 + 2 * 30 + 2 * 10)).cuda()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        fa.forward_batch_prefill(x[:80].contiguous(), kv, 0, slots, [40, 40])
        for t in range(30):
            fa.forward(x[80 + 2 * t:82 + 2 * t].contiguous(), kv, 0, d_slots)
        assert kv.length(0, slots[0]) == 70 and kv.length(0, slots[1]) == 70        # no synchronize before the query
        for t in range(3):
            fa.forward(x[80 + 2 * t:82 + 2 * t].contiguous(), kv, 0, d_slots)
        fa.forward_batch_prefill(x[140:160].contiguous(), kv, 0, slots, [10, 10])     # must append at 73, not at 70
        assert kv.length(0, slots[0]) == 83
        for t in range(2):
            fa.forward(x[80 + 2 * t:82 + 2 * t].contiguous(), kv, 0, d_slots)
        kv.shrink_sequence(slots[1], 64)                                            # 85 -> 64: one page stays
        assert kv.length(0, slots[1]) == 64 and kv.length(0, slots[0]) == 85
        assert kv.pages()[1] == 4 + 1                                                # slot 0 keeps its 4 reserved pages
    assert kv.device_status() == 0


def test_decode_after_free_gives_zero_output(ops, cuda, synth):
    """A released slot keeps no length on the device: a decode-attention launch that still names it writes its defined
    zero output instead of attending over pages that may belong to another sequence by then."""
    torch = cuda
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=2, max_prefill_rows=64)
    kv = ops.KVCache(1, 2, 128, ops.KV_FP16)
    a, b = kv.allocate_sequence(0), kv.allocate_sequence(0)
    k = torch.from_numpy(synth.normal(73, "k", (100, 512), 1.0)).cuda()
    v = torch.from_numpy(synth.normal(73, "v", (100, 512), 0.6)).cuda()
    kv.append(0, [a, b], [60, 40], k, v)
    q = torch.from_numpy(synth.normal(73, "q", (2, 8, 256), 1.0)).cuda()
    d_slots = torch.tensor([a, b], dtype=torch.int32, device="cuda")
    before = fa.decode_core(q, kv, 0, d_slots).clone()
    kv.release_sequence(a)
    after = fa.decode_core(q, kv, 0, d_slots)
    assert not after[0].any(), "released slot still produced attention output"
    assert torch.equal(after[1], before[1])
    assert kv.device_status() == 0
