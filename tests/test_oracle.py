"""CPU: the C restatement (oracle/oracle.c) against the reference's own CPU classes — live when the
compiled reference is present, and always against the committed fixtures generated from it."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_fa_oracle_matches_golden(oracle, synth):
    g = np.load(os.path.join(GOLD, "fa_ref_seed101_t24.npz"))
    seed, T = int(g["seed"]), int(g["tokens"])
    w = synth.fa_weights(seed)
    x = synth.hidden_states(seed, "golden.fa.x", T)
    o = oracle.OracleFullAttention(w, T, kv_mode=0)
    y = o.forward_sequence(x)
    np.testing.assert_array_equal(y, g["y"])          # same operation order, fp32: bit-identical
    np.testing.assert_array_equal(o.k_cache[:T], g["k_cache"])
    np.testing.assert_array_equal(o.v_cache[:T], g["v_cache"])


def test_la_oracle_matches_golden(oracle, synth):
    g = np.load(os.path.join(GOLD, "la_ref_seed202_t24.npz"))
    seed, T = int(g["seed"]), int(g["tokens"])
    w = synth.la_weights(seed)
    x = synth.hidden_states(seed, "golden.la.x", T)
    o = oracle.OracleLinearAttention(w)
    y = o.forward_sequence(x)
    np.testing.assert_array_equal(y, g["y"])
    np.testing.assert_array_equal(o.recurrent[g["recurrent_heads"]], g["recurrent"])
    np.testing.assert_array_equal(o.conv_state, g["conv"])


def test_oracle_matches_compiled_reference_live(oracle, synth):
    if not oracle.have_ref():
        pytest.skip("compiled reference (oracle/_ref) not present")
    w = synth.fa_weights(5)
    x = synth.hidden_states(5, "live.x", 9)
    a = oracle.OracleFullAttention(w, 16).forward_sequence(x)
    b = oracle.RefFullAttention(w, 16).forward_sequence(x)
    np.testing.assert_array_equal(a, b)
    w = synth.la_weights(6)
    o, r = oracle.OracleLinearAttention(w), oracle.RefLinearAttention(w)
    np.testing.assert_array_equal(o.forward_sequence(x), r.forward_sequence(x))
    rec, conv = r.state()
    np.testing.assert_array_equal(o.recurrent, rec)
    np.testing.assert_array_equal(o.conv_state, conv)


def test_la_reference_state_roundtrip(oracle, synth):
    if not oracle.have_ref():
        pytest.skip("compiled reference (oracle/_ref) not present")
    w = synth.la_weights(8)
    x = synth.hidden_states(8, "rt.x", 6)
    a = oracle.RefLinearAttention(w)
    a.forward_sequence(x[:3])
    rec, conv = a.state()
    b = oracle.RefLinearAttention(w)
    b.set_state(rec, conv)
    np.testing.assert_array_equal(a.forward_sequence(x[3:]), b.forward_sequence(x[3:]))


def test_quantiser_known_answers(oracle):
    # absmax -> +-127, scale = absmax/127, half-away-from-zero rounding, clamp, zero row -> scale 1.
    x = np.zeros(256, np.float32)
    x[0], x[1], x[2], x[3] = 127.0, -127.0, 0.5, -0.5
    x[4], x[5], x[6] = 1.5, 2.5, -2.5
    codes, scale = oracle.quantize_head(x)
    assert scale == np.float32(1.0)
    assert list(codes[:7]) == [127, -127, 1, -1, 2, 3, -3]          # roundf, not round-half-even (2, 2, -2)
    codes, scale = oracle.quantize_head(np.zeros(256, np.float32))
    assert scale == np.float32(1.0) and not codes.any()
    tiny = np.full(256, 1e-7, np.float32)                             # absmax/127 < 1e-8 -> scale 1.0
    codes, scale = oracle.quantize_head(tiny)
    assert scale == np.float32(1.0) and not codes.any()


def test_quantiser_vectorised_equals_scalar(oracle, synth):
    x = synth.normal(3, "q.rows", (64, 256), 0.7)
    codes, scales = oracle.quantize_rows(x)
    for i in range(x.shape[0]):
        c, s = oracle.quantize_head(x[i])
        assert s == scales[i]
        np.testing.assert_array_equal(c, codes[i])
    # On N(0, sigma) inputs no quotient lands exactly on a .5 tie, so roundf and round-half-even agree there.
    assert sum(oracle.count_ties(x[i], scales[i]) for i in range(x.shape[0])) == 0


def test_kv_modes_of_the_oracle(oracle, synth):
    w = synth.fa_weights(9)
    x = synth.hidden_states(9, "kv.x", 5)
    o8 = oracle.OracleFullAttention(w, 8, kv_mode=1)
    o8.forward_sequence(x)
    o0 = oracle.OracleFullAttention(w, 8, kv_mode=0)
    o0.forward_sequence(x)
    # what the INT8 cache holds is code*scale of the fp32 K/V
    for t in range(5):
        for h in range(2):
            c, s = oracle.quantize_head(o0.k_cache[t, h * 256:(h + 1) * 256])
            np.testing.assert_array_equal(c, o8.k_codes[t, h * 256:(h + 1) * 256])
            assert s == o8.k_scale[t, h]
            np.testing.assert_array_equal(c.astype(np.float32) * s, o8.k_cache[t, h * 256:(h + 1) * 256])
    o16 = oracle.OracleFullAttention(w, 8, kv_mode=2)
    o16.forward_sequence(x)
    np.testing.assert_array_equal(o16.k_cache[:5], o0.k_cache[:5].astype(np.float16).astype(np.float32))
