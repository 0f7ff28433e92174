"""Generates the golden fixtures in this directory by running the reference's own CPU classes
(qwen::FullAttention / qwen::LinearAttention, compiled from the reference checkout into
oracle/_ref/libqwen_ref.so by oracle/Makefile) on seeded synthetic inputs.

    python tests/golden/make_golden.py

Needs the reference checkout (location: environment variable QWEN_REFERENCE_ROOT); the fixtures it writes are committed so the
tests that use them run anywhere.  Shapes are the real model dims; token counts are kept small so
the files stay a few hundred KB.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402
from oracle import cpu_oracle as O  # noqa: E402

synth = entry.load_package().synth


def main():
    O.build(force=True)
    assert O.have_ref(), "reference checkout not available: cannot regenerate fixtures"
    # Gated full attention: 24 tokens through FullAttention::forward_sequence semantics (position = index).
    seed, T = 101, 24
    w = synth.fa_weights(seed)
    x = synth.hidden_states(seed, "golden.fa.x", T)
    ref = O.RefFullAttention(w, T)
    y = ref.forward_sequence(x)
    k, v = ref.cache()
    np.savez_compressed(os.path.join(HERE, "fa_ref_seed101_t24.npz"), seed=seed, tokens=T, y=y.astype(np.float32),
                        k_cache=k.astype(np.float32), v_cache=v.astype(np.float32))
    # Gated DeltaNet: 24 tokens from a zero state, outputs and final state.
    seed, T = 202, 24
    w = synth.la_weights(seed)
    x = synth.hidden_states(seed, "golden.la.x", T)
    ref = O.RefLinearAttention(w)
    y = ref.forward_sequence(x)
    rec, conv = ref.state()
    heads = np.array([0, 7, 15])   # three of the 16 heads keep the file small
    np.savez_compressed(os.path.join(HERE, "la_ref_seed202_t24.npz"), seed=seed, tokens=T, y=y.astype(np.float32),
                        recurrent_heads=heads, recurrent=rec[heads].astype(np.float32), conv=conv.astype(np.float32))
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
