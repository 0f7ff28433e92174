"""TEST INFRASTRUCTURE ONLY — the hybrid stack composed on the CPU from the per-layer checkers.

Layer wiring follows qwen::LanguageLayer::forward (src/backend/cpu/core/common/language_backbone.cpp:55-91
in the reference): h1 = RMSNorm(x); a = attention(h1); h = x + a; h2 = RMSNorm(h); y = h + MLP(h2); the final
norm and the tied LM head follow LanguageBackbone::forward (language_backbone.cpp:203-229).  qwen::RMSNorm's
constructor throws in the reference (language_common.cpp:9), so the norm is the restated one in oracle.c; the
attention layers and the MLP are either the compiled reference classes (use_ref=True) or the C restatement.
One instance holds the caches of ONE sequence.
"""
from __future__ import annotations

import numpy as np

from . import cpu_oracle as O


def make_stack_weights(synth, seed: int, num_layers: int, inter: int, vocab: int, int8: bool = True, norm_std: float = 0.0) -> dict:
    """Random-init weights of the hybrid stack (matrices ~ N(0, 0.02), norm weights 0 / 1 or, with norm_std, the
    layers' RMSNorm weights ~ N(0, norm_std)), optionally passed through the per-output-channel INT8 quantiser
    (code * scale kept as fp32)."""
    def q(m):
        return O.quantize_weight_rows(m)[0] if int8 else m
    layers = []
    for i in range(num_layers):
        lw = dict(input_norm=np.zeros(1024, np.float32), post_norm=np.zeros(1024, np.float32))
        if norm_std > 0.0:
            lw = dict(input_norm=synth.normal(seed, f"L{i}.input_norm", (1024,), norm_std),
                      post_norm=synth.normal(seed, f"L{i}.post_norm", (1024,), norm_std))
        lw["ffn"] = dict(gate=synth.normal(seed, f"L{i}.gate", (inter, 1024), 0.02),
                         up=synth.normal(seed, f"L{i}.up", (inter, 1024), 0.02),
                         down=synth.normal(seed, f"L{i}.down", (1024, inter), 0.02))
        if synth.is_full_attention_layer(i):
            lw["fa"] = synth.fa_weights(seed, f"L{i}.fa")
        else:
            lw["la"] = synth.la_weights(seed, f"L{i}.la")
        layers.append(lw)
    embed = synth.normal(seed, "embed", (vocab, 1024), 0.02)
    return dict(layers=layers, embed=embed, final_norm=np.zeros(1024, np.float32), int8=int8, quantize=q)


def quantized_view(weights: dict) -> dict:
    """The weights the stack actually computes with when int8_weights is on: every matrix replaced by
    code * scale (norm vectors, conv taps, A_log, dt_bias untouched)."""
    q = weights["quantize"]
    out = dict(layers=[], embed=q(weights["embed"]), final_norm=weights["final_norm"])
    for lw in weights["layers"]:
        n = dict(input_norm=lw["input_norm"], post_norm=lw["post_norm"], ffn={k: q(v) for k, v in lw["ffn"].items()})
        if "fa" in lw:
            n["fa"] = dict(lw["fa"], **{k: q(lw["fa"][k]) for k in ("wq", "wk", "wv", "wo")})
        else:
            n["la"] = dict(lw["la"], **{k: q(lw["la"][k]) for k in ("w_qkv", "w_a", "w_b", "w_z", "w_out")})
        out["layers"].append(n)
    return out


class OracleStackSequence:
    def __init__(self, qweights: dict, max_tokens: int, kv_mode: int = 2, use_ref: bool = False):
        self.w = qweights
        self.ops = []
        for lw in qweights["layers"]:
            if "fa" in lw:
                att = O.RefFullAttention(lw["fa"], max_tokens) if use_ref else O.OracleFullAttention(lw["fa"], max_tokens, kv_mode)
            else:
                att = O.RefLinearAttention(lw["la"]) if use_ref else O.OracleLinearAttention(lw["la"])
            mlp = O.RefMLP(lw["ffn"]["gate"], lw["ffn"]["up"], lw["ffn"]["down"]) if use_ref else None
            self.ops.append((att, mlp))

    def forward_token(self, token: int, want_logits: bool = True):
        h = self.w["embed"][token].astype(np.float32)
        for lw, (att, mlp) in zip(self.w["layers"], self.ops):
            a = att.forward(O.rmsnorm(h, lw["input_norm"]))
            h = (h + a).astype(np.float32)
            h2 = O.rmsnorm(h, lw["post_norm"])
            m = mlp.forward(h2) if mlp is not None else O.mlp(lw["ffn"]["gate"], lw["ffn"]["up"], lw["ffn"]["down"], h2)
            h = (h + m).astype(np.float32)
        hn = O.rmsnorm(h, self.w["final_norm"])
        logits = self.w["embed"] @ hn if want_logits else None
        return hn, logits
