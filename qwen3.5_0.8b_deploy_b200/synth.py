"""Seeded synthetic weights and inputs for the attention hot path.

Every test, fixture and benchmark draws from here so the CPU checker and the GPU path see the
same bits.  The distributions are the ones the workload definitions state: matrices ~ N(0, 0.02),
hidden states ~ N(0, 1), A_log ~ U(0, 2.7), dt_bias ~ N(0, 0.1), q/k norm weights 0 (they enter as
1 + w), DeltaNet norm weight 1.  Generator: numpy Philox, keyed by (seed, stream name).
"""
from __future__ import annotations

import zlib

import numpy as np

HIDDEN = 1024
FA_HEADS, FA_KV_HEADS, FA_HEAD_DIM, FA_ROTARY = 8, 2, 256, 64
ROPE_THETA = 1e7
LA_HEADS, LA_KD, LA_VD, LA_CONV_K = 16, 128, 128, 4
LA_CONV_DIM = LA_HEADS * (2 * LA_KD + LA_VD)          # 6144
FFN_INTER = 3584
VOCAB = 248320
NUM_LAYERS = 24


def is_full_attention_layer(i: int) -> bool:
    """Layers 3, 7, ..., 23 are gated full attention; the other 18 are Gated DeltaNet
    (src/backend/cpu/core/common/language_common.hpp:36-53 in the reference)."""
    return i % 4 == 3


def rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, zlib.crc32(name.encode())]))


def normal(seed, name, shape, std=1.0):
    return (rng(seed, name).standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def fa_weights(seed: int, tag: str = "fa") -> dict:
    """W_q [4096,1024] (per head: 256 q rows then 256 gate rows), W_k/W_v [512,1024],
    q_norm/k_norm [256], W_o [1024,2048]; row-major (out, in)."""
    return dict(
        wq=normal(seed, tag + ".wq", (FA_HEADS * FA_HEAD_DIM * 2, HIDDEN), 0.02),
        wk=normal(seed, tag + ".wk", (FA_KV_HEADS * FA_HEAD_DIM, HIDDEN), 0.02),
        wv=normal(seed, tag + ".wv", (FA_KV_HEADS * FA_HEAD_DIM, HIDDEN), 0.02),
        q_norm=np.zeros(FA_HEAD_DIM, np.float32),
        k_norm=np.zeros(FA_HEAD_DIM, np.float32),
        wo=normal(seed, tag + ".wo", (HIDDEN, FA_HEADS * FA_HEAD_DIM), 0.02),
    )


def la_weights(seed: int, tag: str = "la") -> dict:
    """W_qkv [6144,1024], W_a/W_b [16,1024], W_z [2048,1024], conv [6144,4], A_log/dt_bias [16],
    norm [128], W_out [1024,2048]."""
    return dict(
        w_qkv=normal(seed, tag + ".w_qkv", (LA_CONV_DIM, HIDDEN), 0.02),
        w_a=normal(seed, tag + ".w_a", (LA_HEADS, HIDDEN), 0.02),
        w_b=normal(seed, tag + ".w_b", (LA_HEADS, HIDDEN), 0.02),
        w_z=normal(seed, tag + ".w_z", (LA_HEADS * LA_VD, HIDDEN), 0.02),
        conv_w=normal(seed, tag + ".conv_w", (LA_CONV_DIM, LA_CONV_K), 0.02),
        a_log=rng(seed, tag + ".a_log").uniform(0.0, 2.7, LA_HEADS).astype(np.float32),
        dt_bias=normal(seed, tag + ".dt_bias", (LA_HEADS,), 0.1),
        norm_w=np.ones(LA_VD, np.float32),
        w_out=normal(seed, tag + ".w_out", (HIDDEN, LA_HEADS * LA_VD), 0.02),
    )


def ffn_weights(seed: int, tag: str) -> dict:
    return dict(
        gate=normal(seed, tag + ".gate", (FFN_INTER, HIDDEN), 0.02),
        up=normal(seed, tag + ".up", (FFN_INTER, HIDDEN), 0.02),
        down=normal(seed, tag + ".down", (HIDDEN, FFN_INTER), 0.02),
    )


def hidden_states(seed: int, name: str, rows: int) -> np.ndarray:
    return normal(seed, name, (rows, HIDDEN), 1.0)
