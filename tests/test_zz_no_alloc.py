"""GPU: the allocation-free decode attention entry point (b200attn_fa_decode_core_static).

Some callers of this library cannot allocate device memory while they run — a warm serving loop that must
not hit cudaMalloc / cudaFree (they stall the whole device), or a plugin living inside a fixed memory budget.
For them the library carries its own fixed scratch array.  This file checks, through the C ABI, that the
entry point gives the right result on two calls in a row (the second one with other queries, so left-over
scratch contents from the first call would show) — against b200attn_fa_decode_core and against a float64
softmax over the exported cache — that the free device memory is the same after the two calls as before
them, and that it refuses requests larger than its built-in scratch.  It is named so that pytest collects it after every other test file.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_dtype", [0, 1])
def test_static_scratch_entry_matches_the_handle_based_entry(ops, cuda, synth, kv_dtype):
    torch = cuda
    lengths = [1, 65, 700, 1500]
    n = len(lengths)
    fa = ops.FullAttention(ops.PROJ_FP32, max_batch=8, max_prefill_rows=64)
    kv = ops.KVCache(2, 8, 1536, kv_dtype)
    slots = [kv.allocate_sequence(0) for _ in range(n)]
    k = np.concatenate([synth.normal(71, f"na.k.{i}", (L, 512), 1.0) for i, L in enumerate(lengths)])
    v = np.concatenate([synth.normal(71, f"na.v.{i}", (L, 512), 0.6) for i, L in enumerate(lengths)])
    kv.append(1, slots, lengths, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    d_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    qs = [torch.from_numpy(synth.normal(71, f"na.q.{call}", (n, 8, 256), 1.0)).cuda() for call in range(2)]
    wants = [fa.decode_core(q, kv, 1, d_slots) for q in qs]
    outs = [torch.full((n, 8, 256), float("nan"), dtype=torch.float32, device="cuda") for _ in range(2)]   # caller-owned
    ops.fa_decode_core_static(qs[0], kv, 1, d_slots, outs[0])      # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):
        outs[call].fill_(float("nan"))
        ops.fa_decode_core_static(qs[call], kv, 1, d_slots, outs[call])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the free device memory"
    exported = [kv.export(1, s) for s in slots]
    for call in range(2):
        err = (outs[call] - wants[call]).abs().max().item()
        assert err <= 2e-3, f"call {call}: max abs difference to the handle-based entry {err:.3e}"
        q64 = qs[call].half().double()
        for i in range(n):
            kc, vc, ksc, vsc = exported[i]
            kd, vd = kc.double(), vc.double()
            if ksc is not None:
                kd, vd = kd * ksc.double()[..., None], vd * vsc.double()[..., None]
            for grp in range(2):
                p = torch.softmax(q64[i, 4 * grp:4 * grp + 4] @ kd[:, grp].T / 16.0, dim=1)
                err = (outs[call][i, 4 * grp:4 * grp + 4].double() - p @ vd[:, grp]).abs().max().item()
                assert err <= 2e-3, f"call {call} sequence {i} group {grp}: max abs err against float64 {err:.3e}"
    assert kv.device_status() == 0


def test_static_scratch_entry_rejects_oversized_requests(ops, cuda):
    torch = cuda
    lib = ops.lib()
    kv = ops.KVCache(1, 40, 64, ops.KV_INT8)
    z = torch.zeros((40, 8, 256), device="cuda")
    slots = torch.zeros(40, dtype=torch.int32, device="cuda")
    rc = lib.b200attn_fa_decode_core_static(kv.h, 0, C.c_void_p(slots.data_ptr()), 33, C.c_void_p(z.data_ptr()),
                                            C.c_void_p(z.data_ptr()), None)
    assert rc == ops.ERR_INVALID and b"at most 32" in lib.b200attn_last_error()
    big = ops.KVCache(1, 1, 513 * 64, ops.KV_INT8, num_pages=4)              # block table wider than the scratch is sized for
    rc = lib.b200attn_fa_decode_core_static(big.h, 0, C.c_void_p(slots.data_ptr()), 1, C.c_void_p(z.data_ptr()),
                                            C.c_void_p(z.data_ptr()), None)
    assert rc == ops.ERR_INVALID and b"512" in lib.b200attn_last_error()
    rc = lib.b200attn_fa_decode_core_static(None, 0, None, 1, None, None, None)
    assert rc == ops.ERR_INVALID
