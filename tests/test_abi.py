"""CPU: the C-ABI library loads, exports exactly what include/b200attn.h declares, and rejects bad
arguments with the documented status codes before touching the device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200attn_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(ops):
    assert declared_symbols() == sorted(ops.ABI_SYMBOLS)


def test_library_exports_every_declared_symbol(ops):
    lib = C.CDLL(ops.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert ops.lib().b200attn_abi_version() == 1


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "b200attn.h"\nint main(void){ b200attn_kv_config c; (void)c; return B200ATTN_OK; }\n')
    rc = os.system(f"gcc -std=c99 -Wall -Werror -I{ROOT}/include -c {src} -o {tmp_path}/t.o")
    assert rc == 0


def test_every_entry_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    # each prototype is preceded by a comment block; collect comment + prototype name pairs
    for m in re.finditer(r"/\*((?:(?!\*/).)*)\*/\s*(?:int|long long|const char\*)\s+(b200attn_[a-z0-9_]+)\s*\(", text, flags=re.S):
        comment, name = m.group(1), m.group(2)
        assert re.search(r"\.(cu|cpp|hpp|cuh|h):\d+", comment) or "counterpart" in comment.lower() or name in (
            "b200attn_last_error", "b200attn_abi_version"), name


def test_bad_configs_are_rejected_without_a_device(ops):
    lib = ops.lib()
    h = C.c_void_p()
    # null pointers
    assert lib.b200attn_fa_create(None, C.byref(h)) == ops.ERR_INVALID
    assert b"null" in lib.b200attn_last_error()
    # shapes the kernels are not built for
    cfg = ops.FaConfig(1024, 8, 2, 128, 64, 1e7, ops.PROJ_FP32, 4, 64)
    assert lib.b200attn_fa_create(C.byref(cfg), C.byref(h)) == ops.ERR_UNSUPPORTED
    cfg = ops.LaConfig(1024, 16, 64, 128, 4, ops.PROJ_FP32, 4, 64)
    assert lib.b200attn_la_create(C.byref(cfg), C.byref(h)) == ops.ERR_UNSUPPORTED
    kc = ops.KvConfig(1, 2, 256, 32, 8, 2, 4, ops.KV_INT8)
    assert lib.b200attn_kv_pool_create(C.byref(kc), C.byref(h)) == ops.ERR_UNSUPPORTED
    kc = ops.KvConfig(0, 2, 256, 64, 8, 2, 4, ops.KV_INT8)
    assert lib.b200attn_kv_pool_create(C.byref(kc), C.byref(h)) == ops.ERR_INVALID
    kc = ops.KvConfig(1, 2, 256, 64, 8, 2, 4, 7)
    assert lib.b200attn_kv_pool_create(C.byref(kc), C.byref(h)) == ops.ERR_INVALID
    sc = ops.LaStateConfig(0, 4, 16, 128, 128, 4)
    assert lib.b200attn_la_state_create(C.byref(sc), C.byref(h)) == ops.ERR_INVALID
    # destroying null handles is a no-op
    assert lib.b200attn_fa_destroy(None) == 0 and lib.b200attn_kv_pool_destroy(None) == 0
    assert lib.b200attn_la_destroy(None) == 0 and lib.b200attn_stack_destroy(None) == 0


def test_python_wrapper_raises_typed_errors(ops):
    with pytest.raises(ops.InvalidArgument):
        ops._check(ops.lib().b200attn_kv_seq_len(None, 0, 0, None))
    with pytest.raises(ValueError):   # InvalidArgument is also a ValueError, like std::invalid_argument
        ops._check(ops.lib().b200attn_fa_set_weights(None, None))
