"""GPU: the source-compatible C++ operator classes (qwen::cuda::CudaFullAttention, CudaKVCache,
CudaLinearAttention[V2], CudaLinearAttnState) on top of the C ABI — this repository's own check program and,
when it was built from the reference checkout, the reference's unmodified verify_linear_attn_batch program."""
import os
import subprocess

import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


def test_compat_check_program(cuda):
    exe = os.path.join(entry.PKG_DIR, "compat", "compat_check")
    assert os.path.exists(exe), "compat_check was not built (python __graft_entry__.py build)"
    p = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "compat_check: PASS" in p.stdout, p.stdout + p.stderr


def test_reference_verify_linear_attn_batch_unmodified(cuda):
    exe = os.path.join(entry.ROOT, "oracle", "_ref", "verify_linear_attn_batch")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/verify_linear_attn_batch not built (needs the reference checkout at build time)")
    p = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "PASS" in p.stdout, p.stdout + p.stderr


def test_reference_v2_kernel_accuracy_validate_unmodified(cuda):
    """tests/integration/v2_kernel_accuracy_validate.cu of the reference, built as it is against the compat headers: it
    runs CudaLinearAttentionV2 at hidden 256 / 4 heads / dims 64 (the plain path for sizes other than the model's) and
    checks determinism of forward and forward_batch and that the state moves."""
    exe = os.path.join(entry.ROOT, "oracle", "_ref", "v2_kernel_accuracy_validate")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/v2_kernel_accuracy_validate not built (needs the reference checkout at build time)")
    p = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "FAILED" not in p.stdout, p.stdout + p.stderr
