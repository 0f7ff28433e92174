"""GPU: the tcgen05 / TMA building blocks (operand layouts, descriptors, TMEM read-back) on one tile."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant,n,k", [(0, 64, 256), (0, 256, 64), (0, 128, 128), (1, 256, 64), (1, 128, 128),
                                         (1, 128, 64), (2, 64, 128), (2, 128, 64)])
def test_umma_tile(ops, cuda, synth, variant, n, k):
    torch = cuda
    tf32, bmn = bool(variant & 2), bool(variant & 1)
    a = synth.normal(11, f"umma.a.{variant}.{n}.{k}", (128, k))
    b = synth.normal(11, f"umma.b.{variant}.{n}.{k}", (k, n) if bmn else (n, k))
    if tf32:   # operands exactly representable in tf32 (10-bit mantissa) so truncation is a no-op
        a = (a.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
        b = (b.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    else:
        a = a.astype(np.float16).astype(np.float32)
        b = b.astype(np.float16).astype(np.float32)
    want = a.astype(np.float64) @ (b if bmn else b.T).astype(np.float64)
    d = ops.selftest_umma(variant, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), n, k).cpu().numpy()
    err = np.abs(d - want).max()
    assert err <= 1e-3 * max(1.0, np.abs(want).max()), f"variant {variant} N={n} K={k}: max err {err:.3e}"


def test_tf32_mn_major_is_refused(ops, cuda):
    torch = cuda
    z = torch.zeros((128, 64), device="cuda")
    with pytest.raises(ops.B200AttnError) as e:
        ops.selftest_umma(3, z, z, 128, 64)
    assert e.value.status == ops.ERR_UNSUPPORTED
