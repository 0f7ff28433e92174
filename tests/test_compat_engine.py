"""The reference's engine source compiles, unmodified, against the shim headers, and every attention-side symbol it then
needs is exported by the compat library.

The shims carry the reference's header names (full_attention_cuda.hpp, linear_attention_cuda.hpp, flash_attention.cuh ...)
and are meant to REPLACE those files in the reference's include directory: cuda_engine.hpp includes its siblings with
quotes, so a plain -I in front of the old directory would pick up the old classes.  This test builds that directory the
way a maintainer would (shims over originals, everything else untouched) in a temporary folder, compiles
src/backend/cuda/kernels/cuda_engine.cu and cuda_engine_v3.cu from where they lie, and checks the undefined qwen::cuda
symbols of the object: what is not ours must belong to the reference's own MLP / RMSNorm / LM-head / embedding classes, which stay as they are.

Needs the reference checkout and nvcc; skipped where either is missing (the GPU box has no checkout).
"""
import os
import shutil
import subprocess

import pytest

from oracle.cpu_oracle import reference_root

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMPAT = os.path.join(REPO, "qwen3.5_0.8b_deploy_b200", "compat")
REF_CUDA = os.path.join(reference_root(), "src", "backend", "cuda")

pytestmark = pytest.mark.skipif(
    not os.path.isfile(os.path.join(REF_CUDA, "kernels", "cuda_engine.cu")) or shutil.which("nvcc") is None,
    reason="needs the reference checkout and nvcc")

OUT_OF_SCOPE = ("CudaMLP::", "CudaRMSNorm::", "CudaLMHead::", "CudaTokenEmbedding::")   # the reference's own mlp / rmsnorm / lm_head / token_embedding sources


def _qwen_symbols(args):
    out = subprocess.check_output(["nm", "-C"] + args, text=True)
    syms = set()
    for line in out.splitlines():
        if "qwen::" in line:
            syms.add(line[line.index("qwen::"):].strip())
    return syms


@pytest.mark.parametrize("source", ["cuda_engine.cu", "cuda_engine_v3.cu"])
def test_reference_engine_compiles_and_links_against_the_shims(tmp_path, source):
    lib = os.path.join(REPO, "qwen3.5_0.8b_deploy_b200", "libb200attn_compat.so")
    if not os.path.exists(lib):
        import __graft_entry__
        __graft_entry__.build()
    inc = tmp_path / "include"
    inc.mkdir()
    shims = os.path.join(COMPAT, "include_shims")
    for name in os.listdir(os.path.join(REF_CUDA, "include")):
        shim = os.path.join(shims, name)
        if os.path.isfile(shim):
            text = open(shim).read().replace('"../qwen_cuda_compat.hpp"', '"%s"' % os.path.join(COMPAT, "qwen_cuda_compat.hpp"))
            (inc / name).write_text(text)
        else:
            os.symlink(os.path.join(REF_CUDA, "include", name), inc / name)
    obj = tmp_path / "cuda_engine.o"
    subprocess.check_call(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-c",
                           os.path.join(REF_CUDA, "kernels", source), "-o", str(obj),
                           "-I", str(inc), "-I", os.path.join(REPO, "include")])
    wanted = _qwen_symbols(["-u", str(obj)])
    provided = _qwen_symbols(["-D", "--defined-only", lib])
    ours = {s for s in wanted if not any(k in s for k in OUT_OF_SCOPE)}
    assert ours, "the engine should reference the attention classes"
    missing = sorted(ours - provided)
    assert not missing, "not exported by the compat library: %s" % missing
    if source != "cuda_engine.cu":
        return
    for cls in ("CudaFullAttention::forward(", "CudaFullAttention::forward_batch_prefill(", "CudaLinearAttention::forward(",
                "CudaLinearAttention::forward_batch(", "CudaKVCache::reset(", "CudaLinearAttnState::reset(", "set_fa_weights("):
        assert any(cls in s for s in ours), cls
