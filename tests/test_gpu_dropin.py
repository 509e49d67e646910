"""The drop-in proof: the reference's own attention layer, through its own unmodified launch sites, on this library.

``oracle/_ref/dropin_smoke`` is the reference's ``CudaCausalSelfAttention.cu`` (+ the sources it needs) linked with
``sentinel_b200/csrc/sentinel_compat.cu`` in the place of the reference's ``CudaFlashAttention.cu`` (recipe:
``oracle/Makefile``, target ``dropin``).  It runs the reference's own smokes:

* ``runFlashParitySmokeDemo`` (sentinel/NeuralNet/Cuda/CudaCausalSelfAttention.cu:817-894) with the four argument sets
  of sentinel/main.cpp:640-643 -- it throws when the flash path was not selected and prints flash-versus-dense
  differences of the layer output and of all five gradients;
* ``runGqaCudaSmokeDemo`` (:896-997) -- it throws when flash and dense differ by more than 1e-3 forward / 1e-1 backward.

The harness then reports which kernel family of this library served the calls and how many kernels it launched.
"""
import os
import re
import subprocess

import pytest

from oracle import cpu

pytestmark = pytest.mark.gpu

FLASH_ARGS = [(64, 4, 48, 64), (768, 12, 128, 512), (768, 12, 256, 512), (768, 12, 1024, 1024)]


def _run(exe, *args, reduced=False):
    if not os.path.exists(exe):
        pytest.skip(f"{exe} was not built (reference sources absent at build time)")
    env = dict(os.environ)
    env["SNTL_ATTN_REDUCED_PRECISION"] = "1" if reduced else "0"
    r = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600, env=env)
    out = r.stdout
    fields = dict(re.findall(r"^(\w+)=(.*)$", out, flags=re.M))
    assert r.returncode == 0, (r.returncode, out, r.stderr)
    assert fields["device_status"] == "ok"
    assert int(fields["launches"]) > 0
    return out, fields


def _diffs(out):
    m = re.search(r"fwdDiff=([0-9.e+-]+)\s+bwdDiff=([0-9.e+-]+)", out)
    assert m, out
    return float(m.group(1)), float(m.group(2))


@pytest.mark.parametrize("embed,heads,seq,maxpos", FLASH_ARGS)
def test_reference_flash_parity_smoke_runs_on_this_library_exact(embed, heads, seq, maxpos):
    """fp32 matrices, default setting: the exact fp32 kernels serve the reference's flash call sites."""
    out, f = _run(cpu.DROPIN_SMOKE, "flash", embed, heads, seq, maxpos)
    assert f["path"] == "simt_f32"
    assert f["maxHeadDimension"] == "64"
    fwd, bwd = _diffs(out)
    # flash versus the reference's dense cuBLASLt path (TF32 GEMMs): the reference's own bound for this comparison
    # is 1e-3 forward / 1e-1 backward (CudaCausalSelfAttention.cu:984)
    assert fwd <= 1e-3 and bwd <= 1e-1, (fwd, bwd)


@pytest.mark.parametrize("embed,heads,seq,maxpos", FLASH_ARGS[1:])
def test_reference_flash_parity_smoke_runs_on_tensor_cores(embed, heads, seq, maxpos):
    """head_dim 64 with reduced precision allowed: the tcgen05 kernels behind the same unmodified call sites."""
    out, f = _run(cpu.DROPIN_SMOKE, "flash", embed, heads, seq, maxpos, reduced=True)
    assert f["path"] == "tcgen05_staged"
    fwd, bwd = _diffs(out)
    assert fwd <= 5e-3 and bwd <= 1e-1, (fwd, bwd)


@pytest.mark.parametrize("reduced", [False, True])
def test_reference_gqa_cuda_smoke_runs_on_this_library(reduced):
    """8 query heads, 2 KV heads, head_dim 8: the reference repeats K/V to 8 heads before its flash call; the smoke
    itself enforces host/dense/flash agreement and throws otherwise."""
    out, f = _run(cpu.DROPIN_SMOKE, "gqa", reduced=reduced)
    assert f["path"] == "simt_f32"   # head_dim 8 has no tensor-core kernel
    assert "flashDenseFwd" in out


def test_head_dim_128_variant_reaches_flash():
    """The same link with maxHeadDimension raised to 128 (the one constant an integrator edits): a head_dim-128 layer,
    which the reference sends down its dense path (CudaCausalSelfAttention.cu:48), now takes the flash call sites."""
    out, f = _run(cpu.DROPIN_SMOKE_D128, "flash", 512, 4, 256, 256)
    assert f["maxHeadDimension"] == "128" and f["path"] == "simt_f32"
    fwd, bwd = _diffs(out)
    assert fwd <= 1e-3 and bwd <= 1e-1, (fwd, bwd)
    out, f = _run(cpu.DROPIN_SMOKE_D128, "flash", 1024, 8, 1024, 1024, reduced=True)
    assert f["path"] == "tcgen05_staged"
    fwd, bwd = _diffs(out)
    assert fwd <= 5e-3 and bwd <= 1e-1, (fwd, bwd)
