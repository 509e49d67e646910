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
    if fields["path"] != "reference":
        assert fields["device_status"] == "ok"
        assert int(fields["launches"]) > 0
    return out, fields


def _reference_diffs(*args):
    """The same smoke on the all-reference link (the reference's own flash kernels, fp16 operands): what the
    reference itself measures between its flash and dense paths on this GPU."""
    out, f = _run(cpu.DROPIN_SMOKE_REFERENCE, *args)
    assert f["path"] == "reference"
    return _diffs(out)


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
    # The figures compare the flash layer with the reference's DENSE layer, whose GEMMs run in TF32: that error alone
    # is 1.5e-3 / 4e-3 on a B200 at embed 768 and it is what both the reference's flash kernels (1.3e-3 / 3.2e-3
    # measured with the all-reference link) and these exact kernels (1.5e-3 / 4.1e-3) are seen against.  So the bound
    # is the reference's own figure for the same smoke with room for that shared noise, plus an absolute backstop.
    ref_fwd, ref_bwd = _reference_diffs("flash", embed, heads, seq, maxpos)
    assert fwd <= max(2.0 * ref_fwd, 2e-3) and bwd <= max(2.0 * ref_bwd, 1e-2), (fwd, bwd, ref_fwd, ref_bwd)
    assert fwd <= 5e-3 and bwd <= 1e-1, (fwd, bwd)      # absolute backstop (backward: CudaCausalSelfAttention.cu:984)


@pytest.mark.parametrize("embed,heads,seq,maxpos", FLASH_ARGS[1:])
def test_reference_flash_parity_smoke_runs_on_tensor_cores(embed, heads, seq, maxpos):
    """head_dim 64 with reduced precision allowed: the tcgen05 kernels behind the same unmodified call sites."""
    out, f = _run(cpu.DROPIN_SMOKE, "flash", embed, heads, seq, maxpos, reduced=True)
    assert f["path"] == "tcgen05_staged"
    fwd, bwd = _diffs(out)
    # bf16 operands (8 mantissa bits) against the reference's fp16 operands (11 bits): a few times the reference's own
    # flash-versus-dense figure is expected; the backward bound is the one the reference's GQA smoke enforces (1e-1)
    ref_fwd, ref_bwd = _reference_diffs("flash", embed, heads, seq, maxpos)
    assert fwd <= max(12 * ref_fwd, 3e-2) and bwd <= 1e-1, (fwd, bwd, ref_fwd, ref_bwd)


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
    assert fwd <= 5e-3 and bwd <= 1e-1, (fwd, bwd)      # against the TF32 dense path, as above
    out, f = _run(cpu.DROPIN_SMOKE_D128, "flash", 1024, 8, 1024, 1024, reduced=True)
    assert f["path"] == "tcgen05_staged"
    fwd, bwd = _diffs(out)
    assert fwd <= 3e-2 and bwd <= 1e-1, (fwd, bwd)
    # the unmodified constant still refuses it, exactly as the reference does (CudaCausalSelfAttention.cu:824-825)
    r = subprocess.run([cpu.DROPIN_SMOKE, "flash", "512", "4", "256", "256"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and "headDim exceeds flash max" in r.stdout
