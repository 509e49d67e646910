import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu on the GPU box")


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


GOLDEN_CASES = ["toy_f32_b4_h4_s64_d16", "gqa_h8_kv2_s16_d8", "mha_h4_s48_d16", "gqa_h4_kv1_s200_d64_bf16in",
                "gqa_h4_kv2_s136_d128_bf16in"]
WINDOW_GOLDEN_CASES = ["win4_g2_h2_s16_d16", "win17_g0_h4_kv2_s96_d16", "win64_g5_h4_s200_d32",
                       "win100_g3_h4_kv1_s300_d64_bf16in", "win130_g140_h2_kv1_s520_d128_bf16in"]
ROPE_GOLDEN_CASES = ["rope_h3_d16_c40_base1e4", "rope_h2_d128_c70_base1e6"]
ROPE_LAYER_GOLDEN = "ropelayer_h4_kv2_s160_d64_bf16in"


def max_abs(a, b):
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64))))


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu
    cpu.build()
    return cpu
