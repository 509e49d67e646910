"""Generates the golden fixtures of this directory by running the reference's OWN CPU attention layer
(compiled from the reference sources into oracle/_ref by oracle/Makefile) on seeded inputs.

The reference stores no golden vectors for this path; its tests are parity procedures between two of its own
implementations on LCG/seeded inputs.  These fixtures freeze the outputs of its CPU layer
(CausalSelfAttention::forward/backward through the public API, see oracle/ref_harness.cpp) so that the fp64
restatement and the CUDA kernels can be checked where the reference sources are not available.

Run from the repository root, where the reference is mounted:   python tests/golden/make_golden.py
Each case is stored as <name>.npz with inputs (q, k, v, dout) and reference outputs (o, lse, dq, dk, dv), fp32,
token-major [B, H, S, D]; sliding-window cases also hold the layer's ``window`` and ``global_tokens``.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import cpu  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (B, Hq, Hkv, S, D, input std, seed, round inputs to bf16)
CASES = {
    # BASELINE config 1: the repo-default toy LM attention, fp32
    "toy_f32_b4_h4_s64_d16": (4, 4, 4, 64, 16, 1.0, 101, False),
    # shape of the reference's runGqaHostSmokeDemo (E=64, 8 heads, 2 KV heads, S=16)
    "gqa_h8_kv2_s16_d8": (1, 8, 2, 16, 8, 1.0, 102, False),
    # shape of runFlashParitySmokeDemo(64, 4, 48, 64): S not a multiple of any tile size
    "mha_h4_s48_d16": (2, 4, 4, 48, 16, 1.0, 103, False),
    # tensor-core head sizes at ragged lengths, inputs pre-rounded to bf16 (what the bf16 kernels see)
    "gqa_h4_kv1_s200_d64_bf16in": (1, 4, 1, 200, 64, 0.5, 104, True),
    "gqa_h4_kv2_s136_d128_bf16in": (1, 4, 2, 136, 128, 0.5, 105, True),
}


# sliding window + global tokens (the reference layer's windowSize / globalTokenCount): name: (spec as above, window, global)
WINDOW_CASES = {
    # shape and mask of the reference's runSparseMaskSmokeDemo(32, 2, 16, 32, 4, 2) (main.cpp:759)
    "win4_g2_h2_s16_d16": ((1, 2, 2, 16, 16, 1.0, 111, False), 4, 2),
    "win17_g0_h4_kv2_s96_d16": ((2, 4, 2, 96, 16, 1.0, 112, False), 17, 0),
    "win64_g5_h4_s200_d32": ((1, 4, 4, 200, 32, 1.0, 113, False), 64, 5),
    # tensor-core head sizes: windows that cut through tiles, global tokens, ragged lengths
    "win100_g3_h4_kv1_s300_d64_bf16in": ((1, 4, 1, 300, 64, 0.5, 114, True), 100, 3),
    "win130_g140_h2_kv1_s520_d128_bf16in": ((1, 2, 1, 520, 128, 0.5, 115, True), 130, 140),
}


# rotary embedding: (heads, head_dim, cols, table positions, base, seed): the reference's RotaryEmbedding on a feature-major matrix
ROPE_CASES = {
    "rope_h3_d16_c40_base1e4": (3, 16, 40, 64, 1.0e4, 121),
    "rope_h2_d128_c70_base1e6": (2, 128, 70, 96, 1.0e6, 122),
}
# the reference layer with its rotary embedding active (un-rotated inputs in, gradients w.r.t. them out): (spec, base)
ROPE_LAYER_CASES = {
    "ropelayer_h4_kv2_s160_d64_bf16in": ((1, 4, 2, 160, 64, 0.5, 131, True), 1.0e4),
}


def make_case(B, Hq, Hkv, S, D, std, seed, bf16_inputs):
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal((B, Hq, S, D)) * std).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, S, D)) * std).astype(np.float32)
    v = rng.standard_normal((B, Hkv, S, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, S, D)).astype(np.float32)
    if bf16_inputs:
        q, k, v, dout = (cpu.round_bf16(t) for t in (q, k, v, dout))
    return q, k, v, dout


def main():
    if not cpu.ref_available():
        cpu.build()
    for name, spec in CASES.items():
        q, k, v, dout = make_case(*spec)
        o, lse, dq, dk, dv = cpu.ref_layer_fwd_bwd(q, k, v, dout)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, q=q, k=k, v=v, dout=dout, o=o, lse=lse, dq=dq, dk=dk, dv=dv)
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB")
    for name, (spec, window, global_tokens) in WINDOW_CASES.items():
        q, k, v, dout = make_case(*spec)
        o, lse, dq, dk, dv = cpu.ref_layer_fwd_bwd(q, k, v, dout, window=window, global_tokens=global_tokens)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, q=q, k=k, v=v, dout=dout, o=o, lse=lse, dq=dq, dk=dk, dv=dv,
                            window=np.int32(window), global_tokens=np.int32(global_tokens))
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB")
    for name, (H, D, cols, positions, base, seed) in ROPE_CASES.items():
        m = np.random.default_rng(seed).standard_normal((H * D, cols)).astype(np.float32)
        rotated, cos_t, sin_t = cpu.ref_rope(m, H, D, positions, base)
        unrotated, _, _ = cpu.ref_rope(m, H, D, positions, base, inverse=True)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, matrix=m, cos=cos_t, sin=sin_t, rotated=rotated, inverse_rotated=unrotated,
                            heads=np.int32(H), head_dim=np.int32(D), base=np.float32(base))
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB")
    for name, (spec, base) in ROPE_LAYER_CASES.items():
        q, k, v, dout = make_case(*spec)
        o, dq, dk, dv = cpu.ref_layer_fwd_bwd_rope(q, k, v, dout, base)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, q=q, k=k, v=v, dout=dout, o=o, dq=dq, dk=dk, dv=dv, base=np.float32(base))
        print(f"{name}: wrote {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
