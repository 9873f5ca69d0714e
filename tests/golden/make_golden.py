"""Generates tests/golden/fa_reference_cases.npz with the reference project's OWN attention checker.

The outputs come from oracle/_ref (the reference's compute_reference_attention and its masked
variant, compiled unmodified from the reference tree by oracle/build_oracle.py), so this script only
runs where the reference tree is mounted.  Inputs are regenerated from seeds by `case_inputs`; the
fixture stores the outputs and a SHA-256 of the inputs so that drift of the generator is detected.

The cases are the shapes the reference's tests exercise (tests/test_flash_attention.cpp:141-582):
B=2, H=4, D=64 with S in {1, 4, 16, 32, 128}; S=16 with D in {16, 32, 64, 128}; causal; and the
half-visible [B,S,S] mask.  Inputs are uniform(-1, 1) like the reference's generate_random_data, but
seeded.

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

FIXTURE = os.path.join(HERE, "fa_reference_cases.npz")

# name -> (B, H, S, D, causal, masked, seed)
CASES = {}
for s in (1, 4, 16, 32, 128):
    CASES[f"seq{s}"] = (2, 4, s, 64, False, False, 100 + s)
    CASES[f"seq{s}_causal"] = (2, 4, s, 64, True, False, 200 + s)
for d in (16, 32, 64, 128):
    CASES[f"dim{d}"] = (2, 4, 16, d, False, False, 300 + d)
CASES["mask_half"] = (2, 4, 16, 64, False, True, 400)
CASES["mask_half_s32"] = (2, 4, 32, 64, False, True, 401)


def case_inputs(name):
    B, H, S, D, causal, masked, seed = CASES[name]
    rng = np.random.default_rng(seed)
    q, k, v = (rng.uniform(-1.0, 1.0, (B, H, S, D)).astype(np.float32) for _ in range(3))
    mask = None
    if masked:                       # first half of the keys visible, as in AttentionMaskTest
        mask = np.zeros((B, S, S), dtype=np.float32)
        mask[:, :, : S // 2] = 1.0
    scale = np.float32(1.0) / np.sqrt(np.float32(D))
    return q, k, v, mask, float(scale), causal


def inputs_digest(q, k, v, mask):
    h = hashlib.sha256()
    for a in (q, k, v) + ((mask,) if mask is not None else ()):
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    from oracle import cpu_oracle as o
    assert o.ref_available(), "the reference tree is not mounted: cannot regenerate the fixture"
    out = {}
    for name in CASES:
        q, k, v, mask, scale, causal = case_inputs(name)
        ref = o.ref_masked_attention(q, k, v, mask, scale) if mask is not None else o.ref_attention(q, k, v, scale, causal)
        out[name] = ref
        out[name + "__sha"] = np.frombuffer(inputs_digest(q, k, v, mask).encode(), dtype=np.uint8)
    np.savez_compressed(FIXTURE, **out)
    print(FIXTURE, os.path.getsize(FIXTURE), "bytes,", len(CASES), "cases")


if __name__ == "__main__":
    main()
