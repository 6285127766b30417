"""Generates the committed golden vectors from the reference's own compiled encoder.

Run where the reference tree is mounted (`make -C oracle` builds
oracle/_ref/libSpMM_API_ref.so from the reference sources):

    python tests/golden/make_golden.py

Small cases are stored whole (input bits, words, offsets); large ones as
SHA-256 digests of the outputs.  Inputs come from numpy's PCG64 with the seeds
below, plus hand-placed special values (-0, NaN, subnormals, infinities).
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

SMALL = [  # name, M, K, sparsity, seed
    ("one_tile_p80", 128, 64, 0.8, 11),
    ("one_tile_dense", 128, 64, 0.0, 12),
    ("one_tile_empty", 128, 64, 1.0, 13),
    ("tiles_2x2_p50", 256, 128, 0.5, 14),
    ("tiles_1x3_p999", 128, 192, 0.999, 15),
    ("tiles_3x1_p90_special", 384, 64, 0.9, 16),
]
LARGE = [("m1024_k1024_p80", 1024, 1024, 0.8, 21), ("m2048_k512_p70", 2048, 512, 0.7, 22),
         ("m512_k4096_p90", 512, 4096, 0.9, 23)]


def make_input(M, K, p, seed, special=False):
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((M, K)) * 0.02).astype(np.float16)
    A[rng.random((M, K)) < p] = 0
    bits = A.view(np.uint16).copy()
    if special:
        flat = bits.reshape(-1)
        idx = rng.choice(flat.size, 60, replace=False)
        for i, pattern in enumerate((0x8000, 0x7E00, 0xFE01, 0x0001, 0x83FF, 0x7C00)):
            flat[idx[10 * i:10 * i + 10]] = pattern
    return bits


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    small = {}
    for name, M, K, p, seed in SMALL:
        A = make_input(M, K, p, seed, special="special" in name)
        for variant in ("reorder", "noreorder"):
            w, o = oracle.ref_encode(A, variant)
            small[f"{name}__{variant}__words"] = w
            small[f"{name}__{variant}__offsets"] = o
        small[f"{name}__A"] = A
    np.savez_compressed(os.path.join(HERE, "tiled_csl_small.npz"), **small)
    large = {}
    for name, M, K, p, seed in LARGE:
        A = make_input(M, K, p, seed, special=True)
        entry = {"M": M, "K": K, "p": p, "seed": seed, "A_sha256": digest(A)}
        for variant in ("reorder", "noreorder"):
            w, o = oracle.ref_encode(A, variant)
            entry[variant] = {"n_words": int(w.size), "n_offsets": int(o.size), "words_sha256": digest(w),
                              "offsets_sha256": digest(o)}
        large[name] = entry
    with open(os.path.join(HERE, "tiled_csl_large.json"), "w") as f:
        json.dump(large, f, indent=1, sort_keys=True)
    print("wrote", len(small), "arrays and", len(large), "digests")


if __name__ == "__main__":
    main()
