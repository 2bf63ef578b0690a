"""Generates tests/golden/oft_ref_vectors.npz from the reference's own cpu_oft_tn.

Run in a container that holds the reference tree (oracle/build_ref.sh compiles its unmodified
cpu_oft.hpp into oracle/_ref/).  The vectors pin the plain-C restatement (oracle/oft_oracle.c) on
machines where the reference is absent:
    python tests/golden/make_golden.py
Each case stores the seeded inputs and the reference's output as fp16 bit patterns.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from cute_mma_b200 import inputs  # noqa: E402
from oracle import oracle  # noqa: E402

# name: (m, group_size, n_groups, k, reconn_sz, R kind, input distribution)
CASES = {
    "b8_g2": (16, 32, 2, 64, 8, "qr", "uniform"),
    "b32_g1": (24, 48, 1, 96, 32, "qr", "uniform"),
    "b64_g3": (8, 16, 3, 128, 64, "cayley", "normal"),
    "b128_g2": (5, 24, 2, 256, 128, "qr", "normal"),
    "perm_u01": (12, 40, 1, 64, 16, "perm", "u01"),
    "zero_one": (12, 40, 2, 64, 8, "perm", "01"),
}


def make_inputs(m, gs, G, k, b, kind, dist, seed):
    n = gs * G
    gen = {"uniform": inputs.uniform_pm1, "u01": inputs.uniform_01, "01": inputs.zero_one,
           "normal": lambda s, sd: inputs.normal(s, sd, 1.0)}[dist]
    A, B = gen((m, k), seed), gen((n, k), seed + 1)
    blocks = {"qr": inputs.blocks_qr, "cayley": inputs.blocks_cayley, "perm": inputs.blocks_permutation}[kind](G, k // b, b, seed + 2)
    return A, inputs.pack_r(blocks), B


def main():
    oracle.build(with_reference=True)
    assert oracle.have_reference(), "the reference build (oracle/_ref) is needed to make golden vectors"
    out = {}
    for i, (name, (m, gs, G, k, b, kind, dist)) in enumerate(CASES.items()):
        A, R, B = make_inputs(m, gs, G, k, b, kind, dist, seed=100 + 10 * i)
        C = oracle.ref_cpu_oft_tn(A, R, B, m, gs, G, k, b)
        out[f"{name}__dims"] = np.array([m, gs, G, k, b], dtype=np.int32)
        for key, arr in (("A", A), ("R", R), ("B", B), ("C", C)):
            out[f"{name}__{key}"] = arr.view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "oft_ref_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "oft_ref_vectors.npz"), sorted(CASES))


if __name__ == "__main__":
    main()
