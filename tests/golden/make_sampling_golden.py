"""Generate tests/golden/sampling_cases.npz from the REFERENCE's object code: rows of logits, a
generator seed, the uniform numbers the reference demo's ``sample_row`` consumes from
``std::mt19937(seed)``, and what ``row_logsumexp`` / ``sample_row`` (apps/04_gpt2_grpo.cu:61-78,
compiled into oracle/_ref/libgrpo_ref_sample.so by ``make -C oracle ref-sample``) return.

    make -C oracle oracle ref-sample && python tests/golden/make_sampling_golden.py

Needs the reference tree (to build the library); the committed ``.npz`` travels without it.  Seeds
whose coins fall within 1e-9 of a boundary of the cumulative distribution are skipped, so the
tokens do not hinge on the last bits of a sum.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_SAMPLE = os.path.join(ROOT, "oracle", "_ref", "libgrpo_ref_sample.so")

_fp = C.POINTER(C.c_float)


def load_reference_sampler():
    lib = C.CDLL(REF_SAMPLE)
    lib.grpo_ref_row_logsumexp.restype = C.c_double
    lib.grpo_ref_row_logsumexp.argtypes = [_fp, C.c_int]
    lib.grpo_ref_sample_rows.argtypes = [_fp, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_uint,
                                         C.POINTER(C.c_int)]
    lib.grpo_ref_coins.argtypes = [C.c_uint, C.c_int, C.POINTER(C.c_double)]
    return lib


def reference_draws(lib, x: np.ndarray, seed: int):
    """(lse[n], coins[n], tokens[n]) for one draw per row of ``x`` in row order from mt19937(seed)."""
    n, V = x.shape
    x = np.ascontiguousarray(x, np.float32)
    rows = np.arange(n, dtype=np.int32)
    tokens = np.zeros(n, np.int32)
    coins = np.zeros(n, np.float64)
    lib.grpo_ref_sample_rows(x.ctypes.data_as(_fp), V, V, rows.ctypes.data_as(C.POINTER(C.c_int)), n, seed,
                             tokens.ctypes.data_as(C.POINTER(C.c_int)))
    lib.grpo_ref_coins(seed, n, coins.ctypes.data_as(C.POINTER(C.c_double)))
    lse = np.array([lib.grpo_ref_row_logsumexp(x[i].ctypes.data_as(_fp), V) for i in range(n)])
    return lse, coins, tokens


def main() -> None:
    lib = load_reference_sampler()
    rng = np.random.default_rng(20240611)
    blob = {}
    for V, sigma in ((17, 1.0), (257, 2.0), (4099, 3.0), (50257, 3.0)):
        n = 6
        x = rng.normal(0, sigma, (n, V)).astype(np.float32)
        x[1] = 0.25                 # flat row
        x[2, V // 3] += 30.0        # one dominant token
        seed = 1000 + V
        while True:
            lse, coins, tokens = reference_draws(lib, x, seed)
            margin = min(np.abs(np.cumsum(np.exp(x[i].astype(np.float64) - lse[i])) - coins[i]).min() for i in range(n))
            if margin > 1e-9:
                break
            seed += 1
        logp = np.array([np.float32(np.float64(x[i, tokens[i]]) - lse[i]) for i in range(n)], np.float32)
        key = f"V{V}"
        blob.update({f"{key}/logits": x, f"{key}/seed": np.array(seed, np.uint32), f"{key}/coins": coins,
                     f"{key}/lse": lse, f"{key}/tokens": tokens, f"{key}/logp": logp})
    out = os.path.join(HERE, "sampling_cases.npz")
    np.savez_compressed(out, **blob)
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
