"""Generate tests/golden/sampling_cases.npz: rows of logits, uniform numbers, and what the C
restatement of the reference demo's host-side sampling (apps/04_gpt2_grpo.cu:61-80) returns for
them -- row log-sum-exp, drawn token, fp32 log-probability.

    make -C oracle oracle && python tests/golden/make_sampling_golden.py

Unlike the other golden files these vectors do NOT come from the reference's object code (the demo
cannot be built without the absent llm.c sources): they freeze the restatement, so that it cannot
drift, and give the CUDA path a committed target.  Coins closer than 1e-9 to a boundary of the
cumulative distribution are re-drawn, so the tokens do not hinge on the last bits of a sum.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import oracle_py  # noqa: E402


def main() -> None:
    port = oracle_py.load("port")
    rng = np.random.default_rng(20240611)
    blob = {}
    for V, sigma in ((17, 1.0), (257, 2.0), (4099, 3.0)):
        n = 6
        x = rng.normal(0, sigma, (n, V)).astype(np.float32)
        x[1] = 0.25                 # flat row
        x[2, V // 3] += 30.0        # one dominant token
        coins = rng.random(n)
        lse = np.array([port.row_logsumexp(x[i]) for i in range(n)])
        for i in range(n):
            while True:
                cdf = np.cumsum(np.exp(x[i].astype(np.float64) - lse[i]))
                if np.abs(cdf - coins[i]).min() > 1e-9:
                    break
                coins[i] = rng.random()
        tokens = np.array([port.sample_row(x[i], coins[i]) for i in range(n)], np.int32)
        logp = np.array([np.float32(np.float64(x[i, tokens[i]]) - lse[i]) for i in range(n)], np.float32)
        key = f"V{V}"
        blob.update({f"{key}/logits": x, f"{key}/coins": coins, f"{key}/lse": lse, f"{key}/tokens": tokens,
                     f"{key}/logp": logp})
    out = os.path.join(HERE, "sampling_cases.npz")
    np.savez_compressed(out, **blob)
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
