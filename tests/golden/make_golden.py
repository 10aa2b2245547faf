"""Generate the golden vectors under tests/golden/ from the reference's own CPU code.

Run in a container that has the reference tree (it is absent on the GPU box):

    make -C oracle ref && python tests/golden/make_golden.py

It loads ``oracle/_ref/libgrpo_ref.so`` -- the reference's src/cpu/grpo_loss.cpp compiled
unmodified behind oracle/ref_shim.cpp -- runs it on seeded inputs shaped like the benchmark
configurations (scaled down) and on the reference's own arithmetic fixtures
(bench/bench_grpo_loss_cuda.cu:33-102), and stores inputs and outputs as ``.npz``.
The tests compare the C restatement bit for bit, and the CUDA path within the stated
tolerance, against these files.
"""
from __future__ import annotations

import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import oracle_py  # noqa: E402
import grpo_cpp_b200  # noqa: E402,F401
from grpo_cpp_b200 import workloads as W  # noqa: E402

# (B, G, T, ragged) of the reference's selected-token parity check (bench/...:194-197) and the
# reduction each shape index is paired with there (:210), beta 0.03, alpha 0.5 (:208-211).
TOKEN_FIXTURE_SHAPES = [(1, 1, 1), (1, 1, 255), (1, 1, 256), (1, 1, 257), (1, 1, 4099), (2, 3, 257),
                        (64, 16, 1024)]
# (B, G, T, V, ragged) of the logits parity check (bench/...:252-256), beta 0.03, defaults else.
LOGITS_FIXTURE_SHAPES = [(1, 2, 3, 17, True), (2, 2, 2, 257, False), (1, 1, 2, 4099, False)]


def crc(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).tobytes())


def token_cases():
    out = {}
    for S, T, ragged in ((64, 64, False), (64, 64, True), (24, 37, True)):
        for red, alpha in ((W.SEQUENCE_MEAN, 0.0), (W.TOKEN_MEAN, 0.0), (W.LENGTH_WEIGHTED, 0.5)):
            b = W.selected_token_case(S, T, ragged, seed=42, G=8, reduction=red, length_alpha=alpha)
            out[f"cfg2_S{S}_T{T}_{'ragged' if ragged else 'full'}_red{red}"] = b
    return out


def logits_cases():
    out = {"cfg1": W.tiny_reference_case(42)}
    out["cfg3_scaled"] = W.logits_case(2, 2, 4, 2048, sigma=2.0, reduction=W.TOKEN_MEAN, seed=43)
    for alpha in (0.5, 1.0):
        out[f"cfg4_scaled_alpha{alpha}"] = W.logits_case(
            1, 4, 8, 1500, sigma=2.0, min_len=2, reduction=W.LENGTH_WEIGHTED, length_alpha=alpha, seed=44)
    out["cfg5_scaled"] = W.logits_case(2, 4, 8, 1001, sigma=3.0, min_len=1, reduction=W.TOKEN_MEAN, seed=45)
    return out


def main() -> None:
    if not oracle_py.have_reference():
        raise SystemExit("oracle/_ref/libgrpo_ref.so is missing: run `make -C oracle ref` where the "
                         "reference tree is present")
    ref = oracle_py.load("reference")

    blob = {}
    for name, b in token_cases().items():
        stats, valid, dlogp = ref.loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask,
                                       b.B, b.G, b.T, **b.cfg())
        blob.update({f"{name}/shape": np.array([b.B, b.G, b.T]),
                     f"{name}/cfg": np.array([b.clip_eps, b.beta, b.reduction, b.length_alpha], np.float64),
                     f"{name}/logp_new": b.logp_new, f"{name}/logp_old": b.logp_old,
                     f"{name}/logp_ref": b.logp_ref, f"{name}/advantages": b.advantages,
                     f"{name}/mask": b.mask.astype(np.int8),
                     f"{name}/stats": stats, f"{name}/valid": np.array(valid), f"{name}/dlogp": dlogp})
    np.savez_compressed(os.path.join(HERE, "token_cases.npz"), **blob)

    blob = {}
    for name, b in logits_cases().items():
        stats, valid, dlogits = ref.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages,
                                           b.mask, b.B, b.G, b.T, b.V, **b.cfg())
        blob.update({f"{name}/shape": np.array([b.B, b.G, b.T, b.V]),
                     f"{name}/cfg": np.array([b.clip_eps, b.beta, b.reduction, b.length_alpha], np.float64),
                     f"{name}/logits": b.logits, f"{name}/logp_old": b.logp_old,
                     f"{name}/logp_ref": b.logp_ref, f"{name}/selected": b.selected,
                     f"{name}/advantages": b.advantages, f"{name}/mask": b.mask.astype(np.int8),
                     f"{name}/stats": stats, f"{name}/valid": np.array(valid), f"{name}/dlogits": dlogits})
    np.savez_compressed(os.path.join(HERE, "logits_cases.npz"), **blob)

    # The reference's arithmetic fixtures: inputs are rebuilt from index arithmetic by the tests,
    # so only outputs are stored (a CRC instead of the 1M-token gradient).
    blob = {}
    reductions = (W.SEQUENCE_MEAN, W.TOKEN_MEAN, W.LENGTH_WEIGHTED)
    for i, (B, G, T) in enumerate(TOKEN_FIXTURE_SHAPES):
        b = W.reference_token_fixture(B, G, T, partial=(i == 5))
        stats, valid, dlogp = ref.loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, B, G, T,
                                       clip_eps=0.2, beta=0.03, reduction=reductions[i % 3], length_alpha=0.5)
        key = f"token_{B}x{G}x{T}"
        blob[f"{key}/stats"] = stats
        blob[f"{key}/valid"] = np.array(valid)
        blob[f"{key}/dlogp_crc"] = np.array(crc(dlogp), np.uint64)
        blob[f"{key}/in_crc"] = np.array([crc(b.logp_new), crc(b.logp_old), crc(b.logp_ref),
                                          crc(b.advantages), crc(b.mask)], np.uint64)
        if dlogp.size <= 8192:
            blob[f"{key}/dlogp"] = dlogp
    for (B, G, T, V, partial) in LOGITS_FIXTURE_SHAPES:
        b = W.reference_logits_fixture(B, G, T, V, partial)
        stats, valid, dlogits = ref.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages,
                                           b.mask, B, G, T, V, clip_eps=0.2, beta=0.03)
        key = f"logits_{B}x{G}x{T}x{V}"
        blob[f"{key}/stats"] = stats
        blob[f"{key}/valid"] = np.array(valid)
        blob[f"{key}/dlogits"] = dlogits
        blob[f"{key}/in_crc"] = np.array([crc(b.logits), crc(b.logp_old), crc(b.logp_ref),
                                          crc(b.selected), crc(b.advantages), crc(b.mask)], np.uint64)
    np.savez_compressed(os.path.join(HERE, "reference_fixtures.npz"), **blob)
    for f in ("token_cases.npz", "logits_cases.npz", "reference_fixtures.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
