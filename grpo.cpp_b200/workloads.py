"""Seeded synthetic inputs shaped like the five benchmark configurations.

The reference measures only on synthetic inputs (its deterministic builders in
bench/bench_grpo_loss_cuda.cu:33-102); no public dataset is involved.  These
builders produce the shapes, sizes and value distributions of the benchmark
configurations so that the CPU checker and the CUDA path can be run on
identical arrays.  They are input construction only: nothing here computes a
loss.

Layout (reference include/grpo/grpo_loss.hpp:70-76): ``S = B*G`` responses, each
padded to ``T`` token slots, ``N = S*T`` token rows; ``mask[N]`` int32 0/1;
``advantages[S]``; logits ``[N][P]`` fp32 with the first ``V`` columns valid.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

SEQUENCE_MEAN, TOKEN_MEAN, LENGTH_WEIGHTED = 0, 1, 2


@dataclass
class TokenBatch:
    """Inputs of the selected-token path (reference grpo_loss_cuda, grpo_loss_cuda.cuh:26-37)."""
    B: int
    G: int
    T: int
    logp_new: np.ndarray
    logp_old: np.ndarray
    logp_ref: np.ndarray
    advantages: np.ndarray
    mask: np.ndarray
    clip_eps: float = 0.2
    beta: float = 0.01
    reduction: int = SEQUENCE_MEAN
    length_alpha: float = 0.0
    name: str = ""

    @property
    def S(self) -> int:
        return self.B * self.G

    @property
    def N(self) -> int:
        return self.B * self.G * self.T

    def cfg(self) -> dict:
        return dict(clip_eps=self.clip_eps, beta=self.beta, reduction=self.reduction,
                    length_alpha=self.length_alpha)


@dataclass
class LogitsBatch:
    """Inputs of the logits path (reference grpo_logits_cuda, grpo_loss_cuda.cuh:53-86)."""
    B: int
    G: int
    T: int
    V: int
    logits: np.ndarray  # [N, V] dense
    logp_old: np.ndarray
    logp_ref: np.ndarray
    selected: np.ndarray
    advantages: np.ndarray
    mask: np.ndarray
    clip_eps: float = 0.2
    beta: float = 0.01
    reduction: int = SEQUENCE_MEAN
    length_alpha: float = 0.0
    name: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def S(self) -> int:
        return self.B * self.G

    @property
    def N(self) -> int:
        return self.B * self.G * self.T

    def cfg(self) -> dict:
        return dict(clip_eps=self.clip_eps, beta=self.beta, reduction=self.reduction,
                    length_alpha=self.length_alpha)

    def padded(self, P: int, fill: float = 123.0) -> np.ndarray:
        """Rows re-strided to ``P`` columns, tail pre-filled with a sentinel."""
        out = np.full((self.N, P), fill, np.float32)
        out[:, : self.V] = self.logits.reshape(self.N, self.V)
        return out


def prefix_mask(lengths: np.ndarray, T: int) -> np.ndarray:
    """mask[s, t] = t < lengths[s], flattened to N int32."""
    return (np.arange(T)[None, :] < np.asarray(lengths)[:, None]).astype(np.int32).reshape(-1)


def group_advantages_np(rewards: np.ndarray, B: int, G: int, eps: float = 1e-8) -> np.ndarray:
    """Standardised group-relative advantages for building inputs: per prompt
    ``(r - mean) / sqrt(var + eps)`` with the population variance, all-equal groups -> 0."""
    r = np.asarray(rewards, np.float64).reshape(B, G)
    mean = r.mean(axis=1, keepdims=True)
    var = ((r - mean) ** 2).mean(axis=1, keepdims=True)
    adv = (r - mean) / np.sqrt(var + eps)
    adv[(r == r[:, :1]).all(axis=1)] = 0.0
    return adv.reshape(-1).astype(np.float32)


def row_selected_logp(logits: np.ndarray, selected: np.ndarray) -> np.ndarray:
    """float64 log-softmax of the selected column of each row (input construction)."""
    x = logits.astype(np.float64)
    top = x.max(axis=1)
    lse = top + np.log(np.exp(x - top[:, None]).sum(axis=1))
    return x[np.arange(x.shape[0]), selected] - lse


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def tiny_reference_case(seed: int = 42) -> LogitsBatch:
    """Configuration 1: B=3 x G=16, T=32 ragged, V=24, sequence-mean, uniform fixed reference."""
    B, G, T, V = 3, 16, 32, 24
    rng = _rng(seed)
    S, N = B * G, B * G * T
    lengths = rng.integers(1, T + 1, S)
    mask = prefix_mask(lengths, T)
    logits = rng.standard_normal((N, V)).astype(np.float32)
    selected = rng.integers(0, V, N).astype(np.int32)
    old_logits = logits + (0.05 * rng.standard_normal((N, V))).astype(np.float32)
    logp_old = row_selected_logp(old_logits, selected).astype(np.float32)
    logp_ref = np.full(N, -np.log(float(V)), np.float32)
    rewards = (rng.random(S) < 0.5).astype(np.float32)
    adv = group_advantages_np(rewards, B, G)
    selected = np.where(mask == 1, selected, -1).astype(np.int32)
    logp_old = np.where(mask == 1, logp_old, 0.0).astype(np.float32)
    return LogitsBatch(B, G, T, V, logits, logp_old, logp_ref, selected, adv, mask,
                       0.2, 0.01, SEQUENCE_MEAN, 0.0, "cfg1-tiny", {"rewards": rewards})


def selected_token_case(S: int = 4096, T: int = 256, ragged: bool = False, seed: int = 42,
                        G: int = 8, reduction: int = SEQUENCE_MEAN, length_alpha: float = 0.0
                        ) -> TokenBatch:
    """Configuration 2: per-token logp given; logp ~ ln U(0.01,1), old = logp + N(0,0.02),
    ref = logp + N(0,0.05), advantages ~ N(0,1) per response."""
    assert S % G == 0
    B, N = S // G, S * T
    rng = _rng(seed)
    logp = np.log(rng.uniform(0.01, 1.0, N)).astype(np.float32)
    old = (logp + 0.02 * rng.standard_normal(N)).astype(np.float32)
    ref = (logp + 0.05 * rng.standard_normal(N)).astype(np.float32)
    adv = rng.standard_normal(S).astype(np.float32)
    lengths = rng.integers(1, T + 1, S) if ragged else np.full(S, T)
    mask = prefix_mask(lengths, T)
    return TokenBatch(B, G, T, logp, old, ref, adv, mask, 0.2, 0.01, reduction, length_alpha,
                      f"cfg2-S{S}-T{T}-{'ragged' if ragged else 'full'}")


def logits_case(B: int, G: int, T: int, V: int, *, sigma: float = 2.0, min_len: int | None = None,
                reduction: int = TOKEN_MEAN, length_alpha: float = 0.0, seed: int = 42,
                name: str = "") -> LogitsBatch:
    """Configurations 3-5 at any size: logits ~ N(0, sigma), selected ids uniform, old/ref =
    true selected logp + N(0,0.05), advantages from Bernoulli(0.5) rewards; ``min_len`` set ->
    ragged prefix mask with lengths uniform in [min_len, T], else full mask."""
    rng = _rng(seed)
    S, N = B * G, B * G * T
    logits = (sigma * rng.standard_normal((N, V), dtype=np.float32)).astype(np.float32)
    selected = rng.integers(0, V, N).astype(np.int32)
    now = row_selected_logp(logits, selected)
    old = (now + 0.05 * rng.standard_normal(N)).astype(np.float32)
    ref = (now + 0.05 * rng.standard_normal(N)).astype(np.float32)
    rewards = (rng.random(S) < 0.5).astype(np.float32)
    adv = group_advantages_np(rewards, B, G)
    lengths = rng.integers(min_len, T + 1, S) if min_len is not None else np.full(S, T)
    mask = prefix_mask(lengths, T)
    selected = np.where(mask == 1, selected, -1).astype(np.int32)
    old = np.where(mask == 1, old, 0.0).astype(np.float32)
    ref = np.where(mask == 1, ref, 0.0).astype(np.float32)
    return LogitsBatch(B, G, T, V, logits, old, ref, selected, adv, mask, 0.2, 0.01,
                       reduction, length_alpha, name or f"logits-N{N}-V{V}", {"rewards": rewards})


def fused_v32k_case(seed: int = 42, rows_per_response: int = 64) -> LogitsBatch:
    """Configuration 3: N=1024 x V=32768, full mask, token-mean."""
    return logits_case(2, 8, rows_per_response, 32768, sigma=2.0, reduction=TOKEN_MEAN,
                       seed=seed, name="cfg3-V32768")


def fused_v128k_case(alpha: float, seed: int = 42, rows_per_response: int = 64) -> LogitsBatch:
    """Configuration 4: 16 responses x 64 slots, V=131072, lengths U[16,64], L^alpha weighting."""
    return logits_case(2, 8, rows_per_response, 131072, sigma=2.0, min_len=16,
                       reduction=LENGTH_WEIGHTED, length_alpha=alpha, seed=seed,
                       name=f"cfg4-V131072-alpha{alpha}")


# Configuration 5 (GPT-2-shaped, sharded by token): N = 32*8*256 rows, V=50257 padded to
# P=50304, logits ~ N(0,3), lengths U[32,256], token-mean.  12.3 GiB of logits: built on the
# device by the benchmark and the GPU tests; only the shape constants live here.
GPT2_SHAPE = dict(B=32, G=8, T=256, V=50257, P=50304, sigma=3.0, min_len=32)


# The reference's own deterministic fixtures (bench/bench_grpo_loss_cuda.cu:33-102), restated:
# pure index arithmetic in fp32, so any implementation can rebuild them bit for bit.
def reference_token_fixture(B: int, G: int, T: int, partial: bool) -> TokenBatch:
    f = np.float32
    S, N = B * G, B * G * T
    seq = np.arange(S)
    adv = (np.where(seq % 2 == 0, f(0.4), f(-0.7)) + f(0.03) * (seq % 5).astype(f)).astype(f)
    if partial:
        lengths = np.maximum(1, T // 2 + (seq * 37) % max(1, T // 5 + 1))
    else:
        lengths = np.full(S, T)
    i = np.arange(N)
    old = (f(-2.0) - f(0.000001) * i.astype(f)).astype(f)
    shift = (f(-0.4) + f(0.8) * (i % 17).astype(f) / f(16.0)).astype(f)
    now = (old + shift).astype(f)
    ref = (old + f(0.03) * ((i % 5) - 2).astype(f)).astype(f)
    return TokenBatch(B, G, T, now, old, ref, adv, prefix_mask(lengths, T),
                      name=f"ref-fixture-{B}x{G}x{T}{'-ragged' if partial else ''}")


def reference_logits_fixture(B: int, G: int, T: int, V: int, partial: bool) -> LogitsBatch:
    f = np.float32
    S, N = B * G, B * G * T
    v = np.arange(V)
    base = (f(-0.001) * (v % 257).astype(f)).astype(f)
    base_lse = np.log(np.exp(base.astype(np.float64)).sum())
    seq = np.arange(S)
    adv = (np.where(seq % 2 == 0, f(0.6), f(-0.4)) + f(0.02) * (seq % 3).astype(f)).astype(f)
    lengths = 1 + (seq * 5) % T if partial else np.full(S, T)
    mask = prefix_mask(lengths, T)
    row = np.arange(N)
    active = mask == 1
    selected = np.where(active, (row * 37 + 11) % V, -1).astype(np.int32)
    row_shift = (f(0.01) * (row % 7).astype(f)).astype(f)
    logits = (base[None, :] + row_shift[:, None]).astype(f)
    now = (base[np.maximum(selected, 0)].astype(np.float64) - base_lse).astype(f)
    ratio_shift = (f(-0.25) + f(0.1) * (row % 6).astype(f)).astype(f)
    old = np.where(active, (now - ratio_shift).astype(f), f(0)).astype(f)
    ref = np.where(active, (now + f(0.01) * ((row % 5) - 2).astype(f)).astype(f), f(0)).astype(f)
    return LogitsBatch(B, G, T, V, logits, old, ref, selected, adv, mask, 0.2, 0.0,
                       SEQUENCE_MEAN, 0.0, f"ref-logits-fixture-{B}x{G}x{T}x{V}")


# Counter-based synthetic logits, host restatement of the library's grpo_b200_synthetic_logits kernel
# (csrc/synthetic.cu): element (r, v) of a batch with row stride P depends on (seed, r, v) only, so a
# host can rebuild any row of a batch that exists only on the devices, whatever the sharding.
_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def synthetic_scale(sigma: float) -> np.float32:
    """The fp32 factor that gives the sum of eight 16-bit uniforms standard deviation ``sigma``."""
    return np.float32(sigma / np.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0))


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _fields16(h: np.ndarray) -> np.ndarray:
    m = np.uint64(0xFFFF)
    return ((h & m) + ((h >> np.uint64(16)) & m) + ((h >> np.uint64(32)) & m) + (h >> np.uint64(48))).astype(np.int64)


def synthetic_logits_rows(rows, V: int, P: int, scale, seed: int) -> np.ndarray:
    """``[len(rows), V]`` fp32: the vocabulary columns of the given GLOBAL rows."""
    rows = np.asarray(rows, np.uint64).reshape(-1, 1)
    with np.errstate(over="ignore"):
        c = rows * np.uint64(P) + np.arange(V, dtype=np.uint64)[None, :]
        s = np.uint64(seed) + (np.uint64(2) * c + np.uint64(1)) * _GAMMA
        k = _fields16(_mix64(s)) + _fields16(_mix64(s + _GAMMA)) - 262140
    return k.astype(np.float32) * np.float32(scale)
