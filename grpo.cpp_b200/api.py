"""Reference-facing calls under the reference's names, on numpy arrays.

Mirrors include/grpo/grpo_loss_cuda.cuh:26-102 and the types of include/grpo/grpo_loss.hpp:10-43 of
the reference: same argument order and meaning, same defaults, and ``RuntimeError`` with the same
message wherever the reference throws ``std::runtime_error``.  Each function is one call into the
host layer of the C ABI; the arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from enum import IntEnum

import numpy as np

from . import _lib


class AdvantageMode(IntEnum):
    standardized = 0
    centered = 1


class ReductionMode(IntEnum):
    sequence_mean = 0
    token_mean = 1
    length_weighted = 2


class CudaLossKernel(IntEnum):
    atomic = 0
    block_reduce = 1


class CudaLogitsKernel(IntEnum):
    separate = 0
    fused = 1


@dataclass
class LossConfig:
    clip_eps: float = 0.2
    beta: float = 0.0
    reduction: ReductionMode = ReductionMode.sequence_mean
    length_alpha: float = 0.0


@dataclass
class LossStats:
    loss: float = 0.0
    pg_loss: float = 0.0
    kl: float = 0.0
    valid_tokens: int = 0


@dataclass
class LossResult:
    stats: LossStats = field(default_factory=LossStats)
    dlogp_new: np.ndarray = None


@dataclass
class LogitsLossResult:
    stats: LossStats = field(default_factory=LossStats)
    dlogits: np.ndarray = None


@dataclass
class CudaTiming:
    atomic_ms: float = 0.0
    block_ms: float = 0.0


@dataclass
class CudaLogitsTiming:
    separate_ms: float = 0.0
    fused_ms: float = 0.0


_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int32)


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32).reshape(-1))


def _i32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32).reshape(-1))


def _pf(a):
    return a.ctypes.data_as(_fp), a.size


def _pi(a):
    return a.ctypes.data_as(_ip), a.size


def _prod_ok(*dims):
    p = 1
    for d in dims:
        if d <= 0:
            return 0
        p *= d
    return p if p <= 2**31 - 1 else 0


def _stats(raw, valid):
    return LossStats(float(raw[0]), float(raw[1]), float(raw[2]), int(valid.value))


def grpo_loss_cuda(logp_new, logp_old, logp_ref, advantages, mask, B, G, T,
                   config: LossConfig | None = None,
                   kernel: CudaLossKernel = CudaLossKernel.block_reduce) -> LossResult:
    cfg = config or LossConfig()
    a, b, c, adv, m = _f32(logp_new), _f32(logp_old), _f32(logp_ref), _f32(advantages), _i32(mask)
    dlogp = np.zeros(max(_prod_ok(B, G, T), 1), np.float32)
    raw = np.zeros(3, np.float32)
    valid = C.c_int(0)
    _lib.check(_lib.lib().grpo_b200_loss_host(
        *_pf(a), *_pf(b), *_pf(c), *_pf(adv), *_pi(m), B, G, T, cfg.clip_eps, cfg.beta, int(cfg.reduction),
        cfg.length_alpha, int(kernel), dlogp.ctypes.data_as(_fp), raw.ctypes.data_as(_fp), C.byref(valid)))
    return LossResult(_stats(raw, valid), dlogp)


def benchmark_grpo_loss_cuda(logp_new, logp_old, logp_ref, advantages, mask, B, G, T,
                             config: LossConfig | None = None, warmup: int = 10,
                             iterations: int = 100) -> CudaTiming:
    cfg = config or LossConfig()
    a, b, c, adv, m = _f32(logp_new), _f32(logp_old), _f32(logp_ref), _f32(advantages), _i32(mask)
    t0, t1 = C.c_float(0), C.c_float(0)
    _lib.check(_lib.lib().grpo_b200_benchmark_loss_host(
        *_pf(a), *_pf(b), *_pf(c), *_pf(adv), *_pi(m), B, G, T, cfg.clip_eps, cfg.beta, int(cfg.reduction),
        cfg.length_alpha, warmup, iterations, C.byref(t0), C.byref(t1)))
    return CudaTiming(t0.value, t1.value)


def grpo_logits_cuda(logits_new, logp_old, logp_ref, selected_tokens, advantages, mask, B, G, T, V,
                     config: LossConfig | None = None,
                     kernel: CudaLogitsKernel = CudaLogitsKernel.fused) -> LogitsLossResult:
    cfg = config or LossConfig()
    x, b, c = _f32(logits_new), _f32(logp_old), _f32(logp_ref)
    sel, adv, m = _i32(selected_tokens), _f32(advantages), _i32(mask)
    n = _prod_ok(B, G, T)
    out = np.empty((max(n, 1), max(V, 1)), np.float32)
    raw = np.zeros(3, np.float32)
    valid = C.c_int(0)
    _lib.check(_lib.lib().grpo_b200_logits_host(
        *_pf(x), *_pf(b), *_pf(c), *_pi(sel), *_pf(adv), *_pi(m), B, G, T, V, cfg.clip_eps, cfg.beta,
        int(cfg.reduction), cfg.length_alpha, int(kernel), out.ctypes.data_as(_fp), raw.ctypes.data_as(_fp),
        C.byref(valid)))
    return LogitsLossResult(_stats(raw, valid), out)


def _device_pointer(obj) -> int:
    """Address of caller-owned device memory: an int, or anything with ``data_ptr()``."""
    if obj is None:
        return 0
    if hasattr(obj, "data_ptr"):
        return int(obj.data_ptr())
    return int(obj)


def grpo_logits_cuda_device_inplace(logits_and_dlogits, logp_old, logp_ref, selected_tokens, advantages, mask,
                                    B, G, T, V, P, config: LossConfig | None = None,
                                    kernel: CudaLogitsKernel = CudaLogitsKernel.fused) -> LossStats:
    """``logits_and_dlogits``: device memory of ``B*G*T`` rows of ``P`` floats on the current device
    (a raw address or an object with ``data_ptr()``), replaced in place by dL/dlogits."""
    cfg = config or LossConfig()
    b, c = _f32(logp_old), _f32(logp_ref)
    sel, adv, m = _i32(selected_tokens), _f32(advantages), _i32(mask)
    raw = np.zeros(3, np.float32)
    valid = C.c_int(0)
    _lib.check(_lib.lib().grpo_b200_logits_device_inplace_host(
        _device_pointer(logits_and_dlogits) or None, *_pf(b), *_pf(c), *_pi(sel), *_pf(adv), *_pi(m), B, G, T,
        V, P, cfg.clip_eps, cfg.beta, int(cfg.reduction), cfg.length_alpha, int(kernel),
        raw.ctypes.data_as(_fp), C.byref(valid)))
    return _stats(raw, valid)


def benchmark_grpo_logits_cuda(logits_new, logp_old, logp_ref, selected_tokens, advantages, mask, B, G, T, V,
                               config: LossConfig | None = None, warmup: int = 10,
                               iterations: int = 100) -> CudaLogitsTiming:
    cfg = config or LossConfig()
    x, b, c = _f32(logits_new), _f32(logp_old), _f32(logp_ref)
    sel, adv, m = _i32(selected_tokens), _f32(advantages), _i32(mask)
    t0, t1 = C.c_float(0), C.c_float(0)
    _lib.check(_lib.lib().grpo_b200_benchmark_logits_host(
        *_pf(x), *_pf(b), *_pf(c), *_pi(sel), *_pf(adv), *_pi(m), B, G, T, V, cfg.clip_eps, cfg.beta,
        int(cfg.reduction), cfg.length_alpha, warmup, iterations, C.byref(t0), C.byref(t1)))
    return CudaLogitsTiming(t0.value, t1.value)


class ShardedLogits:
    """One rank of a token-sharded batch: the host-facing call of ``grpo_b200_logits_sharded_host`` with
    numpy metadata, the Python twin of ``grpo::ShardedLogitsBoundary``
    (include/grpo/grpo_loss_sharded.hpp).  Argument meaning and errors follow
    ``grpo_logits_cuda_device_inplace`` (include/grpo/grpo_loss_cuda.cuh:68-86 of the reference) for
    this rank's rows ``[row_offset, row_offset + n_rows)``; the statistics returned are the whole
    batch's.  Create with the rank's device current."""

    def __init__(self, rank: int, world: int, B: int, G: int, T: int, V: int, P: int, row_offset: int, n_rows: int):
        self.world = world
        self._shard = C.c_void_p()
        _lib.check(_lib.lib().grpo_b200_shard_create(rank, world, B * G, T, V, P, row_offset, n_rows,
                                                    C.byref(self._shard)))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        _lib.check(_lib.lib().grpo_b200_shard_export(self._shard, buf))
        return buf.raw

    def connect_ipc(self, handles) -> None:
        """``handles``: every rank's 64 bytes, in rank order (processes, one per device)."""
        if len(handles) != self.world:
            raise ValueError("one handle per rank, in rank order")
        flat = C.create_string_buffer(b"".join(bytes(h) for h in handles), 64 * self.world)
        _lib.check(_lib.lib().grpo_b200_shard_connect_ipc(self._shard, flat))

    def connect_local(self, all_shards) -> None:
        """``all_shards``: every rank's object, in rank order (threads of one process)."""
        arr = (C.c_void_p * self.world)(*[s._shard.value for s in all_shards])
        _lib.check(_lib.lib().grpo_b200_shard_connect_local(self._shard, arr))

    def run(self, logits_and_dlogits, logp_old, logp_ref, selected_tokens, advantages, mask,
            config: LossConfig | None = None, kernel: CudaLogitsKernel = CudaLogitsKernel.fused) -> LossStats:
        cfg = config or LossConfig()
        b, c = _f32(logp_old), _f32(logp_ref)
        sel, adv, m = _i32(selected_tokens), _f32(advantages), _i32(mask)
        raw = np.zeros(3, np.float32)
        valid = C.c_int(0)
        _lib.check(_lib.lib().grpo_b200_logits_sharded_host(
            self._shard, _device_pointer(logits_and_dlogits) or None, *_pf(b), *_pf(c), *_pi(sel), *_pf(adv), *_pi(m),
            cfg.clip_eps, cfg.beta, int(cfg.reduction), cfg.length_alpha, int(kernel), raw.ctypes.data_as(_fp),
            C.byref(valid)))
        return _stats(raw, valid)

    def close(self) -> None:
        if self._shard:
            _lib.lib().grpo_b200_shard_destroy(self._shard)
            self._shard = C.c_void_p()
