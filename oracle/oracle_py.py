"""ctypes bindings of the CPU checkers -- TEST INFRASTRUCTURE ONLY.

Two libraries with the same call shapes:

* ``port``      ``oracle/libgrpo_oracle.so``   the C restatement in ``grpo_oracle.c``
* ``reference`` ``oracle/_ref/libgrpo_ref.so`` the reference's own
  ``src/cpu/grpo_loss.cpp`` compiled behind ``ref_shim.cpp`` (present only when
  it was built in a container that has the reference tree)

Only the tests, the smoke check and the benchmark's CPU-baseline legs may import
this module; the product package never does.  Errors surface as ``RuntimeError``
carrying the reference's exception text, so tests can compare error behaviour
of the two libraries and of the CUDA path word for word.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "libgrpo_oracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libgrpo_ref.so")

SEQUENCE_MEAN, TOKEN_MEAN, LENGTH_WEIGHTED = 0, 1, 2
STANDARDIZED, CENTERED = 0, 1

_f = np.float32
_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def build(force: bool = False) -> None:
    """Compile the C restatement (and the reference library when its tree exists)."""
    if force or not os.path.exists(PORT_PATH):
        subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    subprocess.run(["make", "-s", "-C", _HERE, "ref"], check=True)


def _as(a, dtype):
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


def _dims_ok(*dims) -> bool:
    """True when the reference's shape check (include/grpo/grpo_loss.hpp:51-67) would pass, i.e.
    when array sizes are the next thing it looks at."""
    prod = 1
    for d in dims:
        if d <= 0:
            return False
        prod *= d
    return prod <= 2**31 - 1


def _p(a, ptr_t):
    return a.ctypes.data_as(ptr_t)


class _Lib:
    """One checker library; ``kind`` is ``"port"`` or ``"reference"``."""

    def __init__(self, kind: str):
        self.kind = kind
        prefix = "grpo_oracle_" if kind == "port" else "grpo_ref_"
        path = PORT_PATH if kind == "port" else REF_PATH
        if kind == "port" and not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        self.adv_fn = getattr(self.lib, prefix + "group_advantages")
        self.adv_fn.argtypes = [_fp, C.c_int, C.c_int, C.c_int, C.c_float, _fp]
        self.loss_fn = getattr(self.lib, prefix + "loss")
        self.loss_fn.argtypes = [_fp, _fp, _fp, _fp, _ip, C.c_int, C.c_int, C.c_int,
                                 C.c_float, C.c_float, C.c_int, C.c_float, _fp, _fp, _ip]
        self.logits_fn = getattr(self.lib, prefix + "logits")
        base = [_fp, _fp, _fp, _ip, _fp, _ip, C.c_int, C.c_int, C.c_int, C.c_int,
                C.c_float, C.c_float, C.c_int, C.c_float, _fp, _fp, _ip]
        self.logits_fn.argtypes = base + ([_fp] if kind == "port" else [])
        if kind == "port":
            self.lib.grpo_oracle_strerror.restype = C.c_char_p
            self.lib.grpo_oracle_strerror.argtypes = [C.c_int]
            self.lib.grpo_oracle_logits_rows.argtypes = [_fp, C.c_int, C.c_int, _fp, _fp, _ip, _fp, _fp, C.c_float,
                                                         C.c_float, _fp, _fp, _fp]
            self.lib.grpo_oracle_row_logsumexp.restype = C.c_double
            self.lib.grpo_oracle_row_logsumexp.argtypes = [_fp, C.c_int]
            self.lib.grpo_oracle_sample_row.restype = C.c_int
            self.lib.grpo_oracle_sample_row.argtypes = [_fp, C.c_int, C.c_double]
        else:
            self.lib.grpo_ref_last_error.restype = C.c_char_p

    def _check(self, rc: int) -> None:
        if rc == 0:
            return
        if self.kind == "port":
            raise RuntimeError(self.lib.grpo_oracle_strerror(rc).decode())
        raise RuntimeError(self.lib.grpo_ref_last_error().decode())

    def row_logsumexp(self, row) -> float:
        """apps/04_gpt2_grpo.cu:61-66 (port only; unpinned)."""
        r = _as(row, _f)
        return float(self.lib.grpo_oracle_row_logsumexp(r.ctypes.data_as(_fp), r.size))

    def sample_row(self, row, coin: float) -> int:
        """apps/04_gpt2_grpo.cu:68-80 with the uniform number given (port only; unpinned)."""
        r = _as(row, _f)
        return int(self.lib.grpo_oracle_sample_row(r.ctypes.data_as(_fp), r.size, float(coin)))

    def logits_rows(self, rows, logp_old, logp_ref, selected, adv, w, clip_eps=0.2, beta=0.0):
        """Rows out of a larger batch with their advantages and weights given (port only).
        Returns ``(dlogits[n,V], selected_logp[n], terms[n,3])``."""
        x = _as(rows, _f)
        n, V = x.shape
        b, c, sel = _as(logp_old, _f), _as(logp_ref, _f), _as(selected, np.int32)
        a, ww = _as(adv, _f), _as(w, _f)
        assert b.size == c.size == sel.size == a.size == ww.size == n
        out, lp, terms = np.zeros((n, V), _f), np.zeros(n, _f), np.zeros((n, 3), _f)
        self._check(self.lib.grpo_oracle_logits_rows(_p(x, _fp), n, V, _p(b, _fp), _p(c, _fp), _p(sel, _ip),
                                                     _p(a, _fp), _p(ww, _fp), clip_eps, beta, _p(out, _fp),
                                                     _p(lp, _fp), _p(terms, _fp)))
        return out, lp, terms

    def group_advantages(self, rewards, B, G, mode=STANDARDIZED, eps=1e-8):
        r = _as(rewards, _f)
        n = B * G if _dims_ok(B, G) else 0
        if n and r.size != n:
            raise RuntimeError(f"rewards has size {r.size}, expected {n}")
        out = np.zeros(max(n, 1), _f)
        self._check(self.adv_fn(_p(r, _fp), B, G, mode, eps, _p(out, _fp)))
        return out[:n]

    def loss(self, logp_new, logp_old, logp_ref, advantages, mask, B, G, T,
             clip_eps=0.2, beta=0.0, reduction=SEQUENCE_MEAN, length_alpha=0.0):
        """Returns ``(stats[3] float32, valid_tokens, dlogp[N])``."""
        a, b, c = _as(logp_new, _f), _as(logp_old, _f), _as(logp_ref, _f)
        adv, m = _as(advantages, _f), _as(mask, np.int32)
        if _dims_ok(B, G, T):
            n, s = B * G * T, B * G
            for name, arr, want in (("logp_new", a, n), ("logp_old", b, n), ("logp_ref", c, n),
                                    ("advantages", adv, s), ("mask", m, n)):
                if arr.size != want:
                    raise RuntimeError(f"{name} has size {arr.size}, expected {want}")
        else:
            n = 1
        dlogp = np.zeros(n, _f)
        stats = np.zeros(3, _f)
        valid = C.c_int(0)
        self._check(self.loss_fn(_p(a, _fp), _p(b, _fp), _p(c, _fp), _p(adv, _fp), _p(m, _ip),
                                 B, G, T, clip_eps, beta, reduction, length_alpha,
                                 _p(dlogp, _fp), _p(stats, _fp), C.byref(valid)))
        return stats, valid.value, dlogp

    def logits(self, logits, logp_old, logp_ref, selected, advantages, mask, B, G, T, V,
               clip_eps=0.2, beta=0.0, reduction=SEQUENCE_MEAN, length_alpha=0.0,
               want_selected_logp=False):
        """Returns ``(stats[3], valid_tokens, dlogits[N,V])`` (+ selected_logp[N] for the port)."""
        x = _as(logits, _f)
        b, c = _as(logp_old, _f), _as(logp_ref, _f)
        sel, adv, m = _as(selected, np.int32), _as(advantages, _f), _as(mask, np.int32)
        if _dims_ok(B, G, T) and V > 0:
            n, s = B * G * T, B * G
            for name, arr, want in (("logits_new", x, n * V), ("selected_tokens", sel, n),
                                    ("mask", m, n), ("logp_old", b, n), ("logp_ref", c, n),
                                    ("advantages", adv, s)):
                if arr.size != want:
                    raise RuntimeError(f"{name} has size {arr.size}, expected {want}")
        else:
            n, V = 1, max(V, 1)
        out = np.zeros((n, V), _f)
        stats = np.zeros(3, _f)
        valid = C.c_int(0)
        args = [_p(x, _fp), _p(b, _fp), _p(c, _fp), _p(sel, _ip), _p(adv, _fp), _p(m, _ip),
                B, G, T, V, clip_eps, beta, reduction, length_alpha,
                _p(out, _fp), _p(stats, _fp), C.byref(valid)]
        sel_logp = None
        if self.kind == "port":
            sel_logp = np.zeros(n, _f)
            args.append(_p(sel_logp, _fp))
        self._check(self.logits_fn(*args))
        if want_selected_logp:
            return stats, valid.value, out, sel_logp
        return stats, valid.value, out


_cache: dict[str, _Lib] = {}


def have_reference() -> bool:
    return os.path.exists(REF_PATH)


def load(kind: str = "port") -> _Lib:
    """``kind``: ``"port"``, ``"reference"``, or ``"best"`` (reference when built, else port)."""
    if kind == "best":
        kind = "reference" if have_reference() else "port"
    if kind not in _cache:
        _cache[kind] = _Lib(kind)
    return _cache[kind]
