"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol the header
declares (and the C++ entry points of the reference's API), rejects bad arguments with the
reference's messages before touching CUDA, and has no fallback when there is no device."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

import grpo_cpp_b200 as G
from grpo_cpp_b200 import _lib, workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "grpo_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grpo_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 18
    handle = ctypes.CDLL(G.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/grpo_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"
    assert b"sm_100a" in G.lib().grpo_b200_build_info()


def test_cxx_entry_points_of_the_reference_api_are_exported():
    # mangled names a translation unit compiled against the reference's grpo_loss_cuda.cuh links to
    out = subprocess.run(["nm", "-D", "--defined-only", G.LIB_PATH], capture_output=True, text=True, check=True).stdout
    for fn in ("grpo_loss_cuda", "grpo_logits_cuda", "grpo_logits_cuda_device_inplace",
               "benchmark_grpo_loss_cuda", "benchmark_grpo_logits_cuda"):
        assert re.search(rf"_ZN4grpo\d+{fn}E", out), fn


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(HEADER).read()
    for m in re.finditer(r"/\*((?:(?!\*/).)*)\*/\s*(?:size_t|int|const char\*)\s+(grpo_b200_[a-z0-9_]+)\s*\(", text, re.S):
        comment, name = m.group(1), m.group(2)
        if name in ("grpo_b200_last_error", "grpo_b200_build_info"):
            continue
        assert re.search(r"\.(cu|cpp|hpp|cuh):\d+", comment) or "no counterpart" in comment or \
            "Name " in comment or "Frees" in comment, name


BASE = dict(B=1, G=2, T=1)


@pytest.mark.parametrize("kwargs,msg", [
    (dict(B=0), "B, G and T must be positive"),
    (dict(B=65536, G=65536), "sequence count exceeds INT_MAX"),
    (dict(B=65536, G=1, T=65536), "token count exceeds INT_MAX"),
    (dict(cfg=G.LossConfig(clip_eps=-0.1)), "clip_eps must be finite and in [0, 1)"),
    (dict(cfg=G.LossConfig(clip_eps=1.0)), "clip_eps must be finite and in [0, 1)"),
    (dict(cfg=G.LossConfig(beta=-0.1)), "beta must be finite and non-negative"),
    (dict(cfg=G.LossConfig(beta=float("inf"))), "beta must be finite and non-negative"),
    (dict(cfg=G.LossConfig(length_alpha=1.1, reduction=G.ReductionMode.length_weighted)),
     "length_alpha must be finite and in [0, 1]"),
    (dict(now=[0]), "logp_new has size 1, expected 2"),
    (dict(old=[0]), "logp_old has size 1, expected 2"),
    (dict(adv=[1]), "advantages has size 1, expected 2"),
    (dict(mask=[1]), "mask has size 1, expected 2"),
    (dict(now=[float("inf"), 0]), "log probabilities must be finite"),
    (dict(mask=[1, 2]), "mask values must be 0 or 1"),
    (dict(adv=[float("nan"), 1]), "advantages must be finite"),
    (dict(mask=[1, 0]), "every sequence needs at least one valid token"),
])
def test_host_validation_needs_no_device(kwargs, msg):
    # src/cuda/grpo_loss_cuda.cu:584-618 and :44-46 of the reference: same text, same order
    a = dict(now=[0, 0], old=[0, 0], ref=[0, 0], adv=[1, -1], mask=[1, 1], cfg=None, **BASE)
    a.update(kwargs)
    with pytest.raises(RuntimeError) as e:
        G.grpo_loss_cuda(a["now"], a["old"], a["ref"], a["adv"], a["mask"], a["B"], a["G"], a["T"], a["cfg"])
    assert str(e.value) == msg


def test_logits_validation_needs_no_device():
    b = W.logits_case(1, 2, 3, 8, seed=1)
    call = lambda **k: G.grpo_logits_cuda(k.get("x", b.logits), b.logp_old, b.logp_ref, k.get("sel", b.selected),
                                          b.advantages, b.mask, b.B, b.G, b.T, k.get("V", b.V))
    for kw, msg in ((dict(V=0), "V must be positive"),
                    (dict(x=b.logits[:-1]), "logits_new has size 40, expected 48"),
                    (dict(sel=b.selected[:-1]), "selected_tokens has size 5, expected 6"),
                    (dict(sel=np.full(6, 8)), "selected token is outside the vocabulary")):
        with pytest.raises(RuntimeError) as e:
            call(**kw)
        assert str(e.value) == msg
    # first failing row decides between a bad id and a non-finite logit
    # (src/cuda/grpo_loss_cuda.cu:688-697)
    bad = b.logits.copy()
    bad[0, 3] = np.nan
    sel = b.selected.copy()
    sel[1] = 99
    with pytest.raises(RuntimeError, match="logits must be finite"):
        call(x=bad, sel=sel)
    with pytest.raises(RuntimeError, match="P must be at least V"):
        G.grpo_logits_cuda_device_inplace(4096, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                          b.B, b.G, b.T, b.V, b.V - 1)
    with pytest.raises(RuntimeError, match="logits_and_dlogits must not be null"):
        G.grpo_logits_cuda_device_inplace(None, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                          b.B, b.G, b.T, b.V, b.V)


def test_no_cpu_fallback():
    """A valid call on a machine without a GPU must fail loudly, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(RuntimeError, match="CUDA error"):
        G.grpo_loss_cuda([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1)
    from grpo_cpp_b200 import device as D
    with pytest.raises(TypeError, match="must be a CUDA tensor"):
        D.count_lengths(torch.zeros(4, dtype=torch.int32), 2, 2)


def test_product_never_imports_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "grpo.cpp_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle_py" not in text and "grpo_oracle" not in text and "libgrpo_ref" not in text, f


def test_workload_shapes():
    b = W.tiny_reference_case()
    assert (b.B, b.G, b.T, b.V) == (3, 16, 32, 24) and b.logits.shape == (1536, 24)
    assert set(np.unique(b.mask)) <= {0, 1} and (b.selected[b.mask == 0] == -1).all()
    lengths = b.mask.reshape(b.S, b.T).sum(1)
    assert lengths.min() >= 1 and (b.mask.reshape(b.S, b.T)[:, 0] == 1).all()
    t = W.selected_token_case(64, 16, True)
    assert t.N == 1024 and t.logp_new.max() <= 0 and t.logp_new.min() >= np.log(0.01) - 1e-6
    s = W.GPT2_SHAPE
    assert s["B"] * s["G"] * s["T"] == 65536 and s["P"] % 4 == 0 and s["P"] >= s["V"]


def test_sharded_entry_point_validation_needs_no_device():
    """grpo_b200_logits_sharded, grpo_b200_row_order and the exchange-region calls reject bad
    arguments before they touch the device; fake non-null pointers are never dereferenced."""
    import ctypes as C
    from grpo_cpp_b200 import _lib
    L = _lib.lib()
    p = C.c_void_p(4096)
    regions = (C.c_void_p * 8)(*([4096] * 8))

    def sharded(world=2, rank=0, n_seq=4, next_mask=p, reduction=1, regs=regions, n_rows=8, T=2):
        return L.grpo_b200_logits_sharded(p, p, p, p, p, p, p, p, n_rows, 0, T, 16, 16, 0.2, 0.01, 1, 0, None, None,
                                          p, p, 1 << 20, regs, rank, world, n_seq, next_mask, reduction, 0.0, p, p,
                                          None, None)

    for kw, msg in ((dict(world=9), "world must lie in [1, 8]"), (dict(world=0), "world must lie in [1, 8]"),
                    (dict(rank=2), "rank must lie in [0, world)"),
                    (dict(next_mask=None), "regions, next_mask, next_weights and next_meta must not be null and "
                                           "n_seq must be positive"),
                    (dict(n_seq=0), "regions, next_mask, next_weights and next_meta must not be null and "
                                    "n_seq must be positive"),
                    (dict(reduction=3), "unknown reduction mode"),
                    (dict(n_seq=3), "rows reach beyond the last response"),
                    (dict(regs=(C.c_void_p * 8)(4096, None)), "every rank's exchange region must be mapped")):
        assert sharded(**kw) == 1, kw
        assert _lib.last_error() == msg
    assert L.grpo_b200_row_order(None, 8, p, None) == 1 and _lib.last_error() == "device pointers must not be null"
    assert L.grpo_b200_row_order(p, 0, p, None) == 1 and _lib.last_error() == "n_rows must lie in [1, INT_MAX]"
    assert L.grpo_b200_row_order_bytes(2048) == (2048 + 2 + 2) * 4
    assert L.grpo_b200_exchange_bytes(0) == 0 and L.grpo_b200_exchange_bytes(256) > 2 * 8 * 261 * 16
    assert L.grpo_b200_exchange_create(0, C.byref(C.c_void_p())) == 1
    assert L.grpo_b200_exchange_export(None, C.create_string_buffer(64)) == 1
    assert L.grpo_b200_exchange_open(None, C.byref(C.c_void_p())) == 1
    assert L.grpo_b200_exchange_close(None) == 0 and L.grpo_b200_exchange_destroy(None) == 0
