"""Parity of the fused logits CUDA path (K2) with the CPU oracle -- runs on the B200.

Every call goes through the C ABI of libgrpo_b200.so.  Tolerances stated for this path: loss
terms within 1e-5 relative; dL/dlogits within 1e-7 + 1e-5 * |want|; valid-token counts exact;
padded tail columns and masked rows exactly zero.
"""
import os
import re
import subprocess

import numpy as np
import pytest

import oracle_py
import grpo_cpp_b200 as G
from grpo_cpp_b200 import workloads as W
from test_gpu_token_path import assert_grad, assert_stats, cfg_of

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle():
    return oracle_py.load("best")


def run_oracle(b):
    return oracle().logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                           b.B, b.G, b.T, b.V, **b.cfg())


def check_all_entry_points(b, want, name, pad_to=None):
    """Host-vector call (both selectors), in-place call with P = V, and in-place with a padded,
    sentinel-filled tail -- the four ways the reference's own GPU check drives this path
    (bench/bench_grpo_loss_cuda.cu:251-346)."""
    import torch
    stats_w, valid_w, d_w = want
    for kernel in (G.CudaLogitsKernel.fused, G.CudaLogitsKernel.separate):
        r = G.grpo_logits_cuda(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                               b.B, b.G, b.T, b.V, cfg_of(b), kernel)
        assert_stats(r.stats, stats_w, valid_w, f"{name}/{kernel.name}")
        assert_grad(r.dlogits, d_w, f"{name}/{kernel.name}")
        assert np.abs(r.dlogits.sum(axis=1)).max() <= 3e-5
        assert (r.dlogits.reshape(b.N, b.V)[b.mask == 0] == 0).all()
    pads = [b.V] + ([pad_to] if pad_to else [])
    for P in pads:
        for kernel in (G.CudaLogitsKernel.fused, G.CudaLogitsKernel.separate):
            dev = torch.from_numpy(b.padded(P)).cuda()
            st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                   b.B, b.G, b.T, b.V, P, cfg_of(b), kernel)
            out = dev.cpu().numpy()
            assert_stats(st, stats_w, valid_w, f"{name}/inplace P={P}/{kernel.name}")
            assert_grad(out[:, : b.V], d_w, f"{name}/inplace P={P}/{kernel.name}")
            assert (out[:, b.V:] == 0).all(), "padded tail must come back as zeros"
            assert (out[b.mask == 0] == 0).all(), "masked rows must come back as zeros"


def test_golden_logits_cases(golden_logits):
    for name in golden_logits.cases:
        c = golden_logits.case(name)
        B, Gn, T, V = (int(x) for x in c["shape"])
        eps, beta, red, alpha = c["cfg"]
        b = W.LogitsBatch(B, Gn, T, V, c["logits"].reshape(-1, V), c["logp_old"], c["logp_ref"], c["selected"],
                          c["advantages"], c["mask"].astype(np.int32), float(eps), float(beta), int(red), float(alpha))
        want = (c["stats"], int(c["valid"]), c["dlogits"].reshape(-1, V))
        check_all_entry_points(b, want, name, pad_to=((V + 31) // 32) * 32 + 32)


def test_reference_logits_check_cases(golden_fixtures):
    # (1,2,3,17,ragged) (2,2,2,257) (1,1,2,4099) with beta 0.03, then V=17 padded to P=32
    from make_golden import LOGITS_FIXTURE_SHAPES
    for (B, Gn, T, V, partial) in LOGITS_FIXTURE_SHAPES:
        b = W.reference_logits_fixture(B, Gn, T, V, partial)
        b.beta = 0.03
        c = golden_fixtures.case(f"logits_{B}x{Gn}x{T}x{V}")
        want = (c["stats"], int(c["valid"]), c["dlogits"].reshape(-1, V))
        check_all_entry_points(b, want, b.name, pad_to=32 if V == 17 else None)


def test_zero_advantage_logits():
    # bench/bench_grpo_loss_cuda.cu:348-361: A = 0 with old = ref = -101 must not overflow
    b = W.reference_logits_fixture(1, 1, 1, 3, False)
    b.advantages[:] = 0.0
    b.logp_old[:] = -101.0
    b.logp_ref[:] = -101.0
    want = run_oracle(b)
    r = G.grpo_logits_cuda(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, 1, 1, 1, 3)
    assert_stats(r.stats, want[0], want[1])
    assert_grad(r.dlogits, want[2])


def test_masked_rows_are_never_read():
    import torch
    b = W.logits_case(2, 3, 6, 1024, min_len=1, reduction=W.SEQUENCE_MEAN, seed=11)
    want = run_oracle(b)
    poisoned = b.logits.copy()
    poisoned[b.mask == 0] = np.nan
    for kernel in (G.CudaLogitsKernel.fused, G.CudaLogitsKernel.separate):
        dev = torch.from_numpy(poisoned).cuda()
        st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                               b.B, b.G, b.T, b.V, b.V, cfg_of(b), kernel)
        out = dev.cpu().numpy()
        assert_stats(st, want[0], want[1])
        assert (out[b.mask == 0] == 0).all()
        assert_grad(out, want[2])


@pytest.mark.parametrize("V,P,offset_floats", [
    (1021, 1024, 0),     # rows on 32-byte boundaries: masked rows are filled with 256-bit stores
    (1021, 1024, 4),     # the same rows starting 16 bytes off a 32-byte boundary: 128-bit stores
    (1017, 1020, 0),     # a row pitch that is a multiple of 16 bytes only
    (50257, 50304, 0),   # the benchmark's shape: cluster of eight, slices of an even number of chunks
    (50257, 50308, 0),   # slices of an odd number of chunks
    (40000, 40024, 4),
])
def test_masked_row_fill_alignments(V, P, offset_floats):
    """Masked rows come back as exact zeros over all P columns, and nothing is written outside the
    batch's rows, for every alignment of the row base and pitch (the zero fill picks its store width
    by them).  The rows around the batch are sentinels."""
    import torch
    b = W.logits_case(2, 2, 5, V, min_len=1, reduction=W.TOKEN_MEAN, seed=V + P + offset_floats)
    want = run_oracle(b)
    guard = 64
    flat = torch.full((offset_floats + guard + b.N * P + guard,), 7.25, dtype=torch.float32, device="cuda")
    rows = flat[offset_floats + guard: offset_floats + guard + b.N * P].view(b.N, P)
    padded = b.padded(P)
    padded[b.mask == 0] = np.nan
    rows.copy_(torch.from_numpy(padded))
    st = G.grpo_logits_cuda_device_inplace(rows, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                           b.B, b.G, b.T, V, P, cfg_of(b))
    out = rows.cpu().numpy()
    assert_stats(st, want[0], want[1])
    assert_grad(out[:, :V], want[2])
    assert (out[b.mask == 0] == 0).all() and (out[:, V:] == 0).all()
    edge = flat.cpu().numpy()
    assert (edge[: offset_floats + guard] == 7.25).all() and (edge[offset_floats + guard + b.N * P:] == 7.25).all()


@pytest.mark.parametrize("call,msg", [
    (lambda b: G.grpo_logits_cuda(b.logits, b.logp_old, b.logp_ref, np.where(b.mask == 1, b.V, -1), b.advantages,
                                  b.mask, b.B, b.G, b.T, b.V), "selected token is outside the vocabulary"),
    (lambda b: G.grpo_logits_cuda(np.where(np.arange(b.logits.size).reshape(b.logits.shape) == 5, np.inf, b.logits),
                                  b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T, b.V),
     "logits must be finite"),
    (lambda b: G.grpo_logits_cuda(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G,
                                  b.T, 0), "V must be positive"),
    (lambda b: G.grpo_logits_cuda(b.logits[:-1], b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B,
                                  b.G, b.T, b.V), None),
    (lambda b: G.grpo_logits_cuda_device_inplace(None, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                 b.B, b.G, b.T, b.V, b.V), "logits_and_dlogits must not be null"),
    (lambda b: G.grpo_logits_cuda_device_inplace(1 << 20, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                 b.B, b.G, b.T, b.V, b.V - 1), "P must be at least V"),
])
def test_logits_error_contract(call, msg):
    b = W.logits_case(1, 2, 3, 40, seed=3)
    with pytest.raises(RuntimeError) as e:
        call(b)
    if msg is None:
        assert "logits_new has size" in str(e.value)
    else:
        assert str(e.value) == msg


def test_every_resident_variant_matches_oracle():
    """Each compiled cluster/thread/vector shape of the row-resident kernel, forced in turn, on a
    ragged V it can hold (V not a multiple of 4, P padded), against the oracle."""
    import torch
    from grpo_cpp_b200 import device as D
    names = D.variants()
    try:
        for idx, name in enumerate(names):
            c, t, v = (int(x) for x in re.match(r"(\d+)x(\d+)x(\d+)", name).groups())
            cap = c * t * v * 4
            V = cap - 37 if cap > 2048 else cap - 5
            P = cap
            b = W.logits_case(1, 3, 4, V, sigma=2.5, min_len=2, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5,
                              seed=100 + idx)
            want = run_oracle(b)
            D.set_variant(idx)
            dev = torch.from_numpy(b.padded(P)).cuda()
            assert D.plan(dev, V) == name
            st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                   b.B, b.G, b.T, V, P, cfg_of(b))
            out = dev.cpu().numpy()
            assert_stats(st, want[0], want[1], name)
            assert_grad(out[:, :V], want[2], name)
            assert (out[:, V:] == 0).all() and (out[b.mask == 0] == 0).all(), name
    finally:
        D.set_variant(-1)


def test_variants_with_idle_ctas_and_rows_beyond_one_batch():
    """Each cluster shape forced onto rows much narrower than it holds, so that the cluster's last
    CTAs own padding only or nothing at all, on a batch long enough that every cluster stages its
    rows in more than one round (more than 128 rows per cluster), with masked rows in between."""
    import torch
    from grpo_cpp_b200 import device as D
    names = D.variants()
    try:
        for idx, name in enumerate(names):
            c, t, v = (int(x) for x in re.match(r"(\d+)x(\d+)x(\d+)", name).groups())
            if c == 1:
                continue
            cap = c * t * v * 4
            V = cap // 16 - 3       # a sixteenth of the cluster has columns
            P = cap // 8            # an eighth of it has something to store
            # 74 clusters of eight 128-thread CTAs fit the GPU at once: 12,000 rows are more than 128 per cluster
            long_batch = c == 8 and t == 128
            b = W.logits_case(2, 20 if long_batch else 4, 300 if long_batch else 30, V, sigma=2.0, min_len=10,
                              reduction=W.TOKEN_MEAN, seed=300 + idx)
            want = run_oracle(b)
            D.set_variant(idx)
            dev = torch.from_numpy(b.padded(P)).cuda()
            assert D.plan(dev, V) == name
            st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                   b.B, b.G, b.T, V, P, cfg_of(b))
            out = dev.cpu().numpy()
            assert_stats(st, want[0], want[1], name)
            assert_grad(out[:, :V], want[2], name)
            assert (out[:, V:] == 0).all() and (out[b.mask == 0] == 0).all(), name
    finally:
        D.set_variant(-1)


def test_wide_dynamic_range_rows():
    """Rows whose logits span far more than a float exponent range in e-folds: a few columns near
    the top and everything else one or two thousand below, inside one thread's chunks, inside one
    warp and across warps.  The terms far below vanish against the top ones (the reference's double
    exp gives exactly 0 for them too, src/cpu/grpo_loss.cpp:203-213), and nothing on the way may
    overflow, lose its sign or turn into a NaN."""
    import torch
    V = 50257
    b = W.logits_case(1, 2, 4, V, sigma=2.0, min_len=4, seed=77)
    rng = np.random.Generator(np.random.PCG64(5))
    lg = b.logits.reshape(b.N, V)
    lg[0] = -2000.0 + rng.standard_normal(V).astype(np.float32)
    lg[0, [5, 4097, 50000]] = [3.0, 2.5, 1.0]
    lg[1] = np.where(np.arange(V) % 2 == 0, 300.0, -900.0).astype(np.float32) + rng.standard_normal(V).astype(np.float32)
    lg[2] = -1500.0
    lg[2, 12345] = 40.0
    lg[3, : V // 2] -= 1200.0
    lg[4] = rng.uniform(-1000.0, 1000.0, V).astype(np.float32)
    b.selected[:5] = [5, 2, 12345, V - 1, 7]
    # behaviour-policy and reference log-probs near the new ones, as a rollout has them
    l64 = lg.astype(np.float64)
    top = l64.max(axis=1)
    lp = l64[np.arange(b.N), b.selected] - (top + np.log(np.exp(l64 - top[:, None]).sum(axis=1)))
    b.logp_old[:] = (lp + 0.05).astype(np.float32)
    b.logp_ref[:] = (lp - 0.03).astype(np.float32)
    want = run_oracle(b)
    assert np.isfinite(want[2]).all()
    dev = torch.from_numpy(b.padded(50304)).cuda()
    st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                           b.B, b.G, b.T, V, 50304, cfg_of(b))
    out = dev.cpu().numpy()
    assert_stats(st, want[0], want[1], "wide range")
    assert_grad(out[:, :V], want[2], "wide range")


def test_config3_full_size():
    # N = 1024 x V = 32768, full mask, token-mean
    b = W.fused_v32k_case(42)
    want = run_oracle(b)
    check_all_entry_points(b, want, b.name)


@pytest.mark.parametrize("alpha", [0.5, 1.0])
def test_config4_full_size(alpha):
    # N = 1024 x V = 131072, ragged lengths U[16,64], L^alpha weights; in place on the device
    import torch
    b = W.fused_v128k_case(alpha, 42)
    want = run_oracle(b)
    dev = torch.from_numpy(b.logits).cuda()
    st = G.grpo_logits_cuda_device_inplace(dev, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                           b.B, b.G, b.T, b.V, b.V, cfg_of(b))
    out = dev.cpu().numpy()
    assert_stats(st, want[0], want[1], b.name)
    assert_grad(out, want[2], b.name)
    assert (out[b.mask == 0] == 0).all()


def test_device_layer_selected_logp_and_sharding():
    """Resident (no host hop) pipeline; the gathered log-probability; and the token-sharded path
    emulated rank by rank on one GPU: partial lengths summed, then each rank's rows with its
    row offset, then the records summed -- against one global CPU batch, as the reference checks
    its two-GPU demo (apps/03_two_gpu_train.cu:217-265)."""
    import torch
    from grpo_cpp_b200 import device as D
    from grpo_cpp_b200.sharded import shard_rows
    b = W.logits_case(3, 4, 16, 5003, sigma=3.0, min_len=1, reduction=W.TOKEN_MEAN, seed=21)
    P = 5008
    stats_w, valid_w, d_w, lp_w = oracle_py.load("port").logits(
        b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T, b.V,
        want_selected_logp=True, **b.cfg())
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)

    # single shot, everything resident
    boundary = D.ResidentBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=b.reduction)
    x = t(b.padded(P))
    lp = torch.empty(b.N, device="cuda")
    D.count_lengths(mask, b.S, b.T, 0, boundary.lengths)
    D.weights_from_lengths(boundary.lengths, b.reduction, 0.0, boundary.weights, boundary.meta)
    res = D.logits(x, old, ref, sel, adv, boundary.weights, mask, b.T, b.V, b.clip_eps, b.beta,
                   selected_logp=lp).cpu().numpy()
    assert boundary.meta.tolist() == [valid_w, 0]
    assert np.abs(res[:3] - stats_w).max() <= 1e-5 * np.abs(stats_w).max()
    assert_grad(x.cpu().numpy()[:, : b.V], d_w)
    lp_got = lp.cpu().numpy()
    assert np.abs(lp_got - lp_w).max() <= 2e-6 and (lp_got[b.mask == 0] == 0).all()
    # the gathered logit itself is exact: logp + lse reproduces it only through the right index,
    # so check the index path bit for bit on the inputs instead
    assert (b.logits[np.arange(b.N)[b.mask == 1], b.selected[b.mask == 1]]
            == b.padded(P)[np.arange(b.N)[b.mask == 1], b.selected[b.mask == 1]]).all()

    for world in (2, 3, 8):
        lengths = torch.zeros(b.S, dtype=torch.int32, device="cuda")
        for rank in range(world):  # exchange 1: sum of per-rank partial counts
            off, cnt = shard_rows(b.N, world, rank)
            lengths += D.count_lengths(mask[off:off + cnt].contiguous(), b.S, b.T, off)
        weights, meta = D.weights_from_lengths(lengths, b.reduction, 0.0)
        assert meta.tolist() == [valid_w, 0]
        total = np.zeros(5)
        x = t(b.padded(P))
        for rank in range(world):
            off, cnt = shard_rows(b.N, world, rank)
            sl = slice(off, off + cnt)
            r = D.logits(x[sl], old[sl].contiguous(), ref[sl].contiguous(), sel[sl].contiguous(), adv, weights,
                         mask[sl].contiguous(), b.T, b.V, b.clip_eps, b.beta, row_offset=off)
            total += r.cpu().numpy()  # exchange 2
        assert np.abs(total[:3] - stats_w).max() <= 1e-5 * np.abs(stats_w).max(), world
        assert_grad(x.cpu().numpy()[:, : b.V], d_w, f"world={world}")


def test_gpt2_shaped_config_at_full_size():
    """Configuration 5 at its stated size (65,536 rows x P = 50,304, V = 50,257, lengths U[32,256],
    token-mean), built on the device.  The oracle cannot walk 3.3e9 logits in test time, so parity
    at this size is: (a) size-independent properties -- tail and masked rows exactly zero, every
    active row's gradient sums to ~0, gradient at the selected column has the sign of -dlogp;
    (b) 48 sampled active rows checked element-wise against the oracle, with the global
    token-mean weight; (c) the three sums against a float64 recomputation from the gathered
    log-probabilities through the oracle's selected-token function."""
    import torch
    from grpo_cpp_b200 import device as D
    s = W.GPT2_SHAPE
    B, Gn, T, V, P = s["B"], s["G"], s["T"], s["V"], s["P"]
    S, N = B * Gn, B * Gn * T
    gen = torch.Generator(device="cuda").manual_seed(42)
    x = torch.empty(N, P, device="cuda")
    x.normal_(0.0, s["sigma"], generator=gen)
    rng = np.random.Generator(np.random.PCG64(42))
    lengths = rng.integers(s["min_len"], T + 1, S)
    mask_h = W.prefix_mask(lengths, T)
    sel_h = np.where(mask_h == 1, rng.integers(0, V, N), -1).astype(np.int32)
    rewards = (rng.random(S) < 0.5).astype(np.float32)
    adv_h = W.group_advantages_np(rewards, B, Gn)
    mask, sel, adv = (torch.from_numpy(a).cuda() for a in (mask_h, sel_h, adv_h))
    lse = torch.logsumexp(x[:, :V].double(), dim=1)
    now = (x[torch.arange(N, device="cuda"), sel.clamp(min=0).long()].double() - lse).float()
    old_h = np.where(mask_h == 1, now.cpu().numpy() + 0.05 * rng.standard_normal(N), 0).astype(np.float32)
    ref_h = np.where(mask_h == 1, now.cpu().numpy() + 0.05 * rng.standard_normal(N), 0).astype(np.float32)
    old, ref = torch.from_numpy(old_h).cuda(), torch.from_numpy(ref_h).cuda()
    active = np.flatnonzero(mask_h)
    sample = np.sort(rng.choice(active, 48, replace=False))
    rows_before = x[torch.from_numpy(sample).cuda()].cpu().numpy()

    boundary = D.ResidentBoundary(S, T, V, P, clip_eps=0.2, beta=0.01, reduction=W.TOKEN_MEAN)
    lp = torch.empty(N, device="cuda")
    D.count_lengths(mask, S, T, 0, boundary.lengths)
    D.weights_from_lengths(boundary.lengths, W.TOKEN_MEAN, 0.0, boundary.weights, boundary.meta)
    res = D.logits(x, old, ref, sel, adv, boundary.weights, mask, T, V, 0.2, 0.01, selected_logp=lp,
                   workspace=boundary.workspace).cpu().numpy()
    n_valid = int(mask_h.sum())
    assert boundary.meta.tolist() == [n_valid, 0]
    assert res[3] == 0 and res[4] == 0

    # (a) properties over all 3.3e9 outputs
    assert bool((x[:, V:] == 0).all())
    assert bool((x[mask == 0] == 0).all())
    row_sums = x.sum(dim=1)
    assert float(row_sums.abs().max()) <= 3e-5 / 1.0
    # (c) sums from the gathered log-probabilities through the oracle's token function
    st_w, valid_w, dlogp_w = oracle_py.load("best").loss(lp.cpu().numpy(), old_h, ref_h, adv_h, mask_h, B, Gn, T,
                                                         0.2, 0.01, W.TOKEN_MEAN, 0.0)
    assert valid_w == n_valid
    assert np.abs(res[:3] - st_w).max() <= 1e-5 * np.abs(st_w).max()
    lp_true = np.where(mask_h == 1, now.cpu().numpy(), 0)
    assert np.abs(lp.cpu().numpy() - lp_true).max() <= 3e-6
    # (b) sampled rows against the oracle: a one-row-per-response batch under token_mean weighs each
    # row 1/48; rescale to the true global weight 1/n_valid
    k = len(sample)
    st_s, _, d_s = oracle_py.load("best").logits(rows_before[:, :V], old_h[sample], ref_h[sample], sel_h[sample],
                                                 adv_h[sample // T], np.ones(k, np.int32), 1, k, 1, V,
                                                 0.2, 0.01, W.TOKEN_MEAN, 0.0)
    got = x[torch.from_numpy(sample).cuda()].cpu().numpy()[:, :V]
    scale = np.float64(n_valid) / np.float64(k)  # compare at the oracle's 1/48 weight, where 1e-7 absolute bites
    assert_grad(got.astype(np.float64) * scale, d_s, "sampled rows of the GPT-2-shaped batch")


def test_reference_driver_against_this_library():
    """The reference's own check program (bench/bench_grpo_loss_cuda.cu, --check-only), compiled
    from the reference tree and linked against libgrpo_b200.so instead of the reference's CUDA
    library, must pass.  The binary is built where the reference tree exists
    (make -C oracle ref-dropin) and travels with the repository."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_bench_dropin")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/ref_bench_dropin was not built in this checkout")
    out = subprocess.run([exe, "--check-only"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "CUDA checks passed" in out.stdout and "CUDA logits checks passed" in out.stdout


def test_fused_exchange_pass_single_rank():
    """ShardedBoundary.step_fused at world size 1: lengths counted as doubles into the exchange
    buffer, weights derived from it after the (no-op) collective, two passes over the same batch."""
    import torch
    from grpo_cpp_b200.sharded import ShardedBoundary
    b = W.logits_case(2, 3, 8, 4099, sigma=2.0, min_len=1, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5, seed=31)
    P = 4100
    want = run_oracle(b)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sb = ShardedBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=b.reduction,
                         length_alpha=b.length_alpha, device=torch.device("cuda"))
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
    sb.prepare(mask)
    for _ in range(2):
        x = t(b.padded(P))
        sb.step_fused(x, old, ref, sel, adv, mask)
        got = sb.stats()
        g3 = np.array([got["loss"], got["pg_loss"], got["kl"]])
        assert got["valid_tokens"] == want[1]
        assert (np.abs(g3 - want[0]) <= 1e-5 * np.abs(want[0]) + 1e-9).all()
        assert_grad(x.cpu().numpy()[:, : b.V], want[2])


@pytest.mark.gpu
def test_peer_exchange_pass_single_rank():
    """ShardedBoundary.step_peer at world size 1: the reduce kernel's last block pushes the record
    and the partial lengths into its own exchange region, publishes and waits on its own sequence
    number, and adds the one slot -- the whole exchange code path without a second GPU.  Three
    passes, so that both buffers of the region are reused."""
    import torch
    from grpo_cpp_b200.sharded import ShardedBoundary
    b = W.logits_case(2, 3, 8, 4099, sigma=2.0, min_len=1, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5, seed=32)
    P = 4100
    want = run_oracle(b)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sb = ShardedBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=b.reduction,
                         length_alpha=b.length_alpha, device=torch.device("cuda"))
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
    sb.prepare(mask)
    first = sb.weights.clone()
    sb.enable_peer_exchange()
    sb.prepare(mask)  # now through the exchange region (grpo_b200_lengths_sharded): the same weights, bit for bit
    assert (sb.weights == first).all() and sb.meta.cpu().tolist() == [int(b.mask.sum()), 0]
    try:
        for _ in range(3):
            x = t(b.padded(P))
            sb.step_peer(x, old, ref, sel, adv, mask)
            got = sb.stats()
            g3 = np.array([got["loss"], got["pg_loss"], got["kl"]])
            assert got["valid_tokens"] == want[1]
            assert (np.abs(g3 - want[0]) <= 1e-5 * np.abs(want[0]) + 1e-9).all()
            assert_grad(x.cpu().numpy()[:, : b.V], want[2])
            assert sb.lengths_f64.cpu().numpy().astype(np.int64).tolist() == b.mask.reshape(b.S, b.T).sum(1).tolist()
    finally:
        sb.exchange.close()


def test_row_order_partition_and_invariance():
    """grpo_b200_row_order is the stable partition of the row indices by mask (bit-exact against
    numpy), and a pass that uses it writes the same bits as one that does not, for cluster sizes
    1 to 8 and masks from nearly empty to full."""
    import torch
    from grpo_cpp_b200 import device as D
    rng = np.random.default_rng(8)
    for n in (1, 31, 1024, 70001):
        m = (rng.random(n) < 0.6).astype(np.int32)
        got = D.row_order(torch.from_numpy(m).cuda()).cpu().numpy()[: n + 2]
        idx = np.arange(n, dtype=np.int32)
        want = np.concatenate(([m.sum(), n - m.sum()], idx[m != 0], idx[m == 0])).astype(np.int32)
        assert (got == want).all()
    names = D.variants()
    try:
        for name, V, min_len in (("1x128x16", 1000, 1), ("4x128x16", 30000, 3), ("8x128x16", 50257, 1), ("8x256x16", 40000, 12)):
            P = (V + 3) // 4 * 4 + 8
            b = W.logits_case(3, 4, 12, V, sigma=2.0, min_len=min_len, reduction=W.TOKEN_MEAN, seed=len(name) + V)
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
            old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
            lengths = D.count_lengths(mask, b.S, b.T)
            weights, _ = D.weights_from_lengths(lengths, b.reduction, 0.0)
            D.set_variant(names.index(name))
            outs = []
            for order in (None, D.row_order(mask)):
                x = t(b.padded(P))
                assert D.plan(x, V) == name
                res = D.logits(x, old, ref, sel, adv, weights, mask, b.T, V, b.clip_eps, b.beta, row_order=order)
                outs.append((x.cpu().numpy(), res.cpu().numpy()))
            assert (outs[0][0] == outs[1][0]).all() and (outs[0][1] == outs[1][1]).all()
            want = run_oracle(b)
            assert_grad(outs[1][0][:, :V], want[2], name)
    finally:
        D.set_variant(-1)


@pytest.mark.parametrize("name,B,Gn,T,V,lengths", [
    ("8x128x16", 1, 1, 3, 50257, [1]),           # fewer rows than clusters, one active row
    ("8x128x16", 1, 2, 1, 40000, [1, 1]),        # one token per response
    ("4x128x16", 2, 2, 40, 20000, [1, 40, 2, 39]),  # nearly empty next to full responses
    ("1x128x16", 1, 3, 200, 777, [200, 1, 100]),    # many rows per cluster, several staging batches
])
def test_row_order_edge_shapes(name, B, Gn, T, V, lengths):
    """The balanced row order on shapes at the edges of its index arithmetic: clusters without rows,
    clusters with only masked or only active rows, more rows per cluster than one staging batch."""
    import torch
    from grpo_cpp_b200 import device as D
    P = (V + 3) // 4 * 4
    b = W.logits_case(B, Gn, T, V, sigma=2.0, min_len=1, reduction=W.SEQUENCE_MEAN, seed=V + T)
    b.mask = W.prefix_mask(np.asarray(lengths), T).astype(np.int32)
    b.selected = np.where(b.mask == 1, np.maximum(b.selected, 0), -1).astype(np.int32)
    want = run_oracle(b)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
    lens = D.count_lengths(mask, b.S, b.T)
    weights, _ = D.weights_from_lengths(lens, b.reduction, 0.0)
    try:
        D.set_variant(D.variants().index(name))
        x = t(b.padded(P))
        assert D.plan(x, V) == name
        res = D.logits(x, old, ref, sel, adv, weights, mask, b.T, V, b.clip_eps, b.beta, row_order=D.row_order(mask))
        got = res.cpu().numpy()
        assert (np.abs(got[:3] - want[0]) <= 1e-5 * np.abs(want[0]) + 1e-9).all() and got[3] == 0 and got[4] == 0
        out = x.cpu().numpy()
        assert_grad(out[:, :V], want[2], name)
        assert (out[b.mask == 0] == 0).all() and (out[:, V:] == 0).all()
    finally:
        D.set_variant(-1)
