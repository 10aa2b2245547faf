"""Parity of the selected-token CUDA path (K1) with the CPU oracle -- runs on the B200.

Every call goes through the C ABI of libgrpo_b200.so (host layer via ``grpo_loss_cuda``, device
layer via ``grpo_cpp_b200.device``).  Tolerances are the ones stated for this path: loss terms
within 1e-5 relative, dlogp within 1e-7 + 1e-5 * |want|, valid-token counts and masks exact.
"""
import math

import numpy as np
import pytest

import oracle_py
import grpo_cpp_b200 as G
from grpo_cpp_b200 import workloads as W

pytestmark = pytest.mark.gpu

STAT_RTOL, STAT_ATOL = 1e-5, 1e-9
GRAD_RTOL, GRAD_ATOL = 1e-5, 1e-7


def oracle():
    return oracle_py.load("best")


def assert_stats(got: G.LossStats, want_stats, want_valid, what=""):
    got3 = np.array([got.loss, got.pg_loss, got.kl], np.float64)
    want3 = np.asarray(want_stats, np.float64)
    assert got.valid_tokens == want_valid, what
    err = np.abs(got3 - want3)
    assert (err <= STAT_ATOL + STAT_RTOL * np.abs(want3)).all(), f"{what}: got {got3} want {want3}"


def assert_grad(got, want, what=""):
    got, want = np.asarray(got, np.float64).reshape(-1), np.asarray(want, np.float64).reshape(-1)
    err = np.abs(got - want)
    tol = GRAD_ATOL + GRAD_RTOL * np.abs(want)
    bad = np.flatnonzero(err > tol)
    assert bad.size == 0, f"{what}: {bad.size} elements off, worst {err.max():.3e} at {err.argmax()}"


def cfg_of(b) -> G.LossConfig:
    return G.LossConfig(b.clip_eps, b.beta, G.ReductionMode(b.reduction), b.length_alpha)


def run_host(b, kernel=G.CudaLossKernel.block_reduce):
    return G.grpo_loss_cuda(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, b.B, b.G, b.T, cfg_of(b), kernel)


def run_oracle(b):
    return oracle().loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, b.B, b.G, b.T, **b.cfg())


def test_golden_token_cases(golden_token):
    for name in golden_token.cases:
        c = golden_token.case(name)
        B, Gn, T = (int(x) for x in c["shape"])
        eps, beta, red, alpha = c["cfg"]
        cfg = G.LossConfig(float(eps), float(beta), G.ReductionMode(int(red)), float(alpha))
        r = G.grpo_loss_cuda(c["logp_new"], c["logp_old"], c["logp_ref"], c["advantages"],
                             c["mask"].astype(np.int32), B, Gn, T, cfg)
        assert_stats(r.stats, c["stats"], int(c["valid"]), name)
        assert_grad(r.dlogp_new, c["dlogp"], name)
        assert (r.dlogp_new[c["mask"] == 0] == 0).all(), name


def test_reference_check_shapes(golden_fixtures):
    # the block-boundary shapes of the reference's own GPU parity check
    # (bench/bench_grpo_loss_cuda.cu:193-225), both kernel selectors
    from make_golden import TOKEN_FIXTURE_SHAPES
    reductions = (W.SEQUENCE_MEAN, W.TOKEN_MEAN, W.LENGTH_WEIGHTED)
    for i, (B, Gn, T) in enumerate(TOKEN_FIXTURE_SHAPES):
        b = W.reference_token_fixture(B, Gn, T, partial=(i == 5))
        b.beta, b.reduction, b.length_alpha = 0.03, reductions[i % 3], 0.5
        want = run_oracle(b)
        gold = golden_fixtures.case(f"token_{B}x{Gn}x{T}")
        assert (want[0] == gold["stats"]).all()
        for kernel in (G.CudaLossKernel.atomic, G.CudaLossKernel.block_reduce):
            r = run_host(b, kernel)
            assert_stats(r.stats, want[0], want[1], b.name)
            assert_grad(r.dlogp_new, want[2], b.name)


def test_known_answers_through_cuda():
    # the reference's CPU known answers (tests/test_grpo_loss.cpp:97-167, 243-247), asked of the GPU
    now = np.log(np.array([1.1, 1.5, 0.9, 0.5], np.float32)).astype(np.float32)
    g = G.grpo_loss_cuda(now, np.zeros(4), now, [1, 1, -1, -1], [1, 1, 1, 1], 1, 4, 1).dlogp_new
    assert abs(g[0] + 1.1 / 4) <= 1e-6 and g[1] == 0 and abs(g[2] - 0.9 / 4) <= 1e-6 and g[3] == 0
    r = G.grpo_loss_cuda([0], [0], [math.log(2.0)], [0], [1], 1, 1, 1, G.LossConfig(beta=0.3))
    assert abs(r.stats.kl - (1 - math.log(2.0))) <= 1e-6 and abs(r.dlogp_new[0] + 0.3) <= 1e-6
    for d in (1e-3, 1e-4, 1e-6):
        d32 = float(np.float32(d))
        r = G.grpo_loss_cuda([0], [0], [d32], [0], [1], 1, 1, 1, G.LossConfig(beta=1.0))
        exact_kl, exact_g = math.expm1(d32) - d32, -math.expm1(d32)
        assert abs(r.stats.kl - exact_kl) <= 2e-14 + 0.15 * exact_kl and r.stats.kl >= 0
        assert abs(r.dlogp_new[0] - exact_g) <= 1e-10 + 2e-6 * abs(exact_g)
    z = np.zeros(8, np.float32)
    mask = [1, 0, 0, 0, 1, 1, 1, 1]
    g = G.grpo_loss_cuda(z, z, z, [1, 1], mask, 1, 2, 4, G.LossConfig(reduction=G.ReductionMode.token_mean)).dlogp_new
    assert abs(-g[0] - 0.2) <= 1e-6 and abs(-g[4:].sum() - 0.8) <= 1e-6
    for alpha in (0.0, 0.5, 1.0):
        cfg = G.LossConfig(reduction=G.ReductionMode.length_weighted, length_alpha=alpha)
        g = G.grpo_loss_cuda(z, z, z, [1, 1], mask, 1, 2, 4, cfg).dlogp_new
        assert abs(-g[0] - 0.5) <= 1e-6 and abs(-g[4:].sum() - 4.0 ** alpha / 2) <= 1e-6
    r = G.grpo_loss_cuda([0], [-100], [0], [0], [1], 1, 1, 1)  # zero advantage: ratio never evaluated
    assert r.stats.loss == 0 and r.dlogp_new[0] == 0


@pytest.mark.parametrize("call,msg", [
    (lambda: G.grpo_loss_cuda([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 0, 2, 1), "B, G and T must be positive"),
    (lambda: G.grpo_loss_cuda([0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1), "logp_new has size 1, expected 2"),
    (lambda: G.grpo_loss_cuda([0, 0], [0, 0], [0, 0], [1, -1], [1, 0], 1, 2, 1),
     "every sequence needs at least one valid token"),
    (lambda: G.grpo_loss_cuda([0], [0], [0], [0], [0], 1, 1, 1), "every sequence needs at least one valid token"),
    (lambda: G.grpo_loss_cuda([0], [-100], [0], [-1], [1], 1, 1, 1), "CUDA loss became non-finite"),
])
def test_error_contract_with_device(call, msg):
    # bench/bench_grpo_loss_cuda.cu:227-243: CPU and CUDA must both throw for these
    with pytest.raises(RuntimeError) as e:
        call()
    assert str(e.value) == msg


@pytest.mark.parametrize("T,ragged", [(256, False), (256, True), (1024, False), (1024, True)])
def test_full_size_selected_token_config(T, ragged):
    # configuration 2 at its stated sizes: 4096 responses, N = 1,048,576 and 4,194,304
    b = W.selected_token_case(4096, T, ragged, seed=42)
    want = run_oracle(b)
    r = run_host(b)
    assert_stats(r.stats, want[0], want[1], b.name)
    assert_grad(r.dlogp_new, want[2], b.name)
    assert (r.dlogp_new[b.mask == 0] == 0).all()
    again = run_host(b)  # no atomics: bit-identical from run to run
    assert again.stats == r.stats and (again.dlogp_new.view(np.uint32) == r.dlogp_new.view(np.uint32)).all()


def test_device_layer_offsets_and_unaligned():
    import torch
    from grpo_cpp_b200 import device as D
    b = W.selected_token_case(64, 37, True, seed=9, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5)
    want = run_oracle(b)
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    mask = t(b.mask)
    lengths = D.count_lengths(mask, b.S, b.T)
    assert (lengths.cpu().numpy() == b.mask.reshape(b.S, b.T).sum(1)).all()
    weights, meta = D.weights_from_lengths(lengths, b.reduction, b.length_alpha)
    assert meta.tolist() == [int(b.mask.sum()), 0]
    # the reference's weights, read off its own gradient: with all log-probabilities 0 and A = 1 each
    # active token's dlogp is exactly -weight (src/cpu/grpo_loss.cpp:124-131,160)
    z = np.zeros(b.N, np.float32)
    w_ref = -oracle().loss(z, z, z, np.ones(b.S, np.float32), b.mask, b.B, b.G, b.T, 0.2, 0.0, b.reduction,
                           b.length_alpha)[2].reshape(b.S, b.T)[:, 0]
    assert (weights.cpu().numpy().view(np.uint32) == w_ref.view(np.uint32)).all()
    adv = t(b.advantages)
    # whole batch
    dlogp, res = D.loss(t(b.logp_new), t(b.logp_old), t(b.logp_ref), adv, weights, mask, b.T, b.clip_eps, b.beta)
    res = res.cpu().numpy()
    assert np.abs(res[:3] - want[0]).max() <= 1e-5 * np.abs(want[0]).max()
    assert_grad(dlogp.cpu().numpy(), want[2])
    assert res[3] == 0 and res[4] == 0
    # two shards cut inside a response, the second starting at an address that is not 16-byte aligned
    cut = 1001
    total = np.zeros(5)
    for lo, hi in ((0, cut), (cut, b.N)):
        sl = lambda a: t(a)[lo:hi]
        d2, r2 = D.loss(sl(b.logp_new), sl(b.logp_old), sl(b.logp_ref), adv, weights, mask[lo:hi], b.T,
                        b.clip_eps, b.beta, token_offset=lo,
                        dlogp=torch.empty(b.N, device=dev)[lo:hi])
        assert_grad(d2.cpu().numpy(), want[2][lo:hi])
        total += r2.cpu().numpy()
    assert np.abs(total[:3] - want[0]).max() <= 1e-5 * np.abs(want[0]).max()


def test_group_advantages_bit_exact():
    import torch
    from grpo_cpp_b200 import device as D
    rng = np.random.RandomState(5)
    B, Gn = 37, 16
    rewards = rng.choice([0.0, 1.0, 0.25], size=B * Gn).astype(np.float32)
    rewards[:Gn] = 1.0  # an all-equal group
    for mode in (0, 1):
        want = oracle().group_advantages(rewards, B, Gn, mode, 1e-8)
        got, meta = D.group_advantages(torch.from_numpy(rewards).cuda(), B, Gn, mode, 1e-8)
        assert meta.item() == 0
        assert (got.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all()


@pytest.mark.gpu
def test_global_group_advantages_single_rank_on_device():
    """sharded.global_group_advantages without a process group (world 1): the device kernel on the
    regrouped rewards, bit-exact against the oracle, all-equal groups exactly zero."""
    import torch
    from grpo_cpp_b200.sharded import global_group_advantages
    rng = np.random.RandomState(9)
    prompts, G_local = 7, 8
    rewards = (rng.rand(prompts, G_local) < 0.4).astype(np.float32)
    rewards[3] = 0.0
    mine, meta = global_group_advantages(torch.from_numpy(rewards.reshape(-1)).cuda(), prompts, G_local)
    want = oracle_py.load("best").group_advantages(rewards.reshape(-1), prompts, G_local)
    assert (mine.cpu().numpy() == np.asarray(want)).all() and int(meta.cpu()[0]) == 0
    assert (mine.cpu().numpy().reshape(prompts, G_local)[3] == 0).all()
