"""Pins the CPU checker before anything is compared with it.

Three layers: (1) the known answers the reference's own unit tests hold for this path
(tests/test_grpo_loss.cpp of the reference: clipping, KL, reductions, finite differences,
error contract, zero advantage, logits boundary, advantages); (2) the committed golden vectors,
which were produced by the reference's own object code; (3) when that object code is present
(oracle/_ref), bit-for-bit agreement of the C restatement with it on fresh seeded inputs.
Every comparison between the restatement and reference output is exact (``==`` on the bits).
"""
import math
import zlib

import os

import numpy as np
import pytest

import oracle_py
from grpo_cpp_b200 import workloads as W

KINDS = ["port"] + (["reference"] if oracle_py.have_reference() else [])


@pytest.fixture(params=KINDS)
def lib(request):
    return oracle_py.load(request.param)


def f32(*v):
    return np.array(v, np.float32)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- (1) known answers -------------------------------------------------------------------

def test_clipping_known_answers(lib):
    # reference tests/test_grpo_loss.cpp:97-109: ratios 1.1 / 1.5 / 0.9 / 0.5 with A = +1,+1,-1,-1
    now = np.log(f32(1.1, 1.5, 0.9, 0.5)).astype(np.float32)
    _, _, g = lib.loss(now, np.zeros(4), now, f32(1, 1, -1, -1), np.ones(4, np.int32), 1, 4, 1)
    assert abs(g[0] - (-1.1 / 4)) <= 1e-6
    assert g[1] == 0.0
    assert abs(g[2] - (0.9 / 4)) <= 1e-6
    assert g[3] == 0.0


def test_kl_known_answers(lib):
    # :111-135: k3 estimator at ref/new = 2 -> 1 - ln 2, gradient -beta; expm1 behaviour near zero
    stats, _, g = lib.loss([0], [0], [math.log(2.0)], [0], [1], 1, 1, 1, beta=0.3)
    assert abs(stats[2] - (1 - math.log(2.0))) <= 1e-6
    assert abs(stats[0] - 0.3 * (1 - math.log(2.0))) <= 1e-6
    assert abs(g[0] + 0.3) <= 1e-6
    for d in (1e-3, 1e-4, 1e-6):
        d32 = float(np.float32(d))
        stats, _, g = lib.loss([0], [0], [d32], [0], [1], 1, 1, 1, beta=1.0)
        exact_kl = math.expm1(d32) - d32
        exact_g = -math.expm1(d32)
        assert abs(stats[2] - exact_kl) <= 2e-14 + 0.15 * abs(exact_kl)
        assert abs(g[0] - exact_g) <= 1e-10 + 2e-6 * abs(exact_g)
        assert stats[2] >= 0.0


def test_reduction_gradient_mass(lib):
    # :137-167: lengths {1,4}; gradient mass per response under the three reductions
    z = np.zeros(8, np.float32)
    mask = np.array([1, 0, 0, 0, 1, 1, 1, 1], np.int32)
    _, _, g = lib.loss(z, z, z, [1, 1], mask, 1, 2, 4, reduction=W.SEQUENCE_MEAN)
    assert abs(-g[0] - 0.5) <= 1e-6 and abs(-g[4:].sum() - 0.5) <= 1e-6
    _, _, g = lib.loss(z, z, z, [1, 1], mask, 1, 2, 4, reduction=W.TOKEN_MEAN)
    assert abs(-g[0] - 0.2) <= 1e-6 and abs(-g[4:].sum() - 0.8) <= 1e-6
    for alpha in (0.0, 0.5, 1.0):
        _, _, g = lib.loss(z, z, z, [1, 1], mask, 1, 2, 4, reduction=W.LENGTH_WEIGHTED, length_alpha=alpha)
        assert abs(-g[0] - 0.5) <= 1e-6
        assert abs(-g[4:].sum() - 4.0 ** alpha / 2) <= 1e-6
        assert (g[1:4] == 0).all()


def _fd_problem():
    B, G, T = 2, 3, 4
    rng = np.random.RandomState(7)
    n = B * G * T
    old = rng.uniform(-2.0, -0.5, n).astype(np.float32)
    now = (old + rng.uniform(-0.12, 0.12, n)).astype(np.float32)
    ref = (old + rng.uniform(-0.12, 0.12, n)).astype(np.float32)
    adv = f32(0.7, -0.2, -0.5, -0.8, 0.3, 0.5)
    mask = W.prefix_mask(1 + np.arange(B * G) % T, T)
    return B, G, T, now, old, ref, adv, mask


def test_finite_differences_token_path(lib):
    # :169-208: central differences of the scalar loss vs dlogp, ragged, L^0.5 weights, beta 0.03
    B, G, T, now, old, ref, adv, mask = _fd_problem()
    kw = dict(beta=0.03, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5)
    _, _, g = lib.loss(now, old, ref, adv, mask, B, G, T, **kw)
    h = np.float32(1e-3)
    for i in np.flatnonzero(mask):
        up, dn = now.copy(), now.copy()
        up[i] += h
        dn[i] -= h
        num = (lib.loss(up, old, ref, adv, mask, B, G, T, **kw)[0][0]
               - lib.loss(dn, old, ref, adv, mask, B, G, T, **kw)[0][0]) / (2 * h)
        assert abs(g[i] - num) <= 2e-4 + 3e-3 * abs(num)


@pytest.mark.parametrize("call,msg", [
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 0, 2, 1), "B, G and T must be positive"),
    (lambda L: L.loss([0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1), "logp_new has size 1, expected 2"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1, clip_eps=-0.1),
     "clip_eps must be finite and in [0, 1)"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1, beta=-0.1),
     "beta must be finite and non-negative"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 0], 1, 2, 1),
     "every sequence needs at least one valid token"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1, reduction=2, length_alpha=1.1),
     "length_alpha must be finite and in [0, 1]"),
    (lambda L: L.loss([np.inf, 0], [0, 0], [0, 0], [1, -1], [1, 1], 1, 2, 1), "log probabilities must be finite"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [1, -1], [1, 2], 1, 2, 1), "mask values must be 0 or 1"),
    (lambda L: L.loss([0, 0], [0, 0], [0, 0], [np.nan, -1], [1, 1], 1, 2, 1), "advantages must be finite"),
    (lambda L: L.loss([0], [-100], [0], [-1], [1], 1, 1, 1), "loss became non-finite"),
    (lambda L: L.loss([0], [0], [0], [1], [1], 65536, 65536, 1), "sequence count exceeds INT_MAX"),
    (lambda L: L.loss([0], [0], [0], [1], [1], 65536, 1, 65536), "token count exceeds INT_MAX"),
    (lambda L: L.group_advantages([], 65536, 65536), "sequence count exceeds INT_MAX"),
    (lambda L: L.group_advantages([np.inf, 1], 1, 2), "rewards must be finite"),
    (lambda L: L.group_advantages([0, 1], 1, 2, eps=-1.0), "eps must be finite and non-negative"),
])
def test_error_contract(lib, call, msg):
    # :210-241 plus the remaining throw sites of src/cpu/grpo_loss.cpp
    with pytest.raises(RuntimeError) as e:
        call(lib)
    assert str(e.value) == msg


def test_zero_advantage_short_circuit(lib):
    # :243-247: A == 0 must not evaluate exp(0 - (-100))
    stats, _, g = lib.loss([0], [-100], [0], [0], [1], 1, 1, 1)
    assert stats[0] == 0.0 and g[0] == 0.0


def _boundary_problem():
    logits = f32(1.0, -0.5, 0.2, 0.8, 0.3, 0.1, -0.4, 0.7, -0.2, 0.5, 1.1, 0.0,
                 1000.0, 999.0, 998.0, 997.0).reshape(4, 4)
    sel = np.array([3, 0, 2, -1], np.int32)
    mask = np.array([1, 1, 1, 0], np.int32)
    now = np.zeros(4, np.float32)
    for i in range(3):
        top = logits[i].max()
        z = np.exp((logits[i] - top).astype(np.float64)).sum()
        now[i] = np.float32(logits[i, sel[i]] - top) - np.float32(math.log(z))
    old = f32(now[0] - 0.1, now[1] + 0.05, now[2] - 0.03, 0)
    ref = f32(now[0] + 0.02, now[1] - 0.01, now[2] + 0.04, 0)
    return logits, sel, mask, now, old, ref, f32(0.7, -0.4)


def test_logits_boundary(lib):
    # :257-313: logits path == selected-token path; row sums ~ 0; masked row exactly 0 even with
    # logits of 1000; finite differences through the softmax; the two throws of the logits path
    logits, sel, mask, now, old, ref, adv = _boundary_problem()
    base, _, _ = lib.loss(now, old, ref, adv, mask, 1, 2, 2, beta=0.03)
    stats, valid, d = lib.logits(logits, old, ref, sel, adv, mask, 1, 2, 2, 4, beta=0.03)
    assert valid == 3
    assert np.abs(stats - base).max() <= 1e-7
    assert np.abs(d.sum(axis=1)).max() <= 2e-7
    assert (d[3] == 0).all()
    h = np.float32(1e-3)
    for i in range(3):
        for v in range(4):
            up, dn = logits.copy(), logits.copy()
            up[i, v] += h
            dn[i, v] -= h
            num = (lib.logits(up, old, ref, sel, adv, mask, 1, 2, 2, 4, beta=0.03)[0][0]
                   - lib.logits(dn, old, ref, sel, adv, mask, 1, 2, 2, 4, beta=0.03)[0][0]) / (2 * h)
            assert abs(d[i, v] - num) <= 2e-5 + 4e-3 * abs(num)
    with pytest.raises(RuntimeError, match="selected token is outside the vocabulary"):
        lib.logits(logits, old, ref, [4, 0, 2, -1], adv, mask, 1, 2, 2, 4, beta=0.03)
    bad = logits.copy()
    bad[0, 0] = np.inf
    with pytest.raises(RuntimeError, match="logits must be finite"):
        lib.logits(bad, old, ref, sel, adv, mask, 1, 2, 2, 4, beta=0.03)


def test_group_advantages_known_answers(lib):
    # :51-95
    r = f32(0, 1, 1, 0, 2, 2, 2, 2)
    z = lib.group_advantages(r, 2, 4, oracle_py.STANDARDIZED, 1e-12)
    c = lib.group_advantages(r, 2, 4, oracle_py.CENTERED)
    assert abs(z[0] + 1) <= 1e-5 and abs(z[1] - 1) <= 1e-5
    assert (z[4:] == 0).all()
    assert (lib.group_advantages([2, 2, 2, 2], 1, 4, oracle_py.STANDARDIZED, 0.0) == 0).all()
    assert lib.group_advantages([2], 1, 1, oracle_py.STANDARDIZED, 0.0)[0] == 0
    assert (lib.group_advantages([0.1] * 7, 1, 7, oracle_py.STANDARDIZED, 0.0) == 0).all()
    assert (lib.group_advantages([0.1] * 7, 1, 7, oracle_py.CENTERED) == 0).all()
    assert abs(c[:4].sum()) <= 1e-6 and abs(c[4:].sum()) <= 1e-6
    assert abs(z[:4].mean()) <= 1e-6 and abs(z[:4].var() - 1) <= 2e-5


# ---- (2) golden vectors (reference object code) vs the restatement: exact ----------------

def test_port_matches_golden_token_cases(golden_token):
    port = oracle_py.load("port")
    for name in golden_token.cases:
        c = golden_token.case(name)
        B, G, T = (int(x) for x in c["shape"])
        eps, beta, red, alpha = c["cfg"]
        stats, valid, dlogp = port.loss(c["logp_new"], c["logp_old"], c["logp_ref"], c["advantages"],
                                        c["mask"].astype(np.int32), B, G, T, float(eps), float(beta),
                                        int(red), float(alpha))
        assert valid == int(c["valid"]), name
        assert (bits(stats) == bits(c["stats"])).all(), name
        assert (bits(dlogp) == bits(c["dlogp"])).all(), name


def test_port_matches_golden_logits_cases(golden_logits):
    port = oracle_py.load("port")
    for name in golden_logits.cases:
        c = golden_logits.case(name)
        B, G, T, V = (int(x) for x in c["shape"])
        eps, beta, red, alpha = c["cfg"]
        stats, valid, d = port.logits(c["logits"], c["logp_old"], c["logp_ref"], c["selected"],
                                      c["advantages"], c["mask"].astype(np.int32), B, G, T, V,
                                      float(eps), float(beta), int(red), float(alpha))
        assert valid == int(c["valid"]), name
        assert (bits(stats) == bits(c["stats"])).all(), name
        assert (bits(d) == bits(c["dlogits"].reshape(d.shape))).all(), name


def test_port_matches_golden_reference_fixtures(golden_fixtures):
    from make_golden import LOGITS_FIXTURE_SHAPES, TOKEN_FIXTURE_SHAPES
    port = oracle_py.load("port")
    reductions = (W.SEQUENCE_MEAN, W.TOKEN_MEAN, W.LENGTH_WEIGHTED)
    for i, (B, G, T) in enumerate(TOKEN_FIXTURE_SHAPES):
        b = W.reference_token_fixture(B, G, T, partial=(i == 5))
        c = golden_fixtures.case(f"token_{B}x{G}x{T}")
        got_crc = [zlib.crc32(np.ascontiguousarray(a).tobytes())
                   for a in (b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask)]
        assert got_crc == [int(x) for x in c["in_crc"]], "fixture builder drifted"
        stats, valid, dlogp = port.loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, B, G, T,
                                        0.2, 0.03, reductions[i % 3], 0.5)
        assert valid == int(c["valid"])
        assert (bits(stats) == bits(c["stats"])).all()
        assert zlib.crc32(dlogp.tobytes()) == int(c["dlogp_crc"])
    for (B, G, T, V, partial) in LOGITS_FIXTURE_SHAPES:
        b = W.reference_logits_fixture(B, G, T, V, partial)
        c = golden_fixtures.case(f"logits_{B}x{G}x{T}x{V}")
        stats, valid, d = port.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                      B, G, T, V, 0.2, 0.03)
        assert valid == int(c["valid"])
        assert (bits(stats) == bits(c["stats"])).all()
        assert (bits(d) == bits(c["dlogits"].reshape(d.shape))).all()


# ---- (3) restatement vs the reference's object code on fresh inputs: exact ---------------

needs_ref = pytest.mark.skipif(not oracle_py.have_reference(), reason="oracle/_ref not built here")


@needs_ref
@pytest.mark.parametrize("seed", [1, 2, 3])
@pytest.mark.parametrize("red,alpha", [(0, 0.0), (1, 0.0), (2, 0.0), (2, 0.37), (2, 1.0)])
def test_port_equals_reference_token_path(seed, red, alpha):
    port, ref = oracle_py.load("port"), oracle_py.load("reference")
    b = W.selected_token_case(96, 53, ragged=True, seed=seed, G=8, reduction=red, length_alpha=alpha)
    b.beta = 0.04
    a = port.loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, b.B, b.G, b.T, **b.cfg())
    r = ref.loss(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, b.B, b.G, b.T, **b.cfg())
    assert a[1] == r[1]
    assert (bits(a[0]) == bits(r[0])).all() and (bits(a[2]) == bits(r[2])).all()


@needs_ref
@pytest.mark.parametrize("seed,V", [(5, 7), (6, 300), (7, 1025)])
def test_port_equals_reference_logits_path(seed, V):
    port, ref = oracle_py.load("port"), oracle_py.load("reference")
    b = W.logits_case(2, 3, 5, V, sigma=3.0, min_len=1, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5, seed=seed)
    a = port.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T, V, **b.cfg())
    r = ref.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T, V, **b.cfg())
    assert a[1] == r[1]
    assert (bits(a[0]) == bits(r[0])).all() and (bits(a[2]) == bits(r[2])).all()


@needs_ref
def test_port_equals_reference_advantages():
    port, ref = oracle_py.load("port"), oracle_py.load("reference")
    rng = np.random.RandomState(3)
    r = rng.choice([0.0, 1.0, 0.5], size=12 * 8).astype(np.float32)
    for mode in (0, 1):
        assert (bits(port.group_advantages(r, 12, 8, mode, 1e-8))
                == bits(ref.group_advantages(r, 12, 8, mode, 1e-8))).all()


def test_sampling_helpers_known_answers():
    """row_logsumexp / sample_row (restating apps/04_gpt2_grpo.cu:61-78): uniform rows
    have lse = x + log V and a coin u lands on floor(u * V); a one-hot-like row always returns its
    peak; a coin past the accumulated mass falls back to V - 1."""
    p = oracle_py.load("port")
    x = np.full(1000, -2.25, np.float32)
    assert abs(p.row_logsumexp(x) - (-2.25 + np.log(1000.0))) < 1e-12
    for u in (0.0, 0.0005, 0.2503, 0.4996, 0.7307, 0.9985):  # away from the k/1000 boundaries
        assert p.sample_row(x, u) == int(u * 1000)
    peak = np.full(50, -40.0, np.float32)
    peak[17] = 30.0
    assert abs(p.row_logsumexp(peak) - 30.0) < 1e-12
    assert all(p.sample_row(peak, u) == 17 for u in (1e-9, 0.5, 0.999999))
    assert p.sample_row(peak, 1.0) == 49  # the cumulative sum never exceeds a coin of 1
    two = np.array([np.log(0.25), np.log(0.75)], np.float32)
    assert p.sample_row(two, 0.2499) == 0 and p.sample_row(two, 0.2501) == 1


def test_sampling_helpers_against_committed_vectors():
    """tests/golden/sampling_cases.npz holds what the REFERENCE's own object code of
    apps/04_gpt2_grpo.cu:61-78 returned (tests/golden/make_sampling_golden.py): the restatement must
    give the same log-sum-exp bits and, fed the coins the reference's generator produced, the same
    tokens."""
    from conftest import Golden
    g = Golden("sampling_cases.npz")
    p = oracle_py.load("port")
    assert "V50257" in g.cases
    for name in g.cases:
        c = g.case(name)
        for i in range(len(c["coins"])):
            assert p.row_logsumexp(c["logits"][i]) == c["lse"][i]
            assert p.sample_row(c["logits"][i], c["coins"][i]) == c["tokens"][i]
            assert np.float32(np.float64(c["logits"][i][c["tokens"][i]]) - c["lse"][i]) == c["logp"][i]


def test_sampling_helpers_against_reference_object_code_on_fresh_inputs():
    """Where oracle/_ref/libgrpo_ref_sample.so exists (built from the reference tree): same bits and
    same tokens on inputs that are not in the committed file, including the coin sequence of
    std::uniform_real_distribution<double> over std::mt19937."""
    import make_sampling_golden as M
    if not os.path.exists(M.REF_SAMPLE):
        pytest.skip("reference sampling helpers were not built in this checkout")
    lib = M.load_reference_sampler()
    p = oracle_py.load("port")
    rng = np.random.default_rng(7)
    for V in (5, 1000, 32768):
        x = rng.normal(0, 2.5, (8, V)).astype(np.float32)
        lse, coins, tokens = M.reference_draws(lib, x, seed=99 + V)
        assert ((coins >= 0) & (coins < 1)).all()
        for i in range(8):
            assert p.row_logsumexp(x[i]) == lse[i]
            cdf = np.cumsum(np.exp(x[i].astype(np.float64) - lse[i]))
            if np.abs(cdf - coins[i]).min() > 1e-12:
                assert p.sample_row(x[i], coins[i]) == tokens[i]


def test_rows_entry_matches_the_whole_batch_entry_bit_for_bit():
    """grpo_oracle_logits_rows (rows out of a batch, weights given) against grpo_oracle_logits on the
    whole batch, for the three reductions: same gradient bits, same selected log-probabilities, and
    the per-row fp32 products add up (in double, in row order) to the batch's three sums."""
    from grpo_cpp_b200 import workloads as W
    p = oracle_py.load("port")
    for reduction, alpha in ((0, 0.0), (1, 0.0), (2, 0.5)):
        b = W.logits_case(2, 3, 7, 33, sigma=2.0, min_len=1, reduction=reduction, length_alpha=alpha, seed=3)
        stats, valid, want, want_lp = p.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                               b.B, b.G, b.T, b.V, want_selected_logp=True, **b.cfg())
        lengths = b.mask.reshape(b.S, b.T).sum(1)
        f = np.float32
        if reduction == 0:
            w_seq = f(1.0) / (f(b.S) * lengths.astype(f))
        elif reduction == 1:
            w_seq = np.full(b.S, f(1.0) / f(valid), f)
        else:
            w_seq = np.array([np.float32(np.power(f(L), f(alpha) - f(1.0), dtype=f)) for L in lengths], f) / f(b.S)
        rows = np.flatnonzero(b.mask == 1)
        seq = rows // b.T
        got, got_lp, terms = p.logits_rows(b.logits.reshape(b.N, b.V)[rows], b.logp_old[rows], b.logp_ref[rows],
                                           b.selected[rows], b.advantages[seq], w_seq[seq], b.clip_eps, b.beta)
        assert (got.view(np.uint32) == want.reshape(b.N, b.V)[rows].view(np.uint32)).all()
        assert (got_lp.view(np.uint32) == want_lp[rows].view(np.uint32)).all()
        sums = np.zeros(3)
        for t in terms:
            sums += t.astype(np.float64)
        assert (sums.astype(f) == stats).all()
