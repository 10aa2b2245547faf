"""Parity of grpo_b200_sample_rows with the CPU restatement of the reference demo's host-side
sampling (apps/04_gpt2_grpo.cu:61-78, 138-161; the restatement is pinned to the reference's object
code by tests/test_oracle.py) and with vectors produced by that object code -- runs on the B200,
through the C ABI.

Tolerances: log-sum-exp within 1e-12 relative (both sides sum exp() of the same doubles, in a
different order); fp32 log-probabilities within one unit in the last place of the difference
(1e-6 absolute here); drawn tokens identical for every coin that is not within 1e-12 of a boundary
of the cumulative distribution (such coins are reported, none occur with these seeds).
"""
import numpy as np
import pytest

import oracle_py

pytestmark = pytest.mark.gpu


def _cdf_margin(row, lse, coin):
    c = np.cumsum(np.exp(row.astype(np.float64) - lse))
    return np.abs(c - coin).min()


@pytest.mark.parametrize("V,P,sigma", [(17, 32, 1.0), (4099, 4100, 2.0), (50257, 50304, 3.0), (131072, 131072, 2.0)])
def test_sampling_and_logp_match_the_host_restatement(V, P, sigma):
    import torch
    from grpo_cpp_b200 import device as D
    port = oracle_py.load("port")
    rng = np.random.default_rng(V)
    n_rows, n_sel = 24, 9
    x = np.zeros((n_rows, P), np.float32)
    x[:, :V] = rng.normal(0, sigma, (n_rows, V)).astype(np.float32)
    x[:, V:] = 1e30  # padding columns must never be read
    x[3, :V] = -7.5  # a flat row
    x[5, 11 % V] += 25.0  # a peaked row
    rows = np.array([0, 3, 5, 23, 7, 7, 12, 1, 22], np.int32)
    coins = rng.random(n_sel)
    coins[1] = 0.999999999  # far tail of the flat row
    dev = torch.from_numpy(x).cuda()
    tok, logp, lse = D.sample_rows(dev, V, torch.from_numpy(rows).cuda(), coins=torch.from_numpy(coins).cuda())
    tok, logp, lse = tok.cpu().numpy(), logp.cpu().numpy(), lse.cpu().numpy()
    for i, r in enumerate(rows):
        want_lse = port.row_logsumexp(x[r, :V])
        assert abs(lse[i] - want_lse) <= 1e-12 * max(1.0, abs(want_lse))
        assert _cdf_margin(x[r, :V], want_lse, coins[i]) > 1e-12, "coin too close to a boundary to compare"
        want_tok = port.sample_row(x[r, :V], coins[i])
        assert tok[i] == want_tok
        want_lp = np.float32(np.float64(x[r, want_tok]) - want_lse)
        assert abs(logp[i] - want_lp) <= 1e-6
    # the same tokens under another model's logits (the frozen reference model in the demo)
    y = x.copy()
    y[:, :V] += rng.normal(0, 0.1, (n_rows, V)).astype(np.float32)
    tok2, logp2, lse2 = D.sample_rows(torch.from_numpy(y).cuda(), V, torch.from_numpy(rows).cuda(),
                                      tokens=torch.from_numpy(tok).cuda())
    for i, r in enumerate(rows):
        want_lse = port.row_logsumexp(y[r, :V])
        assert abs(lse2.cpu().numpy()[i] - want_lse) <= 1e-12 * max(1.0, abs(want_lse))
        assert abs(logp2.cpu().numpy()[i] - np.float32(np.float64(y[r, tok[i]]) - want_lse)) <= 1e-6


def test_sampling_rejects_bad_rows_and_arguments():
    import torch
    from grpo_cpp_b200 import device as D, _lib
    x = torch.zeros(4, 8, device="cuda")
    rows = torch.tensor([0, 9, -1], dtype=torch.int32, device="cuda")
    tok, logp, lse = D.sample_rows(x, 8, rows, coins=torch.tensor([0.55, 0.5, 0.5], dtype=torch.float64, device="cuda"))
    assert tok.cpu().tolist() == [4, -1, -1]
    assert np.isnan(lse.cpu().numpy()[1:]).all() and abs(lse.cpu().numpy()[0] - np.log(8.0)) < 1e-15
    with pytest.raises(RuntimeError, match="pass either coins or given_tokens"):
        _lib.check(_lib.lib().grpo_b200_sample_rows(x.data_ptr(), 4, 8, 8, rows.data_ptr(), 3, None, None, None, None,
                                                    None, None))
    with pytest.raises(RuntimeError, match="P must be at least V"):
        _lib.check(_lib.lib().grpo_b200_sample_rows(x.data_ptr(), 4, 9, 8, rows.data_ptr(), 3, rows.data_ptr(), None,
                                                    rows.data_ptr(), None, None, None))


def test_sampling_avoids_the_host_copy():
    """What the call is for: S rows of a GPT-2-sized batch sampled on the device and 3*S numbers
    copied out, against copying all N*P logits to the host first (apps/04_gpt2_grpo.cu:82-90).
    Reports both times; asserts only that the device path is the faster one."""
    import time
    import torch
    from grpo_cpp_b200 import device as D
    N, V, P, S = 4096, 50257, 50304, 64
    x = torch.randn(N, P, device="cuda")
    rows = torch.arange(0, N, N // S, dtype=torch.int32, device="cuda")
    coins = torch.rand(S, dtype=torch.float64, device="cuda")
    host = torch.empty(N, P, pin_memory=True)
    for _ in range(2):
        tok, logp, lse = D.sample_rows(x, V, rows, coins=coins)
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok, logp, lse = D.sample_rows(x, V, rows, coins=coins)
    out = (tok.cpu(), logp.cpu(), lse.cpu())
    t_dev = time.perf_counter() - t0
    t0 = time.perf_counter()
    host.copy_(x)
    torch.cuda.synchronize()
    t_copy = time.perf_counter() - t0
    print(f"\nsample {S} of {N} rows on the device: {t_dev * 1e3:.3f} ms; copying the {N * P * 4 / 1e6:.0f} MB of "
          f"logits to pinned host memory alone: {t_copy * 1e3:.1f} ms")
    assert t_dev < t_copy


def test_sampling_against_committed_vectors():
    import torch
    from conftest import Golden
    from grpo_cpp_b200 import device as D
    g = Golden("sampling_cases.npz")
    for name in g.cases:
        c = g.case(name)
        x = np.ascontiguousarray(c["logits"])
        n, V = x.shape
        tok, logp, lse = D.sample_rows(torch.from_numpy(x).cuda(), V, torch.arange(n, dtype=torch.int32, device="cuda"),
                                       coins=torch.from_numpy(c["coins"]).cuda())
        assert (tok.cpu().numpy() == c["tokens"]).all()
        assert np.abs(lse.cpu().numpy() - c["lse"]).max() <= 1e-12 * np.maximum(1.0, np.abs(c["lse"])).max()
        assert np.abs(logp.cpu().numpy() - c["logp"]).max() <= 1e-6
