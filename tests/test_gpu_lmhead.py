"""The LM-head projection fused with the loss statistics (grpo_b200_lmhead_loss: tcgen05 tensor cores,
TF32 inputs, fp32 accumulation; the logits are never written) -- runs on the B200, through the C ABI.

Checker: the inputs are rounded to TF32 on the host (low 13 mantissa bits cleared), so the tensor
cores' own rounding of the inputs is a no-op and every product is exact; the host forms the logits of
the checked rows in float64 and feeds their float64 log-softmax, rounded to fp32 as the reference
rounds it, to the CPU checker's token loss.  What remains is the order of the fp32 accumulation over
the 768 products of a logit and the fp32 running sum of exponentials.  The tensor cores truncate
when they accumulate, so a logit of magnitude ~10 comes out up to ~2e-5 towards zero and the row
log-sum-exp reads 1e-5 to 2.5e-5 low at C = 768 (measured; far less at small C) -- the same holds for
any tensor-core matmul of this precision.  Tolerances, written below: row log-sum-exp and
log p(selected) within 5e-5 absolute; the three loss sums within 1e-4 relative (measured: 2e-5).
"""
import numpy as np
import pytest

import oracle_py
from grpo_cpp_b200 import workloads as W

pytestmark = pytest.mark.gpu


def to_tf32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def make_case(n_seq, T, C, V, P, seed, min_len=1):
    rng = np.random.default_rng(seed)
    N = n_seq * T
    hidden = to_tf32(rng.standard_normal((N, C)).astype(np.float32))
    lm_head = to_tf32((rng.standard_normal((P, C)) * (3.0 / np.sqrt(C))).astype(np.float32))
    lm_head[V:] = 1e4  # rows beyond the vocabulary must never matter
    lengths = rng.integers(min_len, T + 1, n_seq)
    mask = W.prefix_mask(lengths, T)
    sel = np.where(mask == 1, rng.integers(0, V, N), -1).astype(np.int32)
    adv = W.group_advantages_np((rng.random(n_seq) < 0.5).astype(np.float32), n_seq // 2, 2)
    return hidden, lm_head, mask, sel, adv, rng


def host_rows(hidden, lm_head, V, rows):
    x = hidden[rows].astype(np.float64) @ lm_head[:V].astype(np.float64).T
    top = x.max(axis=1)
    lse = top + np.log(np.exp(x - top[:, None]).sum(axis=1))
    return x, lse


@pytest.mark.parametrize("n_seq,T,C,V,P", [(4, 32, 64, 1000, 1024), (6, 50, 768, 50257, 50304), (2, 64, 128, 300, 512)])
def test_fused_projection_matches_the_host_in_float64(n_seq, T, C, V, P):
    import torch
    from grpo_cpp_b200 import device as D
    hidden, lm_head, mask, sel, adv, rng = make_case(n_seq, T, C, V, P, seed=V + C)
    N = n_seq * T
    x, lse = host_rows(hidden, lm_head, V, np.arange(N))
    now = np.where(mask == 1, (x[np.arange(N), np.maximum(sel, 0)] - lse), 0.0).astype(np.float32)
    old = np.where(mask == 1, now + 0.05 * rng.standard_normal(N), 0).astype(np.float32)
    ref = np.where(mask == 1, now + 0.05 * rng.standard_normal(N), 0).astype(np.float32)
    want = oracle_py.load("best").loss(now, old, ref, adv, mask, n_seq // 2, 2, T, clip_eps=0.2, beta=0.01,
                                       reduction=W.TOKEN_MEAN)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    mask_d = t(mask)
    weights, meta = D.weights_from_lengths(D.count_lengths(mask_d, n_seq, T), W.TOKEN_MEAN, 0.0)
    res, lp, got_lse = D.lmhead_loss(t(hidden), t(lm_head), V, t(old), t(ref), t(sel), t(adv), weights, mask_d, T, 0.2, 0.01,
                                     want_selected_logp=True, want_lse=True)
    rec = res.cpu().numpy()
    assert rec[3] == 0 and rec[4] == 0, rec
    active = mask == 1
    assert np.abs(got_lse.cpu().numpy()[active] - lse[active]).max() <= 5e-5
    assert np.abs(lp.cpu().numpy()[active] - now[active]).max() <= 5e-5
    assert (lp.cpu().numpy()[~active] == 0).all()
    assert (np.abs(rec[:3] - want[0]) <= 1e-4 * np.abs(want[0]) + 1e-7).all(), (rec[:3], want[0])
    assert meta.cpu().tolist()[0] == want[1]


def test_fused_projection_against_the_materialised_path_at_gpt2_size():
    """4,096 rows x V = 50,257 x C = 768: the same batch through (a) an fp32 matmul that writes the 824 MB
    of logits followed by the fused logits kernel, and (b) the fused projection, which writes none; the
    three sums agree within 1e-4 relative, log p(selected) within 5e-5, and 64 rows are checked against
    the host in float64."""
    import torch
    from grpo_cpp_b200 import device as D
    n_seq, T, C, V, P = 16, 256, 768, 50257, 50304
    hidden, lm_head, mask, sel, adv, rng = make_case(n_seq, T, C, V, P, seed=5, min_len=32)
    N = n_seq * T
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    h_d, w_d, mask_d, sel_d, adv_d = t(hidden), t(lm_head), t(mask), t(sel), t(adv)
    weights, _ = D.weights_from_lengths(D.count_lengths(mask_d, n_seq, T), W.TOKEN_MEAN, 0.0)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        logits = h_d @ w_d.T  # exact products (the inputs are TF32-representable), fp32 accumulation
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    active_rows = torch.from_numpy(np.flatnonzero(mask == 1).astype(np.int32)).cuda()
    _, lp_rows, _ = D.sample_rows(logits, V, active_rows, tokens=sel_d[active_rows.long()])
    now = torch.zeros(N, device="cuda")
    now[active_rows.long()] = lp_rows
    noise = lambda: torch.from_numpy((0.05 * rng.standard_normal(N)).astype(np.float32)).cuda()
    old = torch.where(mask_d == 1, now + noise(), torch.zeros_like(now))
    ref = torch.where(mask_d == 1, now + noise(), torch.zeros_like(now))
    lp_a = torch.empty(N, device="cuda")
    rec_a = D.logits(logits, old, ref, sel_d, adv_d, weights, mask_d, T, V, 0.2, 0.01, selected_logp=lp_a).cpu().numpy()
    res, lp_b, lse_b = D.lmhead_loss(h_d, w_d, V, old, ref, sel_d, adv_d, weights, mask_d, T, 0.2, 0.01,
                                     want_selected_logp=True, want_lse=True)
    rec_b = res.cpu().numpy()
    assert rec_b[3] == 0 and rec_b[4] == 0
    assert (np.abs(rec_b[:3] - rec_a[:3]) <= 1e-4 * np.abs(rec_a[:3]) + 1e-7).all(), (rec_b, rec_a)
    assert (lp_a - lp_b).abs().max().item() <= 5e-5
    rows = np.flatnonzero(mask == 1)[:: max(1, int(mask.sum()) // 64)][:64]
    x, lse = host_rows(hidden, lm_head, V, rows)
    assert np.abs(lse_b.cpu().numpy()[rows] - lse).max() <= 5e-5
    assert np.abs(lp_b.cpu().numpy()[rows] - (x[np.arange(rows.size), sel[rows]] - lse)).max() <= 5e-5


def test_fused_projection_rejects_bad_arguments():
    import torch
    from grpo_cpp_b200 import device as D
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 32"):
        D.lmhead_loss(z(8, 40), z(64, 40), 60, z(8), z(8), z(8, dt=torch.int32), z(1), z(1), z(8, dt=torch.int32), 8, 0.2, 0.0)
    with pytest.raises(RuntimeError, match="P must be at least V"):
        D.lmhead_loss(z(8, 64), z(64, 64), 65, z(8), z(8), z(8, dt=torch.int32), z(1), z(1), z(8, dt=torch.int32), 8, 0.2, 0.0)
