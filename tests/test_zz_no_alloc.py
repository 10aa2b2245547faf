"""The allocation-free selected-token entry point against the ordinary one -- runs on the B200.

``grpo_b200_loss_noalloc`` serves callers that cannot allocate device memory and have none to
spare (all of it handed out at start-up, or allocation would stall or is forbidden where they
run): it keeps its partial sums in an array the library owns.  The test drives it through the C
ABI on two different batches in a row -- so that anything left in the shared array by the first
call would show in the second -- and requires the same bits as ``grpo_b200_loss`` on the same
inputs.  It also checks the size limit's error.  The file is named to be collected last.
"""
import numpy as np
import pytest

from grpo_cpp_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _run_both(batch, dev):
    import torch
    from grpo_cpp_b200 import device as D
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    new, old, ref, adv, mask = t(batch.logp_new), t(batch.logp_old), t(batch.logp_ref), t(batch.advantages), t(batch.mask)
    lengths = D.count_lengths(mask, batch.S, batch.T)
    weights, _ = D.weights_from_lengths(lengths, batch.reduction, batch.length_alpha)
    want_g, want_r = D.loss(new, old, ref, adv, weights, mask, batch.T, batch.clip_eps, batch.beta)
    got_g = torch.full((batch.N,), float("nan"), device=dev)
    got_r = torch.full((5,), float("nan"), dtype=torch.float64, device=dev)
    D.loss_noalloc(new, old, ref, adv, weights, mask, batch.T, batch.clip_eps, batch.beta, dlogp=got_g, result=got_r)
    torch.cuda.synchronize()
    return want_g.cpu().numpy(), want_r.cpu().numpy(), got_g.cpu().numpy(), got_r.cpu().numpy()


def test_noalloc_matches_workspace_entry_point_twice():
    import torch
    dev = torch.device("cuda")
    first = W.selected_token_case(512, 300, ragged=True, seed=11)          # 153,600 tokens, many blocks
    second = W.selected_token_case(24, 37, ragged=True, seed=12, reduction=W.LENGTH_WEIGHTED, length_alpha=0.5)
    for batch in (first, second):  # the second, smaller call must not see the first call's partials
        want_g, want_r, got_g, got_r = _run_both(batch, dev)
        assert (got_g.view(np.uint32) == want_g.view(np.uint32)).all()
        assert (got_r.view(np.uint64) == want_r.view(np.uint64)).all()
        assert np.isfinite(got_r).all() and got_r[3] == 0 and got_r[4] == 0


def test_noalloc_scalar_branch_and_capped_grid():
    """Unaligned slices (the kernel's one-token-at-a-time branch), token counts that leave one to
    three tokens past the last group of four, and a batch large enough that the grid is capped
    (above 2M tokens): the same bits as the workspace entry point every time, and the oracle's sums
    within the path's tolerance on the large batch."""
    import torch
    import oracle_py
    from grpo_cpp_b200 import device as D
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    base = W.selected_token_case(8, 131, ragged=True, seed=13)
    new, old, ref, adv, mask = t(base.logp_new), t(base.logp_old), t(base.logp_ref), t(base.advantages), t(base.mask)
    weights, _ = D.weights_from_lengths(D.count_lengths(mask, base.S, base.T), base.reduction, 0.0)
    for first, count in ((1, 1001), (3, 1002), (2, 1003), (0, 1047), (5, 7)):
        sl = slice(first, first + count)  # element offsets 1, 2, 3, 5 break the 16-byte alignment
        args = (new[sl], old[sl], ref[sl], adv, weights, mask[sl], base.T, base.clip_eps, base.beta)
        want_g, want_r = D.loss(*args, token_offset=first)
        got_g = torch.full((count,), float("nan"), device=dev)
        got_r = torch.full((5,), float("nan"), dtype=torch.float64, device=dev)
        D.loss_noalloc(*args, dlogp=got_g, result=got_r, token_offset=first)
        torch.cuda.synchronize()
        assert (got_g.cpu().numpy().view(np.uint32) == want_g.cpu().numpy().view(np.uint32)).all()
        assert (got_r.cpu().numpy().view(np.uint64) == want_r.cpu().numpy().view(np.uint64)).all()
    big = W.selected_token_case(4096, 640, ragged=True, seed=14)  # 2,621,440 tokens: the grid is at its cap
    want_g, want_r, got_g, got_r = _run_both(big, dev)
    assert (got_g.view(np.uint32) == want_g.view(np.uint32)).all()
    assert (got_r.view(np.uint64) == want_r.view(np.uint64)).all()
    ws, wv, wg = oracle_py.load("best").loss(big.logp_new, big.logp_old, big.logp_ref, big.advantages, big.mask,
                                            big.B, big.G, big.T, **big.cfg())
    assert (np.abs(got_r[:3] - ws) <= 1e-5 * np.abs(ws) + 1e-9).all()
    assert (np.abs(got_g - wg) <= 1e-7 + 1e-5 * np.abs(wg)).all()


def test_noalloc_refuses_oversized_calls():
    import torch
    from grpo_cpp_b200 import _lib
    dummy = torch.zeros(8, device="cuda")
    imask = torch.ones(8, dtype=torch.int32, device="cuda")
    res = torch.zeros(5, dtype=torch.float64, device="cuda")
    rc = _lib.lib().grpo_b200_loss_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                           dummy.data_ptr(), imask.data_ptr(), (1 << 24) + 1, 0, 8, 0.2, 0.0,
                                           dummy.data_ptr(), res.data_ptr(), None)
    assert rc == _lib.E_INVALID
    assert "at most 16777216 tokens" in _lib.last_error()
