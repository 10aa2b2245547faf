"""Contracts around the kernels, on the B200 through the C ABI: bounded waits that are made to run
out, a row order that does not belong to the mask, concurrent host threads, the synthetic-logits
generator against its host restatement, and the size check of the exchange regions.

Nothing here faults or hangs the device: the one wait that is made to run out polls memory of its
own device with a limit of about a millisecond and returns a status record.
"""
import threading

import numpy as np
import pytest

import oracle_py
import grpo_cpp_b200 as G
from grpo_cpp_b200 import workloads as W
from test_gpu_token_path import assert_grad, assert_stats, cfg_of

pytestmark = pytest.mark.gpu


def test_exchange_wait_runs_out_and_reports_instead_of_hanging():
    """World of two with nobody playing rank 1: both regions live on this device, rank 0 pushes its
    counts into both and polls its own region for rank 1's words, which never come.  With the limit
    set to ~2 million SM cycles (about a millisecond) the kernel gives up, writes bad_inputs = -2
    into the caller-visible status record, and the host raises -- for the lengths exchange of
    prepare() and for a full pass alike.  The context stays usable afterwards."""
    import torch
    from grpo_cpp_b200 import device as D
    from grpo_cpp_b200.sharded import ShardedBoundary
    b = W.logits_case(2, 2, 8, 4099, sigma=2.0, min_len=1, reduction=W.TOKEN_MEAN, seed=41)
    P = 4100
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
    sb = ShardedBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=b.reduction, device=dev)
    mine = D.PeerExchange(b.S, 0, 2)
    silent = D.PeerExchange(b.S, 1, 2)  # a region nobody ever writes a pass into
    mine.regions[1] = silent.own
    sb.exchange = mine
    D.set_exchange_timeout_cycles(2_000_000)
    try:
        sb.prepare(mask)
        torch.cuda.synchronize()
        assert sb.prepare_status.cpu().tolist()[4] == -2.0
        with pytest.raises(RuntimeError, match="the exchange between ranks timed out"):
            sb.stats()
        sb.prepare_status.zero_()
        x = t(b.padded(P))
        sb.step_peer(x, old, ref, sel, adv, mask)
        torch.cuda.synchronize()
        assert sb.result.cpu().tolist()[4] == -2.0
        with pytest.raises(RuntimeError, match="the exchange between ranks timed out"):
            sb.stats()
    finally:
        D.set_exchange_timeout_cycles(1 << 32)
        torch.cuda.synchronize()
        mine.close()
        silent.close()
    # the device still answers and a plain pass is still right
    want = oracle_py.load("best").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                         b.B, b.G, b.T, b.V, **b.cfg())
    dev_logits = t(b.padded(P))
    st = G.grpo_logits_cuda_device_inplace(dev_logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                           b.B, b.G, b.T, b.V, P, cfg_of(b))
    assert_stats(st, want[0], want[1], "after the timed-out exchange")


def test_sharded_calls_reject_a_response_count_the_region_was_not_made_for():
    import torch
    from grpo_cpp_b200 import device as D, _lib
    dev = torch.device("cuda")
    ex = D.PeerExchange(4, 0, 1)
    try:
        mask = torch.ones(16, dtype=torch.int32, device=dev)
        w = torch.zeros(8, device=dev)
        meta = torch.zeros(2, dtype=torch.int32, device=dev)
        status = torch.zeros(5, dtype=torch.float64, device=dev)
        ws = D.logits_workspace(16, dev)
        with pytest.raises(ValueError, match="created for 4 responses"):
            D.lengths_sharded(mask, 8, 2, 0, exchange=ex, reduction=1, length_alpha=0.0, weights=w, meta=meta,
                              workspace=ws, status=status)
        rc = _lib.lib().grpo_b200_lengths_sharded(mask.data_ptr(), 16, 0, 2, 8, ex.regions, 0, 1, 1, 0.0,
                                                  w.data_ptr(), meta.data_ptr(), None, status.data_ptr(),
                                                  ws.data_ptr(), ws.numel(), None)
        assert rc == _lib.E_INVALID and "created for 4 responses" in _lib.last_error()
        rc = _lib.lib().grpo_b200_lengths_sharded(mask.data_ptr(), 16, 0, 4, 4, ex.regions, 0, 1, 2, 1.5,
                                                  w.data_ptr(), meta.data_ptr(), None, status.data_ptr(),
                                                  ws.data_ptr(), ws.numel(), None)
        assert rc == _lib.E_INVALID and "length_alpha" in _lib.last_error()
    finally:
        ex.close()


def test_row_order_of_another_mask_is_reported_not_obeyed_blindly():
    """A row order made from mask A handed in with mask B: the pass reports bad_inputs = -3 (and the
    host-facing text says so); an order whose counts do not add up is ignored and reported; row
    indices outside the batch are never dereferenced."""
    import torch
    from grpo_cpp_b200 import device as D
    b = W.logits_case(2, 3, 8, 4099, sigma=2.0, min_len=2, reduction=W.TOKEN_MEAN, seed=43)
    P = 4100
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    old, ref, sel, adv, mask = t(b.logp_old), t(b.logp_ref), t(b.selected), t(b.advantages), t(b.mask)
    lengths = D.count_lengths(mask, b.S, b.T)
    weights, _ = D.weights_from_lengths(lengths, b.reduction, 0.0)
    other = b.mask.copy().reshape(b.S, b.T)
    other[:, 1], other[:, -1] = 0, 1  # same count per response, different rows
    wrong = D.row_order(t(other.reshape(-1)))
    res = D.logits(t(b.padded(P)), old, ref, sel, adv, weights, mask, b.T, b.V, b.clip_eps, b.beta, row_order=wrong)
    assert res.cpu().tolist()[4] == -3.0
    short = D.row_order(mask).clone()
    short[0] -= 1  # counts no longer add up to the row count
    x = t(b.padded(P))
    res = D.logits(x, old, ref, sel, adv, weights, mask, b.T, b.V, b.clip_eps, b.beta, row_order=short)
    assert res.cpu().tolist()[4] == -3.0
    want = oracle_py.load("best").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                         b.B, b.G, b.T, b.V, **b.cfg())
    assert_grad(x.cpu().numpy()[:, : b.V], want[2], "ignored order")  # the rows were still processed by mask
    wild = D.row_order(mask).clone()
    wild[2] = 10 ** 9  # an index far outside the batch
    wild[3] = -5
    res = D.logits(t(b.padded(P)), old, ref, sel, adv, weights, mask, b.T, b.V, b.clip_eps, b.beta, row_order=wild)
    torch.cuda.synchronize()
    assert res.cpu().tolist()[4] == -3.0
    # and the right order is accepted
    res = D.logits(t(b.padded(P)), old, ref, sel, adv, weights, mask, b.T, b.V, b.clip_eps, b.beta,
                   row_order=D.row_order(mask))
    assert res.cpu().tolist()[4] == 0.0


def test_concurrent_host_threads_get_the_serial_results():
    """The reference's two-GPU demo calls the library from one host thread per device
    (apps/03_two_gpu_train.cu:200-215).  Here several threads call grpo_logits_cuda and
    grpo_loss_cuda at once -- all on one device, and one per device where two exist -- and every
    result must equal the one the same call gives alone, bit for bit."""
    import torch
    lb = [W.logits_case(2, 2, 6, V, sigma=2.0, min_len=1, reduction=W.TOKEN_MEAN, seed=50 + i)
          for i, V in enumerate((4099, 20000, 40000, 777))]
    tb = [W.selected_token_case(64, 96 + 8 * i, ragged=True, seed=60 + i) for i in range(4)]

    def run_logits(b):
        r = G.grpo_logits_cuda(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T,
                               b.V, cfg_of(b))
        return r.dlogits.copy(), (r.stats.loss, r.stats.pg_loss, r.stats.kl, r.stats.valid_tokens)

    def run_loss(b):
        r = G.grpo_loss_cuda(b.logp_new, b.logp_old, b.logp_ref, b.advantages, b.mask, b.B, b.G, b.T, cfg_of(b))
        return r.dlogp_new.copy(), (r.stats.loss, r.stats.pg_loss, r.stats.kl, r.stats.valid_tokens)

    jobs = [(run_logits, b) for b in lb] + [(run_loss, b) for b in tb]
    serial = [fn(b) for fn, b in jobs]
    n_dev = min(torch.cuda.device_count(), 2)
    for round_ in range(3):
        got = [None] * len(jobs)
        errors = []

        def worker(i):
            try:
                torch.cuda.set_device(i % n_dev)
                fn, b = jobs[i]
                for _ in range(3):
                    got[i] = fn(b)
            except Exception as e:  # pragma: no cover
                errors.append((i, repr(e)))

        threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(jobs))]
        for th in threads:
            th.start()
        for th in threads:
            th.join()
        assert not errors, errors
        for (want_a, want_s), (got_a, got_s) in zip(serial, got):
            assert got_s == want_s
            assert (got_a.view(np.uint32) == want_a.view(np.uint32)).all()
    torch.cuda.set_device(0)


@pytest.mark.parametrize("V,P,rows,offset", [(17, 32, 5, 0), (50257, 50304, 7, 65529), (32768, 32768, 3, 1000)])
def test_synthetic_logits_match_the_host_restatement_bit_for_bit(V, P, rows, offset):
    import torch
    from grpo_cpp_b200 import device as D
    scale = W.synthetic_scale(3.0)
    out = torch.empty(rows, P, device="cuda")
    D.synthetic_logits(out, V, float(scale), 1234, row_offset=offset, tail_fill=-7.0)
    got = out.cpu().numpy()
    want = W.synthetic_logits_rows(np.arange(offset, offset + rows), V, P, scale, 1234)
    assert (got[:, :V].view(np.uint32) == want.view(np.uint32)).all()
    assert (got[:, V:] == -7.0).all()
    # a shard built on its own equals the same rows of the whole
    whole = torch.empty(offset % 7 + rows + 2, P, device="cuda")
    first = offset - offset % 7
    D.synthetic_logits(whole, V, float(scale), 1234, row_offset=first)
    assert (whole[offset - first: offset - first + rows, :V].cpu().numpy() == got[:, :V]).all()


def test_synthetic_logits_have_the_stated_distribution():
    x = W.synthetic_logits_rows(np.arange(64), 50257, 50304, W.synthetic_scale(3.0), 99)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 3.0) < 0.01
    assert 4.0 * 3.0 < float(np.abs(x).max()) <= 4.9 * 3.0


def _message(call):
    try:
        call()
    except RuntimeError as e:
        return str(e)
    return None


def test_in_place_entry_raises_the_complaint_the_ordered_checks_raise():
    """The in-place entry checks its metadata in fused copy-and-check sweeps; whenever several things are
    wrong at once it must still name the complaint that comes first in the reference's order
    (src/cuda/grpo_loss_cuda.cu:584-618, 676-697, 44-46) -- the one the host-vector entry, which walks
    the arrays in that order, raises for the same inputs.  The device logits must stay untouched."""
    import torch
    b = W.logits_case(2, 2, 6, 257, sigma=1.5, min_len=2, seed=73)
    cfg = cfg_of(b)
    clean = b.padded(260)

    def both(**changed):
        args = dict(old=b.logp_old.copy(), ref=b.logp_ref.copy(), sel=b.selected.copy(), adv=b.advantages.copy(),
                    mask=b.mask.copy(), cfg=cfg, kernel=G.CudaLogitsKernel.fused)
        args.update(changed)
        dev = torch.from_numpy(clean.copy()).cuda()
        inplace = _message(lambda: G.grpo_logits_cuda_device_inplace(dev, args["old"], args["ref"], args["sel"], args["adv"],
                                                                     args["mask"], b.B, b.G, b.T, b.V, 260, args["cfg"],
                                                                     args["kernel"]))
        vectors = _message(lambda: G.grpo_logits_cuda(b.logits, args["old"], args["ref"], args["sel"], args["adv"],
                                                      args["mask"], b.B, b.G, b.T, b.V, args["cfg"], args["kernel"]))
        assert inplace == vectors and inplace is not None, (changed.keys(), inplace, vectors)
        assert (dev.cpu().numpy() == clean).all(), "a rejected call must leave the logits as they were"
        return inplace

    def poke(a, i, v):
        a = a.copy()
        a[i] = v
        return a

    active = int(np.flatnonzero(b.mask == 1)[3])
    assert "finite" in both(old=poke(b.logp_old, 5, np.nan))
    assert "mask values" in both(mask=poke(b.mask, 7, 3))
    # a bad mask value early and a non-finite log-probability later, and the other way round
    assert "mask values" in both(mask=poke(b.mask, 2, 5), ref=poke(b.logp_ref, 9, np.inf))
    assert "finite" in both(mask=poke(b.mask, 9, 5), ref=poke(b.logp_ref, 2, np.inf))
    # advantages are looked at after every token, selected ids after the advantages
    assert "advantages" in both(adv=poke(b.advantages, 1, np.nan), sel=poke(b.selected, active, b.V))
    assert "vocabulary" in both(sel=poke(b.selected, active, -3))
    assert "vocabulary" in both(sel=poke(b.selected, active, b.V), kernel=7)
    assert "selector" in both(kernel=7)
    # a response without a valid token is found last
    empty = b.mask.copy()
    empty[: b.T] = 0
    assert "at least one valid token" in both(mask=empty)
    assert "at least one valid token" not in both(mask=empty, old=poke(b.logp_old, 0, np.nan))
