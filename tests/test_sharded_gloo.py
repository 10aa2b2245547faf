"""World-size-2 run of the token-sharded rank logic over the gloo backend (CPU).

The kernels cannot run here, so the per-row arithmetic comes from ``tests/cpu_ops.py`` (the CPU
oracle, one row at a time); what is under test is the product's rank logic in
``grpo_cpp_b200/sharded.py``: contiguous row ranges that cut through a response, the all-reduce of
partial lengths into global weights, the all-reduce of the result record, and the reference's error
contract evaluated on GLOBAL quantities.  Expected values come from one global CPU batch, the way
the reference validates its two-GPU demo (apps/03_two_gpu_train.cu:217-265).
"""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, queue):
    try:
        for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
            sys.path.insert(0, p)
        import cpu_ops
        import oracle_py
        import grpo_cpp_b200  # noqa: F401
        from grpo_cpp_b200 import workloads as W
        from grpo_cpp_b200.sharded import ShardedBoundary, shard_rows
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        reduction, alpha, empty_mode = case[:3]
        fused = len(case) > 3 and case[3]
        peer = fused == "peer"
        b = W.logits_case(2, 3, 5, 33, sigma=2.0, min_len=1, reduction=reduction, length_alpha=alpha, seed=77)
        P = 40
        if empty_mode == "globally_empty":
            b.mask[5:10] = 0  # response 1 has no valid token on any rank
        elif empty_mode == "empty_on_rank1_only":
            # response 3 spans rows 15..19; rank 1 starts at row 15; leave only row 15 valid... it is on
            # rank 1, so instead clear response 2's tail (rows 13,14 on rank 0 / none on rank 1)
            b.mask[10:15] = [1, 0, 0, 0, 0]
        b.selected = np.where(b.mask == 1, np.maximum(b.selected, 0), -1).astype(np.int32)
        sb = ShardedBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=reduction,
                             length_alpha=alpha, ops=cpu_ops)
        off, cnt = shard_rows(b.N, world, rank)
        assert (sb.row_offset, sb.n_local) == (off, cnt)
        sl = slice(off, off + cnt)
        x = torch.from_numpy(b.padded(P)[sl].copy())
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        sb.prepare(t(b.mask[sl]))
        if peer:
            # as below, through the path whose exchange the last kernel of the pass does itself
            sb.enable_peer_exchange()
            sb.prepare(t(b.mask[sl]))  # again, now through the exchange: the same weights
            scratch = x.clone()
            sb.step_peer(scratch, t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages),
                         t(b.mask[sl]))
            sb.step_peer(x, t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages), t(b.mask[sl]))
            assert sb.exchange.passes == 3
        elif fused:
            # two passes over the batch with one collective each: the second pass runs on the weights
            # that rode along with the first pass's result record
            scratch = x.clone()
            sb.step_fused(scratch, t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages),
                          t(b.mask[sl]))
            sb.weights_check = sb.weights.clone()
            sb.step_fused(x, t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages), t(b.mask[sl]))
        else:
            sb.step(x, t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages), t(b.mask[sl]))
        if empty_mode == "globally_empty":
            try:
                sb.stats()
                queue.put((rank, "no error raised"))
            except RuntimeError as e:
                queue.put((rank, "ok" if str(e) == "every sequence needs at least one valid token" else str(e)))
            return
        got = sb.stats()
        want = oracle_py.load("port").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                             b.B, b.G, b.T, b.V, **b.cfg())
        w3 = np.asarray(want[0], np.float64)
        g3 = np.array([got["loss"], got["pg_loss"], got["kl"]])
        assert got["valid_tokens"] == want[1]
        assert (np.abs(g3 - w3) <= 1e-6 * np.abs(w3) + 1e-9).all(), (g3, w3)
        out = x.numpy()
        assert np.abs(out[:, : b.V] - want[2][sl]).max() <= 1e-7
        assert (out[:, b.V:] == 0).all()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("case", [(1, 0.0, None), (2, 0.5, None), (0, 0.0, None), (1, 0.0, None, True),
                                  (2, 0.5, None, True), (1, 0.0, None, "peer"), (2, 1.0, None, "peer"),
                                  (1, 0.0, "empty_on_rank1_only"), (1, 0.0, "globally_empty")])
def test_two_ranks_over_gloo(case):
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(r for r, _ in results) == [0, 1]
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_shard_rows_partition():
    from grpo_cpp_b200.sharded import shard_rows
    for n in (1, 7, 64, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (o0, c0), (o1, _) in zip(spans, spans[1:]):
                assert o0 + c0 == o1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_balanced_shards_cover_and_balance():
    from grpo_cpp_b200 import workloads as W
    from grpo_cpp_b200.sharded import shard_rows_balanced
    rng = np.random.RandomState(0)
    T, S, V, P = 64, 96, 1000, 1024
    mask = W.prefix_mask(rng.randint(8, T + 1, S), T)
    for masked_cost in (1.0, 0.8):  # pure traffic; the default calibrated to the row kernel's times
        cost = np.where(mask != 0, float(V + P), masked_cost * P)
        for world in (1, 2, 3, 8):
            spans = shard_rows_balanced(mask, world, V, P, masked_cost)
            assert spans[0][0] == 0 and sum(c for _, c in spans) == mask.size
            for (o0, c0), (o1, _) in zip(spans, spans[1:]):
                assert o0 + c0 == o1
            work = [cost[o:o + c].sum() for o, c in spans]
            assert max(work) - min(work) <= 2 * (V + P)  # within a row or two of each other
    assert shard_rows_balanced(mask, 8, V, P) == shard_rows_balanced(mask, 8, V, P, 0.8)


def _adv_worker(rank, world, port, queue):
    try:
        for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
            sys.path.insert(0, p)
        import cpu_ops
        import oracle_py
        import grpo_cpp_b200  # noqa: F401
        from grpo_cpp_b200.sharded import global_group_advantages
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        prompts, local_G = 5, 3
        rng = np.random.RandomState(4)
        rewards = (rng.rand(world, prompts, local_G) < 0.5).astype(np.float32)  # [source][prompt][g]
        rewards[:, 2, :] = 1.0  # an all-equal group: advantages exactly zero
        mine, meta = global_group_advantages(torch.from_numpy(rewards[rank].reshape(-1).copy()), prompts, local_G,
                                             ops=cpu_ops)
        global_rewards = rewards.transpose(1, 0, 2).reshape(-1)  # [prompt][source][g], apps/05 layout
        want = oracle_py.load("port").group_advantages(global_rewards, prompts, world * local_G)
        want = np.asarray(want).reshape(prompts, world, local_G)[:, rank, :].reshape(-1)
        assert (mine.numpy() == want).all() and int(meta[0]) == 0
        assert (mine.numpy().reshape(prompts, local_G)[2] == 0).all()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_global_group_advantages_over_gloo():
    """Rewards all-gathered over two ranks, regrouped as the reference's two-GPU demo does, advantages
    of the whole groups, this rank's slice back: equal to the oracle on the global batch."""
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_adv_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
