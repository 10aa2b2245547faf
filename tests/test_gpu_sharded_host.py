"""The host side of token-sharded execution (grpo_b200_shard_* and grpo_b200_logits_sharded_host),
through the C ABI on the B200: one rank on one GPU against the CPU checker; two processes on two
GPUs trading IPC handles; and the C++ face (include/grpo/grpo_loss_sharded.hpp) driven by one host
thread per device, the reference's own pattern (apps/03_two_gpu_train.cu:200-215).

The two-GPU cases are skipped on a one-GPU box.  Every device wait is bounded; the parents bound
their own waits too.
"""
import ctypes as C
import os
import socket
import subprocess
import sys
import traceback

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
THREADS_EXE = os.path.join(ROOT, "tests", "cxx", "build", "sharded_threads")


def test_one_rank_matches_the_cpu_checker_and_the_reference_facing_call():
    import torch
    import oracle_py
    import grpo_cpp_b200 as G
    from grpo_cpp_b200 import workloads as W
    from grpo_cpp_b200.api import ShardedLogits
    for reduction, alpha in ((W.TOKEN_MEAN, 0.0), (W.LENGTH_WEIGHTED, 0.5), (W.SEQUENCE_MEAN, 0.0)):
        b = W.logits_case(2, 4, 16, 8191, sigma=2.0, min_len=1, reduction=reduction, length_alpha=alpha, seed=71)
        P = 8192
        want = oracle_py.load("best").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                             b.B, b.G, b.T, b.V, **b.cfg())
        cfg = G.LossConfig(b.clip_eps, b.beta, G.ReductionMode(reduction), alpha)
        shard = ShardedLogits(0, 1, b.B, b.G, b.T, b.V, P, 0, b.N)
        try:
            for _ in range(2):  # twice: the region's pass counter and buffers are reused
                x = torch.from_numpy(b.padded(P)).cuda()
                st = shard.run(x, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, cfg)
                got = np.array([st.loss, st.pg_loss, st.kl])
                assert st.valid_tokens == want[1]
                assert (np.abs(got - want[0]) <= 1e-5 * np.abs(want[0]) + 1e-9).all()
                out = x.cpu().numpy()
                assert (np.abs(out[:, : b.V] - want[2]) <= 1e-7 + 1e-5 * np.abs(want[2])).all()
                assert (out[:, b.V:] == 0).all() and (out[b.mask == 0] == 0).all()
            x = torch.from_numpy(b.padded(P)).cuda()
            st2 = G.grpo_logits_cuda_device_inplace(x, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                                    b.B, b.G, b.T, b.V, P, cfg)
            assert (st2.loss, st2.pg_loss, st2.kl, st2.valid_tokens) == (st.loss, st.pg_loss, st.kl, st.valid_tokens)
            assert (x.cpu().numpy().view(np.uint32) == out.view(np.uint32)).all()
            # the reference's error contract, same texts
            bad_mask = b.mask.copy()
            bad_mask[: b.T] = 0
            with pytest.raises(RuntimeError, match="every sequence needs at least one valid token"):
                shard.run(torch.from_numpy(b.padded(P)).cuda(), b.logp_old, b.logp_ref,
                          np.where(bad_mask == 1, b.selected, -1), b.advantages, bad_mask, cfg)
            with pytest.raises(RuntimeError, match="selected token is outside the vocabulary"):
                sel = b.selected.copy()
                sel[int(np.flatnonzero(b.mask == 1)[0])] = b.V
                shard.run(x, b.logp_old, b.logp_ref, sel, b.advantages, b.mask, cfg)
            # several things wrong at once: the complaint that comes first in the reference's order
            m2, r2 = b.mask.copy(), b.logp_ref.copy()
            m2[2], r2[9] = 5, np.inf
            with pytest.raises(RuntimeError, match="mask values must be 0 or 1"):
                shard.run(x, b.logp_old, r2, b.selected, b.advantages, m2, cfg)
            m2, r2 = b.mask.copy(), b.logp_ref.copy()
            m2[9], r2[2] = 5, np.inf
            with pytest.raises(RuntimeError, match="log probabilities must be finite"):
                shard.run(x, b.logp_old, r2, b.selected, b.advantages, m2, cfg)
            a2 = b.advantages.copy()
            a2[1] = np.nan
            with pytest.raises(RuntimeError, match="advantages must be finite"):
                shard.run(x, b.logp_old, b.logp_ref, sel, a2, b.mask, cfg)
            assert (x.cpu().numpy().view(np.uint32) == out.view(np.uint32)).all(), "rejected calls leave the logits alone"
            with pytest.raises(RuntimeError, match="logp_old has size 3, expected"):
                shard.run(x, b.logp_old[:3], b.logp_ref, b.selected, b.advantages, b.mask, cfg)
            with pytest.raises(RuntimeError, match="logits_and_dlogits must not be null"):
                shard.run(None, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, cfg)
        finally:
            shard.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, queue):
    try:
        for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
            sys.path.insert(0, p)
        import torch
        import torch.distributed as dist
        import oracle_py
        import grpo_cpp_b200 as G
        from grpo_cpp_b200 import workloads as W
        from grpo_cpp_b200.api import ShardedLogits
        from grpo_cpp_b200.sharded import shard_rows
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        b = W.logits_case(2, 4, 16, 8191, sigma=2.0, min_len=1, reduction=W.TOKEN_MEAN, seed=72)
        P = 8192
        off, cnt = shard_rows(b.N, world, rank)
        sl = slice(off, off + cnt)
        want = oracle_py.load("port").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                             b.B, b.G, b.T, b.V, **b.cfg())
        shard = ShardedLogits(rank, world, b.B, b.G, b.T, b.V, P, off, cnt)
        handles = [None] * world
        dist.all_gather_object(handles, shard.handle())
        shard.connect_ipc(handles)
        cfg = G.LossConfig(b.clip_eps, b.beta, G.ReductionMode(b.reduction), 0.0)
        records = []
        for _ in range(3):
            dist.barrier()  # the ranks line up on the host before each call
            x = torch.from_numpy(b.padded(P)[sl]).cuda()
            st = shard.run(x, b.logp_old[sl], b.logp_ref[sl], b.selected[sl], b.advantages, b.mask[sl], cfg)
            got = np.array([st.loss, st.pg_loss, st.kl])
            assert st.valid_tokens == want[1]
            assert (np.abs(got - want[0]) <= 1e-5 * np.abs(want[0]) + 1e-9).all(), (got, want[0])
            out = x.cpu().numpy()
            assert (np.abs(out[:, : b.V] - want[2][sl]) <= 1e-7 + 1e-5 * np.abs(want[2][sl])).all()
            assert (out[:, b.V:] == 0).all()
            records.append((st.loss, st.pg_loss, st.kl, st.valid_tokens))
        everyone = [None] * world
        dist.all_gather_object(everyone, records)
        assert all(r == everyone[0] for r in everyone), "the ranks' statistics differ"
        dist.barrier()
        shard.close()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_processes_on_two_gpus_through_ipc_handles():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


@pytest.mark.parametrize("world", [1, 2])
def test_cxx_face_with_one_host_thread_per_device(world):
    """tests/cxx/sharded_threads.cu (built by __graft_entry__.build): std::threads, one per device, each
    constructing a grpo::ShardedLogitsBoundary, connecting through peer access, and calling run() --
    statistics identical on every rank and equal to the single-device call, gradient within tolerance,
    and the reference's exception when a response has no valid token."""
    import torch
    if not os.path.exists(THREADS_EXE):
        pytest.fail("tests/cxx/build/sharded_threads is missing: run __graft_entry__.build()")
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run = subprocess.run([THREADS_EXE, str(world)], capture_output=True, text=True, timeout=240)
    print(run.stdout)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all ok" in run.stdout
