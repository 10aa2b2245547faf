"""Two ranks on two GPUs: the token-sharded pass whose exchange the reduce kernel does itself over
NVLink peer memory (``ShardedBoundary.step_peer``), checked against one global CPU batch.

Needs two GPUs; skipped on a one-GPU box.  The ranks use the process group for the first pass's
lengths and to trade the 64-byte handles of their exchange regions; after that every data-path byte
moves through the library's own kernel.  Each rank's waits are bounded on the device, and the parent bounds its own wait too.
"""
import os
import socket
import sys
import traceback

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, reduction, alpha, queue):
    try:
        for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
            sys.path.insert(0, p)
        import torch
        import torch.distributed as dist
        import oracle_py
        import grpo_cpp_b200  # noqa: F401
        from grpo_cpp_b200 import workloads as W
        from grpo_cpp_b200.sharded import ShardedBoundary
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        b = W.logits_case(2, 4, 16, 8191, sigma=2.0, min_len=1, reduction=reduction, length_alpha=alpha, seed=5)
        P = 8192
        dev = torch.device("cuda", rank)
        sb = ShardedBoundary(b.S, b.T, b.V, P, clip_eps=b.clip_eps, beta=b.beta, reduction=reduction,
                             length_alpha=alpha, device=dev)
        sl = slice(sb.row_offset, sb.row_offset + sb.n_local)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        old, ref, sel, adv, mask = t(b.logp_old[sl]), t(b.logp_ref[sl]), t(b.selected[sl]), t(b.advantages), t(b.mask[sl])
        sb.prepare(mask)  # the first pass's weights: one collective call, before the exchange exists
        want = oracle_py.load("port").logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask,
                                             b.B, b.G, b.T, b.V, **b.cfg())
        first = sb.weights.clone()
        sb.enable_peer_exchange()
        sb.prepare(mask)  # again, by the library's own exchange: the same global lengths and weights
        assert (sb.weights == first).all()
        assert sb.lengths_f64.cpu().numpy().astype(np.int64).tolist() == b.mask.reshape(b.S, b.T).sum(1).tolist()
        for _ in range(3):
            x = t(b.padded(P)[sl])
            sb.step_peer(x, old, ref, sel, adv, mask)
            got = sb.stats()
            w3 = np.asarray(want[0], np.float64)
            g3 = np.array([got["loss"], got["pg_loss"], got["kl"]])
            assert got["valid_tokens"] == want[1], (got, want[1])
            assert (np.abs(g3 - w3) <= 1e-5 * np.abs(w3) + 1e-9).all(), (g3, w3)
            out = x.cpu().numpy()
            err = np.abs(out[:, : b.V] - want[2][sl])
            assert (err <= 1e-5 * np.abs(want[2][sl]) + 1e-7).all(), err.max()
            assert (out[:, b.V:] == 0).all()
        dist.barrier()
        sb.exchange.close()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("reduction,alpha", [(1, 0.0), (2, 0.5)])
def test_two_gpus_exchange_through_the_reduce_kernel(reduction, alpha):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, reduction, alpha, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(r for r, _ in results) == [0, 1]
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
