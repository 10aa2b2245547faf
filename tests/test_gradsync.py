"""Gradient all-reduce fused with the 1/world scale (grpo_b200_allreduce_scale): the slice arithmetic on
CPU (alone and as a two-rank reduce-scatter / all-gather over gloo), and the kernel itself on the B200 --
one rank on one GPU, two ranks on two -- against the host sum in rank order times the scale, bit for bit.
"""
import os
import socket
import sys
import traceback

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def expected(buffers, scale):
    """The reference's arithmetic (apps/05_two_gpu_gpt2_grpo.cu:260-268) with the order fixed: fp32 sum of
    the ranks' buffers in rank order, then one fp32 multiply."""
    acc = buffers[0].astype(np.float32).copy()
    for b in buffers[1:]:
        acc = (acc + b.astype(np.float32)).astype(np.float32)
    return (acc * np.float32(scale)).astype(np.float32)


@pytest.mark.parametrize("n", [1, 3, 4, 5, 31, 1024, 124439808, 1000003])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_slices_partition_the_buffer_in_whole_float4s(n, world):
    from grpo_cpp_b200 import device as D
    at = 0
    for r in range(world):
        first, count = D.gradsync_slice(n, world, r)
        assert first == at and count >= 0
        assert first % 4 == 0 and (count % 4 == 0 or r == world - 1)
        at += count
    assert at == n


def _gloo_rank(rank, world, port, n, queue):
    try:
        sys.path.insert(0, ROOT)
        import torch
        import torch.distributed as dist
        import grpo_cpp_b200  # noqa: F401
        from grpo_cpp_b200 import device as D
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        bufs = [np.random.default_rng(100 + r).standard_normal(n).astype(np.float32) for r in range(world)]
        mine = torch.from_numpy(bufs[rank].copy())
        # what the kernel does, with gloo standing in for the peer loads and stores: every rank gathers
        # slice r of all buffers to rank r, rank r adds them in rank order and scales, everyone gets slice r back
        out = torch.empty_like(mine)
        for r in range(world):
            first, count = D.gradsync_slice(n, world, r)
            piece = mine[first:first + count].contiguous()
            gathered = [torch.empty_like(piece) for _ in range(world)] if rank == r else None
            dist.gather(piece, gathered, dst=r)
            if rank == r:
                acc = gathered[0].clone()
                for g in gathered[1:]:
                    acc += g
                acc *= np.float32(1.0 / world)
            else:
                acc = torch.empty_like(piece)
            dist.broadcast(acc, src=r)
            out[first:first + count] = acc
        want = expected(bufs, 1.0 / world)
        assert (out.numpy().view(np.uint32) == want.view(np.uint32)).all()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(target, world, *args):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, *args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_slice_arithmetic_as_a_two_rank_exchange_over_gloo():
    _spawn(_gloo_rank, 2, 1003)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [8, 1003, 1 << 20])
def test_one_rank_scales_in_place(n):
    import torch
    from grpo_cpp_b200 import device as D
    host = np.random.default_rng(n).standard_normal(n).astype(np.float32)
    whole = torch.zeros(n + 8, device="cuda")
    g = whole[4:4 + n]  # inside a larger allocation, 16-byte aligned
    g.copy_(torch.from_numpy(host))
    sync = D.GradSync(g, 0, 1)
    try:
        sync.connect([sync.handle])
        for k in range(3):
            sync.allreduce_scale(0.5)
            host = (host * np.float32(0.5)).astype(np.float32)
            torch.cuda.synchronize()
            assert (g.cpu().numpy().view(np.uint32) == host.view(np.uint32)).all()
        assert not sync.timed_out()
        assert whole[:4].abs().sum().item() == 0 and whole[4 + n:].abs().sum().item() == 0
    finally:
        sync.close()


def _gpu_rank(rank, world, port, n, queue):
    try:
        sys.path.insert(0, ROOT)
        import torch
        import torch.distributed as dist
        import grpo_cpp_b200  # noqa: F401
        from grpo_cpp_b200 import device as D
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        sync = None
        for step in range(3):
            bufs = [np.random.default_rng(1000 * step + r).standard_normal(n).astype(np.float32) for r in range(world)]
            if sync is None:
                g = torch.empty(n, device="cuda")
                sync = D.GradSync(g, rank, world)
                handles = [None] * world
                dist.all_gather_object(handles, sync.handle)
                sync.connect(handles)
            g.copy_(torch.from_numpy(bufs[rank]))
            torch.cuda.synchronize()
            dist.barrier()
            sync.allreduce_scale(1.0 / world)
            torch.cuda.synchronize()
            want = expected(bufs, 1.0 / world)
            assert (g.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all(), f"step {step}"
        assert not sync.timed_out()
        dist.barrier()
        sync.close()
        queue.put((rank, "ok"))
    except Exception:
        queue.put((rank, traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1003, 5_000_001])
def test_two_ranks_on_two_gpus_agree_with_the_host_sum_bit_for_bit(n):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _spawn(_gpu_rank, 2, n)
