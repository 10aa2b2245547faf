#!/usr/bin/env python
"""Benchmark of the GRPO loss boundary on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload: the GPT-2-shaped loss boundary sharded by token (32 prompts x 8 responses x 256
token slots = 65,536 rows, V = 50,257 padded to P = 50,304 fp32 logits ~ N(0,3), ragged lengths
U[32,256], token-mean reduction with the global normaliser all-reduced), the configuration the
headline metric -- fused loss+dlogits tokens/s and HBM GB/s at 1/2/4/8 GPUs -- is quoted on.  The
65,536 rows are split contiguously over the ranks (total work fixed: strong scaling).

A step is one pass of the hot path over the batch, two launches: the fused logits kernel in place (with
the weights the previous pass left), then the reduce kernel (per-row loss terms in double, fixed-order
totals, the next pass's per-response lengths, the exchange between the ranks through NVLink peer memory,
the next pass's weights).  ``--exchange nccl`` runs the older form instead: lengths kernel, logits
kernel, reduce kernel, ONE all-reduce, weights kernel.  The logits are restored from a pristine copy
and L2 is flushed between passes on the same stream, outside the timed event pairs; the K passes are
bracketed by a barrier and a synchronize, each is timed by a CUDA-event pair on the launching stream,
and the per-rank totals are reduced with MAX.  One JSON line is printed by rank 0.

``--impl reference`` times the reference's own CPU implementation of the same path
(oracle/_ref, the reference's src/cpu/grpo_loss.cpp compiled unmodified; the C restatement when
that is absent) on all host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused GRPO loss+dlogits tokens/s"
UNIT = "tokens/s"
CLIP_EPS, BETA = 0.2, 0.01


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
def workload_spec(name: str) -> dict:
    from grpo_cpp_b200 import workloads as W
    if name == "gpt2":
        s = dict(W.GPT2_SHAPE)
        s.update(reduction=W.TOKEN_MEAN, alpha=0.0, label="gpt2-124M-shaped loss boundary, token-sharded")
        return s
    if name == "gpt2s":  # the same row shape with 1/16 of the rows: small enough for multi-pass ncu captures
        s = dict(W.GPT2_SHAPE)
        s.update(B=2, reduction=W.TOKEN_MEAN, alpha=0.0, label="gpt2-124M-shaped loss boundary, 4096 rows")
        return s
    if name == "v32k":
        return dict(B=2, G=8, T=64, V=32768, P=32768, sigma=2.0, min_len=None, reduction=W.TOKEN_MEAN, alpha=0.0,
                    label="fused logits N=1024 x V=32768, full mask, token-mean")
    if name == "v128k":
        return dict(B=2, G=8, T=64, V=131072, P=131072, sigma=2.0, min_len=16, reduction=W.LENGTH_WEIGHTED,
                    alpha=0.5, label="fused logits N=1024 x V=131072, ragged, L^0.5 weights")
    raise SystemExit(f"unknown workload {name}")


def host_metadata(spec: dict, seed: int = 42):
    """Seeded per-token metadata of the whole batch (identical on every rank)."""
    from grpo_cpp_b200 import workloads as W
    rng = np.random.Generator(np.random.PCG64(seed))
    S, T = spec["B"] * spec["G"], spec["T"]
    N = S * T
    lengths = rng.integers(spec["min_len"], T + 1, S) if spec["min_len"] is not None else np.full(S, T)
    mask = W.prefix_mask(lengths, T)
    selected = np.where(mask == 1, rng.integers(0, spec["V"], N), -1).astype(np.int32)
    rewards = (rng.random(S) < 0.5).astype(np.float32)
    adv = W.group_advantages_np(rewards, spec["B"], spec["G"])
    noise_old = (0.05 * rng.standard_normal(N)).astype(np.float32)
    noise_ref = (0.05 * rng.standard_normal(N)).astype(np.float32)
    return mask, selected, adv, noise_old, noise_ref


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------
# CPU arms (the only places that execute anything under oracle/)
# ---------------------------------------------------------------------------------------------
def cpu_sample_batch(spec: dict, responses: int, seed: int):
    """`responses` responses of the workload's shape (T slots, V columns), dense host arrays."""
    from grpo_cpp_b200 import workloads as W
    return W.logits_case(1, responses, spec["T"], spec["V"], sigma=spec["sigma"], min_len=spec["min_len"],
                         reduction=spec["reduction"], length_alpha=spec["alpha"], seed=seed)


def cpu_run(lib, b):
    return lib.logits(b.logits, b.logp_old, b.logp_ref, b.selected, b.advantages, b.mask, b.B, b.G, b.T, b.V,
                      CLIP_EPS, BETA, b.reduction, b.length_alpha)


def cpu_baseline_single(spec: dict, budget_s: float = 12.0) -> dict:
    """The CPU path as shipped (one thread), best of up to 3 runs on a bounded sample."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_py
    lib = oracle_py.load("best")
    responses = 8 if spec["V"] * spec["T"] >= 2 ** 22 else 16
    b = cpu_sample_batch(spec, responses, seed=7)
    best, t_total = None, 0.0
    for _ in range(3):
        t0 = time.perf_counter()
        cpu_run(lib, b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        t_total += dt
        if t_total > budget_s:
            break
    return {"value": b.N / best, "unit": UNIT, "cores": 1, "kind": lib.kind,
            "sample": f"{responses} responses x {spec['T']} slots x V={spec['V']} ({b.N} rows, "
                      f"{int(b.mask.sum())} active), single thread as shipped, best of 3"}


def reference_arm(args, spec: dict) -> None:
    """`--impl reference`: the reference CPU path on all host cores, one response per thread per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_py
    lib = oracle_py.load("best")
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    # memory bound: each thread holds its response's logits and gradient (plus the library's copy)
    per_thread = 3 * spec["T"] * spec["V"] * 4
    cores = max(1, min(cores, int(48e9 // per_thread)))
    batches = [cpu_sample_batch(spec, 1, seed=100 + i) for i in range(min(cores, 4))]
    rows_per_step = cores * spec["T"]

    def one_step():
        threads = [threading.Thread(target=cpu_run, args=(lib, batches[i % len(batches)])) for i in range(cores)]
        t0 = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return time.perf_counter() - t0

    for _ in range(args.warmup):
        one_step()
    times = [one_step() for _ in range(args.steps)]
    total = sum(times)
    value = rows_per_step * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec["label"], "V": spec["V"], "tokens_per_response": spec["T"],
                   "rows_per_step": rows_per_step, "reduction": "token_mean"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": lib.kind,
                         "sample": f"each step = {cores} responses x {spec['T']} slots x V={spec['V']}, one "
                                   f"response per host thread through the reference's grpo_logits_cpu"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def gpu_arm(args, spec: dict) -> None:
    import torch
    import torch.distributed as dist

    import grpo_cpp_b200 as G
    from grpo_cpp_b200 import device as D
    from grpo_cpp_b200.sharded import ShardedBoundary, shard_rows_balanced

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    G.lib()  # fail loudly here if the CUDA library is missing
    if args.variant is not None:
        D.set_variant(args.variant)

    B, Gn, T, V, P = spec["B"], spec["G"], spec["T"], spec["V"], spec["P"]
    S, N = B * Gn, B * Gn * T
    mask_h, sel_h, adv_h, noise_old, noise_ref = host_metadata(spec)
    # contiguous row ranges of equal kernel time (ragged masks make equal row counts unequal work)
    off, cnt = shard_rows_balanced(mask_h, world, V, P, args.masked_cost)[rank]
    sl = slice(off, off + cnt)

    # ---- this rank's rows, built on the device
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    pristine = torch.empty(cnt, P, device=dev)
    pristine.normal_(0.0, spec["sigma"], generator=gen)
    sel_d = torch.from_numpy(sel_h[sl]).to(dev)
    now = torch.empty(cnt, device=dev)
    chunk = 4096
    for r0 in range(0, cnt, chunk):  # true selected log-probability, for realistic old/ref values
        rows = pristine[r0:r0 + chunk, :V].double()
        lse = torch.logsumexp(rows, dim=1)
        idx = sel_d[r0:r0 + chunk].clamp(min=0).long()
        now[r0:r0 + chunk] = (rows.gather(1, idx[:, None])[:, 0] - lse).float()
    m_local = mask_h[sl]
    old_h = np.where(m_local == 1, now.cpu().numpy() + noise_old[sl], 0).astype(np.float32)
    ref_h = np.where(m_local == 1, now.cpu().numpy() + noise_ref[sl], 0).astype(np.float32)
    del now
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    host = {"old": pin(old_h), "ref": pin(ref_h), "sel": pin(sel_h[sl]), "mask": pin(m_local), "adv": pin(adv_h)}
    devt = {k: v.to(dev) for k, v in host.items()}
    work = torch.empty_like(pristine)
    flush = torch.empty(64 * 1024 * 1024, device=dev)  # 256 MB > 126 MB L2
    flush_sink = torch.zeros((), device=dev)

    sb = ShardedBoundary(S, T, V, P, clip_eps=CLIP_EPS, beta=BETA, reduction=spec["reduction"],
                         length_alpha=spec["alpha"], device=dev, rows=(off, cnt))
    n_active_local = int(m_local.sum())
    kernel_bytes = 4 * (n_active_local * V + cnt * P) + cnt * 16
    plan = D.plan(work, V)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def restore():
        work.copy_(pristine)
        flush.fill_(0.0)
        # ... and read back, so that L2 ends up full of CLEAN lines: after the fill alone it holds ~126 MB of dirty
        # ones, and the timed pass would pay for writing them out (about 20 us, whatever the pass's own size)
        torch.sum(flush, dim=(0,), out=flush_sink)

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def device_step(e0, e1, k0, k1):
        e0.record()
        sb.prepare(devt["mask"])
        k0.record()
        sb.ops.logits(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], sb.weights, devt["mask"], T, V,
                      CLIP_EPS, BETA, row_offset=sb.row_offset, result=sb.result, workspace=sb.workspace,
                      row_order=sb.row_order)
        k1.record()
        sb._all_reduce(sb.result)
        e1.record()

    # ---- device-resident steps -------------------------------------------------------------
    # The pass (lengths, row kernel, reduce kernel, weights) is captured once into a
    # CUDA graph and replayed; an eager loop afterwards times the dominant kernel on its own.
    sampler = ClockSampler(local_rank) if rank == 0 else None
    graph = None
    # --exchange peer: the pass is two launches (row kernel, reduce kernel) and the reduce kernel does the
    # exchange itself through the ranks' regions (at one rank: its own region).  --exchange nccl: four launches
    # and one NCCL all-reduce.
    peer = args.exchange == "peer"
    if peer:
        sb.enable_peer_exchange()
    one_pass = sb.step_peer if peer else sb.step_fused
    # With more than one rank the pass stays eager launches: a pass that captured NCCL all-reduces in the
    # graph did not complete on this pool (2 ranks), so graphs are used at one rank only.
    if not args.no_graph and world == 1:
        restore()
        graph = sb.capture(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])

    sb.prepare(devt["mask"])  # weights for the first pass; every later pass gets them from the pass before

    align = torch.zeros(1, device=dev)

    def timed_pass(e0, e1):
        # The restore above takes a different time on every rank (the ranks hold different numbers of rows), and a
        # rank that starts its pass late makes the others wait inside their timed exchange.  A one-element
        # all-reduce, enqueued like everything else and outside the event pair, lines the ranks up first, so the
        # pair measures the pass itself: slowest rank's kernels plus the exchange.
        if world > 1:
            dist.all_reduce(align)
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            one_pass(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])
        e1.record()

    # Restore + flush run on the same stream between the timed passes and the host never waits inside
    # the loop, so every pass's launches are already queued when the device reaches them; the K passes
    # are bracketed by a barrier + synchronize on both sides and timed by one event pair each.
    for _ in range(args.warmup):
        restore()
        timed_pass(ev(), ev())
    barrier()
    pairs = [(ev(), ev()) for _ in range(args.steps)]
    t_wall0 = time.perf_counter()
    for e0, e1 in pairs:
        restore()
        timed_pass(e0, e1)
    barrier()
    t_wall = time.perf_counter() - t_wall0
    step_ms = [e0.elapsed_time(e1) for e0, e1 in pairs]
    # dominant kernel alone (with the reduce kernel behind it): its own event pair inside an eager pass.  The host
    # does not wait between iterations, so the launches are queued while the device is still restoring the
    # logits and the pair brackets device time only, not launch latency.
    kern_pairs = []
    for i in range(3 + min(args.steps, 10)):
        restore()
        e0, e1, k0, k1 = ev(), ev(), ev(), ev()
        device_step(e0, e1, k0, k1)
        if i >= 3:
            kern_pairs.append((k0, k1))
    barrier()
    kern_ms = [k0.elapsed_time(k1) for k0, k1 in kern_pairs]
    stats = sb.stats()  # applies the error contract to the global quantities

    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    per_rank = torch.zeros(world, 2, dtype=torch.float64, device=dev)  # [rank] = (pass ms, dominant kernel ms)
    per_rank[rank, 0] = sum(step_ms) / len(step_ms)
    per_rank[rank, 1] = statistics.mean(kern_ms)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(per_rank)
    total_ms = float(total_ms.item())
    per_rank = per_rank.cpu().tolist()

    # ---- end to end through the public API with host metadata --------------------------------
    h2d = sum(host[k].numel() * host[k].element_size() for k in host)
    cfg = G.LossConfig(CLIP_EPS, BETA, G.ReductionMode(spec["reduction"]), spec["alpha"])
    e2e_s = []
    for i in range(args.warmup + args.steps):
        restore()
        barrier()
        t0 = time.perf_counter()
        if world == 1:
            # the reference-facing call itself: host vectors in, device logits in place, stats out
            st = G.grpo_logits_cuda_device_inplace(work, old_h, ref_h, sel_h, adv_h, mask_h, B, Gn, T, V, P, cfg)
            loss_val = st.loss
        else:
            for k in host:
                devt[k].copy_(host[k], non_blocking=True)
            sb.prepare(devt["mask"])
            if peer:
                sb.step_peer(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])
            else:
                sb.step(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])
            loss_val = sb.stats()["loss"]
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            e2e_s.append(dt)
    e2e_total = torch.tensor([sum(e2e_s)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_total, op=dist.ReduceOp.MAX)
    e2e_total = float(e2e_total.item())
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        k_ms = statistics.mean(kern_ms)
        achieved = kernel_bytes / (k_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": N * args.steps / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": spec["label"], "rows": N, "V": V, "P": P, "responses": S,
                       "tokens_per_response": T, "active_rows": int(mask_h.sum()), "reduction":
                       ["sequence_mean", "token_mean", "length_weighted"][spec["reduction"]],
                       "parallelism": f"token-sharded x{world}", "in_place": True, "kernel": plan,
                       "launch": "eager" if graph is None else "one CUDA graph per pass",
                       "sharding": "contiguous row ranges of equal estimated kernel time" if world > 1 else "single range",
                       "exchange": ("reduce kernel over NVLink peer memory" if peer and world > 1 else
                                    "reduce kernel, own region only" if peer else
                                    "one NCCL all-reduce per pass" if world > 1 else "none"),
                       "l2": "logits restored from a pristine copy and a 256 MB buffer written, then read back, "
                             "between passes on the same stream, outside the timed event pairs; per-rank logits "
                             "far exceed the 126 MB L2"},
            "active_tokens_per_s": int(mask_h.sum()) * args.steps / (total_ms * 1e-3),
            "loss": stats["loss"], "valid_tokens": stats["valid_tokens"],
            "wall_s_timed_loop": t_wall,
            "per_rank_ms": {"pass": [round(p, 4) for p, _ in per_rank], "kernel": [round(k, 4) for _, k in per_rank]},
            "clocks": clocks,
            "e2e": {"value": N * args.steps / e2e_total, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 48, "ms_per_step": 1e3 * e2e_total / args.steps,
                    "api": "grpo_logits_cuda_device_inplace (host metadata, device logits)" if world == 1 else
                           ("ShardedBoundary.prepare+step_peer+stats from pinned host metadata (no collective call)"
                            if peer else "ShardedBoundary.prepare+step+stats from pinned host metadata")},
            # per pass and rank: the row kernel and the reduce kernel (+ lengths and weights kernels with NCCL)
            "gpu_launches": (2 if peer else 4) * args.steps * world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                         "kernel": f"logits_pipelined_kernel<{plan}> (+ reduce kernel)", "ms_per_launch": k_ms,
                         "algorithmic_bytes_per_launch": kernel_bytes,
                         # the ncu-derived figure is for the whole batch on one GPU; a rank's launch moves its share
                         "traffic": (round(TRAFFIC_BYTES[args.workload] * kernel_bytes / FULL_ALGORITHMIC[args.workload])
                                     if args.workload in TRAFFIC_BYTES else None)},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_single(spec)
        print(json.dumps(line), flush=True)
    if peer:
        barrier()  # no rank unmaps a region that another rank's kernel may still write to
        sb.exchange.close()
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel from an ncu
# capture, scaled to the full launch where a smaller case was captured (see profiles/); null
# until a capture exists for that workload.
FULL_ALGORITHMIC = {"gpt2": 20629393828}
TRAFFIC_BYTES: dict = {
    # profiles/logits_pipelined_kernel_gpt2_shaped_4096_rows.txt: reads 1.0001x algorithmic (scaled by
    # active rows), writes = algorithmic minus the ~53 MB still dirty in L2 at kernel end
    "gpt2": 20.58e9,
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gpt2", choices=["gpt2", "gpt2s", "v32k", "v128k"])
    ap.add_argument("--variant", type=int, default=None, help="force a row-resident kernel variant")
    ap.add_argument("--prompts", type=int, default=None,
                    help="override the workload's number of prompts B (rows = B x G x T): the same row shape at "
                         "another batch size, e.g. to see the kernel's steady-state rate on a short configuration")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="at more than one rank: the pass's exchange by the library's own kernel over NVLink peer "
                         "memory, or by one NCCL all-reduce")
    ap.add_argument("--masked-cost", type=float, default=0.8,
                    help="cost of a masked row in units of P floats when cutting the batch into per-rank row ranges")
    ap.add_argument("--no-graph", action="store_true", help="launch each pass eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    import grpo_cpp_b200  # noqa: F401  (registers the package under its importable name)
    spec = workload_spec(args.workload)
    if args.prompts is not None:
        spec["B"] = args.prompts
        spec["label"] += f" (B overridden to {args.prompts})"
    if args.impl == "reference":
        reference_arm(args, spec)
    else:
        gpu_arm(args, spec)


if __name__ == "__main__":
    main()
