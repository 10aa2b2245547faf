#!/usr/bin/env python
"""Benchmark of the GRPO loss boundary on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the GPT-2-shaped loss boundary sharded by token (32 prompts x 8 responses x 256 token
slots = 65,536 rows, V = 50,257 padded to P = 50,304 fp32 logits of standard deviation 3, ragged
lengths U[32,256], token-mean reduction with the global normaliser exchanged between the ranks), the
configuration the headline metric -- fused loss+dlogits tokens/s and HBM GB/s at 1/2/4/8 GPUs -- is
quoted on.  The 65,536 rows are split contiguously over the ranks (total work fixed: strong scaling).
The logits are counter-based (every element a function of seed, global row and column), so every N
sees the same batch and the host can rebuild any row for the parity check.

A step is one pass of the hot path over the batch, two launches: the fused logits kernel in place
(with the weights the previous pass left), then the reduce kernel (per-row loss terms in double,
fixed-order totals, the next pass's per-response lengths, the exchange between the ranks through
NVLink peer memory, the next pass's weights).  The logits are restored from a pristine copy and L2 is
flushed between passes on the same stream, outside the timed event pairs; the K passes are bracketed
by a barrier and a synchronize, each is timed by a CUDA-event pair on the launching stream, and the
per-rank totals are reduced with MAX.  One JSON line is printed by rank 0.  Besides the headline it
carries:

* ``parity``: after the timed loops every rank checks sampled rows of its shard element-wise against
  the CPU checker, and the ranks compare their result records bit for bit;
* ``e2e``: the same pass through the public host-facing call, host metadata in and record out;
* at one GPU, ``other_configs`` (the two short fused-logits configurations and the selected-token
  configuration, each with its own roofline line), ``reference_cuda`` (the reference's own CUDA
  kernels on the same GPU, by its own timing protocol) and ``cpu_baseline``.

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
LOGITS_SEED = 1234
REDUCTION_NAMES = ["sequence_mean", "token_mean", "length_weighted"]


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
def workload_spec(name: str) -> dict:
    from grpo_cpp_b200 import workloads as W
    if name == "gpt2":
        s = dict(W.GPT2_SHAPE)
        s.update(reduction=W.TOKEN_MEAN, alpha=0.0, label="gpt2-124M-shaped loss boundary, token-sharded")
        return s
    if name == "v32k":
        return dict(B=2, G=8, T=64, V=32768, P=32768, sigma=2.0, min_len=None, reduction=W.TOKEN_MEAN, alpha=0.0,
                    label="fused logits N=1024 x V=32768, full mask, token-mean")
    if name in ("v128k_a0.5", "v128k_a1.0"):
        alpha = float(name.split("_a")[1])
        return dict(B=2, G=8, T=64, V=131072, P=131072, sigma=2.0, min_len=16, reduction=W.LENGTH_WEIGHTED,
                    alpha=alpha, label=f"fused logits N=1024 x V=131072, ragged U[16,64], L^{alpha} weights")
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


def host_weights(mask: np.ndarray, S: int, T: int, reduction: int):
    """Per-response weights by the reference's fp32 expressions (src/cpu/grpo_loss.cpp:124-131) for
    the two reductions whose arithmetic numpy reproduces exactly; None for L^alpha (libm's powf)."""
    f = np.float32
    lengths = mask.reshape(S, T).sum(1)
    if reduction == 0:
        return (f(1.0) / (f(S) * lengths.astype(f))).astype(f)
    if reduction == 1:
        return np.full(S, f(1.0) / f(int(lengths.sum())), f)
    return None


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
# CPU arms and checkers (the only places that execute anything under oracle/)
# ---------------------------------------------------------------------------------------------
def _oracle(kind: str):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_py
    return oracle_py.load(kind)


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
    lib = _oracle("best")
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


def reference_cuda_leg(configs) -> dict:
    """The reference's own CUDA kernels compiled for sm_100a (oracle/_ref/ref_cuda_timer, built from
    the reference tree where it was present), timed by the reference's own protocol.  A baseline
    leg like the CPU one: never part of a timed region of this library."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_cuda_timer")
    if not os.path.exists(exe):
        return {"unavailable": "oracle/_ref/ref_cuda_timer was not built (no reference tree at build time)"}
    out = {}
    try:
        run = subprocess.run([exe] + list(configs), capture_output=True, text=True, timeout=240)
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"unavailable": f"ref_cuda_timer did not finish: {e!r}"}
    if run.returncode != 0:
        return {"unavailable": f"ref_cuda_timer exited {run.returncode}: {run.stderr.strip()[-200:]}"}
    for line in run.stdout.splitlines():
        try:
            rec = json.loads(line)
            out[rec.pop("config")] = rec
        except (ValueError, KeyError):
            continue
    return out


def reference_arm(args, spec: dict) -> None:
    """`--impl reference`: the reference CPU path on all host cores, one response per thread per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lib = _oracle("best")
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
                   "rows_per_step": rows_per_step, "reduction": REDUCTION_NAMES[spec["reduction"]]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": lib.kind,
                         "sample": f"each step = {cores} responses x {spec['T']} slots x V={spec['V']}, one "
                                   f"response per host thread through the reference's grpo_logits_cpu"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm: helpers
# ---------------------------------------------------------------------------------------------
class Batch:
    """One rank's rows of a logits workload, resident on the device, plus the host metadata."""

    def __init__(self, spec: dict, dev, world: int = 1, rank: int = 0):
        import torch
        from grpo_cpp_b200 import device as D, workloads as W
        from grpo_cpp_b200.sharded import shard_rows_balanced
        self.spec, self.dev = spec, dev
        self.B, self.G, self.T, self.V, self.P = spec["B"], spec["G"], spec["T"], spec["V"], spec["P"]
        self.S, self.N = self.B * self.G, self.B * self.G * self.T
        self.mask_h, self.sel_h, self.adv_h, noise_old, noise_ref = host_metadata(spec)
        # contiguous row ranges of equal kernel time (ragged masks make equal row counts unequal work)
        self.off, self.cnt = shard_rows_balanced(self.mask_h, world, self.V, self.P)[rank]
        sl = slice(self.off, self.off + self.cnt)
        self.scale = W.synthetic_scale(spec["sigma"])
        self.pristine = torch.empty(self.cnt, self.P, device=dev)
        D.synthetic_logits(self.pristine, self.V, float(self.scale), LOGITS_SEED, row_offset=self.off)
        # log p(selected) of every active local row from the library's own row kernel, for realistic old/ref values
        self.m_local = self.mask_h[sl]
        active = np.flatnonzero(self.m_local == 1).astype(np.int32)
        now = np.zeros(self.cnt, np.float32)
        if active.size:
            rows_d = torch.from_numpy(active).to(dev)
            toks_d = torch.from_numpy(self.sel_h[sl][active]).to(dev)
            _, logp, _ = D.sample_rows(self.pristine, self.V, rows_d, tokens=toks_d)
            now[active] = logp.cpu().numpy()
        self.old_h = np.where(self.m_local == 1, now + noise_old[sl], 0).astype(np.float32)
        self.ref_h = np.where(self.m_local == 1, now + noise_ref[sl], 0).astype(np.float32)
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
        self.host = {"old": pin(self.old_h), "ref": pin(self.ref_h), "sel": pin(self.sel_h[sl]),
                     "mask": pin(self.m_local), "adv": pin(self.adv_h)}
        self.devt = {k: v.to(dev) for k, v in self.host.items()}
        self.work = torch.empty_like(self.pristine)
        self.n_active_local = int(self.m_local.sum())
        self.kernel_bytes = 4 * (self.n_active_local * self.V + self.cnt * self.P) + self.cnt * 16


class Flusher:
    """Restores a working buffer from its pristine copy and leaves L2 full of clean lines of another
    buffer: after a plain fill L2 would hold ~126 MB of dirty lines, and the timed pass would pay
    for writing them out (about 20 us, whatever the pass's own size)."""

    def __init__(self, dev):
        import torch
        self.buf = torch.empty(64 * 1024 * 1024, device=dev)  # 256 MB > 126 MB L2
        self.sink = torch.zeros((), device=dev)

    def __call__(self, work=None, pristine=None):
        import torch
        if work is not None:
            work.copy_(pristine)
        self.buf.fill_(0.0)
        torch.sum(self.buf, dim=(0,), out=self.sink)


def parity_block(batch: Batch, sb, one_pass, flush, world: int, rank: int, rows_per_rank: int = 16) -> dict:
    """Untimed: one more pass on restored logits, then (a) `rows_per_rank` active rows of this rank's
    shard, evenly spaced, are rebuilt on the host from the counter-based generator and checked
    element-wise against the CPU checker's per-row entry at 1e-7 + 1e-5*|want|; (b) tails and sampled
    masked rows must be exactly zero; (c) the ranks' result records are compared bit for bit."""
    import torch
    import torch.distributed as dist
    from grpo_cpp_b200 import workloads as W
    flush(batch.work, batch.pristine)
    d = batch.devt
    one_pass(batch.work, d["old"], d["ref"], d["sel"], d["adv"], d["mask"])
    torch.cuda.synchronize()
    record = sb.result.clone()
    active = np.flatnonzero(batch.m_local == 1)
    masked = np.flatnonzero(batch.m_local == 0)
    pick = active[np.unique(np.linspace(0, active.size - 1, min(rows_per_rank, active.size)).astype(np.int64))] \
        if active.size else active
    pick_masked = masked[[0, masked.size - 1]] if masked.size else masked
    got = batch.work[torch.from_numpy(pick).to(batch.dev)].cpu().numpy()
    got_masked = batch.work[torch.from_numpy(pick_masked).to(batch.dev)].cpu().numpy() if pick_masked.size else None
    x = W.synthetic_logits_rows(batch.off + pick, batch.V, batch.P, batch.scale, LOGITS_SEED)
    w_seq = host_weights(batch.mask_h, batch.S, batch.T, batch.spec["reduction"])
    if w_seq is None:
        w_seq = sb.weights.cpu().numpy()
    seq = (batch.off + pick) // batch.T
    want, _, _ = _oracle("port").logits_rows(x, batch.old_h[pick], batch.ref_h[pick], batch.sel_h[batch.off + pick],
                                            batch.adv_h[seq], w_seq[seq], CLIP_EPS, BETA)
    err = np.abs(got[:, : batch.V].astype(np.float64) - want)
    tol = 1e-7 + 1e-5 * np.abs(want)
    worst = float((err / tol).max()) if pick.size else 0.0
    zeros_ok = bool((got[:, batch.V:] == 0).all() and (got_masked is None or (got_masked == 0).all()))
    info = torch.tensor([float(pick.size), worst, float(err.max()) if pick.size else 0.0, 1.0 if zeros_ok else 0.0],
                        dtype=torch.float64, device=batch.dev)
    bits = record.view(torch.int64).clone()
    if world > 1:
        all_info = [torch.empty_like(info) for _ in range(world)]
        all_bits = [torch.empty_like(bits) for _ in range(world)]
        dist.all_gather(all_info, info)
        dist.all_gather(all_bits, bits)
    else:
        all_info, all_bits = [info], [bits]
    infos = [t.cpu().tolist() for t in all_info]
    return {"rows_checked": int(sum(i[0] for i in infos)), "tolerance": "1e-7 + 1e-5*|want| per element",
            "max_err_over_tolerance": max(i[1] for i in infos), "max_abs_err": max(i[2] for i in infos),
            "tails_and_masked_rows_zero": all(i[3] == 1.0 for i in infos),
            "records_identical": all(bool((b == all_bits[0]).all()) for b in all_bits),
            "passed": bool(max(i[1] for i in infos) <= 1.0 and all(i[3] == 1.0 for i in infos)),
            "checker": "oracle/grpo_oracle.c per-row entry on rows rebuilt on the host from the generator"}


def time_passes(fn, restore, passes: int, warmup: int = 3):
    """Median and mean ms of `fn`, each pass bracketed by its own CUDA-event pair on the current
    stream, `restore` (outside the pair) before each."""
    import torch
    pairs = []
    for i in range(warmup + passes):
        restore()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        if i >= warmup:
            pairs.append((e0, e1))
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in pairs]
    return statistics.median(ms), statistics.mean(ms), min(ms)


def other_logits_config(name: str, dev, flush, peak: float, passes: int = 24) -> dict:
    """One of the short fused-logits configurations on one GPU: the device-resident pass
    (grpo_b200_logits in place, weights and row order prepared once per mask), L2 flushed."""
    import torch
    from grpo_cpp_b200 import device as D
    spec = workload_spec(name)
    b = Batch(spec, dev)
    d = b.devt
    lengths = D.count_lengths(d["mask"], b.S, b.T)
    weights, meta = D.weights_from_lengths(lengths, spec["reduction"], spec["alpha"])
    order = D.row_order(d["mask"])
    result, ws = D.new_result(dev), D.logits_workspace(b.N, dev)

    def one():
        D.logits(b.work, d["old"], d["ref"], d["sel"], d["adv"], weights, d["mask"], b.T, b.V, CLIP_EPS, BETA,
                 result=result, workspace=ws, row_order=order)

    med, mean, best = time_passes(one, lambda: flush(b.work, b.pristine), passes)
    # sampled-row parity on the last pass's output
    from grpo_cpp_b200 import workloads as W
    active = np.flatnonzero(b.mask_h == 1)
    pick = active[np.unique(np.linspace(0, active.size - 1, 6).astype(np.int64))]
    got = b.work[torch.from_numpy(pick).to(dev)].cpu().numpy()
    x = W.synthetic_logits_rows(pick, b.V, b.P, b.scale, LOGITS_SEED)
    w_seq = host_weights(b.mask_h, b.S, b.T, spec["reduction"])
    if w_seq is None:
        w_seq = weights.cpu().numpy()
    want, _, _ = _oracle("port").logits_rows(x, b.old_h[pick], b.ref_h[pick], b.sel_h[pick], b.adv_h[pick // b.T],
                                            w_seq[pick // b.T], CLIP_EPS, BETA)
    ratio = float((np.abs(got[:, : b.V] - want) / (1e-7 + 1e-5 * np.abs(want))).max())
    rec = result.cpu().tolist()
    full_equiv = 2 * b.N * b.V * 4
    return {"workload": spec["label"], "kernel": D.plan(b.work, b.V), "passes": passes, "ms_per_pass": med,
            "ms_per_pass_mean": mean, "ms_per_pass_min": best, "tokens_per_s": b.N / (med * 1e-3),
            "roofline": {"bound": "hbm", "algorithmic_bytes": b.kernel_bytes, "achieved": b.kernel_bytes / med / 1e6,
                         "peak": peak, "unit": "GB/s", "frac": b.kernel_bytes / med / 1e6 / peak},
            "north_star_bytes_2NV4": full_equiv, "active_rows": int(b.mask_h.sum()),
            "launches_per_pass": 2, "loss": rec[0], "bad_inputs": rec[4],
            "parity_max_err_over_tolerance": ratio, "l2": "flushed between passes"}


def other_token_config(tokens_per_seq: int, ragged: bool, dev, flush, peak: float, passes: int = 24) -> dict:
    """The selected-token configuration (4,096 responses) on one GPU: grpo_b200_loss, L2 flushed
    between passes (the whole input is smaller than L2)."""
    import torch
    from grpo_cpp_b200 import device as D, workloads as W
    t = W.selected_token_case(4096, tokens_per_seq, ragged=ragged, seed=42)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    new, old, ref, adv, mask = to(t.logp_new), to(t.logp_old), to(t.logp_ref), to(t.advantages), to(t.mask)
    weights, _ = D.weights_from_lengths(D.count_lengths(mask, t.S, t.T), t.reduction, t.length_alpha)
    dlogp = torch.empty(t.N, device=dev)
    result, ws = D.new_result(dev), D.loss_workspace(dev)

    def one():
        D.loss(new, old, ref, adv, weights, mask, t.T, t.clip_eps, t.beta, dlogp=dlogp, result=result, workspace=ws)

    med, mean, best = time_passes(one, lambda: flush(), passes)
    active = int(t.mask.sum())
    nbytes = 20 * active + 8 * (t.N - active)
    want = _oracle("best").loss(t.logp_new, t.logp_old, t.logp_ref, t.advantages, t.mask, t.B, t.G, t.T, **t.cfg())
    rec = result.cpu().tolist()
    rel = max(abs(rec[k] - float(want[0][k])) / (abs(float(want[0][k])) + 1e-30) for k in range(3))
    g = dlogp.cpu().numpy()
    grad_ratio = float((np.abs(g - want[2]) / (1e-7 + 1e-5 * np.abs(want[2]))).max())
    return {"workload": f"selected-token path, 4096 responses x {tokens_per_seq}, {'ragged' if ragged else 'full'} mask",
            "tokens": t.N, "active_tokens": active, "passes": passes, "ms_per_pass": med, "ms_per_pass_min": best,
            "tokens_per_s": t.N / (med * 1e-3),
            "roofline": {"bound": "hbm", "algorithmic_bytes": nbytes, "achieved": nbytes / med / 1e6, "peak": peak,
                         "unit": "GB/s", "frac": nbytes / med / 1e6 / peak,
                         "note": "84 MB at most: launch-latency bound, not bandwidth bound"},
            "launches_per_pass": 1, "loss_rel_err_vs_cpu": rel, "dlogp_max_err_over_tolerance": grad_ratio,
            "l2": "flushed between passes"}


def lmhead_config(dev, flush, passes: int = 12) -> dict:
    """The LM-head projection fused with the loss statistics on 4,096 GPT-2-shaped rows (hidden 768,
    V = 50,257 padded to 50,304): tcgen05 tensor cores, TF32 inputs, fp32 accumulation, no logits
    written.  Beside it, on the same inputs: a cuBLAS TF32 matmul that writes the 824 MB of logits
    (torch.matmul, a library kernel: the baseline) followed by this library's fused logits pass."""
    import torch
    from grpo_cpp_b200 import device as D, workloads as W
    n_seq, T, C, V, P = 16, 256, 768, 50257, 50304
    N = n_seq * T
    rng = np.random.Generator(np.random.PCG64(11))
    gen = torch.Generator(device=dev).manual_seed(11)
    # inputs exactly representable in TF32 (low 13 mantissa bits cleared), so that the tensor cores' and the
    # library matmul's own roundings of the inputs cannot differ and the two losses below are comparable
    def tf32_representable(x):
        return (x.view(torch.int32) & -8192).view(torch.float32)

    hidden = tf32_representable(torch.empty(N, C, device=dev).normal_(0.0, 1.0, generator=gen))
    lm_head = tf32_representable(torch.empty(P, C, device=dev).normal_(0.0, 3.0 / C ** 0.5, generator=gen))
    mask_h = W.prefix_mask(rng.integers(32, T + 1, n_seq), T)
    sel_h = np.where(mask_h == 1, rng.integers(0, V, N), -1).astype(np.int32)
    adv_h = W.group_advantages_np((rng.random(n_seq) < 0.5).astype(np.float32), n_seq // 8, 8)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    mask, sel, adv = to(mask_h), to(sel_h), to(adv_h)
    weights, _ = D.weights_from_lengths(D.count_lengths(mask, n_seq, T), W.TOKEN_MEAN, 0.0)
    # old/ref log-probabilities near the true ones, as in training: log p(selected) from the fused operator + noise
    _, now, _ = D.lmhead_loss(hidden, lm_head, V, torch.zeros(N, device=dev), torch.zeros(N, device=dev), sel, adv, weights,
                              mask, T, CLIP_EPS, BETA, want_selected_logp=True)
    noise = lambda: to((0.05 * rng.standard_normal(N)).astype(np.float32))
    old = torch.where(mask == 1, now + noise(), torch.zeros_like(now))
    ref = torch.where(mask == 1, now + noise(), torch.zeros_like(now))
    med, mean, best = time_passes(lambda: D.lmhead_loss(hidden, lm_head, V, old, ref, sel, adv, weights, mask, T, CLIP_EPS, BETA),
                                  lambda: flush(), passes)
    fused_rec = D.lmhead_loss(hidden, lm_head, V, old, ref, sel, adv, weights, mask, T, CLIP_EPS, BETA)[0].cpu().tolist()
    logits = torch.empty(N, P, device=dev)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    result, ws, order = D.new_result(dev), D.logits_workspace(N, dev), D.row_order(mask)

    def unfused():
        torch.matmul(hidden, lm_head.T, out=logits)
        D.logits(logits, old, ref, sel, adv, weights, mask, T, V, CLIP_EPS, BETA, result=result, workspace=ws,
                 row_order=order)

    try:
        gemm_med, _, _ = time_passes(lambda: torch.matmul(hidden, lm_head.T, out=logits), lambda: flush(), passes)
        unf_med, _, _ = time_passes(unfused, lambda: flush(), passes)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    unf_rec = result.cpu().tolist()
    flops = 2.0 * N * P * C
    peak_bf16 = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_bf16 = float(json.load(f)["bf16_tflops"])
    except (OSError, KeyError, ValueError):
        peak_bf16 = 1590.0
    peak_tf32 = peak_bf16 / 2.0
    return {"workload": f"LM-head fused with loss statistics, {N} rows x V={V} (P={P}) x C={C}, TF32 in / fp32 accumulate",
            "passes": passes, "ms_per_pass": med, "ms_per_pass_min": best, "tokens_per_s": N / (med * 1e-3),
            "launches_per_pass": 3,
            "roofline": {"bound": "tensor", "flops": flops, "achieved": flops / med / 1e9, "unit": "TFLOP/s",
                         "peak": peak_tf32, "frac": flops / med / 1e9 / peak_tf32,
                         "peak_source": "half of the measured dense bf16 cuBLAS burst figure (TF32 runs at half the bf16 rate)"},
            "cublas_tf32_matmul_writing_logits_ms": gemm_med,
            "cublas_tf32_matmul_tflops": flops / gemm_med / 1e9,
            "cublas_matmul_then_fused_logits_pass_ms": unf_med,
            "loss_fused": fused_rec[0], "loss_matmul_then_logits_pass": unf_rec[0],
            "logits_bytes_not_written": 4 * N * P, "l2": "flushed between passes"}


def same_protocol_leg(dev) -> dict:
    """This library under the reference's own timing protocol (its benchmark entry points, which
    this library exports with the same signatures), for a like-for-like line beside
    `reference_cuda`: warm buffers, back-to-back passes, medians."""
    import torch
    import grpo_cpp_b200 as G
    from grpo_cpp_b200 import device as D, workloads as W
    out = {}
    for name in ("v32k", "v128k_a0.5"):
        spec = workload_spec(name)
        mask, sel, adv, _, _ = host_metadata(spec)
        N = spec["B"] * spec["G"] * spec["T"]
        x_d = torch.empty(N, spec["P"], device=dev)
        D.synthetic_logits(x_d, spec["V"], float(W.synthetic_scale(spec["sigma"])), LOGITS_SEED)
        x = x_d.cpu().numpy()
        del x_d
        typical = np.float32(-np.log(spec["V"]) - 2.0)
        old = np.where(mask == 1, typical, 0).astype(np.float32)
        cfg = G.LossConfig(CLIP_EPS, BETA, G.ReductionMode(spec["reduction"]), spec["alpha"])
        t = G.benchmark_grpo_logits_cuda(x, old, old, sel, adv, mask, spec["B"], spec["G"], spec["T"], spec["V"], cfg,
                                         3, 10)
        out[name] = {"separate_ms": t.separate_ms, "fused_ms": t.fused_ms}
        del x
    for name, T in (("cfg2_1M", 256), ("cfg2_4M", 1024)):
        t = W.selected_token_case(4096, T, ragged=False, seed=42)
        r = G.benchmark_grpo_loss_cuda(t.logp_new, t.logp_old, t.logp_ref, t.advantages, t.mask, t.B, t.G, t.T,
                                       G.LossConfig(t.clip_eps, t.beta), 5, 20)
        out[name] = {"block_ms": r.block_ms}
    return out


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def gpu_arm(args, spec: dict) -> None:
    import torch
    import torch.distributed as dist

    import grpo_cpp_b200 as G
    from grpo_cpp_b200 import device as D
    from grpo_cpp_b200.sharded import ShardedBoundary

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

    batch = Batch(spec, dev, world, rank)
    B, Gn, T, V, P, S, N = batch.B, batch.G, batch.T, batch.V, batch.P, batch.S, batch.N
    off, cnt, devt, host, work = batch.off, batch.cnt, batch.devt, batch.host, batch.work
    mask_h = batch.mask_h
    flush = Flusher(dev)
    restore = lambda: flush(work, batch.pristine)

    sb = ShardedBoundary(S, T, V, P, clip_eps=CLIP_EPS, beta=BETA, reduction=spec["reduction"],
                         length_alpha=spec["alpha"], device=dev, rows=(off, cnt))
    kernel_bytes = batch.kernel_bytes
    plan = D.plan(work, V)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    # ---- device-resident steps -------------------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    graph = None
    # --exchange peer: the pass is two launches (row kernel, reduce kernel) and the reduce kernel does the
    # exchange itself through the ranks' regions (at one rank: its own region).  --exchange nccl: four launches
    # and one NCCL all-reduce.
    peer = args.exchange == "peer"
    if peer:
        sb.enable_peer_exchange()
    one_pass = sb.step_peer if peer else sb.step_fused
    # One CUDA graph per pass at one rank.  With more ranks the pass stays two eager launches: the ranks'
    # kernels wait on one another through the exchange, and launching them the plain way keeps every rank's
    # launch independent of graph replay timing.
    if not args.no_graph and world == 1:
        restore()
        graph = sb.capture(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])

    barrier()  # ranks are lined up on the host before the first exchange of the batch
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
    # dominant kernel (with the reduce kernel behind it): its own event pair inside an eager pass.  The host
    # does not wait between iterations, so the launches are queued while the device is still restoring the
    # logits and the pair brackets device time only, not launch latency.
    kern_pairs = []
    for i in range(3 + min(args.steps, 10)):
        restore()
        if world > 1:
            dist.all_reduce(align)
        k0, k1 = ev(), ev()
        k0.record()
        one_pass(work, devt["old"], devt["ref"], devt["sel"], devt["adv"], devt["mask"])
        k1.record()
        if i >= 3:
            kern_pairs.append((k0, k1))
    barrier()
    kern_ms = [k0.elapsed_time(k1) for k0, k1 in kern_pairs]
    stats = sb.stats()  # applies the error contract to the global quantities
    loss_f64 = float(sb.result.cpu()[0])

    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    per_rank = torch.zeros(world, 2, dtype=torch.float64, device=dev)  # [rank] = (pass ms, dominant kernel ms)
    per_rank[rank, 0] = sum(step_ms) / len(step_ms)
    per_rank[rank, 1] = statistics.mean(kern_ms)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(per_rank)
    total_ms = float(total_ms.item())
    per_rank = per_rank.cpu().tolist()

    # ---- parity (untimed) --------------------------------------------------------------------
    parity = parity_block(batch, sb, one_pass, flush, world, rank)
    parity["loss"] = stats["loss"]
    parity["loss_f64"] = loss_f64

    # ---- end to end through the public API with host metadata --------------------------------
    h2d = sum(host[k].numel() * host[k].element_size() for k in host)
    cfg = G.LossConfig(CLIP_EPS, BETA, G.ReductionMode(spec["reduction"]), spec["alpha"])
    e2e_s = []
    shard = None
    if world > 1:
        # the host-facing sharded call (C ABI grpo_b200_logits_sharded_host; C++ face grpo::ShardedLogitsBoundary):
        # this rank's host metadata in, device logits in place, the global statistics out
        from grpo_cpp_b200.api import ShardedLogits
        shard = ShardedLogits(rank, world, B, Gn, T, V, P, off, cnt)
        handles = [None] * world
        dist.all_gather_object(handles, shard.handle())
        shard.connect_ipc(handles)
        sel_local = np.ascontiguousarray(batch.sel_h[off:off + cnt])
    for i in range(args.warmup + args.steps):
        restore()
        barrier()
        t0 = time.perf_counter()
        if world == 1:
            # the reference-facing call itself: host vectors in, device logits in place, stats out
            st = G.grpo_logits_cuda_device_inplace(work, batch.old_h, batch.ref_h, batch.sel_h, batch.adv_h, mask_h,
                                                   B, Gn, T, V, P, cfg)
        else:
            st = shard.run(work, batch.old_h, batch.ref_h, sel_local, batch.adv_h, batch.m_local, cfg)
        e2e_loss = st.loss
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
        # The dominant launch pair (row kernel + its dependent reduce kernel) is exactly what each timed
        # pass's event pair brackets, on the launching stream: the roofline uses those K durations.  The
        # separate eager loop above re-measures the same two launches afterwards as a cross-check.
        k_ms = statistics.mean(step_ms)
        achieved = kernel_bytes / (k_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": N * args.steps / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": spec["label"], "rows": N, "V": V, "P": P, "responses": S,
                       "tokens_per_response": T, "active_rows": int(mask_h.sum()),
                       "reduction": REDUCTION_NAMES[spec["reduction"]],
                       "parallelism": f"token-sharded x{world}", "in_place": True, "kernel": plan,
                       "inputs": "counter-based generator keyed on (seed, global row, column): the same batch at every N",
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
            "parity": parity,
            "wall_s_timed_loop": t_wall,
            "per_rank_ms": {"pass": [round(p, 4) for p, _ in per_rank], "kernel": [round(k, 4) for _, k in per_rank]},
            "clocks": clocks,
            "e2e": {"value": N * args.steps / e2e_total, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 48, "ms_per_step": 1e3 * e2e_total / args.steps, "loss": e2e_loss,
                    "api": "grpo_logits_cuda_device_inplace (host metadata, device logits)" if world == 1 else
                           "grpo_b200_logits_sharded_host (this rank's host metadata, device logits; lengths exchange, "
                           "row order, row kernel, reduce kernel with the record exchange, one read-back)"},
            # per pass and rank: the row kernel and the reduce kernel (+ lengths and weights kernels with NCCL)
            "gpu_launches": (2 if peer else 4) * args.steps * world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                         "kernel": f"logits_pipelined_kernel<{plan}> (+ reduce kernel)", "ms_per_launch": k_ms,
                         "ms_per_launch_eager_recheck": statistics.mean(kern_ms),
                         "algorithmic_bytes_per_launch": kernel_bytes,
                         # the ncu-derived figure is for the whole batch on one GPU; a rank's launch moves its share
                         "traffic": (round(TRAFFIC_BYTES[args.workload] * kernel_bytes / FULL_ALGORITHMIC[args.workload])
                                     if args.workload in TRAFFIC_BYTES else None)},
        }
    if peer:
        barrier()  # no rank unmaps a region that another rank's kernel may still write to
        sb.exchange.close()
    if shard is not None:
        barrier()
        shard.close()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    if world == 1 and not args.no_others:
        others = {}
        for name in ("v32k", "v128k_a0.5", "v128k_a1.0"):
            others[name] = other_logits_config(name, dev, flush, peak)
            torch.cuda.empty_cache()
        for name, T2, ragged in (("cfg2_1M", 256, False), ("cfg2_1M_ragged", 256, True), ("cfg2_4M", 1024, False),
                                 ("cfg2_4M_ragged", 1024, True)):
            others[name] = other_token_config(T2, ragged, dev, flush, peak)
        others["lmhead_4096"] = lmhead_config(dev, flush)
        line["other_configs"] = others
        line["reference_cuda"] = reference_cuda_leg(["v32k", "v128k_a0.5", "v128k_a1.0", "cfg2_1M", "cfg2_4M"])
        line["same_protocol_as_reference_cuda"] = same_protocol_leg(dev)
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_single(spec)
    print(json.dumps(line), flush=True)


def gradsync_arm(args) -> None:
    """`--workload gradsync`: the in-place sum of one 124,439,808-float gradient buffer per rank times
    1/world -- GPT-2 124M's parameter count, what the reference's two-GPU demo all-reduces and then scales
    (apps/05_two_gpu_gpt2_grpo.cu:216-219, 260-268) -- by the library's one kernel over NVLink peer memory,
    next to ncclAllReduce followed by a scale kernel on the same GPUs.  One JSON line from rank 0."""
    import torch
    import torch.distributed as dist
    from grpo_cpp_b200 import device as D
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    n = 124_439_808
    g = torch.empty(n, device=dev)
    src = torch.empty(n, device=dev).normal_(0.0, 1.0, generator=torch.Generator(device=dev).manual_seed(7 + rank))
    sync = D.GradSync(g, rank, world)
    handles = [None] * world
    if world > 1:
        dist.all_gather_object(handles, sync.handle)
    else:
        handles[0] = sync.handle
    sync.connect(handles)
    align = torch.zeros(1, device=dev)
    scale = 1.0 / world

    def timed(fn, passes):
        pairs = []
        for i in range(3 + passes):
            g.copy_(src)
            if world > 1:
                dist.all_reduce(align)  # lines the ranks up, outside the event pair
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            if i >= 3:
                pairs.append((e0, e1))
        torch.cuda.synchronize()
        t = torch.tensor([statistics.median(a.elapsed_time(b) for a, b in pairs)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def nccl_then_scale():
        if world > 1:
            dist.all_reduce(g)
        g.mul_(scale)

    ours_ms = timed(lambda: sync.allreduce_scale(scale), args.steps)
    ours = g.clone()
    nccl_ms = timed(nccl_then_scale, args.steps)
    same = bool(torch.equal(ours, g)) if world <= 2 else None  # beyond two ranks NCCL's order of additions is its own
    max_diff = float((ours - g).abs().max().item())
    timed_out = sync.timed_out()
    if world > 1:
        dist.barrier()
    sync.close()
    if rank == 0:
        link_bytes = 2 * 4 * n * (world - 1) / world  # per rank and direction: in, the peers' terms of its slice and their results; out, the mirror image
        print(json.dumps({
            "metric": "gradient all-reduce + 1/world scale, ms per call", "workload": "gradsync", "n_gpus": world,
            "floats": n, "steps": args.steps, "fused_kernel_ms": ours_ms, "nccl_allreduce_plus_scale_ms": nccl_ms,
            "speedup_vs_nccl_plus_scale": nccl_ms / ours_ms if ours_ms else None,
            "nvlink_bytes_per_rank_per_direction": link_bytes,
            "nvlink_gbs_per_direction": link_bytes / (ours_ms * 1e-3) / 1e9 if world > 1 else None,
            "nvlink_roofline": {"peak_gbs_per_direction": 770.0, "frac": (link_bytes / (ours_ms * 1e-3) / 1e9 / 770.0) if world > 1 else None,
                                "note": "measured peer-copy bandwidth of this pool; nominal 900"},
            "hbm_gbs_at_one_rank": (2 * 4 * n / (ours_ms * 1e-3) / 1e9) if world == 1 else None,
            "bit_identical_to_nccl_plus_scale": same, "max_abs_diff_vs_nccl_plus_scale": max_diff,
            "timed_out": timed_out}), flush=True)
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
    tune = ap.add_argument_group("tuning and profiling (not used by the default run)")
    tune.add_argument("--workload", default="gpt2", choices=["gpt2", "v32k", "v128k_a0.5", "v128k_a1.0", "gradsync"],
                      help="which configuration the headline line measures; gradsync: the fused gradient "
                           "all-reduce + scale kernel against NCCL + scale (a line of its own)")
    tune.add_argument("--prompts", type=int, default=None,
                      help="override the workload's number of prompts B (rows = B x G x T): the same row shape at "
                           "another batch size, e.g. a few thousand rows for a multi-pass profiler capture")
    tune.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    tune.add_argument("--no-others", action="store_true",
                      help="skip the other configurations and the reference-CUDA leg (one GPU only)")
    tune.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                      help="at more than one rank: the pass's exchange by the library's own kernel over NVLink peer "
                           "memory, or by one NCCL all-reduce")
    tune.add_argument("--no-graph", action="store_true", help="launch each pass eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    import grpo_cpp_b200  # noqa: F401  (registers the package under its importable name)
    if args.workload == "gradsync":
        if args.impl == "b200":
            gradsync_arm(args)
        return
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
