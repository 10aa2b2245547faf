"""Token-sharded execution of the logits path over ``torch.distributed`` (one process per GPU).

The batch of ``N = S*T`` token rows is cut into contiguous row ranges, one per rank; a response
may straddle two ranks.  Rows are independent given the per-response weight, so the ranks only
have to agree on two tiny things, both plain sums over ranks:

1. the per-response valid-token counts (``S`` numbers), so that every rank derives the same
   global lengths, the same token-count normaliser and the same weights;
2. the result record (``float64[5]``: loss, pg, kl and the two error counts).

Three ways to take the sums, by decreasing cost: :meth:`ShardedBoundary.step` (two all-reduces, no
look-ahead), :meth:`~ShardedBoundary.step_fused` (one all-reduce per pass: the next pass's counts
ride with this pass's record) and :meth:`~ShardedBoundary.step_peer` (no collective call: the
pass's last kernel exchanges both through NVLink peer memory and also writes the next weights).

``dL/dlogits`` needs no communication.  The reference has no collective inside its loss path: its
two-GPU demo shards whole responses under ``sequence_mean`` and divides by the device count on
the host (apps/03_two_gpu_train.cu:200-215,247-281); token sharding with ``token_mean`` or
``length_weighted`` needs the global lengths, which is what exchange 1 provides.

``prepare`` depends only on the mask, so it runs once per rollout batch; ``step`` runs once per
optimisation pass over that batch.  ``prepare`` also partitions the local rows into active and
masked ones, which lets the row kernel deal its clusters equal loads.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .api import CudaLogitsKernel, ReductionMode


def shard_rows(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """``(row_offset, row_count)`` of ``rank``: contiguous, sizes differ by at most one row."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must lie in [0, world)")
    base, rem = divmod(n_rows, world)
    return rank * base + min(rank, rem), base + (1 if rank < rem else 0)


def shard_rows_balanced(mask, world: int, V: int, P: int, masked_cost: float = 0.8) -> list[tuple[int, int]]:
    """Contiguous row ranges ``[(row_offset, row_count), ...]`` of nearly equal kernel time.

    An active row moves ``V + P`` floats (one read, one write), a masked row ``P`` (zeros written,
    nothing read), so with ragged masks equal row counts are not equal work: the rank that happens
    to hold the longest responses finishes last and everyone waits for it in the result exchange.
    A masked row's plain zero-fill also runs nearer to the memory rate than an active row's
    read-compute-write, so it is charged ``masked_cost * P`` (0.8 fits the row kernel's measured
    times on the GPT-2-shaped batch: a masked row costs about 0.4 of an active one).
    ``mask`` is the whole batch's host mask; every rank computes the same cut points from it."""
    import numpy as np
    m = np.asarray(mask).reshape(-1) != 0
    cost = np.where(m, float(V + P), masked_cost * P)
    prefix = np.concatenate(([0.0], np.cumsum(cost)))
    total = float(prefix[-1])
    cuts = [0]
    for r in range(1, world):
        target = total * r / world
        cut = int(np.searchsorted(prefix, target, side="left"))
        cuts.append(min(max(cut, cuts[-1]), m.size))
    cuts.append(m.size)
    return [(cuts[r], cuts[r + 1] - cuts[r]) for r in range(world)]


def global_group_advantages(local_rewards: torch.Tensor, n_prompts: int, local_G: int, *, mode: int = 0,
                            eps: float = 1e-8, group=None, ops=None):
    """Group-relative advantages when every rank rolled out ``local_G`` of each prompt's responses.

    ``local_rewards`` is ``[n_prompts * local_G]`` (prompt-major).  The ranks all-gather their rewards,
    lay them out as the global groups ``[prompt][source rank][g]`` -- the layout of the reference's
    two-GPU GPT-2 demo (apps/05_two_gpu_gpt2_grpo.cu:168-202) -- compute the advantages of the whole
    groups with the library's kernel (the reference does this step on the host), and return this
    rank's slice ``[n_prompts * local_G]`` plus the count of non-finite values.  Everything stays on
    the device; the one collective is the all-gather of ``n_prompts * local_G`` floats."""
    if ops is None:
        from . import device as ops  # the CUDA library; fails loudly when it is missing
    if local_rewards.numel() != n_prompts * local_G:
        raise RuntimeError(f"rewards has size {local_rewards.numel()}, expected {n_prompts * local_G}")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    gathered = torch.empty(world, n_prompts, local_G, dtype=local_rewards.dtype, device=local_rewards.device)
    if world > 1:
        dist.all_gather_into_tensor(gathered.view(-1), local_rewards.contiguous().view(-1), group=group)
    else:
        gathered.view(-1).copy_(local_rewards.view(-1))
    global_rewards = gathered.permute(1, 0, 2).contiguous().view(-1)  # [prompt][source][g]
    adv, meta = ops.group_advantages(global_rewards, n_prompts, world * local_G, mode, eps)
    mine = adv.view(n_prompts, world, local_G)[:, rank, :].contiguous().view(-1)
    return mine, meta


class ShardedBoundary:
    """One rank's view of the sharded loss boundary.

    ``ops`` is the module providing ``count_lengths``, ``weights_from_lengths``, ``logits``,
    ``new_result`` and ``logits_workspace`` (default: :mod:`.device`, the CUDA library).  The
    indirection exists so that the rank logic -- offsets, exchanges, error propagation -- can be
    exercised with CPU tensors over the ``gloo`` backend.
    """

    def __init__(self, n_seq: int, tokens_per_seq: int, V: int, P: int, *, clip_eps: float = 0.2,
                 beta: float = 0.0, reduction: int = ReductionMode.token_mean, length_alpha: float = 0.0,
                 group=None, ops=None, device=None, rows: tuple[int, int] | None = None):
        if ops is None:
            from . import device as ops  # the CUDA library; fails loudly when it is missing
        self.ops = ops
        self.S, self.T, self.V, self.P = n_seq, tokens_per_seq, V, P
        self.clip_eps, self.beta, self.reduction, self.alpha = clip_eps, beta, int(reduction), length_alpha
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # `rows` overrides the equal-count split (e.g. one entry of shard_rows_balanced)
        self.row_offset, self.n_local = rows if rows is not None else shard_rows(
            n_seq * tokens_per_seq, self.world, self.rank)
        self.device = device
        self.lengths = torch.zeros(n_seq, dtype=torch.int32, device=device)
        self.weights = torch.zeros(n_seq, dtype=torch.float32, device=device)
        self.meta = torch.zeros(2, dtype=torch.int32, device=device)
        # one buffer for everything a pass exchanges: [0:5) the result record, [5:5+S) partial lengths
        self.xchg = torch.zeros(5 + n_seq, dtype=torch.float64, device=device)
        self.result = self.xchg[:5]
        self.lengths_f64 = self.xchg[5:]
        self.workspace = ops.logits_workspace(self.n_local, device)
        # the record of prepare()'s own exchange: zeros unless a rank did not answer (bad_inputs = -2)
        self.prepare_status = torch.zeros(5, dtype=torch.float64, device=device)
        self.exchange = None  # set by enable_peer_exchange
        self.row_order = None  # set by prepare: the upcoming pass's balanced row order

    def _all_reduce(self, t: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def prepare(self, mask_local: torch.Tensor) -> None:
        """Exchange 1: global lengths and weights from this rank's slice of the mask."""
        if mask_local.numel() != self.n_local:
            raise RuntimeError(f"mask has size {mask_local.numel()}, expected {self.n_local}")
        if self.exchange is not None:  # through the ranks' regions: no collective call
            self.ops.lengths_sharded(mask_local, self.S, self.T, self.row_offset, exchange=self.exchange,
                                     reduction=self.reduction, length_alpha=self.alpha, weights=self.weights,
                                     meta=self.meta, workspace=self.workspace, status=self.prepare_status,
                                     lengths=self.lengths_f64)
        else:
            self.ops.count_lengths(mask_local, self.S, self.T, self.row_offset, self.lengths)
            self._all_reduce(self.lengths)
            self.ops.weights_from_lengths(self.lengths, self.reduction, self.alpha, self.weights, self.meta)
        self.row_order = self.ops.row_order(mask_local, self.row_order)

    def step(self, logits_local, logp_old, logp_ref, selected, advantages, mask_local,
             kernel: int = CudaLogitsKernel.fused) -> torch.Tensor:
        """Kernel on the local rows (in place), then exchange 2.  Returns the global result record."""
        self.ops.logits(logits_local, logp_old, logp_ref, selected, advantages, self.weights, mask_local,
                        self.T, self.V, self.clip_eps, self.beta, row_offset=self.row_offset, kernel=kernel,
                        result=self.result, workspace=self.workspace, row_order=self.row_order)
        self._all_reduce(self.result)
        return self.result

    def step_fused(self, logits_local, logp_old, logp_ref, selected, advantages, mask_local,
                   next_mask_local=None, kernel: int = CudaLogitsKernel.fused) -> torch.Tensor:
        """One pass with ONE collective.  The weights in use come from the previous call (or from
        ``prepare``); the partial lengths of the NEXT pass's mask (the same mask when the batch is
        passed over again) ride in the same all-reduce as this pass's result record, and the next
        pass's weights are derived right after it.  Masks are known long before their logits exist
        -- rollouts precede the forward pass -- so nothing waits on anything new."""
        nxt = mask_local if next_mask_local is None else next_mask_local
        if nxt.numel() != self.n_local:
            raise RuntimeError(f"mask has size {nxt.numel()}, expected {self.n_local}")
        self.ops.count_lengths_f64(nxt, self.S, self.T, self.row_offset, self.lengths_f64)
        self.ops.logits(logits_local, logp_old, logp_ref, selected, advantages, self.weights, mask_local,
                        self.T, self.V, self.clip_eps, self.beta, row_offset=self.row_offset, kernel=kernel,
                        result=self.result, workspace=self.workspace, row_order=self.row_order)
        self._all_reduce(self.xchg)
        self.ops.weights_from_lengths_f64(self.lengths_f64, self.reduction, self.alpha, self.weights, self.meta)
        if next_mask_local is not None:
            self.row_order = self.ops.row_order(next_mask_local, self.row_order)
        return self.result

    def enable_peer_exchange(self) -> None:
        """Set up the library's own exchange over NVLink peer memory (CUDA ranks of one box, at most
        eight): every rank creates its region, the 64-byte handles go round through the process
        group, every rank maps the others' regions.  Afterwards :meth:`step_peer` needs no
        collective call at all."""
        self.exchange = self.ops.PeerExchange(self.S, self.rank, self.world)
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, self.exchange.handle, group=self.group)
        else:
            handles[0] = self.exchange.handle
        self.exchange.open_peers(handles)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody starts a pass before every region is mapped everywhere

    def step_peer(self, logits_local, logp_old, logp_ref, selected, advantages, mask_local,
                  next_mask_local=None, kernel: int = CudaLogitsKernel.fused) -> torch.Tensor:
        """:meth:`step_fused` without a collective call and with two launches per pass: the row
        kernel, then the reduce kernel, which also counts the next mask's valid tokens, exchanges
        them together with the result record through the ranks' regions, and writes the next
        pass's weights.  Works at world size 1 too (the region is then this rank's alone)."""
        nxt = mask_local if next_mask_local is None else next_mask_local
        if nxt.numel() != self.n_local:
            raise RuntimeError(f"mask has size {nxt.numel()}, expected {self.n_local}")
        self.ops.logits_sharded(logits_local, logp_old, logp_ref, selected, advantages, self.weights, mask_local,
                                self.T, self.V, self.clip_eps, self.beta, exchange=self.exchange, next_mask=nxt,
                                reduction=self.reduction, length_alpha=self.alpha, next_weights=self.weights,
                                next_meta=self.meta, next_lengths=self.lengths_f64, result=self.result,
                                workspace=self.workspace, row_offset=self.row_offset, kernel=kernel,
                                row_order=self.row_order)
        if next_mask_local is not None:
            self.row_order = self.ops.row_order(next_mask_local, self.row_order)
        return self.result

    def capture(self, logits_local, logp_old, logp_ref, selected, advantages, mask_local,
                kernel: int = CudaLogitsKernel.fused):
        """Record one pass (``step_peer`` when the exchange is enabled, else ``step_fused``) over these (fixed-address) tensors into a CUDA graph, so that a
        pass is one graph launch and its small launches do not wait on host dispatch.
        One eager pass runs first (kernel attributes, occupancy queries and NCCL set-up must not
        happen under capture); it consumes the logits in place like any pass."""
        one_pass = self.step_peer if self.exchange is not None else self.step_fused
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.prepare(mask_local)
            one_pass(logits_local, logp_old, logp_ref, selected, advantages, mask_local, None, kernel)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass(logits_local, logp_old, logp_ref, selected, advantages, mask_local, None, kernel)
        return graph

    def stats(self) -> dict:
        """Reads the records back (synchronises) and applies the reference's error contract
        (src/cuda/grpo_loss_cuda.cu:44-46, 814-815) to the GLOBAL quantities."""
        # one read-back: the pass's record, prepare()'s record and the two counters
        host = torch.cat([self.result, self.prepare_status, self.meta.to(torch.float64)]).tolist()
        res, prep, meta = host[:5], host[5:10], [int(host[10]), int(host[11])]
        if prep[4] < 0:  # the lengths exchange itself failed: the weights came from partial counts
            raise RuntimeError("the exchange between ranks timed out")
        if res[4] < 0:
            raise RuntimeError({-1.0: "a pipeline wait timed out on some rank",
                                -2.0: "the exchange between ranks timed out"}.get(
                                    res[4], "the row order does not belong to the mask"))
        if meta[1] != 0:
            raise RuntimeError("every sequence needs at least one valid token")
        if res[4] != 0:
            raise RuntimeError("selected token is outside the vocabulary")
        loss, pg, kl = (float(torch.tensor(v, dtype=torch.float64).to(torch.float32)) for v in res[:3])
        if not all(map(_finite, (loss, pg, kl))):
            raise RuntimeError("CUDA logits loss became non-finite")
        return {"loss": loss, "pg_loss": pg, "kl": kl, "valid_tokens": int(meta[0]), "bad_grads": int(res[3])}


def _finite(x: float) -> bool:
    return x == x and abs(x) != float("inf")
