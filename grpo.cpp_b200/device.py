"""Device layer of the C ABI on torch CUDA tensors.

torch supplies device memory and the current stream; every computation below is a kernel of
``libgrpo_b200.so`` enqueued on that stream through the C ABI (``include/grpo_b200.h``).  Nothing
here synchronises or copies to the host; results stay in a device record of five doubles
``[loss, pg_loss, kl, bad_grads, bad_inputs]``.

The calls replace, with everything resident on the device, what the reference does per call on
the host plus its kernels: make_weights (src/cuda/grpo_loss_cuda.cu:21-57), launch_loss (:527-549)
and launch_logits (:551-582).
"""
from __future__ import annotations

import torch

from . import _lib
from .api import CudaLogitsKernel, ReductionMode

RESULT_FIELDS = ("loss", "pg_loss", "kl", "bad_grads", "bad_inputs")


def _check_tensor(t: torch.Tensor, dtype, name: str) -> int:
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise TypeError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def new_result(device=None) -> torch.Tensor:
    return torch.zeros(5, dtype=torch.float64, device=device or torch.cuda.current_device())


def count_lengths(mask: torch.Tensor, n_seq: int, tokens_per_seq: int, row_offset: int = 0,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """Valid tokens per response among the local rows ``[row_offset, row_offset + len(mask))``."""
    m = _check_tensor(mask, torch.int32, "mask")
    if out is None:
        out = torch.empty(n_seq, dtype=torch.int32, device=mask.device)
    o = _check_tensor(out, torch.int32, "lengths")
    _lib.check(_lib.lib().grpo_b200_count_lengths(m, mask.numel(), row_offset, tokens_per_seq, n_seq, o, _stream()))
    return out


def weights_from_lengths(lengths: torch.Tensor, reduction: int, length_alpha: float = 0.0,
                         out: torch.Tensor | None = None, meta: torch.Tensor | None = None):
    """Per-response weights from global lengths; ``meta = [valid_tokens, empty_responses]`` (int32)."""
    l = _check_tensor(lengths, torch.int32, "lengths")
    if out is None:
        out = torch.empty(lengths.numel(), dtype=torch.float32, device=lengths.device)
    if meta is None:
        meta = torch.zeros(2, dtype=torch.int32, device=lengths.device)
    _lib.check(_lib.lib().grpo_b200_weights_from_lengths(
        l, lengths.numel(), int(reduction), float(length_alpha), _check_tensor(out, torch.float32, "weights"),
        _check_tensor(meta, torch.int32, "meta"), _stream()))
    return out, meta


def count_lengths_f64(mask: torch.Tensor, n_seq: int, tokens_per_seq: int, row_offset: int, out: torch.Tensor):
    """As :func:`count_lengths`, writing doubles into ``out[n_seq]`` (a slice of an exchange buffer)."""
    _lib.check(_lib.lib().grpo_b200_count_lengths_f64(_check_tensor(mask, torch.int32, "mask"), mask.numel(),
                                                     row_offset, tokens_per_seq, n_seq,
                                                     _check_tensor(out, torch.float64, "lengths"), _stream()))
    return out


def weights_from_lengths_f64(lengths: torch.Tensor, reduction: int, length_alpha: float, out: torch.Tensor,
                             meta: torch.Tensor):
    """As :func:`weights_from_lengths`, reading the (summed) lengths as doubles."""
    _lib.check(_lib.lib().grpo_b200_weights_from_lengths_f64(
        _check_tensor(lengths, torch.float64, "lengths"), lengths.numel(), int(reduction), float(length_alpha),
        _check_tensor(out, torch.float32, "weights"), _check_tensor(meta, torch.int32, "meta"), _stream()))
    return out, meta


def group_advantages(rewards: torch.Tensor, B: int, G: int, mode: int = 0, eps: float = 1e-8):
    """Group-relative advantages ``[B*G]``; ``meta[0]`` counts non-finite rewards/advantages."""
    r = _check_tensor(rewards, torch.float32, "rewards")
    if rewards.numel() != B * G:
        raise RuntimeError(f"rewards has size {rewards.numel()}, expected {B * G}")
    out = torch.empty(B * G, dtype=torch.float32, device=rewards.device)
    meta = torch.zeros(1, dtype=torch.int32, device=rewards.device)
    _lib.check(_lib.lib().grpo_b200_group_advantages(r, B, G, int(mode), float(eps), out.data_ptr(),
                                                    meta.data_ptr(), _stream()))
    return out, meta


def loss_workspace(device=None) -> torch.Tensor:
    n = _lib.lib().grpo_b200_loss_workspace_bytes(1)
    return torch.empty(n, dtype=torch.uint8, device=device or torch.cuda.current_device())


def loss(logp_new, logp_old, logp_ref, advantages, weights, mask, tokens_per_seq: int, clip_eps: float,
         beta: float, *, token_offset: int = 0, dlogp: torch.Tensor | None = None,
         result: torch.Tensor | None = None, workspace: torch.Tensor | None = None):
    """Selected-token path on device tensors.  Returns ``(dlogp, result)``."""
    n = logp_new.numel()
    if dlogp is None:
        dlogp = torch.empty(n, dtype=torch.float32, device=logp_new.device)
    if result is None:
        result = new_result(logp_new.device)
    if workspace is None:
        workspace = loss_workspace(logp_new.device)
    _lib.check(_lib.lib().grpo_b200_loss(
        _check_tensor(logp_new, torch.float32, "logp_new"), _check_tensor(logp_old, torch.float32, "logp_old"),
        _check_tensor(logp_ref, torch.float32, "logp_ref"), _check_tensor(advantages, torch.float32, "advantages"),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(mask, torch.int32, "mask"),
        n, token_offset, tokens_per_seq, float(clip_eps), float(beta),
        _check_tensor(dlogp, torch.float32, "dlogp"), _check_tensor(result, torch.float64, "result"),
        workspace.data_ptr(), workspace.numel(), _stream()))
    return dlogp, result


def loss_noalloc(logp_new, logp_old, logp_ref, advantages, weights, mask, tokens_per_seq: int, clip_eps: float,
                 beta: float, *, dlogp: torch.Tensor, result: torch.Tensor, token_offset: int = 0):
    """Selected-token path through ``grpo_b200_loss_noalloc``: the caller passes inputs and outputs
    only (``dlogp`` and ``result`` must already exist); the library's own scratch array holds the
    partial sums.  At most 16,777,216 tokens per call; calls that may overlap on the GPU race."""
    _lib.check(_lib.lib().grpo_b200_loss_noalloc(
        _check_tensor(logp_new, torch.float32, "logp_new"), _check_tensor(logp_old, torch.float32, "logp_old"),
        _check_tensor(logp_ref, torch.float32, "logp_ref"), _check_tensor(advantages, torch.float32, "advantages"),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(mask, torch.int32, "mask"),
        logp_new.numel(), token_offset, tokens_per_seq, float(clip_eps), float(beta),
        _check_tensor(dlogp, torch.float32, "dlogp"), _check_tensor(result, torch.float64, "result"), _stream()))
    return dlogp, result


def logits_workspace(n_rows: int, device=None) -> torch.Tensor:
    n = _lib.lib().grpo_b200_logits_workspace_bytes(n_rows)
    return torch.empty(n, dtype=torch.uint8, device=device or torch.cuda.current_device())


def logits(logits_t: torch.Tensor, logp_old, logp_ref, selected, advantages, weights, mask,
           tokens_per_seq: int, V: int, clip_eps: float, beta: float, *, dlogits: torch.Tensor | None = None,
           row_offset: int = 0, kernel: int = CudaLogitsKernel.fused, check_inputs: bool = False,
           selected_logp: torch.Tensor | None = None, result: torch.Tensor | None = None,
           workspace: torch.Tensor | None = None, row_order: torch.Tensor | None = None) -> torch.Tensor:
    """Logits path on device tensors: ``logits_t`` is ``[n_rows, P]`` fp32; ``dlogits=None`` means in
    place.  ``row_order`` (from :func:`row_order` on the same mask) balances the rows over the
    clusters.  Returns the result record."""
    if logits_t.dim() != 2:
        raise ValueError("logits must be [n_rows, P]")
    n_rows, P = logits_t.shape
    x = _check_tensor(logits_t, torch.float32, "logits")
    d = x if dlogits is None else _check_tensor(dlogits, torch.float32, "dlogits")
    if dlogits is not None and tuple(dlogits.shape) != (n_rows, P):
        raise ValueError("dlogits must have the shape of logits")
    if result is None:
        result = new_result(logits_t.device)
    if workspace is None:
        workspace = logits_workspace(n_rows, logits_t.device)
    _lib.check(_lib.lib().grpo_b200_logits(
        x, d, _check_tensor(logp_old, torch.float32, "logp_old"), _check_tensor(logp_ref, torch.float32, "logp_ref"),
        _check_tensor(selected, torch.int32, "selected"), _check_tensor(advantages, torch.float32, "advantages"),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(mask, torch.int32, "mask"),
        n_rows, row_offset, tokens_per_seq, V, P, float(clip_eps), float(beta), int(kernel), int(check_inputs),
        None if selected_logp is None else _check_tensor(selected_logp, torch.float32, "selected_logp"),
        _order_ptr(row_order, n_rows),
        _check_tensor(result, torch.float64, "result"), workspace.data_ptr(), workspace.numel(), _stream()))
    return result


def _order_ptr(row_order, n_rows: int):
    if row_order is None:
        return None
    if row_order.numel() != _lib.lib().grpo_b200_row_order_bytes(n_rows) // 4:
        raise ValueError("row_order must come from row_order() on a mask over the same rows")
    return _check_tensor(row_order, torch.int32, "row_order")


def row_order(mask: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``[n_active, n_masked, active rows..., masked rows...]`` (int32, ``len(mask) + 2`` entries and a
    scratch tail): the stable partition of the local row indices by ``mask`` that :func:`logits`
    takes as ``row_order``."""
    m = _check_tensor(mask, torch.int32, "mask")
    if out is None:
        out = torch.empty(_lib.lib().grpo_b200_row_order_bytes(mask.numel()) // 4, dtype=torch.int32,
                          device=mask.device)
    _lib.check(_lib.lib().grpo_b200_row_order(m, mask.numel(), _check_tensor(out, torch.int32, "row_order"), _stream()))
    return out


class PeerExchange:
    """This rank's exchange region plus the other ranks' regions mapped into this process.

    ``handle`` (64 bytes) is what the ranks trade; ``open_peers`` takes the list of all ranks'
    handles in rank order.  The region belongs to one :class:`~.sharded.ShardedBoundary`: it counts its
    passes on the device, and every rank must make the same sequence of calls (``passes`` mirrors the
    count on the host for bookkeeping only)."""

    def __init__(self, n_seq: int, rank: int, world: int):
        import ctypes as C
        if not (1 <= world <= 8 and 0 <= rank < world):
            raise ValueError("world must lie in [1, 8] and rank in [0, world)")
        self.n_seq, self.rank, self.world = n_seq, rank, world
        region = C.c_void_p()
        _lib.check(_lib.lib().grpo_b200_exchange_create(n_seq, C.byref(region)))
        self.own = region.value
        buf = C.create_string_buffer(64)
        _lib.check(_lib.lib().grpo_b200_exchange_export(self.own, buf))
        self.handle = buf.raw
        self.regions = (C.c_void_p * world)()
        self.regions[rank] = self.own
        self.passes = 0
        self._opened = []

    def open_peers(self, handles: list[bytes]) -> None:
        import ctypes as C
        if len(handles) != self.world:
            raise ValueError("one handle per rank, in rank order")
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            peer = C.c_void_p()
            _lib.check(_lib.lib().grpo_b200_exchange_open(C.create_string_buffer(bytes(h), 64), C.byref(peer)))
            self.regions[r] = peer.value
            self._opened.append(peer.value)

    def close(self) -> None:
        for p in self._opened:
            _lib.lib().grpo_b200_exchange_close(p)
        self._opened = []
        if self.own:
            _lib.lib().grpo_b200_exchange_destroy(self.own)
            self.own = None


def logits_sharded(logits_t: torch.Tensor, logp_old, logp_ref, selected, advantages, weights, mask,
                   tokens_per_seq: int, V: int, clip_eps: float, beta: float, *, exchange: PeerExchange,
                   next_mask: torch.Tensor, reduction: int, length_alpha: float, next_weights: torch.Tensor,
                   next_meta: torch.Tensor, result: torch.Tensor, workspace: torch.Tensor,
                   next_lengths: torch.Tensor | None = None, row_offset: int = 0,
                   kernel: int = CudaLogitsKernel.fused, check_inputs: bool = False,
                   selected_logp: torch.Tensor | None = None, row_order: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`logits` in place on this rank's rows; the pass's last kernel also counts ``next_mask``'s
    valid tokens, sums the result record and the counts over the ranks through their exchange
    regions, and writes the next pass's weights (``next_weights`` may be ``weights``) and
    ``next_meta = [valid_tokens, empty_responses]``."""
    n_rows, P = logits_t.shape
    x = _check_tensor(logits_t, torch.float32, "logits")
    if next_mask.numel() != n_rows:
        raise ValueError("next_mask must cover the same rows as mask")
    if next_weights.numel() != exchange.n_seq:
        raise ValueError("next_weights must hold one entry per response of the exchange region")
    exchange.passes += 1
    _lib.check(_lib.lib().grpo_b200_logits_sharded(
        x, x, _check_tensor(logp_old, torch.float32, "logp_old"), _check_tensor(logp_ref, torch.float32, "logp_ref"),
        _check_tensor(selected, torch.int32, "selected"), _check_tensor(advantages, torch.float32, "advantages"),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(mask, torch.int32, "mask"),
        n_rows, row_offset, tokens_per_seq, V, P, float(clip_eps), float(beta), int(kernel), int(check_inputs),
        None if selected_logp is None else _check_tensor(selected_logp, torch.float32, "selected_logp"),
        _order_ptr(row_order, n_rows),
        _check_tensor(result, torch.float64, "result"), workspace.data_ptr(), workspace.numel(),
        exchange.regions, exchange.rank, exchange.world, exchange.n_seq,
        _check_tensor(next_mask, torch.int32, "next_mask"), int(reduction), float(length_alpha),
        _check_tensor(next_weights, torch.float32, "next_weights"), _check_tensor(next_meta, torch.int32, "next_meta"),
        None if next_lengths is None else _check_tensor(next_lengths, torch.float64, "next_lengths"), _stream()))
    return result


def lengths_sharded(mask: torch.Tensor, n_seq: int, tokens_per_seq: int, row_offset: int, *, exchange: PeerExchange,
                    reduction: int, length_alpha: float, weights: torch.Tensor, meta: torch.Tensor,
                    workspace: torch.Tensor, status: torch.Tensor, lengths: torch.Tensor | None = None) -> torch.Tensor:
    """Global per-response lengths of ``mask`` (this rank's rows) summed over the ranks through their
    exchange regions, and the weights derived from them: what the first pass needs, without a
    collective call.  ``status`` (five doubles) receives the exchanged record: zeros, or
    ``bad_inputs = -2`` when a rank did not answer in time.  Counts as one pass of the region."""
    if n_seq != exchange.n_seq:
        raise ValueError(f"n_seq is {n_seq} but the exchange region was created for {exchange.n_seq} responses")
    exchange.passes += 1
    _lib.check(_lib.lib().grpo_b200_lengths_sharded(
        _check_tensor(mask, torch.int32, "mask"), mask.numel(), row_offset, tokens_per_seq, n_seq, exchange.regions,
        exchange.rank, exchange.world, int(reduction), float(length_alpha),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(meta, torch.int32, "meta"),
        None if lengths is None else _check_tensor(lengths, torch.float64, "lengths"),
        _check_tensor(status, torch.float64, "status"), workspace.data_ptr(), workspace.numel(), _stream()))
    return weights


def set_exchange_timeout_cycles(cycles: int) -> None:
    """Process-wide limit of the exchange's wait for the other ranks, in SM clock cycles."""
    _lib.check(_lib.lib().grpo_b200_exchange_set_timeout_cycles(int(cycles)))


def synthetic_logits(out: torch.Tensor, V: int, scale: float, seed: int, *, row_offset: int = 0,
                     tail_fill: float = 123.0) -> torch.Tensor:
    """Fills ``out`` (``[n_rows, P]`` fp32) with the counter-based synthetic logits of global rows
    ``[row_offset, row_offset + n_rows)``; :func:`..workloads.synthetic_logits_rows` is the host
    restatement of the same function."""
    n_rows, P = out.shape
    _lib.check(_lib.lib().grpo_b200_synthetic_logits(_check_tensor(out, torch.float32, "logits"), n_rows, row_offset,
                                                    V, P, float(scale), int(seed), float(tail_fill), _stream()))
    return out


def sample_rows(logits_t: torch.Tensor, V: int, rows: torch.Tensor, *, coins: torch.Tensor | None = None,
                tokens: torch.Tensor | None = None):
    """For the rows of ``logits_t`` (``[n_rows, P]`` fp32) named in ``rows`` (int32): the row
    log-sum-exp (float64), a token per row -- drawn by inverse CDF from ``coins`` (float64 uniforms in
    [0, 1)) or taken from ``tokens`` (int32) -- and its fp32 log-probability.  Returns
    ``(tokens, logp, lse)``; nothing but these few numbers needs to leave the device."""
    n_rows, P = logits_t.shape
    n = rows.numel()
    dev = logits_t.device
    out_tokens = torch.empty(n, dtype=torch.int32, device=dev) if coins is not None else None
    logp = torch.empty(n, dtype=torch.float32, device=dev)
    lse = torch.empty(n, dtype=torch.float64, device=dev)
    _lib.check(_lib.lib().grpo_b200_sample_rows(
        _check_tensor(logits_t, torch.float32, "logits"), n_rows, V, P, _check_tensor(rows, torch.int32, "rows"), n,
        None if coins is None else _check_tensor(coins, torch.float64, "coins"),
        None if tokens is None else _check_tensor(tokens, torch.int32, "tokens"),
        None if out_tokens is None else out_tokens.data_ptr(), logp.data_ptr(), lse.data_ptr(), _stream()))
    return (out_tokens if coins is not None else tokens), logp, lse


def set_variant(variant: int) -> None:
    """Force a row-resident kernel variant (index into :func:`variants`), ``-1`` for automatic."""
    _lib.check(_lib.lib().grpo_b200_logits_set_variant(variant))


def variants() -> list[str]:
    out, i = [], 0
    while True:
        name = _lib.lib().grpo_b200_logits_variant_name(i)
        if name is None:
            return out
        out.append(name.decode())
        i += 1


def plan(logits_t: torch.Tensor, V: int, kernel: int = CudaLogitsKernel.fused,
         dlogits: torch.Tensor | None = None) -> str:
    """Name of the kernel the dispatcher runs for this layout."""
    d = logits_t if dlogits is None else dlogits
    return _lib.lib().grpo_b200_logits_plan(logits_t.data_ptr(), d.data_ptr(), V, logits_t.shape[1],
                                            logits_t.shape[0], int(kernel)).decode()


class ResidentBoundary:
    """The whole loss boundary with nothing on the host: mask -> lengths -> weights -> fused logits
    kernel -> result record, all enqueued on the current stream.  Buffers are allocated once."""

    def __init__(self, n_seq: int, tokens_per_seq: int, V: int, P: int, *, clip_eps: float = 0.2,
                 beta: float = 0.0, reduction: int = ReductionMode.sequence_mean, length_alpha: float = 0.0,
                 device=None):
        self.S, self.T, self.V, self.P = n_seq, tokens_per_seq, V, P
        self.clip_eps, self.beta, self.reduction, self.alpha = clip_eps, beta, int(reduction), length_alpha
        dev = device or torch.cuda.current_device()
        self.lengths = torch.empty(n_seq, dtype=torch.int32, device=dev)
        self.weights = torch.empty(n_seq, dtype=torch.float32, device=dev)
        self.meta = torch.zeros(2, dtype=torch.int32, device=dev)
        self.result = new_result(dev)
        self.workspace = logits_workspace(n_seq * tokens_per_seq, dev)

    def __call__(self, logits_t, logp_old, logp_ref, selected, advantages, mask,
                 kernel: int = CudaLogitsKernel.fused) -> torch.Tensor:
        count_lengths(mask, self.S, self.T, 0, self.lengths)
        weights_from_lengths(self.lengths, self.reduction, self.alpha, self.weights, self.meta)
        return logits(logits_t, logp_old, logp_ref, selected, advantages, self.weights, mask, self.T, self.V,
                      self.clip_eps, self.beta, kernel=kernel, result=self.result, workspace=self.workspace)


def gradsync_slice(n: int, world: int, rank: int) -> tuple[int, int]:
    """``(first, count)`` in floats of the slice rank ``rank`` reduces in :class:`GradSync` (the
    library's own arithmetic: whole float4s, the last rank takes the tail).  Needs no device."""
    import ctypes as C
    first, count = C.c_int64(), C.c_int64()
    _lib.lib().grpo_b200_gradsync_slice(n, world, rank, C.byref(first), C.byref(count))
    return first.value, count.value


class GradSync:
    """In-place sum of one fp32 buffer per rank times ``scale``, by the library's own kernel over
    NVLink peer memory (``grpo_b200_allreduce_scale``): what the reference's two-GPU GPT-2 demo does
    with ncclAllReduce followed by scale_kernel (apps/05_two_gpu_gpt2_grpo.cu:216-219, 260-268).
    ``grads`` is this rank's flat fp32 CUDA tensor; every rank registers a buffer of the same size,
    the ranks trade :attr:`handle` (192 bytes) and call :meth:`connect`."""

    def __init__(self, grads: torch.Tensor, rank: int, world: int):
        import ctypes as C
        self.grads, self.rank, self.world = grads, rank, world
        self._h = C.c_void_p()
        _lib.check(_lib.lib().grpo_b200_gradsync_create(rank, world, _check_tensor(grads, torch.float32, "grads"),
                                                       grads.numel(), C.byref(self._h)))
        buf = C.create_string_buffer(192)
        _lib.check(_lib.lib().grpo_b200_gradsync_export(self._h, buf))
        self.handle = buf.raw

    def connect(self, handles) -> None:
        import ctypes as C
        if len(handles) != self.world:
            raise ValueError("one handle per rank, in rank order")
        flat = C.create_string_buffer(b"".join(bytes(h) for h in handles), 192 * self.world)
        _lib.check(_lib.lib().grpo_b200_gradsync_connect_ipc(self._h, flat))

    def allreduce_scale(self, scale: float) -> None:
        """Enqueues the kernel on the current stream; every rank makes the same calls."""
        _lib.check(_lib.lib().grpo_b200_allreduce_scale(self._h, float(scale), _stream()))

    def timed_out(self) -> bool:
        import ctypes as C
        flag = C.c_int(0)
        _lib.check(_lib.lib().grpo_b200_gradsync_status(self._h, C.byref(flag)))
        return flag.value != 0

    def close(self) -> None:
        if self._h:
            _lib.lib().grpo_b200_gradsync_destroy(self._h)
            self._h = None


def lmhead_loss(hidden: torch.Tensor, lm_head: torch.Tensor, V: int, logp_old, logp_ref, selected, advantages, weights,
                mask, tokens_per_seq: int, clip_eps: float, beta: float, *, row_offset: int = 0,
                want_selected_logp: bool = False, want_lse: bool = False):
    """LM-head projection fused with the loss statistics (``grpo_b200_lmhead_loss``): ``hidden`` is
    ``[n_rows, C]`` and ``lm_head`` ``[P, C]`` fp32 (read as TF32 by the tensor cores); the logits are
    never materialised.  Returns ``(result, selected_logp or None, lse or None)``."""
    n_rows, C = hidden.shape
    P = lm_head.shape[0]
    if lm_head.shape[1] != C:
        raise ValueError("hidden and lm_head must share the inner dimension")
    dev = hidden.device
    result = new_result(dev)
    ws = torch.empty(_lib.lib().grpo_b200_lmhead_workspace_bytes(n_rows, P), dtype=torch.uint8, device=dev)
    lp = torch.empty(n_rows, dtype=torch.float32, device=dev) if want_selected_logp else None
    lse = torch.empty(n_rows, dtype=torch.float64, device=dev) if want_lse else None
    _lib.check(_lib.lib().grpo_b200_lmhead_loss(
        _check_tensor(hidden, torch.float32, "hidden"), _check_tensor(lm_head, torch.float32, "lm_head"), n_rows, C, V, P,
        _check_tensor(logp_old, torch.float32, "logp_old"), _check_tensor(logp_ref, torch.float32, "logp_ref"),
        _check_tensor(selected, torch.int32, "selected"), _check_tensor(advantages, torch.float32, "advantages"),
        _check_tensor(weights, torch.float32, "weights"), _check_tensor(mask, torch.int32, "mask"), row_offset,
        tokens_per_seq, float(clip_eps), float(beta), None if lp is None else lp.data_ptr(),
        None if lse is None else lse.data_ptr(), result.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
    return result, lp, lse
