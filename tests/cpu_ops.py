"""CPU stand-in for ``grpo_cpp_b200.device`` -- TEST ONLY.

Lets the rank logic of ``grpo_cpp_b200.sharded`` (row offsets, the two all-reduces, error
propagation) run under the ``gloo`` backend on a machine without a GPU.  Per-row arithmetic is
delegated to the CPU oracle one row at a time (a 1x1x1 batch has weight exactly 1), then scaled
by the rank-agreed weight.  The product never imports this module.
"""
import numpy as np
import torch

import oracle_py


def new_result(device=None):
    return torch.zeros(5, dtype=torch.float64)


def logits_workspace(n_rows, device=None):
    return torch.empty(0, dtype=torch.uint8)


def count_lengths(mask, n_seq, tokens_per_seq, row_offset=0, out=None):
    m = mask.numpy()
    seq = (row_offset + np.arange(m.size)) // tokens_per_seq
    counts = np.bincount(seq[m != 0], minlength=n_seq).astype(np.int32)
    if out is None:
        return torch.from_numpy(counts)
    out.copy_(torch.from_numpy(counts))
    return out


def weights_from_lengths(lengths, reduction, length_alpha=0.0, out=None, meta=None):
    L = lengths.numpy()
    f = np.float32
    S = f(L.size)
    with np.errstate(divide="ignore"):
        if reduction == 0:
            w = f(1.0) / (S * L.astype(f))
        elif reduction == 1:
            w = np.full(L.size, f(1.0) / f(int(L.sum())), f)
        else:
            w = np.power(L.astype(f), f(length_alpha) - f(1.0)) / S
    w = np.where(L > 0, w, 0).astype(f)
    out.copy_(torch.from_numpy(w))
    meta.copy_(torch.tensor([int(L.sum()), int((L == 0).sum())], dtype=torch.int32))
    return out, meta


def group_advantages(rewards, B, G, mode=0, eps=1e-8):
    adv = oracle_py.load("port").group_advantages(rewards.numpy(), B, G, mode, eps)
    bad = int((~np.isfinite(adv)).sum())
    return torch.from_numpy(np.asarray(adv, np.float32)), torch.tensor([bad], dtype=torch.int32)


def row_order(mask, out=None):
    m = mask.numpy() != 0
    idx = np.arange(m.size, dtype=np.int32)
    order = np.concatenate(([int(m.sum()), int((~m).sum())], idx[m], idx[~m])).astype(np.int32)
    return torch.from_numpy(order)


def count_lengths_f64(mask, n_seq, tokens_per_seq, row_offset, out):
    out.copy_(count_lengths(mask, n_seq, tokens_per_seq, row_offset).to(torch.float64))
    return out


def weights_from_lengths_f64(lengths, reduction, length_alpha, out, meta):
    return weights_from_lengths(lengths.to(torch.int32), reduction, length_alpha, out, meta)


def logits(logits_t, logp_old, logp_ref, selected, advantages, weights, mask, tokens_per_seq, V, clip_eps, beta,
           *, row_offset=0, kernel=1, result=None, workspace=None, **_):
    port = oracle_py.load("port")
    x = logits_t.numpy()
    n_rows, P = x.shape
    total = np.zeros(5)
    for r in range(n_rows):
        if mask[r].item() == 0:
            x[r, :] = 0.0
            continue
        seq = (row_offset + r) // tokens_per_seq
        w = np.float32(weights[seq].item())
        stats, _, d = port.logits(x[r, :V].copy(), [logp_old[r].item()], [logp_ref[r].item()], [selected[r].item()],
                                  [advantages[seq].item()], [1], 1, 1, 1, V, clip_eps, beta, 0, 0.0)
        total[:3] += (w * stats.astype(np.float32)).astype(np.float64)
        x[r, :V] = w * d[0]
        x[r, V:] = 0.0
    result.copy_(torch.from_numpy(total))
    return result


class PeerExchange:
    """Stand-in for the device-side exchange region: the sums over ranks that the reduce kernel
    takes over NVLink are taken by a gloo all-reduce here.  The handle round trip is kept so that
    ``ShardedBoundary.enable_peer_exchange`` runs unchanged."""

    def __init__(self, n_seq, rank, world):
        self.n_seq, self.rank, self.world = n_seq, rank, world
        self.handle = bytes([rank]) * 64
        self.passes = 0
        self.peers = None

    def open_peers(self, handles):
        assert [h[0] for h in handles] == list(range(self.world))
        self.peers = handles

    def close(self):
        self.peers = None


def logits_sharded(logits_t, logp_old, logp_ref, selected, advantages, weights, mask, tokens_per_seq, V, clip_eps,
                   beta, *, exchange, next_mask, reduction, length_alpha, next_weights, next_meta, result, workspace,
                   next_lengths=None, row_offset=0, kernel=1, **_):
    import torch.distributed as dist
    assert exchange.peers is not None, "regions must be mapped before the first pass"
    exchange.passes += 1
    logits(logits_t, logp_old, logp_ref, selected, advantages, weights, mask, tokens_per_seq, V, clip_eps, beta,
           row_offset=row_offset, kernel=kernel, result=result)
    counts = count_lengths(next_mask, exchange.n_seq, tokens_per_seq, row_offset).to(torch.float64)
    if exchange.world > 1:
        dist.all_reduce(result)
        dist.all_reduce(counts)
    if next_lengths is not None:
        next_lengths.copy_(counts)
    weights_from_lengths(counts.to(torch.int32), reduction, length_alpha, next_weights, next_meta)
    return result


def lengths_sharded(mask, n_seq, tokens_per_seq, row_offset, *, exchange, reduction, length_alpha, weights, meta,
                    workspace, status, lengths=None):
    import torch.distributed as dist
    assert exchange.peers is not None, "regions must be mapped before the first pass"
    exchange.passes += 1
    status.zero_()  # this stand-in's exchange cannot time out
    counts = count_lengths(mask, n_seq, tokens_per_seq, row_offset).to(torch.float64)
    if exchange.world > 1:
        dist.all_reduce(counts)
    if lengths is not None:
        lengths.copy_(counts)
    weights_from_lengths(counts.to(torch.int32), reduction, length_alpha, weights, meta)
    return weights
