"""Multi-GPU data path: whole sequences are bin-packed over the ranks (replicated
weights, no collective inside the layers), each rank runs its share, and one
variable-size gather of the final hidden states restores input order.

The reference has no multi-GPU path; this lifts its longest-processing-time greedy
(python/util.py:11-34, used there across CTAs) to GPUs.
"""
import numpy as np
import torch
import torch.distributed as dist

from . import metadata


def sequence_costs(cfg, lens_tokens):
    """FLOPs per sequence and layer: dense GEMMs + listed attention blocks."""
    costs = []
    for n in lens_tokens:
        visits = metadata.count_visits(cfg, [int(n)])
        costs.append(metadata.sequence_cost(int(n), cfg.hidden, cfg.ffn, cfg.heads, visits))
    return costs


def partition_batch(cfg, lens_tokens, world_size):
    """-> list over ranks of sequence indices (ascending within a rank)."""
    bins = metadata.binpack_sequences(sequence_costs(cfg, lens_tokens), world_size)
    return [sorted(np.nonzero(bins == r)[0].tolist()) for r in range(world_size)]


def gather_outputs(local_out, assignment, lens_tokens, group=None):
    """All ranks end up with the packed [T_total, H] output in input order.

    local_out: this rank's packed rows for its sequences, in `assignment[rank]` order.
    One all_gather on buffers padded to the largest share."""
    world = dist.get_world_size(group)
    tokens_of = [sum(int(lens_tokens[i]) for i in assignment[r]) for r in range(world)]
    pad = max(tokens_of)
    H = local_out.shape[1]
    send = local_out
    if local_out.shape[0] != pad:
        send = torch.zeros(pad, H, dtype=local_out.dtype, device=local_out.device)
        send[: local_out.shape[0]] = local_out
    recv = torch.empty(world * pad, H, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    return unpermute(recv.view(world, pad, H), assignment, lens_tokens)


def unpermute(per_rank, assignment, lens_tokens):
    """per_rank[r] holds rank r's packed rows; returns rows in input sequence order."""
    starts = np.concatenate([[0], np.cumsum(lens_tokens)]).astype(np.int64)
    out = torch.empty(int(starts[-1]), per_rank.shape[-1], dtype=per_rank.dtype, device=per_rank.device)
    for r, seqs in enumerate(assignment):
        off = 0
        for i in seqs:
            n = int(lens_tokens[i])
            out[starts[i]: starts[i] + n] = per_rank[r, off: off + n]
            off += n
    return out
