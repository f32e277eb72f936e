"""CPU oracle: BigBird block-sparse encoder, restated from the reference's validation model.

TEST INFRASTRUCTURE - never imported by the product package.

Every function names the place in the reference it follows (paths are relative
to the reference project root).  Integer outputs (random-block tables, CSR
block lists, varlen offsets, work partitions) are the bit-exact targets for the
CUDA library's host code; floating-point outputs are computed in fp32 with
torch on the CPU and are the target the 16-bit GPU path must match within
max-abs 2e-2 / mean-abs 2e-3 on final hidden states.

Sequences are always evaluated one at a time, un-padded, with an all-ones
attention mask, so every table is a pure function of
(layer seed, head, number of blocks, max_position_embeddings).
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

__all__ = [
    "EncoderConfig",
    "UnsupportedLength",
    "rand_block_table",
    "kv_block_lists",
    "build_block_csr",
    "seq_block_prefix",
    "lpt_partition",
    "visits_per_head",
    "make_weights",
    "gelu_new",
    "sparse_attention_ref",
    "attention_sublayer_ref",
    "layer_ref",
    "embeddings_ref",
    "encoder_ref",
    "binpack_sequences",
]


class UnsupportedLength(ValueError):
    """Raised for sequence lengths the reference's validation model cannot run.

    12 blocks (768 tokens) takes the "old plan" branch whose random ids reach 15,
    so its gather indexes past the sequence (python/modeling_big_bird.py:573-580
    followed by torch_gather_b2 at :978-998 raising IndexError).
    """


@dataclass
class EncoderConfig:
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    layers: int = 12
    block: int = 64
    num_rand: int = 3
    max_pos: int = 4096
    vocab: int = 50358
    type_vocab: int = 2
    eps: float = 1e-12
    # "bigbird": global + window(3) + random per head (the reference model);
    # "band":    first block global + window of 2*band_half+1 blocks, no random
    #            blocks (Longformer-shaped pattern; generic block-table path).
    pattern: str = "bigbird"
    band_half: int = 4
    layer_seeds: List[int] = field(default_factory=list)

    def seed_of(self, layer: int) -> int:
        # python/modeling_big_bird.py:1577 - BigBirdLayer(config, seed=layer_idx)
        return self.layer_seeds[layer] if self.layer_seeds else layer

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


# ----------------------------------------------------------------------------
# random-block tables
# ----------------------------------------------------------------------------

def _old_plan_rows(n_blocks: int, r: int, last_idx_tokens: int, block: int) -> np.ndarray:
    """python/modeling_big_bird.py:1072-1125 (_bigbird_block_rand_mask).

    Uses the process-global legacy numpy RNG exactly as the reference does: one
    np.random.permutation per row, rows 1 .. n_blocks-2.
    """
    rand_attn = np.zeros((n_blocks - 2, r), dtype=np.int32)
    middle_seq = np.arange(1, n_blocks - 1, dtype=np.int32)
    last = n_blocks - 1
    if last_idx_tokens > 2 * block:
        last = last_idx_tokens // block - 1
    for i in range(1, n_blocks - 1):
        start = i - 2
        end = i
        if i == 1:
            rand_attn[i - 1, :] = np.random.permutation(middle_seq[2:last])[:r]
        elif i == 2:
            rand_attn[i - 1, :] = np.random.permutation(middle_seq[3:last])[:r]
        elif i == n_blocks - 3:
            rand_attn[i - 1, :] = np.random.permutation(middle_seq[:last])[:r]
        elif i == n_blocks - 2:
            rand_attn[i - 1, :] = np.random.permutation(middle_seq[:last])[:r]
        else:
            if start > last:
                start = last
                rand_attn[i - 1, :] = np.random.permutation(middle_seq[:start])[:r]
            elif (end + 1) == last:
                rand_attn[i - 1, :] = np.random.permutation(middle_seq[:start])[:r]
            else:
                rand_attn[i - 1, :] = np.random.permutation(
                    np.concatenate((middle_seq[:start], middle_seq[end + 1:last]))
                )[:r]
    return rand_attn


def _rand_attn_plan(n_blocks: int, r: int) -> Tuple[List[int], List[int]]:
    """python/modeling_big_bird.py:1039-1069 (_get_rand_attn_plan), in block units."""
    if 2 * r + 5 < n_blocks:
        return [2 * r + 5, n_blocks], [r, 0]
    if r + 5 < n_blocks:
        return [r + 5, n_blocks], [r // 2, r - r // 2]
    return [n_blocks], [r]


def _single_row(block_id: int, to_start: int, to_end: int, r: int) -> np.ndarray:
    """python/modeling_big_bird.py:1288-1314 (_get_single_block_row_attention)."""
    perm = np.random.permutation(np.arange(to_start, to_end, dtype=np.int32))
    illegal = [block_id - 1, block_id, block_id + 1, 0, to_end - 1]
    if block_id == 1:
        illegal.append(to_end - 2)
    if block_id == to_end - 2:
        illegal.append(1)
    picked: List[int] = []
    for i in range(to_end - to_start):
        if perm[i] not in illegal:
            picked.append(int(perm[i]))
        if len(picked) == r:
            break
    return np.array(picked, dtype=np.int32)


def _with_head_rows(n_blocks: int, heads: int, r: int) -> np.ndarray:
    """python/modeling_big_bird.py:1127-1286 (_bigbird_block_rand_mask_with_head)."""
    plan_len, plan_r = _rand_attn_plan(n_blocks, r)
    max_plan_idx = plan_len.index(n_blocks)
    width = int(np.sum(plan_r[: max_plan_idx + 1]))
    rand_attn = [np.zeros((n_blocks, width), dtype=np.int32) for _ in range(heads)]
    for plan_idx in range(max_plan_idx + 1):
        rnd_r_cnt = 0
        if plan_idx > 0:
            if plan_r[plan_idx] > 0:
                rnd_r_cnt = int(np.sum(plan_r[:plan_idx]))
                curr_r_cnt = int(np.sum(plan_r[: plan_idx + 1]))
                for row in range(1, plan_len[plan_idx - 1]):
                    for h in range(heads):
                        rand_attn[h][row, rnd_r_cnt:curr_r_cnt] = _single_row(
                            row, plan_len[plan_idx - 1], plan_len[plan_idx], plan_r[plan_idx])
            for pl_id in range(plan_idx):
                if plan_r[pl_id] == 0:
                    continue
                for row in range(plan_len[plan_idx - 1], plan_len[plan_idx]):
                    rnd_r_cnt = 0
                    to_start = 0
                    if pl_id > 0:
                        rnd_r_cnt = int(np.sum(plan_r[:pl_id]))
                        to_start = plan_len[pl_id - 1]
                    curr_r_cnt = int(np.sum(plan_r[: pl_id + 1]))
                    for h in range(heads):
                        rand_attn[h][row, rnd_r_cnt:curr_r_cnt] = _single_row(
                            row, to_start, plan_len[pl_id], plan_r[pl_id])
        if plan_r[plan_idx] == 0:
            continue
        curr_r_cnt = int(np.sum(plan_r[: plan_idx + 1]))
        from_start = 1
        to_start = 0
        if plan_idx > 0:
            rnd_r_cnt = int(np.sum(plan_r[:plan_idx]))
            from_start = plan_len[plan_idx - 1]
            to_start = plan_len[plan_idx - 1]
        for row in range(from_start, plan_len[plan_idx]):
            for h in range(heads):
                rand_attn[h][row, rnd_r_cnt:curr_r_cnt] = _single_row(
                    row, to_start, plan_len[plan_idx], plan_r[plan_idx])
    return np.stack([t[1: n_blocks - 1, :] for t in rand_attn], axis=0)


def rand_block_table(seed: int, heads: int, n_blocks: int, r: int = 3,
                     max_pos: int = 4096, block: int = 64) -> np.ndarray:
    """Random-block ids [heads, n_blocks-2, r] for one (layer, sequence length).

    python/modeling_big_bird.py:573-600: np.random.seed(layer seed); when the
    token length is a multiple of 256 the "old plan" table is built for
    max_position_embeddings once per head (head-major RNG order) and cut to the
    first n_blocks-2 rows; otherwise the with-head plan (row-major, heads
    innermost).
    """
    if n_blocks <= 5 + 2 * r:
        raise ValueError("full-attention length: no random table exists")
    np.random.seed(seed)
    if (n_blocks * block) % 256 == 0:
        max_blocks = max_pos // block
        rows = [_old_plan_rows(max_blocks, r, 1024, block)[: n_blocks - 2] for _ in range(heads)]
        table = np.stack(rows, axis=0)
        if table.shape[1] != n_blocks - 2:
            raise UnsupportedLength(f"{n_blocks} blocks exceed max_position_embeddings={max_pos}")
    else:
        table = _with_head_rows(n_blocks, heads, r)
    if int(table.max()) >= n_blocks:
        raise UnsupportedLength(
            f"{n_blocks * block} tokens: the reference model's random ids reach block "
            f"{int(table.max())} >= {n_blocks}")
    return table.astype(np.int32)


# ----------------------------------------------------------------------------
# block lists / CSR / varlen offsets / work partition
# ----------------------------------------------------------------------------

def kv_block_lists(n_blocks: int, cfg: EncoderConfig, rand: np.ndarray | None, head: int) -> List[List[int]]:
    """Key/value block list of every query block of one (sequence, head).

    Order = the concatenation order of the reference's five-part computation
    (python/modeling_big_bird.py:626-851): first/last query block -> every block;
    second -> [0,1,2,last]+random; middle -> [0, i-1,i,i+1]+random+[last];
    second-last -> [0,last-2,last-1,last]+random.  A block that appears twice is
    kept twice: the reference's softmax runs over the concatenated keys.
    Lengths at or below (5+2r) blocks use full attention (:2076-2094).
    """
    L = n_blocks
    if cfg.pattern == "band":
        out = [list(range(L))]
        for i in range(1, L):
            lo, hi = max(0, i - cfg.band_half), min(L - 1, i + cfg.band_half)
            blocks = list(range(lo, hi + 1))
            if lo > 0:
                blocks = [0] + blocks
            out.append(blocks)
        return out
    if L <= 5 + 2 * cfg.num_rand:
        return [list(range(L)) for _ in range(L)]
    assert rand is not None
    out = [list(range(L))]
    out.append([0, 1, 2, L - 1] + [int(x) for x in rand[head, 0]])
    for i in range(2, L - 2):
        out.append([0, i - 1, i, i + 1] + [int(x) for x in rand[head, i - 1]] + [L - 1])
    out.append([0, L - 3, L - 2, L - 1] + [int(x) for x in rand[head, L - 3]])
    out.append(list(range(L)))
    return out


def seq_block_prefix(lens_tokens: Sequence[int], block: int = 64) -> List[int]:
    """python/util.py:37,45 - prefix sums of per-sequence block counts (len B+1)."""
    out = [0]
    for n in lens_tokens:
        if n % block:
            raise ValueError("sequence length must be a multiple of the block size")
        out.append(out[-1] + n // block)
    return out


def build_block_csr(lens_tokens: Sequence[int], cfg: EncoderConfig, layer: int) -> Tuple[np.ndarray, np.ndarray]:
    """CSR block table of one layer for a packed varlen batch.

    Returns (kv_ptr int32 [N+1], kv_idx int32 [heads, total_visits]) with
    sequence-local block ids; the counterpart of to_select_index_position /
    to_select_index built by layers/multi_headed_attention.cpp:15-140, with the
    head dimension the validation model needs (its tables are per head).
    """
    ptr = [0]
    per_head: List[List[int]] = [[] for _ in range(cfg.heads)]
    cache: Dict[int, np.ndarray | None] = {}
    for n in lens_tokens:
        L = n // cfg.block
        if L not in cache:
            if cfg.pattern == "bigbird" and L > 5 + 2 * cfg.num_rand:
                cache[L] = rand_block_table(cfg.seed_of(layer), cfg.heads, L, cfg.num_rand, cfg.max_pos, cfg.block)
            else:
                cache[L] = None
        for h in range(cfg.heads):
            lists = kv_block_lists(L, cfg, cache[L], h)
            for q in range(L):
                per_head[h].extend(lists[q])
                if h == 0:
                    ptr.append(ptr[-1] + len(lists[q]))
    return np.asarray(ptr, dtype=np.int32), np.asarray(per_head, dtype=np.int32)


def visits_per_head(lens_tokens: Sequence[int], cfg: EncoderConfig) -> int:
    """Sum over query blocks of listed key/value blocks, for one head (the
    unit of the attention FLOP count: 4*64*64*64 FLOPs per visit)."""
    total = 0
    for n in lens_tokens:
        L = n // cfg.block
        total += sum(len(x) for x in kv_block_lists(L, cfg, np.zeros((cfg.heads, max(L - 2, 1), cfg.num_rand), np.int32), 0))
    return total


def lpt_partition(cost_per_qblock: Sequence[int], seq_prefix: Sequence[int], n_parts: int,
                  heads: int) -> Tuple[List[int], List[int]]:
    """python/util.py:11-34 (generate_parition_plan), restated.

    Work item id = first_block_of_sequence*heads + head*blocks_in_sequence + local_block.
    Items are visited in descending-cost order (stable), heads innermost; each
    goes to the least-loaded part (ties: lowest part index, as heapq on
    (load, part) tuples does).  Returns (offsets [n_parts+1], ids [heads*N]).
    """
    order = sorted(range(len(cost_per_qblock)), key=lambda i: -cost_per_qblock[i])
    parts: List[List[int]] = [[] for _ in range(n_parts)]
    heap = [(0, i) for i in range(n_parts)]
    starts = [(seq_prefix[i], seq_prefix[i + 1] - seq_prefix[i]) for i in range(len(seq_prefix) - 1)]
    for g in order:
        for h in range(heads):
            load, p = heapq.heappop(heap)
            first, nblk = (0, 0)
            for s in starts:
                if g >= s[0]:
                    first, nblk = s
                else:
                    break
            parts[p].append(g - first + h * nblk + first * heads)
            heapq.heappush(heap, (load + cost_per_qblock[g], p))
    offsets = [0]
    ids: List[int] = []
    for p in parts:
        ids.extend(p)
        offsets.append(len(ids))
    return offsets, ids


def binpack_sequences(costs: Sequence[float], n_bins: int) -> List[List[int]]:
    """Longest-processing-time greedy over whole sequences: descending cost
    (ties by index), each to the least-loaded bin (ties by bin index).  The same
    greedy python/util.py:11-34 applies to CTAs, lifted to GPUs."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * n_bins
    bins: List[List[int]] = [[] for _ in range(n_bins)]
    for i in order:
        b = min(range(n_bins), key=lambda j: (loads[j], j))
        bins[b].append(i)
        loads[b] += costs[i]
    return bins


# ----------------------------------------------------------------------------
# weights
# ----------------------------------------------------------------------------

_LAYER_PARAMS = [
    ("attention.self.query.weight", "w_hh"), ("attention.self.query.bias", "b_h"),
    ("attention.self.key.weight", "w_hh"), ("attention.self.key.bias", "b_h"),
    ("attention.self.value.weight", "w_hh"), ("attention.self.value.bias", "b_h"),
    ("attention.output.dense.weight", "w_hh"), ("attention.output.dense.bias", "b_h"),
    ("attention.output.LayerNorm.weight", "g_h"), ("attention.output.LayerNorm.bias", "b_h"),
    ("intermediate.dense.weight", "w_fh"), ("intermediate.dense.bias", "b_f"),
    ("output.dense.weight", "w_hf"), ("output.dense.bias", "b_h"),
    ("output.LayerNorm.weight", "g_h"), ("output.LayerNorm.bias", "b_h"),
]


def make_weights(cfg: EncoderConfig, seed: int = 0, nonzero_bias: bool = False,
                 embeddings: bool = True) -> Dict[str, torch.Tensor]:
    """Seeded synthetic parameters, named and ordered like the state_dict of the
    reference's BigBirdModel (embeddings, then encoder.layer.{i}.*; torch Linear
    layout [out, in]).  Weights ~ N(0, 0.02).  Default: biases 0, LayerNorm
    gamma 1 / beta 0.  nonzero_bias=True draws biases ~ N(0, 0.02), gamma ~
    1 + N(0, 0.1), beta ~ N(0, 0.1) so that every bias path is exercised.
    """
    g = torch.Generator().manual_seed(seed)
    H, F = cfg.hidden, cfg.ffn

    def w(*shape):
        return torch.randn(*shape, generator=g) * 0.02

    def bias(n):
        return torch.randn(n, generator=g) * 0.02 if nonzero_bias else torch.zeros(n)

    def gamma(n):
        return 1.0 + torch.randn(n, generator=g) * 0.1 if nonzero_bias else torch.ones(n)

    def beta(n):
        return torch.randn(n, generator=g) * 0.1 if nonzero_bias else torch.zeros(n)

    P: Dict[str, torch.Tensor] = {}
    if embeddings:
        P["embeddings.word_embeddings.weight"] = w(cfg.vocab, H)
        P["embeddings.position_embeddings.weight"] = w(cfg.max_pos, H)
        P["embeddings.token_type_embeddings.weight"] = w(cfg.type_vocab, H)
        P["embeddings.LayerNorm.weight"] = gamma(H)
        P["embeddings.LayerNorm.bias"] = beta(H)
    for i in range(cfg.layers):
        for name, kind in _LAYER_PARAMS:
            key = f"encoder.layer.{i}.{name}"
            if kind == "w_hh":
                P[key] = w(H, H)
            elif kind == "w_fh":
                P[key] = w(F, H)
            elif kind == "w_hf":
                P[key] = w(H, F)
            elif kind == "b_h":
                P[key] = beta(H) if name.endswith("LayerNorm.bias") else bias(H)
            elif kind == "b_f":
                P[key] = bias(F)
            elif kind == "g_h":
                P[key] = gamma(H)
    return P


# ----------------------------------------------------------------------------
# floating-point reference (fp32, torch CPU)
# ----------------------------------------------------------------------------

def gelu_new(x: torch.Tensor) -> torch.Tensor:
    """tanh-form GELU ("gelu_new", the activation of bigbird-roberta-base;
    python/modeling_big_bird.py:1424-1437 via ACT2FN; the same formula as
    layers/kernels/add_bias_act.cu:42-48)."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))


def sparse_attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         lists_per_head: Sequence[Sequence[Sequence[int]]], block: int = 64) -> torch.Tensor:
    """softmax(q k_listed^T / sqrt(d)) v_listed per (head, query block).

    q, k, v: [heads, S, d] fp32 of ONE sequence.  lists_per_head[h][qb] is the
    key/value block list (duplicates kept).  Returns [heads, S, d].
    Follows python/modeling_big_bird.py:626-851 with an all-ones mask (the
    additive -10000 penalties vanish).
    """
    nh, S, d = q.shape
    L = S // block
    scale = 1.0 / math.sqrt(d)
    kb = k.view(nh, L, block, d)
    vb = v.view(nh, L, block, d)
    qb = q.view(nh, L, block, d)
    out = torch.empty_like(q).view(nh, L, block, d)
    # group query blocks by list length so that each group is one batched matmul
    by_len: Dict[int, List[int]] = {}
    for i in range(L):
        by_len.setdefault(len(lists_per_head[0][i]), []).append(i)
    for n, rows in by_len.items():
        idx = torch.tensor([[lists_per_head[h][i] for i in rows] for h in range(nh)], dtype=torch.long)  # [nh, R, n]
        R = len(rows)
        hsel = torch.arange(nh).view(nh, 1, 1).expand(nh, R, n)
        kg = kb[hsel, idx].reshape(nh, R, n * block, d)
        vg = vb[hsel, idx].reshape(nh, R, n * block, d)
        qq = qb[:, rows]  # [nh, R, block, d]
        s = torch.matmul(qq, kg.transpose(-1, -2)) * scale
        p = torch.softmax(s, dim=-1)
        out[:, rows] = torch.matmul(p, vg)
    return out.view(nh, S, d)


def _lin(x, W, b):
    return torch.nn.functional.linear(x, W, b)


def attention_sublayer_ref(x: torch.Tensor, P: Dict[str, torch.Tensor], layer: int, cfg: EncoderConfig,
                           return_context: bool = False):
    """Attention half of one layer on ONE un-padded sequence x [S, hidden] fp32:
    q/k/v projections, block-sparse attention, output projection, residual +
    LayerNorm (python/modeling_big_bird.py:444-498, 1318-1329)."""
    S = x.shape[0]
    L = S // cfg.block
    pre = f"encoder.layer.{layer}."
    nh, d = cfg.heads, cfg.head_dim

    def heads(t):
        return t.view(S, nh, d).permute(1, 0, 2).contiguous()

    q = heads(_lin(x, P[pre + "attention.self.query.weight"], P[pre + "attention.self.query.bias"]))
    k = heads(_lin(x, P[pre + "attention.self.key.weight"], P[pre + "attention.self.key.bias"]))
    v = heads(_lin(x, P[pre + "attention.self.value.weight"], P[pre + "attention.self.value.bias"]))
    rand = None
    if cfg.pattern == "bigbird" and L > 5 + 2 * cfg.num_rand:
        rand = rand_block_table(cfg.seed_of(layer), nh, L, cfg.num_rand, cfg.max_pos, cfg.block)
    lists = [kv_block_lists(L, cfg, rand, h) for h in range(nh)]
    ctx = sparse_attention_ref(q, k, v, lists, cfg.block)  # [nh, S, d]
    ctx = ctx.permute(1, 0, 2).reshape(S, nh * d)
    a = _lin(ctx, P[pre + "attention.output.dense.weight"], P[pre + "attention.output.dense.bias"])
    a = torch.nn.functional.layer_norm(a + x, (cfg.hidden,), P[pre + "attention.output.LayerNorm.weight"],
                                       P[pre + "attention.output.LayerNorm.bias"], cfg.eps)
    if return_context:
        return a, ctx
    return a


def layer_ref(x: torch.Tensor, P: Dict[str, torch.Tensor], layer: int, cfg: EncoderConfig) -> torch.Tensor:
    """One encoder layer on ONE sequence (python/modeling_big_bird.py:1485-1562)."""
    pre = f"encoder.layer.{layer}."
    a = attention_sublayer_ref(x, P, layer, cfg)
    f = gelu_new(_lin(a, P[pre + "intermediate.dense.weight"], P[pre + "intermediate.dense.bias"]))
    o = _lin(f, P[pre + "output.dense.weight"], P[pre + "output.dense.bias"])
    return torch.nn.functional.layer_norm(o + a, (cfg.hidden,), P[pre + "output.LayerNorm.weight"],
                                          P[pre + "output.LayerNorm.bias"], cfg.eps)


def embeddings_ref(ids: torch.Tensor, P: Dict[str, torch.Tensor], cfg: EncoderConfig,
                   position_ids: torch.Tensor | None = None, type_ids: torch.Tensor | None = None) -> torch.Tensor:
    """word + token-type + position embeddings, LayerNorm
    (python/modeling_big_bird.py:269-308, rescale_embeddings False)."""
    n = ids.shape[0]
    if position_ids is None:
        position_ids = torch.arange(n)
    if type_ids is None:
        type_ids = torch.zeros(n, dtype=torch.long)
    e = (P["embeddings.word_embeddings.weight"][ids.long()]
         + P["embeddings.token_type_embeddings.weight"][type_ids.long()]
         + P["embeddings.position_embeddings.weight"][position_ids.long()])
    return torch.nn.functional.layer_norm(e, (cfg.hidden,), P["embeddings.LayerNorm.weight"],
                                          P["embeddings.LayerNorm.bias"], cfg.eps)


@torch.no_grad()
def encoder_ref(seqs: Sequence[torch.Tensor], P: Dict[str, torch.Tensor], cfg: EncoderConfig,
                from_ids: bool = True, n_layers: int | None = None) -> torch.Tensor:
    """Full encoder on a varlen batch, one sequence at a time; returns the
    packed [T, hidden] fp32 final hidden states in input order.  seqs are token
    id vectors (from_ids) or [S, hidden] fp32 hidden states."""
    outs = []
    for s in seqs:
        h = embeddings_ref(s, P, cfg) if from_ids else s.float()
        for i in range(cfg.layers if n_layers is None else n_layers):
            h = layer_ref(h, P, i, cfg)
        outs.append(h)
    return torch.cat(outs, dim=0)
