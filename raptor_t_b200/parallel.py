"""Multi-GPU data path: whole sequences are bin-packed over the ranks (replicated
weights, no collective inside the layers), each rank runs its share, and one
variable-size gather of the final hidden states restores input order.

Two forms of that gather: RootGatherer delivers the batch to ONE rank (the caller that
submitted it) - every rank sends each of its sequences straight to that sequence's rows of
the root's output buffer, so no padding, no permutation pass and 1/N of an all-gather's
traffic; OutputGatherer / gather_outputs leave the full output on every rank (padded
all_gather + one index_select).

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


def gather_permutation(assignment, lens_tokens, pad):
    """Row index into the gathered [world * pad, H] buffer for every output row (input order)."""
    starts = np.concatenate([[0], np.cumsum(lens_tokens)]).astype(np.int64)
    perm = np.empty(int(starts[-1]), dtype=np.int64)
    for r, seqs in enumerate(assignment):
        off = 0
        for i in seqs:
            n = int(lens_tokens[i])
            perm[starts[i]: starts[i] + n] = r * pad + off + np.arange(n, dtype=np.int64)
            off += n
    return perm


class OutputGatherer:
    """The gather of one batch layout with everything set up once: padded send buffer,
    receive buffers, the row permutation on the device.  gather() costs one all_gather and
    one index_select.  On CUDA the two run on a side stream (start()/finish()), so a caller
    that keeps two batches in flight overlaps the gather of one with the kernels of the next;
    `depth` result buffers rotate."""

    def __init__(self, assignment, lens_tokens, hidden, dtype, device, group=None, depth=2):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        tokens_of = [sum(int(lens_tokens[i]) for i in assignment[r]) for r in range(self.world)]
        self.pad, self.local_tokens, self.total = max(tokens_of), tokens_of[self.rank], int(sum(tokens_of))
        self.device = torch.device(device)
        self.perm = torch.from_numpy(gather_permutation(assignment, lens_tokens, self.pad)).to(self.device)
        self.send = [torch.zeros(self.pad, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
        self.recv = [torch.empty(self.world * self.pad, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
        self.out = [torch.empty(self.total, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
        self.cuda = self.device.type == "cuda"
        self.side = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.done = [torch.cuda.Event() for _ in range(depth)] if self.cuda else None
        self.n = 0

    def _run(self, local_out, k):
        self.send[k][: self.local_tokens].copy_(local_out)
        dist.all_gather_into_tensor(self.recv[k], self.send[k], group=self.group)
        torch.index_select(self.recv[k], 0, self.perm, out=self.out[k])
        return self.out[k]

    def gather(self, local_out):
        """Synchronous with the current stream: returns the [T_total, H] tensor in input order."""
        k = self.n % len(self.out)
        self.n += 1
        return self._run(local_out, k)

    def start(self, local_out):
        """Enqueue the gather behind the work already on the current stream, on the side
        stream; returns a ticket for finish().  local_out must stay untouched until then."""
        k = self.n % len(self.out)
        self.n += 1
        if not self.cuda:
            self._run(local_out, k)
            return k
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            self._run(local_out, k)
            self.done[k].record()
        return k

    def finish(self, ticket):
        """Makes the current stream wait for that gather and returns its result buffer."""
        if self.cuda:
            torch.cuda.current_stream().wait_event(self.done[ticket])
        return self.out[ticket]


class RootGatherer:
    """Gather of one batch layout to a single rank, set up once.  A sequence's rows are a
    contiguous range of the packed output in input order, so every rank sends each of its
    sequences as one message and the root receives it in place (grouped send/recv: one NCCL
    group per gather).  The root's own sequences are local copies.  On CUDA the gather runs on a
    side stream (start()/finish()), `depth` result buffers rotate; finish() returns the
    [T_total, H] tensor on the root and None elsewhere."""

    def __init__(self, assignment, lens_tokens, hidden, dtype, device, group=None, depth=2, root=0):
        self.group, self.root = group, root
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.starts = np.concatenate([[0], np.cumsum(lens_tokens)]).astype(np.int64)
        self.total = int(self.starts[-1])
        self.lens = [int(n) for n in lens_tokens]
        self.assignment = [list(a) for a in assignment]
        self.local_tokens = sum(self.lens[i] for i in self.assignment[self.rank])
        self.is_root = self.rank == root
        self.out = ([torch.empty(self.total, hidden, dtype=dtype, device=self.device) for _ in range(depth)]
                    if self.is_root else [None] * depth)
        self.cuda = self.device.type == "cuda"
        self.side = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.done = [torch.cuda.Event() for _ in range(depth)] if self.cuda else None
        self.n = 0

    def _run(self, local_out, k):
        ops = []
        if self.is_root:
            out = self.out[k]
            for r, seqs in enumerate(self.assignment):
                off = 0
                for i in seqs:
                    n, s0 = self.lens[i], int(self.starts[i])
                    if r == self.rank:
                        out[s0:s0 + n].copy_(local_out[off:off + n])
                    else:
                        ops.append(dist.P2POp(dist.irecv, out[s0:s0 + n], r, group=self.group))
                    off += n
        else:
            off = 0
            for i in self.assignment[self.rank]:
                n = self.lens[i]
                ops.append(dist.P2POp(dist.isend, local_out[off:off + n], self.root, group=self.group))
                off += n
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return self.out[k]

    def gather(self, local_out):
        """Synchronous with the current stream."""
        k = self.n % len(self.out)
        self.n += 1
        return self._run(local_out, k)

    def start(self, local_out, host_out=None):
        """Enqueue the gather behind the work already on the current stream, on the side stream;
        returns a ticket for finish().  local_out must stay untouched until then.  host_out
        (root only, pinned [>= T_total, H]): the gathered batch is also copied there, still on the
        side stream, so the device-to-host copy overlaps the next steps' kernels as well."""
        k = self.n % len(self.out)
        self.n += 1
        if not self.cuda:
            full = self._run(local_out, k)
            if host_out is not None and full is not None:
                host_out[: self.total].copy_(full)
            return k
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            full = self._run(local_out, k)
            if host_out is not None and full is not None:
                host_out[: self.total].copy_(full, non_blocking=True)
            self.done[k].record()
        return k

    def finish(self, ticket):
        """Makes the current stream wait for that gather; the result buffer on the root, None elsewhere."""
        if self.cuda:
            torch.cuda.current_stream().wait_event(self.done[ticket])
        return self.out[ticket]


class PeerGatherer:
    """RootGatherer's job without kernels on the SMs: the root's result buffers live in symmetric memory
    (every rank maps them), a sending rank copies each of its sequences straight into the root's buffer with
    device-to-device copies (copy engines over NVLink), and hand-offs are 4-byte copies of a generation
    number into the peer's flag words, waited for with stream memory operations.  Nothing of it occupies an
    SM, so the compute kernels of the next steps keep all of them (NCCL's send/receive kernels wait for
    their peer on SMs whose registers and shared memory the compute kernels want whole).

    Same interface as RootGatherer (start / finish, `depth` buffers in rotation).  Flow control: a sender
    writes buffer k of generation g only after the root has released generation g - depth of it (the root's
    flag copy follows whatever consumed the buffer on the side stream, e.g. the copy to the host).
    Needs CUDA, torch symmetric memory and the cuda-python driver bindings; `available()` says so."""

    @staticmethod
    def available():
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            from cuda.bindings import driver  # noqa: F401
            return torch.cuda.is_available()
        except Exception:
            return False

    def __init__(self, assignment, lens_tokens, hidden, dtype, device, group=None, depth=2, root=0):
        import torch.distributed._symmetric_memory as symm
        from cuda.bindings import driver
        self._drv = driver
        self.group = group if group is not None else dist.group.WORLD
        self.root = root
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.starts = np.concatenate([[0], np.cumsum(lens_tokens)]).astype(np.int64)
        self.total = int(self.starts[-1])
        self.lens = [int(n) for n in lens_tokens]
        self.assignment = [list(a) for a in assignment]
        self.is_root = self.rank == root
        self.depth = depth
        # result buffers: allocated on every rank (symmetric), used on the root
        self._buf = symm.empty((depth, self.total, hidden), dtype=dtype, device=self.device)
        self._hbuf = symm.rendezvous(self._buf, self.group.group_name)
        self._root_buf = self._hbuf.get_buffer(root, (depth, self.total, hidden), dtype)
        # flag words: [0 : world*depth] "rank r has filled buffer k" (read on the root),
        #             [world*depth : world*depth + depth] "buffer k is free again" (read on the senders)
        self._flags = symm.empty((self.world * depth + depth,), dtype=torch.int32, device=self.device)
        self._flags.zero_()
        self._hflags = symm.rendezvous(self._flags, self.group.group_name)
        self._peer_flags = [self._hflags.get_buffer(r, (self.world * depth + depth,), torch.int32) for r in range(self.world)]
        self._gen_limit = 1 << 16
        self._gen_src = torch.arange(0, self._gen_limit, dtype=torch.int32, device=self.device)  # source of the 4-byte copies
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.out = [self._buf[k] for k in range(depth)] if self.is_root else [None] * depth
        self.side = torch.cuda.Stream(device=self.device)
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.n = 0

    def _wait(self, flag_index, value):
        addr = self._flags.data_ptr() + 4 * flag_index
        err, = self._drv.cuStreamWaitValue32(self.side.cuda_stream, addr, value,
                                             self._drv.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)
        if int(err) != 0:
            raise RuntimeError(f"cuStreamWaitValue32 failed: {err}")

    def _signal(self, peer, flag_index, value):
        self._peer_flags[peer][flag_index:flag_index + 1].copy_(self._gen_src[value:value + 1], non_blocking=True)

    def start(self, local_out, host_out=None):
        if self.n // self.depth + 1 >= self._gen_limit:
            self._restart()
        k = self.n % self.depth
        gen = self.n // self.depth + 1
        self.n += 1
        ready = torch.cuda.Event()
        ready.record()
        W, D = self.world, self.depth
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            if self.is_root:
                out = self._buf[k]
                off = 0
                for i in self.assignment[self.rank]:
                    n, s0 = self.lens[i], int(self.starts[i])
                    out[s0:s0 + n].copy_(local_out[off:off + n], non_blocking=True)
                    off += n
                for r in range(W):
                    if r != self.rank:
                        self._wait(r * D + k, gen)
                if host_out is not None:
                    host_out[: self.total].copy_(out, non_blocking=True)
                self.done[k].record()
                # the buffer may be refilled once this point of the side stream is reached; a caller that reads it
                # on another stream does so between finish() and its next start(), `depth` gathers earlier
                for r in range(W):
                    if r != self.rank:
                        self._signal(r, W * D + k, gen)
            else:
                if gen > 1:
                    self._wait(W * D + k, gen - 1)
                dst = self._root_buf[k]
                off = 0
                for i in self.assignment[self.rank]:
                    n, s0 = self.lens[i], int(self.starts[i])
                    dst[s0:s0 + n].copy_(local_out[off:off + n], non_blocking=True)
                    off += n
                self._signal(self.root, self.rank * D + k, gen)
                self.done[k].record()
        return k

    def finish(self, ticket):
        torch.cuda.current_stream().wait_event(self.done[ticket])
        return self.out[ticket]

    def _restart(self):
        """Generation numbers are drawn from a table; when it is used up all ranks drain, clear their flag words and
        start again at generation 1 (every rank reaches this at the same gather)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self._flags.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.n = 0


def make_root_gatherer(assignment, lens_tokens, hidden, dtype, device, group=None, depth=2, root=0, kind=None):
    """PeerGatherer where it can be built (kind "peer"), RootGatherer (NCCL / gloo send-recv) otherwise."""
    if kind == "peer":
        return PeerGatherer(assignment, lens_tokens, hidden, dtype, device, group=group, depth=depth, root=root)
    if kind is None and torch.device(device).type == "cuda" and PeerGatherer.available():
        # every rank must take the same branch: agree on it
        ok = torch.ones(1, device=device)
        try:
            g = PeerGatherer(assignment, lens_tokens, hidden, dtype, device, group=group, depth=depth, root=root)
        except Exception:
            g, ok = None, torch.zeros(1, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() > 0:
            return g
    return RootGatherer(assignment, lens_tokens, hidden, dtype, device, group=group, depth=depth, root=root)
