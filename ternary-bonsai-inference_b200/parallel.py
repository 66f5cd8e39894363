"""Sharding of the KV path over the GPUs of one node (one process per GPU).

The reference is single-device, so nothing here has a counterpart in it.  Two ways to
shard, both natural for this path:

* independent sequences: each rank owns whole sequences (all layers); no collective touches
  the data path.  `shard_sequences` balances bytes (context lengths) greedily.
* one long sequence: contiguous context chunks per rank.  Every rank attends over its chunk
  with the same (replicated) q and produces, per q head, the triple (acc[hd], m, l); one
  all-gather of those 24 x 258 floats per layer and a log-sum-exp merge give the output.
  New tokens are appended on the rank that owns the tail chunk.

torch.distributed is only the transport (NCCL on GPUs, gloo in the CPU tests).
"""
import numpy as np


def shard_sequences(lengths, world):
    """Greedy longest-first assignment of sequences to ranks; returns a list of index lists.
    Ties keep the lower rank, so every rank computes the same plan."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    loads = [0] * world
    plan = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        plan[r].append(i)
        loads[r] += int(lengths[i])
    for p in plan:
        p.sort()
    return plan


def split_context(n_pos, world, granularity=128):
    """Contiguous chunks [begin, end) per rank, sizes multiples of `granularity` except the last
    non-empty one; trailing ranks may be empty when n_pos is small."""
    per = -(-n_pos // world)
    per = -(-per // granularity) * granularity
    out = []
    for r in range(world):
        b = min(r * per, n_pos)
        out.append((b, min(b + per, n_pos)))
    return out


def tail_owner(chunks):
    """Rank that owns the last position (where new tokens are appended)."""
    owner = 0
    for r, (b, e) in enumerate(chunks):
        if e > b:
            owner = r
    return owner


def merge_partials_host(parts):
    """Log-sum-exp merge of partial results on the host (numpy): parts [n_parts, rows, hd+2] with
    (acc, m, l) per row.  The GPU path uses bk_lse_merge; this is for tests of the exchange."""
    parts = np.asarray(parts, dtype=np.float64)
    acc, m, l = parts[..., :-2], parts[..., -2], parts[..., -1]
    valid = l > 0
    M = np.max(np.where(valid, m, -np.inf), axis=0)
    w = np.where(valid, np.exp(np.where(valid, m - M, 0.0)), 0.0)
    L = (l * w).sum(0)
    out = (acc * w[..., None]).sum(0)
    with np.errstate(invalid="ignore", divide="ignore"):
        return np.where(L[..., None] > 0, out / L[..., None], 0.0).astype(np.float32)


def all_gather_partials(dist, part, world):
    """All-gather of one rank's [rows, hd+2] partial tensor -> [world, rows, hd+2] (torch)."""
    import torch
    out = torch.empty((world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(out.view(-1), part.contiguous().view(-1)) if part.is_cuda else \
        dist.all_gather(list(out.unbind(0)), part.contiguous())
    return out


class ContextSplit:
    """One long sequence split into contiguous context chunks over the ranks, with the exchange of
    the partial results fused into their merge over peer memory (bk_decode_attn_split) instead
    of an all-gather.  `cache` holds this rank's chunk (created with rope_positions = the full
    context).  Handles travel through torch.distributed's object all-gather (any backend)."""

    def __init__(self, cache, dist, rank, world):
        import ctypes as C
        from . import _abi
        self.cache, self.ctx, self.rank, self.world = cache, cache.ctx, rank, world
        self.seqno = 0
        handle = (C.c_ubyte * 64)()
        mb = C.c_void_p()
        self.ctx.check(self.ctx.lib.bk_mailbox_create(self.ctx.h, world, rank, cache.n_head, cache.hd, C.byref(mb), handle))
        self.mb = mb
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle))
        else:
            handles[0] = bytes(handle)
        blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(handles))
        self.ctx.check(self.ctx.lib.bk_mailbox_open_peers(self.mb, blob))
        if world > 1:
            dist.barrier()  # nobody sends before every mailbox is mapped everywhere

    def attend_device(self, il, q_ptr, out_ptr, q_pos, n_pos=None, seq=0):
        """Scan the local chunk, exchange, merge: every rank ends with the full output."""
        if n_pos is None:
            n_pos = self.cache.n_pos(il, seq)
        self.seqno += 1
        self.ctx.check(self.ctx.lib.bk_decode_attn_split(self.cache.h, il, seq, n_pos, q_pos, q_ptr, out_ptr,
                                                         self.mb, self.seqno))

    def step_device(self, il, q_ptr, k_ptr, v_ptr, out_ptr, q_pos, seq=0):
        """The whole step in one launch per rank: the tail owner passes the new token's k/v
        device pointers (appended as its next row, roped at q_pos), the others pass None."""
        self.seqno += 1
        self.ctx.check(self.ctx.lib.bk_attn_step_split(self.cache.h, il, seq, q_pos, q_ptr, k_ptr, v_ptr, out_ptr,
                                                       self.mb, self.seqno))

    def open_layers_mailbox(self, dist, n_layers):
        """A second mailbox with a row for every (layer, q head), for steps whose layers do not depend on one
        another: all layers are scanned first and the partial rows of all of them cross in ONE exchange."""
        import ctypes as C
        handle = (C.c_ubyte * 64)()
        mb = C.c_void_p()
        self.ctx.check(self.ctx.lib.bk_mailbox_create(self.ctx.h, self.world, self.rank, n_layers * self.cache.n_head,
                                                      self.cache.hd, C.byref(mb), handle))
        self.mb_layers, self.n_layers_mb, self.seqno_layers = mb, n_layers, 0
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle))
        else:
            handles[0] = bytes(handle)
        blob = (C.c_ubyte * (64 * self.world)).from_buffer_copy(b"".join(handles))
        self.ctx.check(self.ctx.lib.bk_mailbox_open_peers(self.mb_layers, blob))
        self.part_layers = self.ctx.alloc(n_layers * self.cache.n_head * (self.cache.hd + 2) * 4)
        if self.world > 1:
            dist.barrier()

    def step_layers_device(self, q_ptr, k_ptr, v_ptr, out_ptr, q_pos, seq=0):
        """One token through all layers of the layers mailbox with a single exchange: q_ptr [n_layers][n_head][hd],
        out_ptr the same shape; the tail owner passes the new token's k/v (the same rows for every layer here),
        the others None.  Only for callers whose layer l + 1 does not need layer l's output."""
        nh, hd = self.cache.n_head, self.cache.hd
        for il in range(self.n_layers_mb):
            if k_ptr is not None:
                self.cache.append_device(il, k_ptr, v_ptr, n_tokens=1, pos=q_pos, seq=seq)
            self.cache.decode_device(il, q_ptr + il * nh * hd * 4, self.part_layers.ptr + il * nh * (hd + 2) * 4,
                                     q_pos=[q_pos], partial=True)
        self.seqno_layers += 1
        self.ctx.check(self.ctx.lib.bk_exchange_merge(self.mb_layers, nh // self.cache.n_kv, self.part_layers.ptr, out_ptr,
                                                      self.seqno_layers))

    def close(self):
        if getattr(self, "mb", None):
            self.ctx.lib.bk_mailbox_destroy(self.mb)
            self.mb = None
        if getattr(self, "mb_layers", None):
            self.ctx.lib.bk_mailbox_destroy(self.mb_layers)
            self.mb_layers = None
            self.part_layers.free()
