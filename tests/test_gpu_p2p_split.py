"""Context split over two GPUs with the peer-memory exchange (bk_decode_attn_split).

Spawns one process per GPU (skipped with fewer than two GPUs): each holds one half of a
sequence, rank 0 also holds the whole sequence in a second cache as the reference.  The merged
output on BOTH ranks must equal the whole-cache output, over several layers and steps (the
mailbox slots alternate with the call's parity and are reused), with new tokens appended on
the rank that owns the tail.  NVLS/multimem is not involved (plain peer stores); the ranks
leave only between steps.
"""
import importlib
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NH, NKV, HD = 24, 4, 256


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_q, variant="attend"):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if variant == "unfused":
        os.environ["BONSAI_KV_SPLIT_UNFUSED"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok, worst = True, 0.0
    try:
        bk = importlib.import_module("ternary-bonsai-inference_b200")
        par = importlib.import_module("ternary-bonsai-inference_b200.parallel")
        ctx = bk.Context(rank)
        rng = np.random.default_rng(3)       # same stream on both ranks
        n0, steps, layers = 6000, 3, 2
        n_total = n0 + steps
        k = rng.standard_normal((n_total, NKV, HD), dtype=np.float32)
        v = rng.standard_normal((n_total, NKV, HD), dtype=np.float32)
        k[:, :, [9, 100, 222]] *= np.float32(20.0)
        v[:, :, [9, 100, 222]] *= np.float32(20.0)
        q = rng.standard_normal((steps, layers, NH, HD), dtype=np.float32)
        chunks = par.split_context(n0, world)
        b, e = chunks[rank]
        owner = par.tail_owner(chunks)
        mode = bk.parse_mode("planar4")
        mine = bk.AttnCache(ctx, mode, n_layers=layers, n_ctx=(e - b) + steps, rope_positions=n_total)
        whole = bk.AttnCache(ctx, mode, n_layers=layers, n_ctx=n_total) if rank == 0 else None
        for il in range(layers):
            mine.append(il, k[b:e], v[b:e], pos=b)
            if whole:
                whole.append(il, k[:n0], v[:n0])
        split = par.ContextSplit(mine, dist, rank, world)
        d_out = ctx.alloc(NH * HD * 4)
        for s in range(steps):
            pos = n0 + s
            for il in range(layers):
                d_q = ctx.to_device(q[s, il])
                if variant == "step":      # one launch per rank: the tail owner's append is part of it
                    d_k, d_v = ctx.to_device(k[pos]), ctx.to_device(v[pos])
                    own = rank == owner
                    split.step_device(il, d_q.ptr, d_k.ptr if own else None, d_v.ptr if own else None, d_out.ptr, q_pos=pos)
                else:
                    if rank == owner:
                        mine.append(il, k[pos], v[pos], pos=pos)
                    split.attend_device(il, d_q.ptr, d_out.ptr, q_pos=pos)
                got = d_out.download((NH, HD), np.float32)   # synchronises: reports a timed-out wait
                d_q.free()
                if whole:
                    whole.append(il, k[pos], v[pos])
                    want = whole.attend(il, q[s, il])[0]
                    worst = max(worst, float(np.max(np.abs(got - want))))
                gathered = [None] * world
                dist.all_gather_object(gathered, got.tobytes())
                ok = ok and all(g == gathered[0] for g in gathered)   # both ranks hold the same output
        split.close()
        out_q.put((rank, ok, worst))
    except Exception as ex:  # report instead of hanging the parent
        out_q.put((rank, False, repr(ex)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("variant", ["attend", "step", "unfused"])
def test_split_context_over_peer_memory(variant):
    """attend: exchange and merge inside the decode launch's finishing CTAs; step: the tail owner's
    append in the same launch too; unfused: partial rows, then the separate exchange kernel."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, variant)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(60)
    for rank, ok, worst in results:
        assert ok is True, (rank, worst)
    worst0 = [w for r, ok, w in results if r == 0][0]
    assert worst0 < 2e-4, worst0
