"""CPU tests of the multi-GPU host logic: partition plans, and the exchange + log-sum-exp merge of
the context split on two gloo ranks (world_size 2, no GPU)."""
import importlib
import os
import socket

import numpy as np
import pytest

par = importlib.import_module("ternary-bonsai-inference_b200.parallel")


def test_shard_sequences_balances_and_is_deterministic():
    rng = np.random.default_rng(0)
    lens = rng.integers(2048, 16385, 64)
    for world in (1, 2, 4, 8):
        plan = par.shard_sequences(lens, world)
        assert sorted(i for p in plan for i in p) == list(range(64))
        loads = [int(lens[p].sum()) for p in plan]
        assert max(loads) - min(loads) <= lens.max()
        assert plan == par.shard_sequences(list(lens), world)
    assert par.shard_sequences([5, 5, 5], 2) == [[0, 2], [1]]
    assert par.shard_sequences([], 2) == [[], []]


def test_split_context_covers_without_overlap():
    for n, world in ((262144, 8), (262144, 1), (1000, 4), (1, 8), (131073, 2), (129, 2)):
        chunks = par.split_context(n, world)
        assert chunks[0][0] == 0 and max(e for _, e in chunks) == n
        for (b0, e0), (b1, e1) in zip(chunks, chunks[1:]):
            assert e0 == b1 or (b1 == e1 == n)
        assert all((e - b) % 128 == 0 for b, e in chunks[:-1] if e < n)
        assert chunks[par.tail_owner(chunks)][1] == n


def _partials(scores, values):
    """(acc, m, l) of softmax(scores) @ values, rows = heads."""
    m = scores.max(1)
    p = np.exp(scores - m[:, None])
    return np.concatenate([p @ values, m[:, None], p.sum(1)[:, None]], axis=1).astype(np.float32)


def test_merge_partials_equals_whole():
    rng = np.random.default_rng(1)
    s = rng.standard_normal((24, 1000)) * 3
    v = rng.standard_normal((1000, 256))
    whole = _partials(s, v)
    want = whole[:, :256] / whole[:, 257:258]
    cuts = [0, 130, 131, 700, 1000]
    parts = [_partials(s[:, a:b], v[a:b]) for a, b in zip(cuts, cuts[1:])]
    parts.append(np.zeros_like(parts[0]))  # a rank with an empty chunk: l = 0
    got = par.merge_partials_host(np.stack(parts))
    assert np.max(np.abs(got - want)) < 1e-5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # same stream on every rank: replicated q, shared K/V
        n = 1000
        s = rng.standard_normal((24, n)) * 3
        v = rng.standard_normal((n, 256))
        b, e = par.split_context(n, world, granularity=128)[rank]
        mine = _partials(s[:, b:e], v[b:e]) if e > b else np.zeros((24, 258), np.float32)
        gathered = par.all_gather_partials(dist, torch.from_numpy(mine), world).numpy()
        got = par.merge_partials_host(gathered)
        whole = _partials(s, v)
        out_q.put((rank, float(np.max(np.abs(got - whole[:, :256] / whole[:, 257:258])))))
    finally:
        dist.destroy_process_group()


def test_context_split_exchange_on_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    assert set(results) == {0, 1} and max(results.values()) < 1e-5


def _rank_main_layers(rank, world, port, out_q):
    """The layers-batched form of the context split: every rank scans all layers first and the partial rows of
    all of them cross in ONE exchange per token (bk_exchange_merge); the merge is row-wise, so stacking the
    layers' rows changes nothing but the row count."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)
        n_layers, n = 3, 700
        s = rng.standard_normal((n_layers, 24, n)) * 3
        v = rng.standard_normal((n_layers, n, 256))
        b, e = par.split_context(n, world, granularity=128)[rank]
        mine = np.concatenate([_partials(s[il][:, b:e], v[il][b:e]) if e > b else np.zeros((24, 258), np.float32)
                               for il in range(n_layers)])                      # [n_layers * 24][258]
        gathered = par.all_gather_partials(dist, torch.from_numpy(mine), world).numpy()
        got = par.merge_partials_host(gathered)                                 # ONE exchange, ONE merge
        worst = 0.0
        for il in range(n_layers):
            whole = _partials(s[il], v[il])
            worst = max(worst, float(np.max(np.abs(got[il * 24:(il + 1) * 24] - whole[:, :256] / whole[:, 257:258]))))
        out_q.put((rank, worst))
    finally:
        dist.destroy_process_group()


def test_layers_batched_exchange_on_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main_layers, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    assert set(results) == {0, 1} and max(results.values()) < 1e-5
