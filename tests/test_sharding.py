"""Context sharding (the N > 1 path of bench.py) on CPU: per-shard partial records from
the oracle, exchanged between two gloo ranks and merged, must reproduce the unsharded
attention. This is the host-side logic of the multi-GPU path; the records themselves
come from the GPU kernels on a B200 (tests/test_gpu_attn.py covers shards there)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.oracle import Oracle

NH, NKV, HD = 24, 4, 256


def shard_bounds(n_keys, world, rank):
    per = (n_keys + world - 1) // world
    return rank * per, min(n_keys, (rank + 1) * per)


def test_shard_bounds_cover_everything():
    for n in (1, 2, 7, 100, 131001):
        for w in (1, 2, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and max(e for _, e in spans) == n
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert b1 == max(e0, b1) and b1 >= e0 or e1 <= b1  # contiguous or empty tail
            assert sum(max(0, e - b) for b, e in spans) == n


@pytest.mark.parametrize("n_keys,world", [(300, 2), (5, 4), (1000, 8)])
def test_sharded_records_merge_to_the_whole(oracle, n_keys, world):
    rng = np.random.default_rng(n_keys)
    K = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(3, K), oracle.kv_store_rows(3, V)
    want = oracle.attn(q[None], kc, vc, [n_keys - 1], NKV, 1 / 16, 3, 3)[0]
    recs = []
    for r in range(world):
        b, e = shard_bounds(n_keys, world, r)
        recs.append(oracle.attn_partials(q, kc, vc, b, max(b, e), NKV, 1 / 16, 3, 3, 1))
    merged = oracle.attn_merge(np.concatenate(recs, axis=1))
    assert np.abs(merged - want).max() <= 5e-6
    if world > n_keys:
        assert np.isneginf(recs[-1][:, 0, 0]).all()  # a shard without keys: the empty record


def _rank_main(rank, world, port, n_keys, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ora = Oracle()
    rng = np.random.default_rng(1234)  # every rank builds the same cache, keeps its slice
    K = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    b, e = shard_bounds(n_keys, world, rank)
    row = ora.row_bytes(2)
    kc = ora.kv_store_rows(2, K[b:e]) if e > b else np.zeros(row * NKV, np.uint8)
    vc = ora.kv_store_rows(2, V[b:e]) if e > b else np.zeros(row * NKV, np.uint8)
    mine = torch.from_numpy(ora.attn_partials(q, kc, vc, 0, max(0, e - b), NKV, 1 / 16, 2, 2, 1))
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)                       # [rank][head][1][258]
    recs = torch.cat(gathered, dim=1).numpy()             # [head][rank][258]
    merged = ora.attn_merge(recs)
    if rank == 0:
        want = ora.attn(q[None], ora.kv_store_rows(2, K), ora.kv_store_rows(2, V), [n_keys - 1], NKV,
                        1 / 16, 2, 2)[0]
        np.save(out_path, np.array([np.abs(merged - want).max()]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_all_gather_and_merge(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "err.npy")
    mp.spawn(_rank_main, args=(2, port, 257, out), nprocs=2, join=True)
    assert float(np.load(out)[0]) <= 5e-6


def test_sequence_dealing_is_a_balanced_partition():
    """bench.py's sequence sharding (benchmark config 5 over N GPUs): every sequence lands on
    exactly one rank, every rank derives the same table, and the loads differ by less than
    the longest sequence."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "bench_module", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    lens = [int(x) for x in np.random.default_rng(7).integers(1024, 32769, size=64)]
    for world in (1, 2, 4, 8):
        table = bench.deal_sequences(lens, world)
        assert table == bench.deal_sequences(list(lens), world)
        assert sorted(i for r in table for i in r) == list(range(64))
        loads = [sum(lens[i] for i in r) for r in table]
        assert max(loads) - min(loads) < max(lens)
    assert bench.deal_sequences([5, 5, 5], 2) == [[0, 2], [1]]
