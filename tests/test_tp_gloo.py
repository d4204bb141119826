"""Tensor-parallel sharding of a decoder block checked on CPU with two gloo ranks (no GPU)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from leankv_b200.engine import DecodeEngine, DecoderConfig

CFG = DecoderConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_layers=2, num_q_heads=8,
                    num_kv_heads=2, head_dim=128)


def _full_weights():
    gen = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=gen) * 0.05
    full = {"embed": r(64, 256), "final_norm": torch.ones(256), "lm_head": r(64, 256), "layers": []}
    for _ in range(CFG.num_layers):
        full["layers"].append({"ln1": torch.ones(256), "ln2": torch.ones(256),
                               "q_proj": r(1024, 256), "k_proj": r(256, 256), "v_proj": r(256, 256),
                               "o_proj": r(256, 1024), "gate_proj": r(512, 256), "up_proj": r(512, 256),
                               "down_proj": r(256, 512)})
    return full


def _block(x, lw, nq, nkv, t, reduce):
    """One token through one block with per-head 'attention' = v of its kv head (keeps the test about
    the projections' sharding); masks use the same thresholds on every rank."""
    m = lambda a, thr: a * (a.abs() > thr)
    qkv = m(x, t) @ lw["wqkv_t"]
    v = qkv[(nq + nkv) * 128:].reshape(nkv, 128)
    attn = v.repeat_interleave(nq // nkv, dim=0).reshape(-1)
    o = m(attn, t) @ lw["wo_t"]
    o = reduce(o)
    h = x + o
    mlp = F.silu(m(h, t) @ lw["wgate_t"]) * (m(h, t) @ lw["wup_t"])
    d = m(mlp, t) @ lw["wdown_t"]
    return h + reduce(d)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = DecodeEngine.shard_weights(_full_weights(), CFG, rank, world)
        x = torch.randn(256, generator=torch.Generator().manual_seed(1))

        def reduce(t):
            dist.all_reduce(t)
            return t

        for lw in w["layers"]:
            x = _block(x, lw, CFG.num_q_heads // world, CFG.num_kv_heads // world, 0.3, reduce)
        if rank == 0:
            torch.save(x, out)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_equals_single_rank(tmp_path):
    out = str(tmp_path / "tp2.pt")
    mp.spawn(_worker, args=(2, 29731, out), nprocs=2, join=True)
    got = torch.load(out)
    w = DecodeEngine.shard_weights(_full_weights(), CFG, 0, 1)
    x = torch.randn(256, generator=torch.Generator().manual_seed(1))
    for lw in w["layers"]:
        x = _block(x, lw, CFG.num_q_heads, CFG.num_kv_heads, 0.3, lambda t: t)
    assert torch.allclose(got, x, rtol=1e-4, atol=2e-4)


def test_shard_shapes():
    for tp in (1, 2):
        w = DecodeEngine.shard_weights(_full_weights(), CFG, tp - 1, tp)
        lw = w["layers"][0]
        assert lw["wqkv_t"].shape == (256, (8 + 2 + 2) * 128 // tp)
        assert lw["wo_t"].shape == (1024 // tp, 256) and lw["wdown_t"].shape == (512 // tp, 256)
        assert lw["wgate_t"].shape == (256, 512 // tp) and w["lm_head_t"].shape == (256, 64)
        assert all(t.is_contiguous() for t in lw.values())
    with pytest.raises(RuntimeError):
        DecodeEngine(DecoderConfig(num_q_heads=8, num_kv_heads=8), {}, "cpu")


def _batch_worker(rank, world, port, out):
    """Batch-sharded decode has no data-path collective: each rank only needs to know its slice.
    The ranks gather their slices (control plane only) so the test can see the whole partition."""
    from leankv_b200.batch_engine import partition_batch

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = partition_batch(81, world, rank)
        counts = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([mine.start, mine.stop]))
        # per-rank token throughput adds up: sum of "tokens per step" over ranks == the batch
        tok = torch.tensor([len(mine)], dtype=torch.int64)
        dist.all_reduce(tok)
        if rank == 0:
            torch.save({"ranges": [c.tolist() for c in counts], "total": int(tok)}, out)
    finally:
        dist.destroy_process_group()


def test_batch_partition_covers_every_sequence_once(tmp_path):
    from leankv_b200.batch_engine import partition_batch

    out = str(tmp_path / "part.pt")
    mp.spawn(_batch_worker, args=(2, 29741, out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["ranges"] == [[0, 41], [41, 81]] and r["total"] == 81
    for total, world in ((80, 1), (80, 2), (80, 4), (80, 8), (7, 8), (0, 2)):
        seen = [i for rk in range(world) for i in partition_batch(total, world, rk)]
        assert seen == list(range(total))
        sizes = [len(partition_batch(total, world, rk)) for rk in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        partition_batch(8, 2, 2)
