"""Tensor-parallel partitioning on CPU: two gloo ranks, each holding its shard, compute
partial results with the oracle; the collectives must reproduce the unsharded layer."""

import os
import socket

import numpy as np
import pytest

import oracle
from quantibbler_b200 import tp
from quantibbler_b200.decoder import DecoderConfig, random_layer, random_model


def test_shards_tile_the_layer():
    rng = np.random.default_rng(0)
    layer = random_layer(rng, 64, 96, 40, with_bias=True)
    cols = [tp.shard_column_parallel(layer, r, 4) for r in range(4)]
    assert np.array_equal(np.concatenate([c["ub_rows"] for c in cols]), layer["ub_rows"])
    assert np.array_equal(np.concatenate([c["s1"] for c in cols]), layer["s1"])
    assert all(np.array_equal(c["vb_t_rows"], layer["vb_t_rows"]) for c in cols)
    rows = [tp.shard_row_parallel(layer, r, 4) for r in range(4)]
    assert np.array_equal(np.concatenate([c["vb_t_rows"] for c in rows], axis=1), layer["vb_t_rows"])
    assert rows[0]["bias"] is not None and all(c["bias"] is None for c in rows[1:])
    with pytest.raises(ValueError, match="not divisible"):
        tp.shard_column_parallel(layer, 0, 5)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    import torch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)
    col = random_layer(rng, 64, 96, 40, with_bias=True)      # e.g. gate
    row = random_layer(rng, 96, 64, 40, with_bias=True)      # e.g. down
    x = rng.standard_normal(96).astype(np.float32)

    def apply(layer, v):
        return oracle.layer_apply(layer["ub_rows"], layer["vb_t_rows"], layer["dout"], layer["din"],
                                  layer["r"], layer["s1"], layer["s2"], layer["bias"], v)

    full_mid = apply(col, x)
    full_out = apply(row, full_mid)
    # column-parallel: the output stays sharded by feature
    mine = apply(tp.shard_column_parallel(col, rank, world), x)
    lo = rank * (64 // world)
    ok_col = np.array_equal(mine, full_mid[lo:lo + 64 // world])
    # row-parallel on the sharded activations: one all-reduce completes the sum
    part = apply(tp.shard_row_parallel(row, rank, world), mine)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    err = float(np.abs(t.numpy() - full_out).max() / np.abs(full_out).max())
    # greedy over a vocabulary-sharded head: the first maximum wins across ranks
    logits = np.zeros(32, np.float32)
    logits[5] = logits[20] = 3.0
    shard = logits[rank * 16:(rank + 1) * 16]
    pair = torch.tensor([float(shard.max()), float(np.argmax(shard) + rank * 16)])
    pairs = [torch.zeros(2) for _ in range(world)]
    dist.all_gather(pairs, pair)
    vals = torch.stack([p[0] for p in pairs])
    winner = int(pairs[int(torch.argmax(vals))][1])
    q.put((rank, ok_col, err, winner))
    dist.destroy_process_group()


def test_two_rank_partition_reproduces_the_layer():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_col, err, winner in results:
        assert ok_col, rank
        assert err <= 1e-6, (rank, err)
        assert winner == 5


def test_shard_model_shapes():
    cfg = DecoderConfig(n_layers=1, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                        vocab=128)
    w = random_model(cfg, {n: 16 for n in ("q", "k", "v", "o", "gate", "up", "down")}, seed=1)
    s = tp.shard_model(w, cfg, 1, 2)
    lw = s["layers"][0]
    assert lw["q"]["dout"] == 32 and lw["k"]["dout"] == 16 and lw["gate"]["dout"] == 64
    assert lw["o"]["din"] == 32 and lw["down"]["din"] == 64
    assert s["lm_head"].shape == (64, 64) and s["vocab_offset"] == 64
    with pytest.raises(ValueError, match="must divide"):
        tp.shard_model(w, cfg, 0, 4)


def _model_worker(rank, world, port, q):
    """One tensor-parallel rank of the reference's parity-tiny model in NumPy: its shard of
    every linear and of the head, local heads only, one gloo all-reduce per sub-block."""
    import dataclasses
    import json

    import torch
    import torch.distributed as dist

    from conftest import GOLDEN
    from oracle import decoder_np
    from quantibbler_b200 import model_dir
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    fixture = os.path.join(GOLDEN, "parity-tiny")
    cfg, weights = model_dir.decoder_inputs(model_dir.load(fixture), max_seq=16)
    with open(os.path.join(fixture, "goldens.json")) as f:
        g = json.load(f)
    local = dataclasses.replace(cfg, n_heads=cfg.n_heads // world,
                                n_kv_heads=cfg.n_kv_heads // world, d_ff=cfg.d_ff // world)

    def reduce(part):
        t = torch.from_numpy(np.ascontiguousarray(part, dtype=np.float32).copy())
        dist.all_reduce(t)
        return t.numpy()

    mine = decoder_np.Session(local, tp.shard_model(weights, cfg, rank, world), reduce=reduce)
    whole = decoder_np.Session(cfg, weights)
    worst_whole = worst_golden = 0.0
    for pos, tok in enumerate(g["input_ids"]):
        _, part = mine.step(tok)                      # this rank's slice of the vocabulary
        parts = [torch.zeros(cfg.vocab // world) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(part.copy()))
        logits = torch.cat(parts).numpy()
        _, want = whole.step(tok)
        worst_whole = max(worst_whole, float(np.abs(logits - want).max()))
        worst_golden = max(worst_golden, float(
            np.abs(logits - np.asarray(g["logits"][pos], np.float32)).max()))
    q.put((rank, worst_whole, worst_golden, "q_norm" in mine.w["layers"][0]))
    dist.destroy_process_group()


def test_two_rank_model_reproduces_the_reference_goldens():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_model_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, worst_whole, worst_golden, has_qk_norm in results:
        assert has_qk_norm, rank                    # the per-head norm vectors are replicated
        assert worst_whole <= 2e-5, (rank, worst_whole)    # partial sums round differently
        assert worst_golden <= 1e-2, (rank, worst_golden)  # parity_tiny.rs:26


def test_decoder_refuses_positions_beyond_the_cache():
    # host-side refusal (the device skips and reports such a token as well)
    from quantibbler_b200.decoder import check_cache_capacity
    check_cache_capacity([0, 5], 3, 8)           # reaches position 7 of 8: fits
    check_cache_capacity([], 3, 8)
    with pytest.raises(ValueError, match="position 8 does not fit the KV cache of 8 positions"):
        check_cache_capacity([0, 5], 4, 8)
    with pytest.raises(ValueError, match="position 8 does not fit"):
        check_cache_capacity([8], 1, 8)
    with pytest.raises(ValueError, match="negative position -1"):
        check_cache_capacity([-1], 1, 8)
