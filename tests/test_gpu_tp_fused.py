"""Tensor-parallel decode on two GPUs: the all-reduce fused into the RMSNorm (tagged stores
into the peers' inboxes, sum in rank order) against the NCCL all-reduce, eagerly and through a
CUDA graph.

Needs two GPUs; skipped otherwise.  Ranks are child processes (one per GPU) that rendezvous
on 127.0.0.1."""

import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RANKS = {n: 24 for n in ("q", "k", "v", "o", "gate", "up", "down")}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    from quantibbler_b200.decoder import Decoder, DecoderConfig, random_model
    from quantibbler_b200.gpu import GpuContext

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    ctx = GpuContext.init_at(rank)
    results = {}
    for serving, batch in (("float32", 3), ("bfloat16", 16)):
        base = dict(n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                    vocab=128, max_seq=32, max_batch=batch, kv_dtype="float32", serving=serving)
        first = [(5 * i + 3) % 128 for i in range(batch)]
        for fused in (True, False):
            cfg = DecoderConfig(fused_allreduce=fused, **base)
            weights = random_model(cfg, RANKS, seed=11)
            dec = Decoder(ctx, cfg, weights, tp_rank=rank, tp_size=world, group=dist.group.WORLD)
            assert dec.fused_ar == fused, getattr(dec, "fused_ar_error", "")
            dec.start(first, [0] * batch)
            toks, logits = [], []
            for _ in range(5):
                dec.step()
                ctx.synchronize()
                logits.append(dec.logits.cpu().numpy().copy())
                dec.advance()
                toks.append(dec.token_ids.cpu().numpy().copy())
            results[(serving, fused)] = (np.array(toks), np.array(logits))
            if fused:  # the same through a CUDA graph: the device-side call counter keeps counting
                graph = Decoder(ctx, cfg, weights, tp_rank=rank, tp_size=world,
                                group=dist.group.WORLD)
                graph.capture()
                graph.start(first, [0] * batch)
                results[(serving, "graph")] = (graph.decode(5), None)
            dist.barrier()
        if rank == 0:
            # the same model unsharded, on this GPU alone: what the sharded run must reproduce
            cfg = DecoderConfig(**base)
            single = Decoder(ctx, cfg, random_model(cfg, RANKS, seed=11))
            single.start(first, [0] * batch)
            toks, logits = [], []
            for _ in range(5):
                single.step()
                ctx.synchronize()
                logits.append(single.logits.cpu().numpy().copy())
                single.advance()
                toks.append(single.token_ids.cpu().numpy().copy())
            results[(serving, "single")] = (np.array(toks), np.array(logits))
        dist.barrier()
    # The all-reduce INSIDE the plans (o / down push their outputs into the peers' inboxes, the
    # norm inside gate,up / q,k,v sums what arrived) against the all-reduce + norm kernel between
    # the plain plans: the same sum in the same rank order, so the same bits.
    for serving in ("float32", "bfloat16"):
        base = dict(n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                    vocab=128, max_seq=32, max_batch=2, kv_dtype="float32", serving=serving)
        for inside in (True, False):
            cfg = DecoderConfig(norm_fused_max_batch_tp=4 if inside else 0, **base)
            dec = Decoder(ctx, cfg, random_model(cfg, RANKS, seed=12), tp_rank=rank, tp_size=world,
                          group=dist.group.WORLD)
            assert dec.fused_ar and dec.allreduce_in_plans == inside
            dec.capture()
            dec.start([7, 99], [0, 3])
            logits = []
            for _ in range(4):
                dec.graph.replay()
                ctx.synchronize()
                logits.append(dec.logits.cpu().numpy().copy())
                dec.advance()
            results[(serving, f"inplan{int(inside)}")] = (np.array(logits), None)
            dist.barrier()
    np.savez(os.path.join(out_dir, f"tp_rank{rank}.npz"),
             **{f"{s}_{f}_tok": v[0] for (s, f), v in results.items()},
             **{f"{s}_{f}_log": v[1] for (s, f), v in results.items() if v[1] is not None})
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)   # a captured graph holds NCCL kernels: leave without the communicator teardown


def test_fused_allreduce_matches_nccl(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    got, other = np.load(tmp_path / "tp_rank0.npz"), np.load(tmp_path / "tp_rank1.npz")
    from oracle import decoder_np
    from quantibbler_b200.decoder import DecoderConfig, random_model
    for serving in ("float32", "bfloat16"):
        for r in (got, other):
            assert np.array_equal(r[f"{serving}_inplan1_tok"], r[f"{serving}_inplan0_tok"]), serving
    for serving, batch, tol in (("float32", 3, 2e-4), ("bfloat16", 16, 3e-2)):
        a, b = got[f"{serving}_True_log"], got[f"{serving}_False_log"]
        # NCCL adds the two partials in its own order; with two ranks a + b == b + a, so the
        # fused path must agree bit for bit on the first step and stay within rounding after
        assert np.abs(a - b).max() <= tol * np.abs(b).max()
        assert np.array_equal(got[f"{serving}_True_tok"], got[f"{serving}_False_tok"])
        assert np.array_equal(got[f"{serving}_graph_tok"], got[f"{serving}_True_tok"])
        # both ranks end every step with the same greedy tokens
        assert np.array_equal(other[f"{serving}_True_tok"], got[f"{serving}_True_tok"])
        # the two vocabulary shards side by side are the logits of the whole model: against
        # the unsharded decoder on one GPU (row-parallel layers sum two partial products
        # instead of one long one, so equal up to rounding) ...
        full = np.concatenate([got[f"{serving}_True_log"], other[f"{serving}_True_log"]], axis=-1)
        single = got[f"{serving}_single_log"]
        assert full.shape == single.shape
        assert np.abs(full[0] - single[0]).max() <= tol * np.abs(single).max()
        exact_serving = serving == "float32"   # bfloat16 rounds each rank's partial t and u, so a
        if exact_serving:                      # near-tie may pick another token there
            assert np.array_equal(got[f"{serving}_True_tok"], got[f"{serving}_single_tok"])
        # ... and against the CPU restatement of the reference's forward
        cfg = DecoderConfig(n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                            vocab=128, max_seq=32, max_batch=batch, kv_dtype="float32",
                            serving=serving)
        weights = random_model(cfg, RANKS, seed=11)
        for b_i in range(min(batch, 3)):
            session = decoder_np.Session(cfg, weights)
            tok = (5 * b_i + 3) % 128
            for step in range(5):
                want_tok, want = session.step(tok)
                assert np.abs(full[step, b_i] - want).max() <= 5 * tol * np.abs(want).max()
                if exact_serving:
                    assert want_tok == got[f"{serving}_True_tok"][step, b_i]
                tok = int(got[f"{serving}_True_tok"][step, b_i])   # feed what the device chose
