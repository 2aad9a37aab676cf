"""Tensor-parallel host logic on CPU: two gloo ranks cut the same full weights with shard_weight, run
their shard of the projections through the oracle (the reference's arithmetic), exchange with the
collectives the GPU path uses (all-reduce after a row-parallel projection, gather of logits / argmax
pairs after the column-parallel output), and must reproduce the unsharded result: bit for bit where
only rows are split, to f32 summation order where K is split."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.bindings import Oracle, Q4_K, Q8_0
from tensorlisp_b200.programs import DecoderConfig, combine_argmax, decoder_step, decoder_weights, shard_weight

D, FFN, VOCAB, TOK = 512, 1024, 768, 5


def full_weights():
    rng = np.random.default_rng(21)
    return {"blk.0.ffn_gate": (rng.standard_normal((FFN, D)) * 0.05).astype(np.float32),
            "blk.0.ffn_up": (rng.standard_normal((FFN, D)) * 0.05).astype(np.float32),
            "blk.0.ffn_down": (rng.standard_normal((D, FFN)) * 0.05).astype(np.float32),
            "output": (rng.standard_normal((VOCAB, D)) * 0.05).astype(np.float32)}


def ffn_and_logits(o, W, x):
    q = {k: o.quantize(Q8_0 if k == "output" else Q4_K, v) for k, v in W.items()}
    g = o.mul_mat(Q4_K, q["blk.0.ffn_gate"], D, x)
    u = o.mul_mat(Q4_K, q["blk.0.ffn_up"], D, x)
    h = o.silu_mul(g, u)
    y = o.mul_mat(Q4_K, q["blk.0.ffn_down"], h.shape[1], h)
    return y, o.mul_mat(Q8_0, q["output"], D, x)


def rank_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = Oracle()
        x = np.random.default_rng(3).standard_normal((TOK, D)).astype(np.float32)
        W = {k: shard_weight(k, v, rank, world) for k, v in full_weights().items()}
        y, logits = ffn_and_logits(o, W, x)
        ty = torch.from_numpy(np.ascontiguousarray(y))
        dist.all_reduce(ty)                                   # ALLREDUCE after the row-parallel ffn_down
        parts = [torch.empty_like(torch.from_numpy(logits)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(logits)))
        pair = torch.from_numpy(np.stack([logits.max(axis=1), logits.argmax(axis=1).astype(np.float32)]))
        pairs = [torch.empty_like(pair) for _ in range(world)]
        dist.all_gather(pairs, pair)
        if rank == 0:
            ret["y"] = ty.numpy().copy()
            ret["logits"] = np.concatenate([p.numpy() for p in parts], axis=1)
            mx = np.stack([p.numpy()[0] for p in pairs])
            ix = np.stack([p.numpy()[1] for p in pairs]).astype(np.int64)
            ret["argmax"] = combine_argmax(mx, ix, VOCAB // world)
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_projections():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(rank_main, args=(2, port, ret), nprocs=2, join=True)
    o = Oracle()
    x = np.random.default_rng(3).standard_normal((TOK, D)).astype(np.float32)
    y, logits = ffn_and_logits(o, full_weights(), x)
    # K split on 256-element boundaries: same quantization blocks, same integer sums, another f32 order
    assert np.abs(ret["y"] - y).max() <= 1e-5 * np.abs(y).max()
    # rows split: every logit is computed exactly as in the unsharded matrix
    assert np.array_equal(ret["logits"], logits)
    assert np.array_equal(ret["argmax"], logits.argmax(axis=1))


def test_shard_shapes_partition_the_model():
    cfg = DecoderConfig(n_layers=1, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ffn=1024, vocab=768)
    full = {s.name: s for s in decoder_weights(cfg, 1)}
    for tp in (2,):
        shards = [{s.name: s for s in decoder_weights(cfg, tp)} for _ in range(tp)]
        for name, f in full.items():
            ne = [sh[name].ne for sh in shards]
            if len(f.ne) == 1 or name == "token_embd":
                assert all(n == f.ne for n in ne)
                continue
            w = np.zeros((f.ne[1], f.ne[0]), np.float32)
            for r in range(tp):
                cut = shard_weight(name, w, r, tp)
                assert list(cut.shape) == [ne[r][1], ne[r][0]], name
        g = decoder_step(cfg, 4, 64, 16, tp=tp)
        ops = [g.graph.tensors[n].op for n in g.graph.nodes]
        assert ops.count("ALLREDUCE") == 2 * cfg.n_layers


def test_combine_argmax_breaks_ties_like_a_single_argmax():
    mx = np.array([[1.0, 5.0, 2.0], [1.0, 4.0, 7.0]], np.float32)
    ix = np.array([[3, 0, 1], [0, 2, 4]], np.int64)
    assert combine_argmax(mx, ix, 10).tolist() == [3, 0, 14]
