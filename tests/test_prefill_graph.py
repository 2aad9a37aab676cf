"""Host-side checks of the prompt-pass program (no GPU): node counts, shapes and the tensor-parallel shards."""
import numpy as np

from tensorlisp_b200.graph import F16, F32, Q8_0
from tensorlisp_b200.programs import DecoderConfig, decoder_weights, prefill_step


def small_cfg():
    return DecoderConfig(n_layers=3, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ffn=1024, vocab=2048, wtype=Q8_0)


def ops_of(g):
    out = {}
    for t in g.nodes:
        op = g.tensors[t].op
        out[op] = out.get(op, 0) + 1
    return out


def test_prefill_graph_shapes():
    cfg = small_cfg()
    S, L = 3, 40
    dg = prefill_step(cfg, S, L)
    g = dg.graph
    ops = ops_of(g)
    assert ops["FLASH_ATTN_EXT"] == cfg.n_layers
    assert ops["MUL_MAT"] == 7 * cfg.n_layers + 1
    assert ops["CUSTOM"] == cfg.n_layers           # one cache write per layer
    assert "ALLREDUCE" not in ops
    assert g.tensors[dg.logits].ne[:2] == [cfg.vocab, S]
    assert dg.inputs == dict(ids=0, pos=1, mask=2, last=3, slots=4)
    blocks = S * ((L + cfg.block_size - 1) // cfg.block_size)
    assert dg.state_bytes == [blocks * cfg.n_kv_heads * cfg.block_size * cfg.head_dim * 2] * (2 * cfg.n_layers)
    # attention operands are views [head_dim, tokens, heads, prompts] over [head_dim, heads, tokens*prompts] storage
    fa = [g.tensors[t] for t in g.nodes if g.tensors[t].op == "FLASH_ATTN_EXT"][0]
    q, k, v, m = (g.tensors[s] for s in fa.src[:4])
    assert q.ty == F32 and q.ne == [128, L, cfg.n_heads, S] and q.nb[1] == 128 * cfg.n_heads * 4 and q.nb[2] == 128 * 4
    assert k.ty == F16 and k.ne == [128, L, cfg.n_kv_heads, S] and k.nb[1] == 128 * cfg.n_kv_heads * 2
    assert v.ty == F16 and v.ne == k.ne
    assert m.ty == F16 and m.ne[:2] == [L, L]
    assert fa.ne == [128, cfg.n_heads, L, S]


def test_prefill_graph_without_cache():
    cfg = small_cfg()
    dg = prefill_step(cfg, 2, 16, write_cache=False)
    assert "CUSTOM" not in ops_of(dg.graph)
    assert dg.state_bytes == [] and "slots" not in dg.inputs


def test_prefill_graph_tensor_parallel():
    cfg = small_cfg()
    S, L, tp = 2, 32, 2
    dg = prefill_step(cfg, S, L, tp=tp)
    g = dg.graph
    ops = ops_of(g)
    assert ops["ALLREDUCE"] == 2 * cfg.n_layers
    assert g.tensors[dg.logits].ne[:2] == [cfg.vocab // tp, S]
    assert [(s.name, s.ne) for s in dg.weights] == [(s.name, s.ne) for s in decoder_weights(cfg, tp)]
    fa = [g.tensors[t] for t in g.nodes if g.tensors[t].op == "FLASH_ATTN_EXT"][0]
    assert g.tensors[fa.src[0]].ne[2] == cfg.n_heads // tp and g.tensors[fa.src[1]].ne[2] == cfg.n_kv_heads // tp
    blocks = S * (L // cfg.block_size)
    assert dg.state_bytes[0] == blocks * (cfg.n_kv_heads // tp) * cfg.block_size * cfg.head_dim * 2
    # every all-reduce sums a full-width [d_model, tokens] activation
    for t in g.nodes:
        T = g.tensors[t]
        if T.op == "ALLREDUCE":
            assert T.ne[:2] == [cfg.d_model, S * L] and T.ty == F32
