"""The graphs of the benchmark configurations, written against ``Graph`` the way the reference's
Scheme programs are written against the generated ``(ggml-*)`` ops: each helper is the stdlib form
it restates (crates/tensorlisp/src/scheme/stdlib/nn.ss, attn.ss; ports/gemma4/concurrency.ss for
the paged decode loop). Weights are declared in a fixed order so a caller can lay the weight buffer
out once and compile any number of shapes against it.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .graph import F16, F32, I32, Q4_K, Q8_0, Graph, row_size


@dataclass
class DecoderConfig:
    """Llama-style decoder. Defaults are the Llama-3-8B shape of benchmark config 4."""
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    d_ffn: int = 14336
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 500000.0
    block_size: int = 16
    wtype: int = Q4_K        # projections and FFN matrices
    etype: int = Q8_0        # token_embd and output


@dataclass
class WeightSpec:
    name: str
    ty: int
    ne: list   # ggml order: [K (row length), M (rows)]

    def nbytes(self) -> int:
        n = row_size(self.ty, self.ne[0])
        for d in self.ne[1:]:
            n *= d
        return n


def rms_norm_w(g: Graph, x: int, w: int, eps: float, name: str = "") -> int:
    """nn:rms-norm (stdlib/nn.ss:38-43) = ggml_mul(ggml_rms_norm(x, eps), w)."""
    return g.mul(g.rms_norm(x, eps), w, name)


def swiglu_ffn(g: Graph, x: int, norm_w: int, gate: int, up: int, down: int, eps: float, p: str = "") -> int:
    """benchmark config 2: RMSNorm -> gate/up -> SiLU(gate)*up -> down (gated MLP of ports/gemma4/gemma4.ss:62-64)."""
    h = rms_norm_w(g, x, norm_w, eps, p + "ffn_in")
    a = g.mul_mat(gate, h, p + "ffn_gate_out")
    b = g.mul_mat(up, h, p + "ffn_up_out")
    m = g.mul(g.silu(a), b, p + "ffn_act")
    return g.mul_mat(down, m, p + "ffn_down_out")


def rope_neox(g: Graph, x: int, pos: int, head_dim: int, theta: float) -> int:
    """attn:rope (stdlib/attn.ss:95-101): ggml_rope_ext(x, pos, NULL, dims, 2, 0, base, 1, 0, 1, 32, 1)."""
    return g.rope_ext(x, pos, None, head_dim, 2, 0, theta, 1.0, 0.0, 1.0, 32.0, 1.0)


@dataclass
class DecoderGraph:
    graph: Graph
    weights: list            # WeightSpec, in weight-index order
    state_bytes: list        # per state tensor
    inputs: dict             # name -> input index
    logits: int
    token: int
    cfg: DecoderConfig = None
    tp: int = 1
    extras: dict = field(default_factory=dict)


def decoder_weights(cfg: DecoderConfig, tp: int = 1) -> list:
    """Weight list of one rank. Column-parallel matrices (wq, wk, wv, gate, up, output) keep K and split
    their rows; row-parallel ones (wo, down) split K (on 256-element boundaries) and keep their rows."""
    d, hd = cfg.d_model, cfg.head_dim
    qd, kvd = cfg.n_heads * hd // tp, cfg.n_kv_heads * hd // tp
    ffn = cfg.d_ffn // tp
    assert cfg.n_kv_heads % tp == 0 and cfg.d_ffn % (tp * 256) == 0 and (cfg.n_heads * hd // tp) % 256 == 0
    ws = [WeightSpec("token_embd", cfg.etype, [d, cfg.vocab])]
    for i in range(cfg.n_layers):
        p = "blk.%d." % i
        ws += [WeightSpec(p + "attn_norm", F32, [d]), WeightSpec(p + "wq", cfg.wtype, [d, qd]),
               WeightSpec(p + "wk", cfg.wtype, [d, kvd]), WeightSpec(p + "wv", cfg.wtype, [d, kvd]),
               WeightSpec(p + "wo", cfg.wtype, [qd, d]), WeightSpec(p + "ffn_norm", F32, [d]),
               WeightSpec(p + "ffn_gate", cfg.wtype, [d, ffn]), WeightSpec(p + "ffn_up", cfg.wtype, [d, ffn]),
               WeightSpec(p + "ffn_down", cfg.wtype, [ffn, d])]
    assert cfg.vocab % tp == 0
    ws += [WeightSpec("output_norm", F32, [d]), WeightSpec("output", cfg.etype, [d, cfg.vocab // tp])]
    return ws


COLUMN_PARALLEL = ("wq", "wk", "wv", "ffn_gate", "ffn_up", "output")   # rows split across ranks
ROW_PARALLEL = ("wo", "ffn_down")                                        # K split across ranks, results summed


def shard_weight(name: str, w: np.ndarray, rank: int, tp: int) -> np.ndarray:
    """This rank's part of a full f32 weight `w` ([rows, K], or [n] for norms), cut BEFORE quantization:
    rows of column-parallel matrices (whole heads / FFN units / vocabulary entries), K ranges of
    row-parallel ones (multiples of 256, so every quantization block stays whole), everything else whole."""
    base = name.rsplit(".", 1)[-1]
    if tp == 1 or w.ndim != 2:
        return w
    if base in COLUMN_PARALLEL:
        assert w.shape[0] % tp == 0
        n = w.shape[0] // tp
        return np.ascontiguousarray(w[rank * n:(rank + 1) * n])
    if base in ROW_PARALLEL:
        assert w.shape[1] % (tp * 256) == 0
        n = w.shape[1] // tp
        return np.ascontiguousarray(w[:, rank * n:(rank + 1) * n])
    return w


def combine_argmax(local_max: np.ndarray, local_idx: np.ndarray, vocab_per_rank: int) -> np.ndarray:
    """Global argmax of column-parallel logits from every rank's (max, index) per token: arrays
    [ranks, tokens]. Ties go to the lowest global index, as a single argmax over the full row would."""
    best = np.argmax(local_max, axis=0)   # first rank holding the maximum
    tok = np.arange(local_max.shape[1])
    return (best * vocab_per_rank + local_idx[best, tok]).astype(np.int64)


def decoder_step(cfg: DecoderConfig, batch: int, max_ctx: int, pool_blocks: int, tp: int = 1,
                 with_argmax: bool = True, taps: bool = False) -> DecoderGraph:
    """One batched decode step over a paged f16 KV pool (the loop body of ports/gemma4/concurrency.ss:120-158):
    inputs are the token ids, their positions, the block tables, the context lengths (after this
    token) and the cache slots of the new tokens. With tp > 1 this is one rank's shard: attention over
    its own KV heads, an ALLREDUCE after each row-parallel projection, logits for its vocabulary slice."""
    g = Graph()
    d, hd = cfg.d_model, cfg.head_dim
    heads, kvh = cfg.n_heads // tp, cfg.n_kv_heads // tp
    specs = decoder_weights(cfg, tp)
    wid = {s.name: g.weight(s.ty, s.ne, s.name) for s in specs}
    max_blocks = (max_ctx + cfg.block_size - 1) // cfg.block_size
    pool_elems = pool_blocks * kvh * cfg.block_size * hd
    pools = [(g.state(F16, [pool_elems], "k_pool.%d" % i), g.state(F16, [pool_elems], "v_pool.%d" % i))
             for i in range(cfg.n_layers)]
    ids = g.input(I32, [batch], "ids")
    pos = g.input(I32, [batch], "pos")
    tables = g.input(I32, [max_blocks, batch], "tables")
    lens = g.input(I32, [batch], "lens")
    slots = g.input(I32, [2 * batch], "slots")
    scale = 1.0 / float(np.sqrt(hd))

    x = x0 = g.get_rows(wid["token_embd"], ids, "embd")
    for i in range(cfg.n_layers):
        p = "blk.%d." % i
        h = rms_norm_w(g, x, wid[p + "attn_norm"], cfg.eps, p + "attn_in")
        q = g.mul_mat(wid[p + "wq"], h, p + "q")
        k = g.mul_mat(wid[p + "wk"], h, p + "k")
        v = g.mul_mat(wid[p + "wv"], h, p + "v")
        q = g.set_name(rope_neox(g, g.reshape(q, [hd, heads, batch]), pos, hd, cfg.rope_theta), p + "q_rope")
        k = g.set_name(rope_neox(g, g.reshape(k, [hd, kvh, batch]), pos, hd, cfg.rope_theta), p + "k_rope")
        kc, vc = pools[i]
        g.paged_cache_write(g.cast(g.reshape(k, [hd * kvh, batch]), F16), g.cast(v, F16), kc, vc, slots,
                            cfg.block_size, kvh, p + "cache_write")
        a = g.paged_attention(g.cast(q, F16), kc, vc, tables, lens, cfg.block_size, max_ctx, scale, kvh, p + "attn")
        a = g.reshape(g.cast(a, F32), [hd * heads, batch])
        o = g.mul_mat(wid[p + "wo"], a, p + "attn_out")
        if tp > 1:
            o = g.allreduce(o, p + "attn_out_sum")
        x = g.add(x, o, p + "res1")
        f = swiglu_ffn(g, x, wid[p + "ffn_norm"], wid[p + "ffn_gate"], wid[p + "ffn_up"], wid[p + "ffn_down"], cfg.eps, p)
        if tp > 1:
            f = g.allreduce(f, p + "ffn_down_sum")
        x = g.add(x, f, p + "res2")
    x = rms_norm_w(g, x, wid["output_norm"], cfg.eps, "final_norm")
    logits = g.output(g.mul_mat(wid["output"], x, "logits"))
    token = g.output(g.cast(g.argmax(logits, "argmax"), F32, "token")) if with_argmax else -1
    extras = {}
    if taps:
        # every named intermediate stays readable after the run (the reference's `taps`, native_ir.rs:117-132)
        names = ("attn_in", "q", "k", "v", "q_rope", "k_rope", "attn", "attn_out", "res1", "ffn_in", "ffn_gate_out",
                 "ffn_up_out", "ffn_act", "ffn_down_out", "res2")
        tap = {"embd": x0, "final_norm": x}
        for t in g.nodes:
            nm = g.tensors[t].name
            if nm.startswith("blk.") and nm.split(".", 2)[2] in names:
                tap[nm] = t
        for t in tap.values():
            if t not in g.keep:
                g.keep.append(t)
        extras["taps"] = tap
    return DecoderGraph(g, specs, [pool_elems * 2] * (2 * cfg.n_layers),
                        dict(ids=0, pos=1, tables=2, lens=3, slots=4), logits, token, cfg, tp, extras)


def prefill_step(cfg: DecoderConfig, n_seqs: int, n_tokens: int, tp: int = 1, write_cache: bool = True) -> DecoderGraph:
    """Prompt pass of benchmark config 5: `n_seqs` prompts of `n_tokens` tokens each through the whole decoder with
    dense causal attention (attn:flash of stdlib/attn.ss over permuted views, the way the reference's ports
    build prefill), the new keys and values written to the paged pools, logits for the last token of every
    prompt. Inputs: token ids [n_seqs*n_tokens], positions, the f16 causal mask [n_tokens, n_tokens] shared by
    all heads and prompts, the row index of every prompt's last token, and the cache slots."""
    g = Graph()
    hd = cfg.head_dim
    heads, kvh = cfg.n_heads // tp, cfg.n_kv_heads // tp
    T = n_seqs * n_tokens
    specs = decoder_weights(cfg, tp)
    wid = {s.name: g.weight(s.ty, s.ne, s.name) for s in specs}
    pool_blocks = n_seqs * ((n_tokens + cfg.block_size - 1) // cfg.block_size)
    pool_elems = pool_blocks * kvh * cfg.block_size * hd
    pools = [(g.state(F16, [pool_elems], "k_pool.%d" % i), g.state(F16, [pool_elems], "v_pool.%d" % i))
             for i in range(cfg.n_layers)] if write_cache else []
    ids = g.input(I32, [T], "ids")
    pos = g.input(I32, [T], "pos")
    mask = g.input(F16, [n_tokens, n_tokens], "mask")
    last = g.input(I32, [n_seqs], "last")
    slots = g.input(I32, [2 * T], "slots") if write_cache else -1
    scale = 1.0 / float(np.sqrt(hd))

    x = g.get_rows(wid["token_embd"], ids, "embd")
    for i in range(cfg.n_layers):
        p = "blk.%d." % i
        h = rms_norm_w(g, x, wid[p + "attn_norm"], cfg.eps, p + "attn_in")
        q = g.mul_mat(wid[p + "wq"], h, p + "q")
        k = g.mul_mat(wid[p + "wk"], h, p + "k")
        v = g.mul_mat(wid[p + "wv"], h, p + "v")
        q = g.set_name(rope_neox(g, g.reshape(q, [hd, heads, T]), pos, hd, cfg.rope_theta), p + "q_rope")
        k = g.set_name(rope_neox(g, g.reshape(k, [hd, kvh, T]), pos, hd, cfg.rope_theta), p + "k_rope")
        k16 = g.cast(g.reshape(k, [hd * kvh, T]), F16, p + "k16")
        v16 = g.cast(v, F16, p + "v16")
        if write_cache:
            kc, vc = pools[i]
            g.paged_cache_write(k16, v16, kc, vc, slots, cfg.block_size, kvh, p + "cache_write")
        # [hd, heads, tokens, prompts] -> views [hd, tokens, heads, prompts], as ggml_flash_attn_ext wants them
        qv = g.permute(g.reshape(q, [hd, heads, n_tokens, n_seqs]), 0, 2, 1, 3)
        kv = g.permute(g.reshape(k16, [hd, kvh, n_tokens, n_seqs]), 0, 2, 1, 3)
        vv = g.permute(g.reshape(v16, [hd, kvh, n_tokens, n_seqs]), 0, 2, 1, 3)
        a = g.flash_attn_ext(qv, kv, vv, mask, scale, name=p + "attn")      # [hd, heads, tokens, prompts]
        o = g.mul_mat(wid[p + "wo"], g.reshape(a, [hd * heads, T]), p + "attn_out")
        if tp > 1:
            o = g.allreduce(o, p + "attn_out_sum")
        x = g.add(x, o, p + "res1")
        f = swiglu_ffn(g, x, wid[p + "ffn_norm"], wid[p + "ffn_gate"], wid[p + "ffn_up"], wid[p + "ffn_down"], cfg.eps, p)
        if tp > 1:
            f = g.allreduce(f, p + "ffn_down_sum")
        x = g.add(x, f, p + "res2")
    x = g.get_rows(x, last, "last_rows")
    x = rms_norm_w(g, x, wid["output_norm"], cfg.eps, "final_norm")
    logits = g.output(g.mul_mat(wid["output"], x, "logits"))
    names = dict(ids=0, pos=1, mask=2, last=3)
    if write_cache:
        names["slots"] = 4
    return DecoderGraph(g, specs, [pool_elems * 2] * (2 * len(pools)), names, logits, -1, cfg, tp)


class DecodeLoop:
    """The host side of a batched greedy decode loop over the paged pool: the loop of ports/gemma4/concurrency.ss:120-158
    (the reference's callers in crates/tensorlisp/tests/native_concurrency.rs:100-143 drive it step by step). One compiled
    decode-step program is replayed; per step the host uploads the three small arrays that advance (positions, context
    lengths, cache slots), and the token ids never leave the GPU: the ARGMAX of a step is copied into the id input of the
    next one on the device stream (`tlb_program_feed_input`). Block tables are assigned up front for `max_ctx` tokens per
    sequence, so no step has to allocate a page."""

    def __init__(self, native, cfg: DecoderConfig, batch: int, max_ctx: int, tables: np.ndarray) -> None:
        from .native import NativeProgram

        self.cfg, self.batch, self.max_ctx = cfg, batch, max_ctx
        self.tables = np.ascontiguousarray(tables, np.int32)
        max_blocks = (max_ctx + cfg.block_size - 1) // cfg.block_size
        assert self.tables.shape == (batch, max_blocks)
        pool_blocks = int(self.tables.max()) + 1
        self.dg = decoder_step(cfg, batch, max_ctx, pool_blocks)
        g = self.dg.graph
        self.argmax = [t for t in g.nodes if g.tensors[t].name == "argmax"][0]
        g.keep.append(self.argmax)   # its i32 bytes feed the next step
        self.native = native
        if not native.state_offsets:
            native.alloc_states(self.dg.state_bytes)
        self.prog = NativeProgram.compile(native, g)
        self.pos = None
        self.steps = 0

    def begin(self, first_ids: np.ndarray, cached_tokens: np.ndarray) -> None:
        """`first_ids`: the token each sequence feeds first; `cached_tokens`: how many tokens of it the pools already hold."""
        self.pos = np.ascontiguousarray(cached_tokens, np.int32).copy()
        self.prog.set_input(self.dg.inputs["ids"], np.ascontiguousarray(first_ids, np.int32))
        self.prog.set_input(self.dg.inputs["tables"], self.tables)
        self.steps = 0

    def step(self, wait: bool = True) -> None:
        """One token for every sequence; afterwards the id input already holds the tokens just chosen."""
        bs = self.cfg.block_size
        assert self.pos is not None and int(self.pos.max()) < self.max_ctx
        slots = self.tables[np.arange(self.batch), self.pos // bs].astype(np.int64) * bs + self.pos % bs
        self.prog.set_input(self.dg.inputs["pos"], self.pos)
        self.prog.set_input(self.dg.inputs["lens"], self.pos + 1)
        self.prog.set_input(self.dg.inputs["slots"], slots.view(np.int32))
        self.prog.enqueue()
        self.prog.feed_input(self.dg.inputs["ids"], self.argmax)
        if wait:
            self.native.sync()
        self.pos = self.pos + 1
        self.steps += 1

    def tokens(self) -> np.ndarray:
        """The tokens the last step chose (reads them back: waits for the step)."""
        return self.prog.read(self.argmax).reshape(self.batch).astype(np.int64)

    def logits(self) -> np.ndarray:
        return self.prog.read(self.dg.logits).reshape(self.batch, -1)

    def free(self) -> None:
        self.prog.free()
