"""Seeded synthetic models of the benchmark shapes, generated and quantised on the device.

Weights are i.i.d. N(0, 0.02) (router N(0, 0.1)), norm weights 1.0; element (r, c) of tensor
`stream` is a pure function of (seed, stream, r*cols + c), so any shard can be regenerated on
any rank.  Tensor names follow GGUF (`blk.N.attn_q.weight`, ... — src/model.rs:1660-1666 and
:1844-1870 in the Camelid tree).
"""
from __future__ import annotations

from dataclasses import replace

import numpy as np

from . import shard
from .engine import F32, Q4_K, Q6_K, Q8_0, EngineConfig, ResidentDecode, Weight

SHAPES = {
    # name: (hidden, layers, heads, kv_heads, head_dim, ffn, vocab, rope_theta, experts, experts_used)
    "tiny": (256, 2, 4, 2, 64, 512, 512, 10000.0, 0, 0),
    "tiny-moe": (256, 2, 4, 2, 64, 512, 512, 10000.0, 4, 2),
    "tiny-tp": (512, 2, 8, 2, 64, 1024, 512, 10000.0, 0, 0),  # smallest shape that splits over two ranks
    "small": (4096, 2, 32, 8, 128, 8192, 2048, 500000.0, 0, 0),  # two layers at the 8B width: every matvec takes the staged kernel
    "llama-1b": (2048, 16, 32, 8, 64, 8192, 128256, 500000.0, 0, 0),
    "llama-3b": (3072, 28, 24, 8, 128, 8192, 128256, 500000.0, 0, 0),
    "llama-8b": (4096, 32, 32, 8, 128, 14336, 128256, 500000.0, 0, 0),
    "mixtral-8x7b": (4096, 32, 32, 8, 128, 14336, 32000, 1000000.0, 8, 2),
}

SLOTS = ("q", "k", "v", "o", "gate", "up", "down")
STREAM_EMBD, STREAM_OUTPUT = 1_000_000, 1_000_001


def engine_config(shape: str, max_pos: int, max_seqs: int = 1, n_layers: int | None = None, **kw) -> EngineConfig:
    hidden, layers, heads, kv, hd, ffn, vocab, theta, ne, nu = SHAPES[shape]
    return EngineConfig(n_layers=n_layers or layers, n_heads=heads, n_kv_heads=kv, head_dim=hd, hidden=hidden, ffn_dim=ffn,
                        max_pos=max_pos, vocab=vocab, rope_dim=hd, eps=1e-5, rope_theta=theta, max_seqs=max_seqs,
                        n_experts=ne, n_experts_used=nu, **kw)


def quant_plan(mix: str) -> dict:
    """Tensor role -> GGUF type.  "q8_0": everything Q8_0.  "q4_k_m": Q4_K except attn_v,
    ffn_down and output in Q6_K (the mix the benchmark configurations name)."""
    if mix == "q8_0":
        return {r: Q8_0 for r in SLOTS + ("token_embd", "output")}
    if mix == "q4_k_m":
        plan = {r: Q4_K for r in SLOTS + ("token_embd", "output")}
        plan.update(v=Q6_K, down=Q6_K, output=Q6_K)
        return plan
    if mix == "q4_k":
        return {r: Q4_K for r in SLOTS + ("token_embd", "output")}
    if mix == "q6_k":
        return {r: Q6_K for r in SLOTS + ("token_embd", "output")}
    raise ValueError(f"unknown quantisation mix {mix!r}")


def stream_of(layer: int, slot: int) -> int:
    return layer * 16 + slot


def proj_shapes(cfg: EngineConfig) -> dict:
    qw, kvw = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    return {"q": (qw, cfg.hidden), "k": (kvw, cfg.hidden), "v": (kvw, cfg.hidden), "o": (cfg.hidden, qw),
            "gate": (cfg.ffn_dim, cfg.hidden), "up": (cfg.ffn_dim, cfg.hidden), "down": (cfg.hidden, cfg.ffn_dim)}


def _synth_slice(qt: int, seed: int, stream: int, rows: int, cols: int, sigma: float, sl) -> Weight:
    """The slice ``sl`` of synthetic tensor ``stream``.  Whole-row blocks are generated directly
    (an element depends only on its global index); anything else is cut out of the full tensor."""
    if sl is None:
        return Weight.synth(qt, seed, stream, rows, cols, sigma)
    if sl.contiguous_rows and sl.col0 == 0 and sl.n_cols == cols:
        return Weight.synth(qt, seed, stream, sl.rows, cols, sigma, row0=sl.row0)
    full = Weight.synth(qt, seed, stream, rows, cols, sigma)
    part = full.shard(sl)
    full.free()
    return part


def build_engine(cfg: EngineConfig, mix: str, seed: int, tap=None, sigma: float = 0.02) -> ResidentDecode:
    """Creates an engine and fills it with the synthetic model; with ``cfg.tp_size`` or
    ``cfg.ep_size`` above 1, with this rank's shard of the very same model.  ``tap(role, layer,
    weight)``, if given, sees every device-resident tensor before the engine takes it over (used
    to copy the very same bytes into a CPU checker; unsharded engines only)."""
    plan = quant_plan(mix)
    eng = ResidentDecode(cfg)
    shapes = proj_shapes(cfg)
    ones = np.ones(cfg.hidden, np.float32)
    moe = cfg.n_experts > 0
    tp = shard.tp_slices(cfg, cfg.tp_rank, cfg.tp_size) if cfg.tp_size > 1 else {}
    ep = shard.ep_slices(cfg, cfg.ep_rank, cfg.ep_size) if cfg.ep_size > 1 else {}
    if tap and (tp or ep):
        raise ValueError("tap sees whole tensors: build the unsharded engine for that")
    for layer in range(cfg.n_layers):
        projs = {}
        for slot, name in enumerate(SLOTS):
            if moe and slot >= 4:
                continue
            rows, cols = shapes[name]
            w = _synth_slice(plan[name], seed, stream_of(layer, slot), rows, cols, sigma, tp.get(name))
            if tap:
                tap(name, layer, w)
            projs[name] = w
        eng.adopt_layer(layer, projs, ones, ones)
        if moe:
            router = Weight.synth(F32, seed, stream_of(layer, 12), cfg.n_experts, cfg.hidden, 0.1)
            exps = []
            for i, name in enumerate(("gate", "up", "down")):
                rows, cols = shapes[name]
                w = _synth_slice(plan[name] if name != "down" else Q4_K, seed, stream_of(layer, 8 + i), cfg.n_experts * rows, cols,
                                 sigma, ep.get(name + "_exps"))
                exps.append(w)
            if tap:
                tap("router", layer, router)
                for name, w in zip(("gate_exps", "up_exps", "down_exps"), exps):
                    tap(name, layer, w)
            eng.adopt_layer_moe(layer, router, *exps)
    out = _synth_slice(plan["output"], seed, STREAM_OUTPUT, cfg.vocab, cfg.hidden, sigma, tp.get("output"))
    emb = Weight.synth(plan["token_embd"], seed, STREAM_EMBD, cfg.vocab, cfg.hidden, sigma)
    if tap:
        tap("output", -1, out)
        tap("token_embd", -1, emb)
    eng.adopt_output(ones, out)
    eng.adopt_token_embd(emb)
    return eng


def weight_bytes_per_token(cfg: EngineConfig, mix: str) -> int:
    """Wire bytes of every weight one decode step reads once (the roofline numerator's weight
    term): all layer projections (top-k experts for MoE), norms, the output matrix and one
    embedding row."""
    plan = quant_plan(mix)
    bpw = {Q8_0: 34 / 32, Q4_K: 144 / 256, Q6_K: 210 / 256, F32: 4.0}
    shapes = proj_shapes(cfg)
    per_layer = 0.0
    for slot, name in enumerate(SLOTS):
        rows, cols = shapes[name]
        if cfg.n_experts > 0 and slot >= 4:
            qt = plan[name] if name != "down" else Q4_K
            per_layer += cfg.n_experts_used * rows * cols * bpw[qt]
        else:
            per_layer += rows * cols * bpw[plan[name]]
    if cfg.n_experts > 0:
        per_layer += cfg.n_experts * cfg.hidden * 4
    per_layer += 2 * cfg.hidden * 4
    total = cfg.n_layers * per_layer + cfg.vocab * cfg.hidden * bpw[plan["output"]] + cfg.hidden * 4
    total += cfg.hidden * bpw[plan["token_embd"]]
    return int(total)


def kv_bytes_per_position(cfg: EngineConfig) -> int:
    return cfg.n_layers * 2 * cfg.n_kv_heads * cfg.head_dim * 2
