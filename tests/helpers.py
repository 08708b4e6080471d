"""Shared test plumbing: the same synthetic model in the CPU checker and in the engine."""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc


def has_gpu() -> bool:
    try:
        import camelid_b200 as cm

        return cm.device_count() > 0
    except Exception:
        return False


def close_enough(got, ref, rel=1e-4, floor=1e-5):
    """|got-ref| <= rel*|ref| + floor*max|ref| elementwise (the reference's GPU tests use
    close(.., 1e-4), src/cuda_resident/tests.rs:7805-7825)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    tol = rel * np.abs(ref) + floor * (np.abs(ref).max() + 1e-30)
    bad = np.abs(got - ref) > tol
    return not bad.any(), float(np.abs(got - ref).max()), int(bad.sum())


def hidden_gate(got, ref):
    """The acceptance gate per layer: max-abs 2e-2 and relative 1e-2 (relative to the row's RMS)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    max_abs = float(np.abs(got - ref).max())
    rel = float(np.abs(got - ref).max() / (np.sqrt((ref ** 2).mean()) + 1e-30))
    return max_abs <= 2e-2 and rel <= 1e-2, max_abs, rel


class ModelPair:
    """An engine and a CPU checker holding byte-identical weights."""

    def __init__(self, cfg, mix: str, seed: int, via: str = "device"):
        import camelid_b200 as cm
        from camelid_b200 import synth

        self.cfg, self.mix, self.seed = cfg, mix, seed
        self.oracle = orc.OracleModel(cfg.oracle_dict())
        o = self.oracle
        layer_projs: dict[int, dict] = {}
        moe: dict[int, dict] = {}

        def tap(role, layer, w):
            wire = w.export_wire()
            if role in synth.SLOTS:
                layer_projs.setdefault(layer, {})[role] = (w.qt, wire)
            elif role == "output":
                o.set_output(np.ones(cfg.hidden, np.float32), w.qt, wire)
            elif role == "token_embd":
                o.set_token_embd(w.qt, wire)
            else:
                moe.setdefault(layer, {})[role] = (w.qt, wire)

        if via == "device":
            self.engine = synth.build_engine(cfg, mix, seed, tap=tap)
        else:  # generate on the CPU checker, upload wire bytes through set_layer
            self.engine = cm.ResidentDecode(cfg)
            plan = synth.quant_plan(mix)
            shapes = synth.proj_shapes(cfg)
            ones = np.ones(cfg.hidden, np.float32)
            for layer in range(cfg.n_layers):
                projs = {}
                for slot, name in enumerate(synth.SLOTS):
                    rows, cols = shapes[name]
                    projs[name] = (plan[name], orc.synth_tensor(plan[name], seed, synth.stream_of(layer, slot), rows, cols, 0.02))
                layer_projs[layer] = projs
                self.engine.set_layer(layer, projs, ones, ones)
            out = orc.synth_tensor(plan["output"], seed, synth.STREAM_OUTPUT, cfg.vocab, cfg.hidden, 0.02)
            emb = orc.synth_tensor(plan["token_embd"], seed, synth.STREAM_EMBD, cfg.vocab, cfg.hidden, 0.02)
            self.engine.set_output(ones, (plan["output"], out))
            self.engine.set_token_embd((plan["token_embd"], emb))
            o.set_output(ones, plan["output"], out)
            o.set_token_embd(plan["token_embd"], emb)
        ones = np.ones(cfg.hidden, np.float32)
        for layer in range(cfg.n_layers):
            projs = layer_projs.get(layer, {})
            if cfg.n_experts > 0:
                zero = np.zeros(4, np.uint8)  # dense FFN slots unused by a MoE layer
                for name in ("gate", "up", "down"):
                    projs.setdefault(name, (8, zero))
            o.set_layer(layer, projs, ones, ones)
            if layer in moe:
                m = moe[layer]
                o.set_moe(layer, m["router"][1].view(np.float32), m["gate_exps"], m["up_exps"], m["down_exps"])

    def rope(self, position: int):
        c = self.cfg
        return orc.rope_table(position, c.rope_dim or c.head_dim, c.rope_theta)

    @property
    def scale(self) -> float:
        return float(np.float32(1.0) / np.sqrt(np.float32(self.cfg.head_dim)))


def greedy_match(got, ref_tokens, gaps):
    """(number of leading equal tokens, the checker's top-2 logit gap where they first differ)."""
    got, ref_tokens = np.asarray(got), np.asarray(ref_tokens)
    diff = np.nonzero(got != ref_tokens)[0]
    if diff.size == 0:
        return len(ref_tokens), None
    return int(diff[0]), float(gaps[diff[0]])
