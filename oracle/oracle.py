"""ctypes front end of the CPU checker (``camelid_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libcamelid_oracle.so"

Q8_0, Q4_K, Q6_K, F32 = 8, 12, 14, 0
QT_NAMES = {"Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K, "F32": F32}


def build(march: str | None = None, out: str | None = None) -> Path:
    """Compile the checker with gcc (``make -C oracle``); returns the .so path."""
    args = ["make", "-s", "-C", str(_HERE)]
    target = Path(out) if out else _LIB_PATH
    if march:
        args.append(f"ORACLE_MARCH={march}")
    if out:
        args += [f"OUT={out}", "-B"]
    subprocess.run(args, check=True)
    return target


_lib = None


def lib(path: str | os.PathLike | None = None):
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else _LIB_PATH
    if not p.exists():
        build()
    L = C.CDLL(str(p))
    vp, i32, i64, u64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float
    sig = {
        "orc_f32_to_f16_bits": (C.c_uint16, [f32]),
        "orc_f16_bits_to_f32": (f32, [C.c_uint16]),
        "orc_kv_f32_to_f16_bits": (C.c_uint16, [f32]),
        "orc_kv_round_row": (None, [vp, vp, i64]),
        "orc_row_bytes": (i64, [C.c_int, i64]),
        "orc_dequant": (C.c_int, [C.c_int, vp, i64, vp]),
        "orc_quantize": (C.c_int, [C.c_int, vp, i64, vp]),
        "orc_synth_normal": (None, [u64, u64, i64, i64, f32, vp]),
        "orc_synth_tokens": (None, [u64, u64, i64, i32, vp]),
        "orc_synth_tensor": (C.c_int, [C.c_int, u64, u64, i64, i64, i64, f32, vp]),
        "orc_quantize_act_q8_0": (None, [vp, i64, vp, vp]),
        "orc_quantize_act_q8_k": (None, [vp, i64, vp, vp]),
        "orc_matvec": (C.c_int, [C.c_int, vp, i64, i64, vp, vp]),
        "orc_matvec_quantised": (C.c_int, [C.c_int, vp, i64, i64, vp, vp, vp]),
        "orc_matvec_dequant_f32": (C.c_int, [C.c_int, vp, i64, i64, vp, vp]),
        "orc_rms_norm": (None, [vp, vp, i64, f32, vp]),
        "orc_rope_table": (None, [i64, i32, f32, vp, vp]),
        "orc_rope_apply": (None, [vp, i32, i32, i32, vp, vp, i32]),
        "orc_attention_head": (C.c_int, [vp, vp, vp, i64, i64, i32, f32, vp, vp]),
        "orc_silu_mul": (None, [vp, vp, i64, vp]),
        "orc_argmax": (i32, [vp, i64]),
        "orc_softmax_top_k": (C.c_int, [vp, i32, i32, vp, vp]),
        "orc_model_create": (vp, [i32] * 9 + [f32, f32, i32, i32, i32]),
        "orc_model_destroy": (None, [vp]),
        "orc_model_set_proj": (C.c_int, [vp, i32, i32, i32, vp]),
        "orc_model_set_norms": (C.c_int, [vp, i32, vp, vp]),
        "orc_model_set_moe": (C.c_int, [vp, i32, vp, i32, vp, i32, vp, i32, vp]),
        "orc_model_set_output": (None, [vp, vp, i32, vp]),
        "orc_model_set_token_embd": (None, [vp, i32, vp]),
        "orc_embedding": (C.c_int, [vp, i32, vp]),
        "orc_model_read_kv": (C.c_int, [vp, i32, i64, vp, vp]),
        "orc_model_write_kv": (C.c_int, [vp, i32, i64, vp, vp]),
        "orc_sample_uniform": (f32, [C.c_uint64, C.c_uint32]),
        "orc_sample_uniform_clamped_count": (i32, []),
        "orc_min_p_candidate": (i32, [f32, f32, f32, i32]),
        "orc_sample_gumbel": (i32, [vp, i32, f32, C.c_uint64, vp]),
        "orc_sample_gumbel_filtered": (i32, [vp, i32, f32, f32, C.c_uint64, vp]),
        "orc_model_set_rope_frequencies": (C.c_int, [vp, vp, i32]),
        "orc_model_set_kv_q8": (C.c_int, [vp, i32]),
        "orc_kv_q8_0_quantize_block": (f32, [vp, vp]),
        "orc_attention_head_q8": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i32, f32, vp, vp]),
        "orc_rope_llama3_frequency": (f32, [f32, f32, f32, f32, f32]),
        "orc_forward": (C.c_int, [vp, vp, i64, vp, vp, vp]),
        "orc_generate": (C.c_int, [vp, vp, i32, i32, i64, vp, vp]),
        "orc_generate_gaps": (C.c_int, [vp, vp, i32, i32, i64, vp, vp, vp]),
        "orc_expf_twin": (f32, [f32]),
        "orc_expf_twin_mismatches": (i64, [f32, f32, i64]),
        "orc_num_threads": (C.c_int, []),
        "orc_set_num_threads": (None, [C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = L
    return L


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def row_bytes(qt: int, cols: int) -> int:
    return int(lib().orc_row_bytes(qt, cols))


def dequant(qt: int, wire: np.ndarray, n: int) -> np.ndarray:
    wire = np.ascontiguousarray(wire, dtype=np.uint8)
    out = np.empty(n, np.float32)
    assert lib().orc_dequant(qt, _p(wire), n, _p(out)) == 0
    return out


def quantize(qt: int, x) -> np.ndarray:
    x = _f32(x).ravel()
    blk = 32 if qt == Q8_0 else 256
    assert x.size % blk == 0
    out = np.empty(row_bytes(qt, x.size), np.uint8)
    assert lib().orc_quantize(qt, _p(x), x.size, _p(out)) == 0
    return out


def synth_normal(seed: int, stream: int, start: int, n: int, sigma: float) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_synth_normal(seed, stream, start, n, sigma, _p(out))
    return out


def synth_tokens(seed: int, stream: int, n: int, vocab: int) -> np.ndarray:
    out = np.empty(n, np.int32)
    lib().orc_synth_tokens(seed, stream, n, vocab, _p(out))
    return out


def synth_tensor(qt: int, seed: int, stream: int, rows: int, cols: int, sigma: float, row0: int = 0) -> np.ndarray:
    out = np.empty(rows * row_bytes(qt, cols), np.uint8)
    assert lib().orc_synth_tensor(qt, seed, stream, row0, rows, cols, sigma, _p(out)) == 0
    return out


def quantize_act_q8_0(x):
    x = _f32(x)
    qs = np.empty(x.size, np.int8)
    sc = np.empty(x.size // 32, np.float32)
    lib().orc_quantize_act_q8_0(_p(x), x.size, _p(qs), _p(sc))
    return qs, sc


def quantize_act_q8_k(x):
    x = _f32(x)
    qs = np.empty(x.size, np.int8)
    d = np.empty(x.size // 256, np.float32)
    lib().orc_quantize_act_q8_k(_p(x), x.size, _p(qs), _p(d))
    return qs, d


def matvec(qt: int, w: np.ndarray, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x)
    y = np.empty(rows, np.float32)
    assert lib().orc_matvec(qt, _p(w), rows, cols, _p(x), _p(y)) == 0
    return y


def matvec_quantised(qt: int, w: np.ndarray, rows: int, cols: int, xq: np.ndarray, xs: np.ndarray) -> np.ndarray:
    y = np.empty(rows, np.float32)
    assert lib().orc_matvec_quantised(qt, _p(w), rows, cols, _p(xq), _p(xs), _p(y)) == 0
    return y


def matvec_dequant_f32(qt: int, w: np.ndarray, rows: int, cols: int, x) -> np.ndarray:
    x = _f32(x)
    y = np.empty(rows, np.float32)
    assert lib().orc_matvec_dequant_f32(qt, _p(w), rows, cols, _p(x), _p(y)) == 0
    return y


def rms_norm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(w), x.size, eps, _p(out))
    return out


def rope_table(position: int, rope_dim: int, base: float):
    c = np.empty(rope_dim // 2, np.float32)
    s = np.empty(rope_dim // 2, np.float32)
    lib().orc_rope_table(position, rope_dim, base, _p(c), _p(s))
    return c, s


def rope_apply(x, heads: int, head_dim: int, rope_dim: int, cosv, sinv, split_half: bool = False) -> np.ndarray:
    x = _f32(x).copy()
    cosv, sinv = _f32(cosv), _f32(sinv)
    lib().orc_rope_apply(_p(x), heads, head_dim, rope_dim, _p(cosv), _p(sinv), int(split_half))
    return x


def attention_head(q, k, v, n_pos: int, head_dim: int, scale: float, stride: int | None = None) -> np.ndarray:
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(head_dim, np.float32)
    scores = np.empty(n_pos, np.float32)
    rc = lib().orc_attention_head(_p(q), _p(k), _p(v), stride or head_dim, n_pos, head_dim, scale, _p(out), _p(scores))
    assert rc == 0
    return out


def silu_mul(g, u) -> np.ndarray:
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


def argmax(x) -> int:
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), x.size))


def sample_gumbel(logits, inv_temp: float, seed: int):
    """Index and per-token scores of the temperature draw (sample_gumbel)."""
    x = _f32(logits)
    scores = np.empty(x.size, np.float32)
    return int(lib().orc_sample_gumbel(_p(x), x.size, inv_temp, seed, _p(scores))), scores


def sample_gumbel_filtered(logits, temperature: float, min_p: float, seed: int):
    """Index (-1 = hand the row to the CPU sampler) and scores (-inf where filtered) of the min-p draw."""
    x = _f32(logits)
    scores = np.empty(x.size, np.float32)
    return int(lib().orc_sample_gumbel_filtered(_p(x), x.size, temperature, min_p, seed, _p(scores))), scores


def softmax_top_k(logits, k: int):
    logits = _f32(logits)
    idx = np.empty(max(k, 1), np.int32)
    w = np.empty(max(k, 1), np.float32)
    n = lib().orc_softmax_top_k(_p(logits), logits.size, k, _p(idx), _p(w))
    return [(int(idx[i]), float(w[i])) for i in range(n)]


class OracleModel:
    """A Llama/Mixtral-shaped model held as GGUF wire bytes, stepped on the CPU."""

    SLOTS = ("q", "k", "v", "o", "gate", "up", "down")

    def __init__(self, cfg: dict):
        self.cfg = dict(cfg)
        c = self.cfg
        self._keep = []
        self._h = lib().orc_model_create(
            c["n_layers"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["hidden"], c["ffn_dim"],
            c.get("rope_dim", c["head_dim"]), c["max_pos"], c["vocab"], c.get("eps", 1e-5),
            c.get("rope_theta", 10000.0), int(c.get("split_half_pairing", False)),
            c.get("n_experts", 0), c.get("n_experts_used", 0))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_model_destroy(self._h)
            self._h = None

    def _hold(self, a, dtype):
        a = np.ascontiguousarray(a, dtype=dtype)
        self._keep.append(a)
        return a

    def set_layer(self, layer: int, projs: dict, attn_norm, ffn_norm):
        for slot, name in enumerate(self.SLOTS):
            if name in projs:
                qt, data = projs[name]
                assert lib().orc_model_set_proj(self._h, layer, slot, qt, _p(self._hold(data, np.uint8))) == 0
        lib().orc_model_set_norms(self._h, layer, _p(self._hold(attn_norm, np.float32)),
                                  _p(self._hold(ffn_norm, np.float32)))

    def set_moe(self, layer: int, router, gate, up, down):
        lib().orc_model_set_moe(self._h, layer, _p(self._hold(router, np.float32)),
                                gate[0], _p(self._hold(gate[1], np.uint8)), up[0], _p(self._hold(up[1], np.uint8)),
                                down[0], _p(self._hold(down[1], np.uint8)))

    def set_output(self, final_norm, qt: int, data):
        lib().orc_model_set_output(self._h, _p(self._hold(final_norm, np.float32)), qt, _p(self._hold(data, np.uint8)))

    def set_token_embd(self, qt: int, data):
        lib().orc_model_set_token_embd(self._h, qt, _p(self._hold(data, np.uint8)))

    def embedding(self, token: int) -> np.ndarray:
        out = np.empty(self.cfg["hidden"], np.float32)
        assert lib().orc_embedding(self._h, token, _p(out)) == 0
        return out

    def read_kv_layer(self, layer: int, n_positions: int):
        shape = (self.cfg["n_kv_heads"], n_positions, self.cfg["head_dim"])
        ck, cv = np.empty(shape, np.float32), np.empty(shape, np.float32)
        assert lib().orc_model_read_kv(self._h, layer, n_positions, _p(ck), _p(cv)) == 0
        return ck, cv

    def set_kv_q8(self, on: bool = True):
        """Keeps the KV cache as Q8_0 blocks (src/tensor/kv_quant.rs) from the next forward on."""
        assert lib().orc_model_set_kv_q8(self._h, int(on)) == 0

    def set_rope_frequencies(self, freq):
        f = _f32(freq)
        assert lib().orc_model_set_rope_frequencies(self._h, _p(f), f.size) == 0

    def write_kv_layer(self, layer: int, ck, cv):
        """Plants positions 0..n-1 of one layer's cache ([kv_head][n][head_dim] each), rounded to f16."""
        ck, cv = _f32(ck), _f32(cv)
        assert ck.shape == cv.shape and ck.shape[0] == self.cfg["n_kv_heads"] and ck.shape[2] == self.cfg["head_dim"]
        assert lib().orc_model_write_kv(self._h, layer, ck.shape[1], _p(ck), _p(cv)) == 0

    def forward(self, x, position: int, want_logits=True, want_taps=False):
        x = _f32(x)
        c = self.cfg
        logits = np.empty(c["vocab"], np.float32) if want_logits else None
        hidden = np.empty(c["hidden"], np.float32)
        taps = np.empty((c["n_layers"], c["hidden"]), np.float32) if want_taps else None
        rc = lib().orc_forward(self._h, _p(x), position, _p(logits) if want_logits else None, _p(hidden),
                               _p(taps) if want_taps else None)
        assert rc == 0, f"oracle forward failed rc={rc}"
        return logits, hidden, taps

    def generate(self, prompt, n_gen: int, start_pos: int = 0, want_gaps: bool = False):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(n_gen, np.int32)
        logits = np.empty(self.cfg["vocab"], np.float32)
        gaps = np.empty(n_gen, np.float32)
        rc = lib().orc_generate_gaps(self._h, _p(prompt), prompt.size, n_gen, start_pos, _p(out), _p(logits), _p(gaps))
        assert rc == 0
        return (out, logits, gaps) if want_gaps else (out, logits)
