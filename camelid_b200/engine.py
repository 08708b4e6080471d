"""Host-side mirror of Camelid's resident decode engine over the C ABI.

``ResidentDecode`` follows ``cuda_resident::CudaResidentDecode`` (src/cuda_resident.rs:15093
in the Camelid tree) method for method — ``new`` → constructor, ``set_layer_located`` →
``set_layer``, ``set_output``, ``forward_token``, ``forward_token_logits``,
``forward_token_hidden``, ``prefill``/``prefill_from``, ``verify_batch``, ``seed_layer``,
``read_kv_layer``, ``weights_ready``, ``filled``/``set_filled``, ``max_pos``, ``n_layers`` —
with errors raised as ``CmldError`` where the Rust returns ``Err(String)``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field, asdict

import numpy as np

from ._lib import Config, Tensor, check, lib

F32, Q8_0, Q4_K, Q6_K, Q8_0_HOST36 = 0, 8, 12, 14, 108
ACT_Q8_0, ACT_Q8_K = 1, 2
QT_NAMES = {"F32": F32, "Q8_0": Q8_0, "Q4_K": Q4_K, "Q6_K": Q6_K}
PROJ_NAMES = ("q", "k", "v", "o", "gate", "up", "down")


def device_count() -> int:
    return int(lib().cmld_device_count())


def act_row_bytes(cols: int) -> int:
    return int(lib().cmld_act_row_bytes(cols))


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class DeviceBuffer:
    """A raw device allocation made through the library (no torch involved)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(lib().cmld_malloc(C.byref(p), self.nbytes))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        check(lib().cmld_memcpy_h2d(buf.ptr, _np_ptr(a), a.nbytes))
        return buf

    def to_numpy(self, dtype, count: int | None = None) -> np.ndarray:
        dt = np.dtype(dtype)
        n = self.nbytes // dt.itemsize if count is None else count
        out = np.empty(n, dt)
        check(lib().cmld_memcpy_d2h(_np_ptr(out), self.ptr, n * dt.itemsize))
        return out

    def zero(self):
        check(lib().cmld_memset(self.ptr, 0, self.nbytes))

    def free(self):
        if getattr(self, "ptr", None):
            lib().cmld_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _tensor_of(obj) -> tuple[Tensor, object]:
    """(cmld_tensor, keep-alive) from (qtype, numpy bytes) | (qtype, Weight) | (qtype, ptr, nbytes)."""
    qt = obj[0]
    src = obj[1]
    if isinstance(src, np.ndarray):
        a = np.ascontiguousarray(src).view(np.uint8).reshape(-1)
        return Tensor(a.ctypes.data, a.nbytes, qt, 0), a
    if isinstance(src, DeviceBuffer):
        return Tensor(src.ptr, src.nbytes if len(obj) < 3 else obj[2], qt, 0), src
    return Tensor(int(src), int(obj[2]), qt, 0), None


class Weight:
    """A quantised matrix resident on the device (operator-level API)."""

    def __init__(self, handle, qt: int, rows: int, cols: int):
        self._h, self.qt, self.rows, self.cols = handle, qt, rows, cols

    @classmethod
    def from_wire(cls, qt: int, rows: int, cols: int, wire: np.ndarray) -> "Weight":
        wire = np.ascontiguousarray(wire).view(np.uint8).reshape(-1)
        h = C.c_void_p()
        check(lib().cmld_weight_create(qt, rows, cols, _np_ptr(wire), wire.nbytes, C.byref(h)))
        return cls(h.value, Q8_0 if qt == Q8_0_HOST36 else qt, rows, cols)

    @classmethod
    def synth(cls, qt: int, seed: int, stream: int, rows: int, cols: int, sigma: float, row0: int = 0) -> "Weight":
        h = C.c_void_p()
        check(lib().cmld_weight_synth(qt, seed, stream, row0, rows, cols, sigma, C.byref(h)))
        return cls(h.value, qt, rows, cols)

    def shard(self, sl) -> "Weight":
        """The part of this matrix that ``sl`` (a ``shard.Slice``) names, as a new device matrix."""
        h = C.c_void_p()
        check(lib().cmld_weight_shard(self._h, sl.block_rows, sl.first_block, sl.block_step, sl.n_blocks, sl.col0, sl.n_cols,
                                      C.byref(h)))
        return Weight(h.value, self.qt, sl.rows, sl.n_cols)

    @property
    def wire_bytes(self) -> int:
        return int(lib().cmld_weight_wire_bytes(self._h))

    def export_wire(self) -> np.ndarray:
        out = np.empty(self.wire_bytes, np.uint8)
        check(lib().cmld_weight_export_wire(self._h, _np_ptr(out)))
        return out

    def dequant(self, row0: int = 0, nrows: int | None = None) -> np.ndarray:
        nrows = self.rows - row0 if nrows is None else nrows
        buf = DeviceBuffer(nrows * self.cols * 4)
        check(lib().cmld_weight_dequant(self._h, row0, nrows, buf.ptr))
        return buf.to_numpy(np.float32).reshape(nrows, self.cols)

    def gemv(self, act: DeviceBuffer, batch: int, residual: DeviceBuffer | None = None) -> np.ndarray:
        y = DeviceBuffer(batch * self.rows * 4)
        check(lib().cmld_gemv(self._h, act.ptr, batch, y.ptr, residual.ptr if residual else None))
        return y.to_numpy(np.float32).reshape(batch, self.rows)

    def free(self):
        if getattr(self, "_h", None):
            lib().cmld_weight_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def quantize_activation(kind: int, x: np.ndarray) -> DeviceBuffer:
    """Quantise f32 rows x[batch][cols] on the device; returns the operand buffer."""
    x = np.ascontiguousarray(x, np.float32)
    batch, cols = (1, x.size) if x.ndim == 1 else x.shape
    xd = DeviceBuffer.from_numpy(x)
    act = DeviceBuffer(batch * act_row_bytes(cols))
    act.zero()
    check(lib().cmld_act_quantize(kind, xd.ptr, cols, batch, act.ptr))
    return act


def export_activation(kind: int, act: DeviceBuffer, cols: int, batch: int):
    codes = np.empty((batch, cols), np.int8)
    scales = np.empty((batch, cols // (32 if kind == ACT_Q8_0 else 256)), np.float32)
    check(lib().cmld_act_export(kind, act.ptr, cols, batch, _np_ptr(codes), _np_ptr(scales)))
    return codes, scales


@dataclass
class EngineConfig:
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    hidden: int
    ffn_dim: int
    max_pos: int
    vocab: int
    rope_dim: int = 0
    eps: float = 1e-5
    split_half_pairing: bool = False
    rope_theta: float = 10000.0
    max_seqs: int = 1
    n_experts: int = 0
    n_experts_used: int = 0
    tp_rank: int = 0
    tp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    device: int = -1
    flags: int = 0

    def to_c(self) -> Config:
        d = asdict(self)
        d["rope_dim"] = self.rope_dim or self.head_dim
        d["split_half_pairing"] = int(self.split_half_pairing)
        return Config(**d)

    def oracle_dict(self) -> dict:
        d = asdict(self)
        d["rope_dim"] = self.rope_dim or self.head_dim
        return d


class ResidentDecode:
    """CudaResidentDecode (src/cuda_resident.rs:15093) over the C ABI."""

    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        h = C.c_void_p()
        c = cfg.to_c()
        check(lib().cmld_engine_create(C.byref(c), C.byref(h)))
        self._h = h.value

    def close(self):
        if getattr(self, "_h", None):
            lib().cmld_engine_destroy(self._h)
            self._h = None

    # -- sharded engines ---------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        """Made on rank 0 and sent to the other ranks by the caller."""
        buf = (C.c_uint8 * 128)()
        check(lib().cmld_comm_unique_id(buf))
        return bytes(buf)

    def comm_init(self, unique_id: bytes, rank: int, world: int):
        """Collective over the ranks of the tensor- or expert-parallel group."""
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(lib().cmld_engine_comm_init(self._h, buf, rank, world))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- weights ---------------------------------------------------------------
    def set_layer(self, layer: int, projs: dict, attn_norm, ffn_norm):
        """set_layer_located (src/cuda_resident.rs:16133): projs maps q,k,v,o,gate,up,down to
        (qtype, wire bytes)."""
        arr = (Tensor * 7)()
        keep = []
        for i, name in enumerate(PROJ_NAMES):
            if name in projs and projs[name] is not None:
                arr[i], k = _tensor_of(projs[name])
                keep.append(k)
            else:
                arr[i] = Tensor(None, 0, 0, 0)
        an = np.ascontiguousarray(attn_norm, np.float32)
        fn = np.ascontiguousarray(ffn_norm, np.float32)
        check(lib().cmld_engine_set_layer(self._h, layer, arr, _np_ptr(an), _np_ptr(fn)))

    def set_layer_moe(self, layer: int, router, gate_exps, up_exps, down_exps):
        r = np.ascontiguousarray(router, np.float32)
        ts, keep = [], []
        for obj in (gate_exps, up_exps, down_exps):
            t, k = _tensor_of(obj)
            ts.append(t)
            keep.append(k)
        check(lib().cmld_engine_set_layer_moe(self._h, layer, _np_ptr(r), C.byref(ts[0]), C.byref(ts[1]), C.byref(ts[2])))

    def set_output(self, final_norm, output):
        fnorm = np.ascontiguousarray(final_norm, np.float32)
        t, keep = _tensor_of(output)
        check(lib().cmld_engine_set_output(self._h, _np_ptr(fnorm), C.byref(t)))

    def set_token_embd(self, token_embd):
        t, keep = _tensor_of(token_embd)
        check(lib().cmld_engine_set_token_embd(self._h, C.byref(t)))

    # -- device-resident weights (handles are consumed) ----------------------------
    def adopt_layer(self, layer: int, projs: dict, attn_norm, ffn_norm):
        arr = (C.c_void_p * 7)()
        for i, name in enumerate(PROJ_NAMES):
            w = projs.get(name)
            arr[i] = w._h if w is not None else None
        an = np.ascontiguousarray(attn_norm, np.float32)
        fn = np.ascontiguousarray(ffn_norm, np.float32)
        check(lib().cmld_engine_adopt_layer(self._h, layer, arr, _np_ptr(an), _np_ptr(fn)))
        for w in projs.values():
            if w is not None:
                w._h = None

    def adopt_layer_moe(self, layer: int, router: "Weight", gate_exps: "Weight", up_exps: "Weight", down_exps: "Weight"):
        check(lib().cmld_engine_adopt_layer_moe(self._h, layer, router._h, gate_exps._h, up_exps._h, down_exps._h))
        for w in (router, gate_exps, up_exps, down_exps):
            w._h = None

    def adopt_output(self, final_norm, output: "Weight"):
        fnorm = np.ascontiguousarray(final_norm, np.float32)
        check(lib().cmld_engine_adopt_output(self._h, _np_ptr(fnorm), output._h))
        output._h = None

    def adopt_token_embd(self, token_embd: "Weight"):
        check(lib().cmld_engine_adopt_token_embd(self._h, token_embd._h))
        token_embd._h = None

    # -- bookkeeping -----------------------------------------------------------
    def weights_ready(self) -> bool:
        return bool(lib().cmld_engine_weights_ready(self._h))

    def filled(self) -> int:
        return int(lib().cmld_engine_filled(self._h))

    def set_filled(self, n: int):
        check(lib().cmld_engine_set_filled(self._h, n))

    def max_pos(self) -> int:
        return int(lib().cmld_engine_max_pos(self._h))

    def n_layers(self) -> int:
        return int(lib().cmld_engine_n_layers(self._h))

    # -- forward_token family ----------------------------------------------------
    def _f(self, a):
        return np.ascontiguousarray(a, np.float32)

    def set_rope_frequencies(self, freq):
        """Per-pair angular frequencies of the engine-owned RoPE table (``rope_pair_frequency`` of the model:
        rope_freqs.weight and linear / llama3 scaling folded in); the table is recomputed for every position."""
        f = self._f(freq)
        check(lib().cmld_engine_set_rope_frequencies(self._h, _np_ptr(f), f.size))

    def rope_row(self, position: int):
        half = (self.cfg.rope_dim or self.cfg.head_dim) // 2
        c, s = np.empty(half, np.float32), np.empty(half, np.float32)
        check(lib().cmld_engine_rope_row(self._h, position, _np_ptr(c), _np_ptr(s)))
        return c, s

    def forward_token(self, embedding, cos, sin, position: int, scale: float, compute_logits: bool = True):
        e, c, s = self._f(embedding), self._f(cos), self._f(sin)
        tok = C.c_uint32(0)
        check(lib().cmld_engine_forward_token(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), position, scale,
                                              int(compute_logits), C.byref(tok)))
        return int(tok.value) if compute_logits else None

    def forward_token_sample(self, embedding, cos, sin, position: int, scale: float, temperature: float, seed: int, min_p: float = 0.0):
        """Forward, then a temperature draw on the device (``forward_token_sample``; with ``min_p`` the filtered draw).
        Returns the token, or (None, logits) when the filter hands the row back to the CPU."""
        e, c, s = self._f(embedding), self._f(cos), self._f(sin)
        tok = C.c_uint32(0)
        logits = np.empty(self.cfg.vocab, np.float32) if min_p > 0 else None
        check(lib().cmld_engine_forward_token_sample(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), position, scale, temperature, min_p,
                                                     seed, C.byref(tok), _np_ptr(logits) if logits is not None else None))
        if tok.value == 0xFFFFFFFF:
            return None, logits
        return int(tok.value)

    def forward_token_logits(self, embedding, cos, sin, position: int, scale: float) -> np.ndarray:
        e, c, s = self._f(embedding), self._f(cos), self._f(sin)
        out = np.empty(self.cfg.vocab, np.float32)
        check(lib().cmld_engine_forward_token_logits(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), position, scale, _np_ptr(out)))
        return out

    def forward_token_hidden(self, embedding, cos, sin, position: int, scale: float, taps: bool = False):
        e, c, s = self._f(embedding), self._f(cos), self._f(sin)
        out = np.empty(self.cfg.hidden, np.float32)
        t = np.empty((self.cfg.n_layers, self.cfg.hidden), np.float32) if taps else None
        check(lib().cmld_engine_forward_token_hidden(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), position, scale,
                                                     _np_ptr(out), _np_ptr(t) if taps else None))
        return (out, t) if taps else out

    def forward_layer(self, layer: int, hidden_in, cos, sin, position: int, scale: float) -> np.ndarray:
        h, c, s = self._f(hidden_in), self._f(cos), self._f(sin)
        out = np.empty(self.cfg.hidden, np.float32)
        check(lib().cmld_engine_forward_layer(self._h, layer, _np_ptr(h), _np_ptr(c), _np_ptr(s), position, scale, _np_ptr(out)))
        return out

    def prefill(self, embeddings, cos_all, sin_all, n: int, scale: float):
        self.prefill_from(embeddings, cos_all, sin_all, n, scale, 0)

    def prefill_from(self, embeddings, cos_all, sin_all, n: int, scale: float, start: int):
        e, c, s = self._f(embeddings), self._f(cos_all), self._f(sin_all)
        half = (self.cfg.rope_dim or self.cfg.head_dim) // 2
        if e.size < n * self.cfg.hidden or c.size < n * half or s.size < n * half:
            raise ValueError("prefill: input slices too short")
        check(lib().cmld_engine_prefill_from(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), n, scale, start))

    def verify_batch(self, embeddings, cos_all, sin_all, base_position: int, k: int, scale: float) -> np.ndarray:
        e, c, s = self._f(embeddings), self._f(cos_all), self._f(sin_all)
        out = np.empty(k, np.uint32)
        check(lib().cmld_engine_verify_batch(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), base_position, k, scale, _np_ptr(out)))
        return out

    def verify_tree(self, embeddings, cos_all, sin_all, parents, base_position: int, scale: float) -> np.ndarray:
        """Greedy token after every node of a draft tree in one batched pass (``verify_tree``).  ``parents[i]`` is the
        breadth-first index of node i's parent (-1 for the root, node 0); the nodes' K/V rows land at
        base_position + i."""
        n = len(parents)
        bits = np.zeros(n, np.uint32)
        for i, par in enumerate(parents):
            if par >= 0:
                bits[i] = bits[par] | np.uint32(1 << par)
        e, c, s = self._f(embeddings), self._f(cos_all), self._f(sin_all)
        slots = (base_position + np.arange(n)).astype(np.int32)
        out = np.empty(n, np.uint32)
        check(lib().cmld_engine_verify_tree(self._h, _np_ptr(e), _np_ptr(c), _np_ptr(s), _np_ptr(slots), _np_ptr(bits), 1,
                                            base_position, n, scale, _np_ptr(out)))
        return out

    def compact_tree_kv_path(self, path, base_position: int):
        p = np.ascontiguousarray(path, np.int32)
        check(lib().cmld_engine_compact_tree_kv_path(self._h, _np_ptr(p), p.size, base_position))

    def seed_layer(self, layer: int, ck, cv, n_positions: int):
        ck, cv = self._f(ck), self._f(cv)
        check(lib().cmld_engine_seed_layer(self._h, layer, _np_ptr(ck), _np_ptr(cv), n_positions))

    def read_kv_layer(self, layer: int, n_positions: int):
        shape = (self.cfg.n_kv_heads // max(1, self.cfg.tp_size), n_positions, self.cfg.head_dim)
        ck, cv = np.empty(shape, np.float32), np.empty(shape, np.float32)
        check(lib().cmld_engine_read_kv_layer(self._h, layer, n_positions, _np_ptr(ck), _np_ptr(cv)))
        return ck, cv

    # -- token-id driven ---------------------------------------------------------
    def prefill_tokens(self, seq: int, tokens, start_pos: int = 0) -> int:
        t = np.ascontiguousarray(tokens, np.int32)
        nxt = C.c_uint32(0)
        check(lib().cmld_engine_prefill_tokens(self._h, seq, _np_ptr(t), t.size, start_pos, C.byref(nxt)))
        return int(nxt.value)

    def decode_greedy(self, seqs, tokens_in, positions, n_steps: int) -> np.ndarray:
        s = np.ascontiguousarray(seqs, np.int32)
        t = np.ascontiguousarray(tokens_in, np.int32)
        p = np.ascontiguousarray(positions, np.int64)
        out = np.empty((n_steps, s.size), np.uint32)
        check(lib().cmld_engine_decode_greedy(self._h, s.size, _np_ptr(s), _np_ptr(t), _np_ptr(p), n_steps, _np_ptr(out)))
        return out

    def step_batch(self, seqs, tokens_in, positions, want_logits=False, want_hidden=False):
        s = np.ascontiguousarray(seqs, np.int32)
        t = np.ascontiguousarray(tokens_in, np.int32)
        p = np.ascontiguousarray(positions, np.int64)
        toks = np.empty(s.size, np.uint32)
        logits = np.empty((s.size, self.cfg.vocab), np.float32) if want_logits else None
        hidden = np.empty((s.size, self.cfg.hidden), np.float32) if want_hidden else None
        check(lib().cmld_engine_step_batch(self._h, s.size, _np_ptr(s), _np_ptr(t), _np_ptr(p), _np_ptr(toks),
                                           _np_ptr(logits) if want_logits else None,
                                           _np_ptr(hidden) if want_hidden else None))
        return toks, logits, hidden

    def last_timing(self):
        ms = C.c_float(0)
        n = C.c_int64(0)
        check(lib().cmld_engine_last_timing(self._h, C.byref(ms), C.byref(n)))
        return float(ms.value), int(n.value)
