"""GGUF v3 files for the models this engine runs: write the seeded synthetic models, read any
llama-architecture GGUF with F32 / Q8_0 / Q4_K / Q6_K tensors into an engine.

The layout is the one Camelid's reader accepts (src/gguf/reader.rs:378-555 in the Camelid tree): magic
"GGUF", u32 version (2 or 3), i64 tensor count, i64 metadata count, the metadata pairs, the tensor
directory (name, u32 n_dims, i64 dims innermost first, i32 type id, u64 offset relative to the data
section), padding to `general.alignment` (32 when absent), then every tensor's bytes, each starting on
an alignment boundary and contiguous in directory order.  Tensor names and metadata keys are the ones
Camelid's model loader looks up (src/model.rs:320-540, :1660-1666, :1844-1870): `{arch}.block_count`,
`{arch}.embedding_length`, ..., `token_embd.weight`, `blk.N.attn_q.weight`, ..., `output.weight`, and for
Mixtral shapes `blk.N.ffn_gate_inp.weight` and the stacked `blk.N.ffn_{gate,up,down}_exps.weight`.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32
F32, F16, Q8_0, Q4_K, Q6_K = 0, 1, 8, 12, 14
# (values per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}

# metadata value type ids of the GGUF format
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<?",
           T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


def tensor_nbytes(qt: int, dims) -> int:
    """dims innermost first (ne[0] = row length)."""
    per, size = BLOCK[qt]
    n = 1
    for d in dims:
        n *= int(d)
    if dims[0] % per:
        raise ValueError(f"tensor first dimension {dims[0]} is not divisible by block size {per} (type {qt})")
    return n // per * size


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


def _pack_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(v) -> bytes:
    """(type id, payload) for the Python value: bool, int (u32 if it fits, else u64; negative i32/i64),
    float (f32), str, or a list of one of these; a tuple (type_id, value) forces the type."""
    if isinstance(v, tuple):
        t, x = v
        if t == T_STR:
            return struct.pack("<I", t) + _pack_str(x)
        if t == T_ARR:
            raise ValueError("force the element type inside the list instead")
        return struct.pack("<I", t) + struct.pack(_SCALAR[t], x)
    if isinstance(v, bool):
        return struct.pack("<I", T_BOOL) + struct.pack("<?", v)
    if isinstance(v, int):
        if v < 0:
            t = T_I32 if v >= -(1 << 31) else T_I64
        else:
            t = T_U32 if v < (1 << 32) else T_U64
        return struct.pack("<I", t) + struct.pack(_SCALAR[t], v)
    if isinstance(v, float):
        return struct.pack("<I", T_F32) + struct.pack("<f", v)
    if isinstance(v, str):
        return struct.pack("<I", T_STR) + _pack_str(v)
    if isinstance(v, (list, np.ndarray)):
        items = list(v)
        if not items:
            return struct.pack("<IIQ", T_ARR, T_I32, 0)
        first = items[0]
        if isinstance(first, str):
            body = b"".join(_pack_str(x) for x in items)
            et = T_STR
        elif isinstance(first, (float, np.floating)):
            body = np.asarray(items, "<f4").tobytes()
            et = T_F32
        else:
            body = np.asarray(items, "<i4").tobytes()
            et = T_I32
        return struct.pack("<IIQ", T_ARR, et, len(items)) + body
    raise TypeError(f"no GGUF metadata type for {type(v)}")


@dataclass
class TensorInfo:
    name: str
    qt: int
    dims: tuple  # innermost first
    offset: int  # relative to the data section
    nbytes: int


def write_gguf(path, metadata: dict, tensors, alignment: int = DEFAULT_ALIGNMENT) -> list[TensorInfo]:
    """tensors: iterable of (name, type id, dims innermost first, bytes-like or callable returning bytes).
    A callable is invoked when its turn comes, so a large model never sits in host memory at once."""
    tensors = list(tensors)
    if alignment <= 0 or alignment & (alignment - 1):
        raise ValueError("alignment must be a power of two")
    meta = dict(metadata)
    if alignment != DEFAULT_ALIGNMENT:
        meta["general.alignment"] = (T_U32, alignment)
    infos, off = [], 0
    names = set()
    for name, qt, dims, _ in tensors:
        if name in names:
            raise ValueError(f"duplicate tensor name {name}")
        if len(name.encode()) >= 64:
            raise ValueError(f"tensor name {name} is too long")
        names.add(name)
        nb = tensor_nbytes(qt, dims)
        infos.append(TensorInfo(name, qt, tuple(int(d) for d in dims), off, nb))
        off = _align(off + nb, alignment)
    head = bytearray()
    head += MAGIC + struct.pack("<Iqq", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += _pack_str(k) + _pack_value(v)
    for ti in infos:
        head += _pack_str(ti.name) + struct.pack("<I", len(ti.dims))
        for d in ti.dims:
            head += struct.pack("<q", d)
        head += struct.pack("<iQ", ti.qt, ti.offset)
    data_start = _align(len(head), alignment)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (data_start - len(head)))
        pos = 0
        for ti, (_, _, _, src) in zip(infos, tensors):
            if pos != ti.offset:
                f.write(b"\0" * (ti.offset - pos))
                pos = ti.offset
            data = src() if callable(src) else src
            data = np.ascontiguousarray(data).view(np.uint8).reshape(-1) if isinstance(data, np.ndarray) else memoryview(data)
            if len(data) != ti.nbytes:
                raise ValueError(f"tensor {ti.name}: {len(data)} bytes given, {ti.nbytes} expected")
            f.write(data)
            pos += ti.nbytes
        # the reader checks every tensor's end against the file length; no trailing padding is required
    return infos


class GgufFile:
    """Read-only view of a GGUF file: `.metadata` (dict), `.tensors` (name -> TensorInfo), `.data(name)`
    (a numpy uint8 view into the memory-mapped file)."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        mm = self._mm
        if mm[:4] != MAGIC:
            raise ValueError("bad magic; expected GGUF")
        self._pos = 4
        self.version = self._read("<I")
        if self.version not in (2, 3):
            raise ValueError(f"version {self.version}; expected v2 or v3")
        n_tensors, n_meta = self._read("<q"), self._read("<q")
        if n_tensors < 0 or n_meta < 0:
            raise ValueError("negative tensor or metadata count")
        self.metadata = {}
        for _ in range(n_meta):
            key = self._read_str()
            if key in self.metadata:
                raise ValueError(f"duplicate metadata key {key}")
            self.metadata[key] = self._read_value()
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            raise ValueError(f"invalid alignment {self.alignment}")
        raw = []
        for _ in range(n_tensors):
            name = self._read_str()
            nd = self._read("<I")
            if nd == 0 or nd > 4:
                raise ValueError(f"tensor {name} has invalid dimension count {nd}")
            dims = tuple(self._read("<q") for _ in range(nd))
            qt = self._read("<i")
            raw.append((name, qt, dims, self._read("<Q")))
        self.data_start = _align(self._pos, self.alignment)
        self.tensors = {}
        expected = 0
        for name, qt, dims, off in raw:
            if name in self.tensors:
                raise ValueError(f"duplicate tensor name {name}")
            if qt not in BLOCK:
                raise ValueError(f"tensor {name}: type {qt} is not one of F32/F16/Q8_0/Q4_K/Q6_K")
            if off != expected:
                raise ValueError(f"tensor {name} offset {off} is not contiguous; expected {expected}")
            nb = tensor_nbytes(qt, dims)
            if self.data_start + off + nb > len(mm):
                raise ValueError(f"tensor {name} data extends beyond end of file")
            self.tensors[name] = TensorInfo(name, qt, dims, off, nb)
            expected = _align(off + nb, self.alignment)

    def _read(self, fmt):
        (v,) = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += struct.calcsize(fmt)
        return v

    def _read_str(self):
        n = self._read("<Q")
        s = bytes(self._mm[self._pos:self._pos + n]).decode("utf-8")
        self._pos += n
        return s

    def _read_value(self, t=None):
        t = self._read("<I") if t is None else t
        if t in _SCALAR:
            return self._read(_SCALAR[t])
        if t == T_STR:
            return self._read_str()
        if t == T_ARR:
            et, n = self._read("<I"), self._read("<Q")
            if et in _SCALAR and et != T_BOOL:
                dt = np.dtype(_SCALAR[et])
                out = np.frombuffer(self._mm, dt, n, self._pos).copy()
                self._pos += n * dt.itemsize
                return out
            return [self._read_value(et) for _ in range(n)]
        raise ValueError(f"unknown metadata value type {t}")

    def data(self, name: str) -> np.ndarray:
        ti = self.tensors[name]
        return np.frombuffer(self._mm, np.uint8, ti.nbytes, self.data_start + ti.offset)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass  # views handed out by data() are still alive: the mapping goes when the last of them does
        self._f.close()


# ------------------------------------------------------------------ the models of this engine

def model_metadata(cfg, name: str, arch: str = "llama") -> dict:
    md = {
        "general.architecture": arch,
        "general.name": name,
        f"{arch}.block_count": cfg.n_layers,
        f"{arch}.context_length": cfg.max_pos,
        f"{arch}.embedding_length": cfg.hidden,
        f"{arch}.feed_forward_length": cfg.ffn_dim,
        f"{arch}.attention.head_count": cfg.n_heads,
        f"{arch}.attention.head_count_kv": cfg.n_kv_heads,
        f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.eps),
        f"{arch}.rope.dimension_count": cfg.rope_dim or cfg.head_dim,
        f"{arch}.rope.freq_base": float(cfg.rope_theta),
        f"{arch}.vocab_size": cfg.vocab,
        f"{arch}.attention.key_length": cfg.head_dim,
        f"{arch}.attention.value_length": cfg.head_dim,
    }
    if cfg.n_experts > 0:
        md[f"{arch}.expert_count"] = cfg.n_experts
        md[f"{arch}.expert_used_count"] = cfg.n_experts_used
    return md


_PROJ_NAMES = {"q": "attn_q", "k": "attn_k", "v": "attn_v", "o": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}


def emit_synthetic(path, shape: str, mix: str, seed: int, max_pos: int = 8192, n_layers: int | None = None, sigma: float = 0.02,
                   extra_metadata: dict | None = None, rope_freqs=None):
    """Writes the seeded synthetic model (the very tensors `synth.build_engine` generates) as a GGUF file.
    Tensors are generated and quantised on the current CUDA device one at a time and streamed to the file."""
    from . import synth
    from .engine import F32 as E_F32, Q4_K as E_Q4_K, Weight

    cfg = synth.engine_config(shape, max_pos=max_pos, n_layers=n_layers)
    plan = synth.quant_plan(mix)
    shapes = synth.proj_shapes(cfg)
    ones = np.ones(cfg.hidden, np.float32)

    def gen(qt, stream, rows, cols, s=sigma):
        def make():
            w = Weight.synth(qt, seed, stream, rows, cols, s)
            try:
                return w.export_wire()
            finally:
                w.free()
        return make

    tensors = [("token_embd.weight", plan["token_embd"], (cfg.hidden, cfg.vocab), gen(plan["token_embd"], synth.STREAM_EMBD, cfg.vocab, cfg.hidden))]
    moe = cfg.n_experts > 0
    for layer in range(cfg.n_layers):
        tensors.append((f"blk.{layer}.attn_norm.weight", F32, (cfg.hidden,), ones))
        for slot, name in enumerate(synth.SLOTS):
            if moe and slot >= 4:
                continue
            rows, cols = shapes[name]
            tensors.append((f"blk.{layer}.{_PROJ_NAMES[name]}.weight", plan[name], (cols, rows), gen(plan[name], synth.stream_of(layer, slot), rows, cols)))
        tensors.append((f"blk.{layer}.ffn_norm.weight", F32, (cfg.hidden,), ones))
        if moe:
            tensors.append((f"blk.{layer}.ffn_gate_inp.weight", F32, (cfg.hidden, cfg.n_experts),
                            gen(E_F32, synth.stream_of(layer, 12), cfg.n_experts, cfg.hidden, 0.1)))
            for i, name in enumerate(("gate", "up", "down")):
                rows, cols = shapes[name]
                qt = plan[name] if name != "down" else E_Q4_K
                tensors.append((f"blk.{layer}.ffn_{name}_exps.weight", qt, (cols, rows, cfg.n_experts),
                                gen(qt, synth.stream_of(layer, 8 + i), cfg.n_experts * rows, cols)))
    tensors.append(("output_norm.weight", F32, (cfg.hidden,), ones))
    tensors.append(("output.weight", plan["output"], (cfg.hidden, cfg.vocab), gen(plan["output"], synth.STREAM_OUTPUT, cfg.vocab, cfg.hidden)))
    md = model_metadata(cfg, f"synthetic-{shape}-{mix}-seed{seed}")
    md["general.file_type"] = 7 if mix == "q8_0" else 15  # LLAMA_FTYPE_MOSTLY_Q8_0 / MOSTLY_Q4_K_M
    if rope_freqs is not None:  # llama.cpp's freq_factors: one divisor per rotated pair
        rf = np.ascontiguousarray(rope_freqs, np.float32)
        tensors.append(("rope_freqs.weight", F32, (rf.size,), lambda: rf.view(np.uint8)))
    md.update(extra_metadata or {})
    return write_gguf(path, md, tensors)


def engine_config_from(g: GgufFile, max_pos: int | None = None, **kw):
    from .engine import EngineConfig

    md = g.metadata
    arch = md["general.architecture"]
    heads = int(md[f"{arch}.attention.head_count"])
    hidden = int(md[f"{arch}.embedding_length"])
    head_dim = int(md.get(f"{arch}.attention.key_length", hidden // heads))
    emb = g.tensors["token_embd.weight"]
    return EngineConfig(
        n_layers=int(md[f"{arch}.block_count"]), n_heads=heads, n_kv_heads=int(md.get(f"{arch}.attention.head_count_kv", heads)),
        head_dim=head_dim, hidden=hidden, ffn_dim=int(md[f"{arch}.feed_forward_length"]),
        max_pos=int(max_pos or md[f"{arch}.context_length"]), vocab=int(md.get(f"{arch}.vocab_size", emb.dims[1])),
        rope_dim=int(md.get(f"{arch}.rope.dimension_count", head_dim)), eps=float(md.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)),
        rope_theta=float(md.get(f"{arch}.rope.freq_base", 10000.0)), n_experts=int(md.get(f"{arch}.expert_count", 0)),
        n_experts_used=int(md.get(f"{arch}.expert_used_count", 0)), **kw)


def _powf(base: float, exponent: float) -> np.float32:
    """f32 power by the C library, which is what the reference's ``f32::powf`` and the engine's own table call
    (numpy's float32 power differs from it in the last bit for some exponents)."""
    import ctypes
    import ctypes.util

    global _LIBM
    if _LIBM is None:
        _LIBM = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
        _LIBM.powf.restype = ctypes.c_float
        _LIBM.powf.argtypes = [ctypes.c_float, ctypes.c_float]
    return np.float32(_LIBM.powf(float(base), float(exponent)))


_LIBM = None


def rope_frequencies(md: dict, rope_dim: int, rope_freqs=None) -> np.ndarray:
    """Per-pair RoPE frequency of a model file, in f32 like ``rope_pair_frequency`` (src/inference/rope.rs:532-560
    in the Camelid tree): freq_base^(-2i/rope_dim), divided by ``rope_freqs.weight[i]`` when the file carries that
    tensor, then the metadata's scaling: none, "linear" (divide by the factor) or "llama3" (wavelength-dependent
    blend, :733-757).  Any other scaling type (YaRN also rescales the rotation's magnitude) raises."""
    arch = md["general.architecture"]
    f32 = np.float32
    half = rope_dim // 2
    base = f32(md.get(f"{arch}.rope.freq_base", 10000.0))
    kind = md.get(f"{arch}.rope.scaling.type")
    kind = None if kind in (None, "", "none") else str(kind)
    if kind not in (None, "linear", "llama3"):
        raise ValueError(f"rope scaling type {kind!r} is not supported by the engine-owned RoPE table")
    factor = f32(md.get(f"{arch}.rope.scaling.factor", 1.0))
    out = np.empty(half, f32)
    for i in range(half):
        freq = _powf(base, f32(-(f32(i) * f32(2.0)) / f32(rope_dim)))
        if rope_freqs is not None:
            freq = f32(freq / f32(rope_freqs[i]))
        if kind == "linear":
            freq = f32(freq / factor)
        elif kind == "llama3":
            ctx = f32(md[f"{arch}.rope.scaling.original_context_length"])
            lo, hi = f32(md[f"{arch}.rope.scaling.low_freq_factor"]), f32(md[f"{arch}.rope.scaling.high_freq_factor"])
            wavelength = f32(f32(f32(2.0) * f32(np.pi)) / freq)
            if wavelength < f32(ctx / hi):
                pass
            elif wavelength > f32(ctx / lo):
                freq = f32(freq / factor)
            else:
                smooth = f32(f32(f32(ctx / wavelength) - lo) / f32(hi - lo))
                freq = f32(f32(f32(f32(f32(1.0) - smooth) * freq) / factor) + f32(smooth * freq))
        out[i] = freq
    return out


def load_engine(path, max_pos: int | None = None, **kw):
    """An engine filled from a GGUF file (unsharded).  Tensors go from the memory-mapped file straight into
    `set_layer` / `set_output` / `set_token_embd`; `output.weight` falls back to `token_embd.weight` when the
    file ties them."""
    from .engine import ResidentDecode

    g = GgufFile(path)
    try:
        cfg = engine_config_from(g, max_pos, **kw)
        eng = ResidentDecode(cfg)
        f32 = lambda name: g.data(name).view(np.float32)  # noqa: E731
        for layer in range(cfg.n_layers):
            projs = {}
            for short, long in _PROJ_NAMES.items():
                name = f"blk.{layer}.{long}.weight"
                if name in g.tensors:
                    projs[short] = (g.tensors[name].qt, g.data(name))
            eng.set_layer(layer, projs, f32(f"blk.{layer}.attn_norm.weight"), f32(f"blk.{layer}.ffn_norm.weight"))
            if cfg.n_experts > 0:
                exps = [(g.tensors[f"blk.{layer}.ffn_{n}_exps.weight"].qt, g.data(f"blk.{layer}.ffn_{n}_exps.weight")) for n in ("gate", "up", "down")]
                eng.set_layer_moe(layer, f32(f"blk.{layer}.ffn_gate_inp.weight"), *exps)
        out_name = "output.weight" if "output.weight" in g.tensors else "token_embd.weight"
        eng.set_output(f32("output_norm.weight"), (g.tensors[out_name].qt, g.data(out_name)))
        eng.set_token_embd((g.tensors["token_embd.weight"].qt, g.data("token_embd.weight")))
        # the engine-owned RoPE table: rope_freqs.weight and the metadata's scaling, as the reference applies them
        arch = g.metadata["general.architecture"]
        scaled = g.metadata.get(f"{arch}.rope.scaling.type") not in (None, "", "none")
        if "rope_freqs.weight" in g.tensors or scaled:
            factors = f32("rope_freqs.weight") if "rope_freqs.weight" in g.tensors else None
            if factors is not None and factors.size != cfg.rope_dim // 2:
                raise ValueError(f"rope_freqs.weight holds {factors.size} values, {cfg.rope_dim // 2} pairs are rotated")
            eng.set_rope_frequencies(rope_frequencies(g.metadata, cfg.rope_dim, factors))
        return eng
    finally:
        g.close()
