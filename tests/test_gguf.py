"""GGUF writer / reader (CPU): the byte layout Camelid's reader checks (src/gguf/reader.rs:378-555) and a
round trip of metadata and tensor bytes."""
import struct

import numpy as np
import pytest

from camelid_b200 import gguf


def _tensors(rng):
    specs = [("token_embd.weight", gguf.Q8_0, (64, 10)), ("blk.0.attn_norm.weight", gguf.F32, (64,)),
             ("blk.0.attn_q.weight", gguf.Q4_K, (256, 3)), ("blk.0.attn_v.weight", gguf.Q6_K, (256, 5)),
             ("blk.0.ffn_gate_exps.weight", gguf.Q4_K, (256, 2, 4))]
    return [(n, t, d, rng.integers(0, 256, gguf.tensor_nbytes(t, d), dtype=np.uint8)) for n, t, d in specs]


def test_sizes_follow_the_block_layouts():
    assert gguf.tensor_nbytes(gguf.Q8_0, (64, 10)) == 64 // 32 * 34 * 10
    assert gguf.tensor_nbytes(gguf.Q4_K, (4096, 14336)) == 4096 // 256 * 144 * 14336
    assert gguf.tensor_nbytes(gguf.Q6_K, (256, 2, 3)) == 210 * 6
    assert gguf.tensor_nbytes(gguf.F32, (7,)) == 28
    with pytest.raises(ValueError):
        gguf.tensor_nbytes(gguf.Q4_K, (128, 2))


def test_round_trip_and_layout(tmp_path):
    rng = np.random.default_rng(3)
    tensors = _tensors(rng)
    md = {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 500000.0,
          "llama.attention.layer_norm_rms_epsilon": 1e-5, "some.flag": True, "some.negative": -7,
          "big.count": 1 << 40, "tokenizer.ggml.tokens": ["a", "bc", ""], "tokenizer.ggml.scores": [0.5, -1.0],
          "tokenizer.ggml.token_type": [1, 2, 3]}
    path = tmp_path / "m.gguf"
    infos = gguf.write_gguf(path, md, tensors)
    raw = path.read_bytes()
    # header as the reference parses it
    assert raw[:4] == b"GGUF"
    version, n_t, n_kv = struct.unpack_from("<Iqq", raw, 4)
    assert (version, n_t, n_kv) == (3, len(tensors), len(md))
    g = gguf.GgufFile(path)
    assert g.data_start % 32 == 0 and g.alignment == 32
    # directory: offsets relative to the data section, aligned and contiguous in order
    expected = 0
    for ti, (name, qt, dims, data) in zip(infos, tensors):
        assert ti.offset == expected and ti.offset % 32 == 0
        got = g.tensors[name]
        assert (got.qt, got.dims, got.offset, got.nbytes) == (qt, tuple(dims), ti.offset, len(data))
        assert np.array_equal(g.data(name), data)
        expected = (ti.offset + ti.nbytes + 31) // 32 * 32
    assert len(raw) == g.data_start + infos[-1].offset + infos[-1].nbytes
    # metadata
    assert g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 1
    assert g.metadata["some.flag"] is True and g.metadata["some.negative"] == -7 and g.metadata["big.count"] == 1 << 40
    assert g.metadata["tokenizer.ggml.tokens"] == ["a", "bc", ""]
    assert np.allclose(g.metadata["tokenizer.ggml.scores"], [0.5, -1.0]) and list(g.metadata["tokenizer.ggml.token_type"]) == [1, 2, 3]
    assert abs(g.metadata["llama.rope.freq_base"] - 500000.0) < 1e-3
    g.close()


def test_other_alignment_is_recorded_and_used(tmp_path):
    rng = np.random.default_rng(4)
    path = tmp_path / "a.gguf"
    gguf.write_gguf(path, {"general.architecture": "llama"}, _tensors(rng), alignment=128)
    g = gguf.GgufFile(path)
    assert g.alignment == 128 and g.data_start % 128 == 0
    assert all(t.offset % 128 == 0 for t in g.tensors.values())
    g.close()


def test_reader_rejects_what_the_reference_rejects(tmp_path):
    rng = np.random.default_rng(5)
    path = tmp_path / "m.gguf"
    gguf.write_gguf(path, {"general.architecture": "llama"}, _tensors(rng))
    raw = bytearray(path.read_bytes())
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + raw[4:])
    with pytest.raises(ValueError, match="magic"):
        gguf.GgufFile(bad)
    bad.write_bytes(raw[:4] + struct.pack("<I", 4) + raw[8:])
    with pytest.raises(ValueError, match="version"):
        gguf.GgufFile(bad)
    bad.write_bytes(raw[:-10])  # last tensor cut short
    with pytest.raises(ValueError, match="beyond end of file"):
        gguf.GgufFile(bad)
    with pytest.raises(ValueError, match="duplicate"):
        gguf.write_gguf(bad, {}, [("x", gguf.F32, (4,), np.zeros(16, np.uint8))] * 2)
    with pytest.raises(ValueError, match="bytes given"):
        gguf.write_gguf(bad, {}, [("x", gguf.F32, (4,), np.zeros(15, np.uint8))])


def test_model_metadata_keys_are_the_loader_keys():
    from camelid_b200 import synth

    md = gguf.model_metadata(synth.engine_config("mixtral-8x7b", max_pos=4096), "m")
    for key in ("general.architecture", "llama.block_count", "llama.context_length", "llama.embedding_length",
                "llama.feed_forward_length", "llama.attention.head_count", "llama.attention.head_count_kv",
                "llama.attention.layer_norm_rms_epsilon", "llama.rope.dimension_count", "llama.rope.freq_base",
                "llama.expert_count", "llama.expert_used_count", "llama.vocab_size"):
        assert key in md, key
    assert md["llama.expert_count"] == 8 and md["llama.expert_used_count"] == 2 and md["llama.attention.head_count_kv"] == 8


def test_rope_frequencies_follow_the_reference_function():
    """gguf.rope_frequencies restates rope_pair_frequency (src/inference/rope.rs:532-560): the plain form has the C
    library's powf bits, the llama3 form equals the checker's C restatement of llama3_scaled_rope_frequency
    (:733-757), linear scaling and rope_freqs.weight divide, and an unknown scaling type is refused."""
    import ctypes
    import ctypes.util

    from camelid_b200 import gguf
    from oracle import oracle as orc

    libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
    libm.powf.restype, libm.powf.argtypes = ctypes.c_float, [ctypes.c_float, ctypes.c_float]
    md = {"general.architecture": "llama", "llama.rope.freq_base": 500000.0}
    plain = gguf.rope_frequencies(md, 128)
    want = np.array([libm.powf(500000.0, np.float32(-(np.float32(i) * np.float32(2.0)) / np.float32(128))) for i in range(64)], np.float32)
    assert np.array_equal(plain.view(np.uint32), want.view(np.uint32))
    l3 = dict(md, **{"llama.rope.scaling.type": "llama3", "llama.rope.scaling.factor": 32.0, "llama.rope.scaling.original_context_length": 8192,
                     "llama.rope.scaling.low_freq_factor": 1.0, "llama.rope.scaling.high_freq_factor": 4.0})
    got = gguf.rope_frequencies(l3, 128)
    ref = np.array([orc.lib().orc_rope_llama3_frequency(float(f), 32.0, 8192.0, 1.0, 4.0) for f in plain], np.float32)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    assert got[0] == plain[0] and got[-1] == np.float32(plain[-1] / np.float32(32.0)) and np.any((got != plain) & (got != plain / np.float32(32.0)))
    lin = gguf.rope_frequencies(dict(md, **{"llama.rope.scaling.type": "linear", "llama.rope.scaling.factor": 4.0}), 128)
    assert np.array_equal(lin, (plain / np.float32(4.0)).astype(np.float32))
    fac = (1.0 + np.arange(64, dtype=np.float32)).astype(np.float32)
    assert np.array_equal(gguf.rope_frequencies(md, 128, fac), (plain / fac).astype(np.float32))
    with pytest.raises(ValueError):
        gguf.rope_frequencies(dict(md, **{"llama.rope.scaling.type": "yarn"}), 128)


# ---- files built the way the reference's own tests build them (tests/tensor_store.rs:1062-1090 in the Camelid
# tree: magic, u32 version 3, i64 tensor count, i64 metadata count, one string KV, the tensor record with i64
# dims, i32 type and u64 offset, zero padding to 32 bytes, payload) — written here field by field, not through
# gguf.write_gguf, so the reader is pinned to the reference's byte recipe and not only to this package's writer.

def _ref_style_file(path, name, type_id, dims, payload, extra_kv=()):
    def s(v):
        raw = v.encode()
        return struct.pack("<Q", len(raw)) + raw

    b = bytearray(b"GGUF")
    b += struct.pack("<I", 3)
    b += struct.pack("<q", 1)
    b += struct.pack("<q", 1 + len(extra_kv))
    b += s("general.architecture") + struct.pack("<i", 8) + s("llama")
    for key, type_code, packed in extra_kv:
        b += s(key) + struct.pack("<i", type_code) + packed
    b += s(name) + struct.pack("<I", len(dims))
    for d in dims:
        b += struct.pack("<q", d)
    b += struct.pack("<i", type_id) + struct.pack("<Q", 0)
    while len(b) % 32:
        b.append(0)
    b += payload
    path.write_bytes(bytes(b))


def test_reader_takes_the_reference_test_files(tmp_path):
    # loads_f32_tensor_payload (tests/tensor_store.rs:15-31)
    p = tmp_path / "f32.gguf"
    _ref_style_file(p, "test.weight", 0, [2], struct.pack("<ff", 1.0, 2.5))
    g = gguf.GgufFile(p)
    assert g.version == 3 and g.alignment == 32 and g.metadata == {"general.architecture": "llama"}
    t = g.tensors["test.weight"]
    assert t.dims == (2,) and t.qt == gguf.F32 and t.offset == 0 and g.data_start % 32 == 0
    assert g.data("test.weight").view(np.float32).tolist() == [1.0, 2.5]
    g.close()
    # loads_q8_0_tensor_payload_as_f32 (:68-85): scale 1.0 (f16 0x3c00), codes 0..31 -> values 0..31
    from oracle import oracle as orc

    p = tmp_path / "q8.gguf"
    payload = struct.pack("<H", 0x3C00) + bytes(range(32))
    _ref_style_file(p, "test.weight", 8, [32], payload)
    g = gguf.GgufFile(p)
    t = g.tensors["test.weight"]
    assert t.qt == gguf.Q8_0 and t.dims == (32,) and t.nbytes == 34
    vals = orc.dequant(8, g.data("test.weight"), 32)
    assert vals[0] == 0.0 and vals[31] == 31.0 and np.array_equal(vals, np.arange(32, dtype=np.float32))
    g.close()
    # K-quant superblocks and a 2-D tensor with its dims in GGUF order (innermost first)
    rng = np.random.default_rng(11)
    for type_id, block in ((12, 144), (14, 210)):
        p = tmp_path / f"k{type_id}.gguf"
        payload = rng.integers(0, 256, 3 * 2 * block, dtype=np.uint8).tobytes()
        _ref_style_file(p, "blk.0.attn_q.weight", type_id, [512, 3], payload)
        g = gguf.GgufFile(p)
        t = g.tensors["blk.0.attn_q.weight"]
        assert t.dims == (512, 3) and t.qt == type_id and t.nbytes == len(payload)
        assert g.data("blk.0.attn_q.weight").tobytes() == payload
        g.close()
    # a second KV of another type before the tensor table: u32 value (type 4)
    p = tmp_path / "kv.gguf"
    key_val = struct.pack("<I", 16)
    _ref_style_file(p, "test.weight", 0, [2], struct.pack("<ff", 3.0, 4.0), extra_kv=[("llama.block_count", 4, key_val)])
    g = gguf.GgufFile(p)
    assert g.metadata["llama.block_count"] == 16 and g.data("test.weight").view(np.float32).tolist() == [3.0, 4.0]
    g.close()


def test_reader_refuses_a_q8_0_tensor_that_is_not_block_aligned(tmp_path):
    # rejects_q8_0_tensor_with_non_block_aligned_first_dimension (tests/tensor_store.rs:1023-1032)
    p = tmp_path / "bad-q8.gguf"
    _ref_style_file(p, "test.weight", 8, [31], b"")
    with pytest.raises(ValueError) as ei:
        gguf.GgufFile(p)
    assert "first dimension 31" in str(ei.value) and "block size 32" in str(ei.value)


def test_engine_config_reads_the_llama_keys_of_the_reference_loader(tmp_path):
    """The metadata keys ModelConfig::from_gguf reads for a llama-architecture file (src/model.rs:320-540):
    block_count, context_length, embedding_length, feed_forward_length, attention.head_count(_kv),
    attention.layer_norm_rms_epsilon, rope.dimension_count, rope.freq_base, expert_count, expert_used_count,
    vocab_size, attention.key_length — engine_config_from picks each of them up, and falls back the same way
    (kv heads = heads, head_dim = embedding/heads, vocab from token_embd's second dim)."""
    md = {"general.architecture": "llama", "llama.block_count": 3, "llama.context_length": 4096, "llama.embedding_length": 256,
          "llama.feed_forward_length": 768, "llama.attention.head_count": 8, "llama.attention.head_count_kv": 2,
          "llama.attention.layer_norm_rms_epsilon": 1e-6, "llama.rope.dimension_count": 32, "llama.rope.freq_base": 500000.0,
          "llama.expert_count": 4, "llama.expert_used_count": 2}
    emb = np.zeros(gguf.tensor_nbytes(gguf.F32, (256, 1000)), np.uint8)
    path = tmp_path / "cfg.gguf"
    gguf.write_gguf(path, md, [("token_embd.weight", gguf.F32, (256, 1000), emb)])
    g = gguf.GgufFile(path)
    c = gguf.engine_config_from(g)
    g.close()
    assert (c.n_layers, c.max_pos, c.hidden, c.ffn_dim, c.n_heads, c.n_kv_heads) == (3, 4096, 256, 768, 8, 2)
    assert c.head_dim == 32 and c.rope_dim == 32 and c.vocab == 1000 and c.n_experts == 4 and c.n_experts_used == 2
    assert abs(c.eps - 1e-6) < 1e-12 and c.rope_theta == 500000.0
    for drop in ("llama.attention.head_count_kv", "llama.rope.dimension_count", "llama.expert_count", "llama.expert_used_count"):
        md.pop(drop)
    gguf.write_gguf(path, md, [("token_embd.weight", gguf.F32, (256, 1000), emb)])
    g = gguf.GgufFile(path)
    c = gguf.engine_config_from(g, max_pos=128)
    g.close()
    assert c.n_kv_heads == 8 and c.rope_dim == 32 and c.n_experts == 0 and c.max_pos == 128
