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
