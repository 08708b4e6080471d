"""The synthetic models as GGUF files: written from the device, read back into an engine, same bits as the engine
built directly (the file holds the very bytes the direct build quantises)."""
import numpy as np
import pytest

from helpers import has_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not has_gpu(), reason="needs a GPU")
@pytest.mark.parametrize("shape,mix", [("tiny", "q4_k_m"), ("tiny", "q8_0"), ("tiny-moe", "q4_k_m")])
def test_emitted_file_loads_to_the_same_model(cm, tmp_path, shape, mix):
    from camelid_b200 import gguf, synth

    path = tmp_path / f"{shape}-{mix}.gguf"
    infos = gguf.emit_synthetic(path, shape, mix, seed=77, max_pos=96)
    g = gguf.GgufFile(path)
    cfg = synth.engine_config(shape, max_pos=96)
    assert g.metadata["llama.block_count"] == cfg.n_layers and g.metadata["llama.embedding_length"] == cfg.hidden
    assert g.tensors["token_embd.weight"].dims == (cfg.hidden, cfg.vocab)
    assert g.tensors["blk.0.attn_q.weight"].dims == (cfg.hidden, cfg.n_heads * cfg.head_dim)
    if cfg.n_experts:
        assert g.tensors["blk.1.ffn_down_exps.weight"].dims == (cfg.ffn_dim, cfg.hidden, cfg.n_experts)
        assert g.tensors["blk.0.ffn_gate_inp.weight"].dims == (cfg.hidden, cfg.n_experts)
    assert len(infos) == len(g.tensors)
    g.close()
    direct = synth.build_engine(cfg, mix, 77)
    loaded = gguf.load_engine(path, max_pos=96)
    prompt = np.array([3, 1, 4, 1, 5, 9, 2, 6], np.int32)
    outs = []
    for eng in (direct, loaded):
        first = eng.prefill_tokens(0, prompt, 0)
        toks = eng.decode_greedy([0], [first], [len(prompt)], 12)[:, 0]
        nxt, logits, hidden = eng.step_batch([0], [int(toks[-1])], [len(prompt) + 12], want_logits=True, want_hidden=True)
        outs.append((first, toks, logits, hidden))
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1])
    assert np.array_equal(outs[0][2], outs[1][2]) and np.array_equal(outs[0][3], outs[1][3])
    direct.close()
    loaded.close()


@pytest.mark.skipif(not has_gpu(), reason="needs a GPU")
@pytest.mark.parametrize("scaling", ["llama3", "linear", "freq_factors"])
def test_scaled_rope_file_decodes_like_the_checker(cm, orc, tmp_path, scaling):
    """A file with scaled RoPE (Llama-3.1/3.2 style metadata) or a rope_freqs.weight tensor: load_engine hands the
    reference's per-pair frequencies (rope_pair_frequency, src/inference/rope.rs:532-560) to the engine-owned table,
    and the greedy tokens and logits equal the CPU checker's, which rotates by the same frequencies."""
    from camelid_b200 import gguf, synth
    from helpers import ModelPair

    cfg = synth.engine_config("tiny", max_pos=96)
    half = cfg.head_dim // 2
    extra, factors = {}, None
    if scaling == "llama3":
        extra = {"llama.rope.scaling.type": "llama3", "llama.rope.scaling.factor": 8.0, "llama.rope.scaling.original_context_length": 32,
                 "llama.rope.scaling.low_freq_factor": 1.0, "llama.rope.scaling.high_freq_factor": 4.0}
    elif scaling == "linear":
        extra = {"llama.rope.scaling.type": "linear", "llama.rope.scaling.factor": 4.0}
    else:
        factors = (1.0 + np.arange(half, dtype=np.float32) / 7.0).astype(np.float32)
    path = tmp_path / f"scaled-{scaling}.gguf"
    gguf.emit_synthetic(path, "tiny", "q4_k_m", seed=5, max_pos=96, extra_metadata=extra, rope_freqs=factors)
    g = gguf.GgufFile(path)
    freq = gguf.rope_frequencies(g.metadata, cfg.rope_dim, g.data("rope_freqs.weight").view(np.float32) if factors is not None else None)
    g.close()
    plain = gguf.rope_frequencies({"general.architecture": "llama", "llama.rope.freq_base": cfg.rope_theta}, cfg.rope_dim)
    assert not np.array_equal(freq, plain)  # the case does change the rotation
    loaded = gguf.load_engine(path, max_pos=96)
    pair = ModelPair(cfg, "q4_k_m", seed=5)  # the same tensors, built directly, with the CPU checker beside them
    pair.oracle.set_rope_frequencies(freq)
    prompt = orc.synth_tokens(5, 5, 12, cfg.vocab)
    ref_tokens, ref_logits = pair.oracle.generate(prompt, 20)
    first = loaded.prefill_tokens(0, prompt, 0)
    rest = loaded.decode_greedy([0], [first], [len(prompt)], 19)[:, 0]
    got = np.concatenate([[first], rest])
    assert np.array_equal(got, ref_tokens), (got, ref_tokens)
    c, s = loaded.rope_row(40)  # the host-side row a forward_token caller asks for follows the same frequencies
    ang = (np.float32(40) * freq).astype(np.float64)
    assert np.allclose(c, np.cos(ang), atol=1e-6) and np.allclose(s, np.sin(ang), atol=1e-6)
    loaded.close()
