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
