"""Parity at the benchmark's model shapes (B200, through the C ABI).

Config 1 runs in full: Llama-3.2-1B-shaped, all Q8_0, 32-token prompt, 128 greedy tokens, against
the CPU checker holding byte-identical weights.  The larger configs are run at their true widths
(hidden, heads, ffn, vocab) but with fewer layers so the CPU checker finishes in seconds; the
arithmetic of a layer does not depend on how many follow it.

The reference quantises every matvec operand to int8, so a value 1e-6 away (one f32 reassociation)
from a rounding boundary gets the neighbouring code and the layer output jumps by more than the
acceptance gate allows; the only way to meet the gates (per-layer hidden states and logits within
max-abs 2e-2 / relative 1e-2, at least 32 equal greedy tokens) on every input is to keep the CPU
path's order of f32 operations.  The engine does, in its default mode — the mode the benchmark
times — so the bar here is zero difference: the residual stream after every layer, the logits and
every greedy token are BIT-IDENTICAL to the checker's.  CMLD_FLAG_EXACT_ORDER selects the plain
(one lane per sum) kernels, which must give the same bits again.
"""
import numpy as np
import pytest

from helpers import ModelPair, greedy_match, hidden_gate

pytestmark = pytest.mark.gpu

EXACT = 16  # CMLD_FLAG_EXACT_ORDER


def _greedy(pair, orc, prompt, n_gen, seq=0):
    eng, ref = pair.engine, pair.oracle
    ref_tokens, _, gaps = ref.generate(prompt, n_gen, want_gaps=True)
    first = eng.prefill_tokens(seq, prompt, 0)
    rest = eng.decode_greedy([seq], [first], [len(prompt)], n_gen - 1)[:, 0]
    got = np.concatenate([[first], rest])
    return greedy_match(got, ref_tokens, gaps)


def _bit_identity(pair, orc, prompt, n_positions):
    """Whole forward passes (no teacher forcing): residual stream after every layer, and logits.
    Returns the counts of positions with identical taps / logits and the acceptance gate's verdict."""
    eng, ref, cfg = pair.engine, pair.oracle, pair.cfg
    equal_taps = equal_logits = total = gate_ok = 0
    worst = 0.0
    for pos in range(n_positions):
        emb = ref.embedding(int(prompt[pos]))
        c, s = pair.rope(pos)
        ref_logits, _, ref_taps = ref.forward(emb, pos, want_taps=True)
        _, taps = eng.forward_token_hidden(emb, c, s, pos, pair.scale, taps=True)
        logits = eng.forward_token_logits(emb, c, s, pos, pair.scale)
        equal_taps += int(np.array_equal(taps.view(np.uint32), ref_taps.view(np.uint32)))
        equal_logits += int(np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32)))
        gate_ok += int(all(hidden_gate(taps[l], ref_taps[l])[0] for l in range(cfg.n_layers)) and hidden_gate(logits, ref_logits)[0])
        worst = max(worst, float(np.abs(taps - ref_taps).max()), float(np.abs(logits - ref_logits).max()))
        total += 1
    return equal_taps, equal_logits, total, worst, gate_ok


@pytest.mark.parametrize("flags", [0, EXACT])
def test_config1_llama_1b_q8_0_is_bit_identical(cm, orc, flags):
    """Config 1 in full: the residual stream after each of the 16 layers, the logits and all 128 greedy
    tokens equal the CPU checker's bit for bit (default engine; and the plain reference-order kernels)."""
    from camelid_b200 import synth

    cfg = synth.engine_config("llama-1b", max_pos=512, flags=flags)
    pair = ModelPair(cfg, "q8_0", seed=20261125)
    prompt = orc.synth_tokens(20261125, 5, 32, cfg.vocab)
    eq_t, eq_l, total, worst, gate = _bit_identity(pair, orc, prompt, 6)
    print(f"config 1 flags={flags}: taps bit-identical at {eq_t}/{total} positions, logits at {eq_l}/{total}, worst abs diff {worst:.2e}")
    assert gate == total and eq_t == total and eq_l == total, (eq_t, eq_l, total, worst)
    n_match, gap = _greedy(pair, orc, prompt, 128)
    print(f"config 1 flags={flags}: {n_match}/128 greedy tokens equal")
    assert n_match == 128, (n_match, gap)


@pytest.mark.parametrize("shape,layers,flags", [("llama-3b", 6, 0), ("llama-8b", 8, 0), ("llama-3b", 3, EXACT), ("llama-8b", 2, EXACT)])
def test_k_quant_mix_is_bit_identical(cm, orc, shape, layers, flags):
    """Configs 3 and 4 (Q4_K_M mix) at their true widths: 100 % of (position, layer) pairs and the logits
    inside the acceptance gate — with zero difference — and every greedy token equal."""
    from camelid_b200 import synth

    cfg = synth.engine_config(shape, max_pos=256, n_layers=layers, flags=flags)
    pair = ModelPair(cfg, "q4_k_m", seed=20261125)
    prompt = orc.synth_tokens(20261125, 5, 24, cfg.vocab)
    eq_t, eq_l, total, worst, gate = _bit_identity(pair, orc, prompt, 5)
    print(f"{shape} x{layers} flags={flags}: taps bit-identical at {eq_t}/{total} positions, logits {eq_l}/{total}, worst {worst:.2e}")
    assert gate == total and eq_t == total and eq_l == total, (eq_t, eq_l, total, worst)
    n_match, gap = _greedy(pair, orc, prompt, 40)
    assert n_match == 40, (n_match, gap)


def test_llama_8b_long_context_stays_bit_identical(cm, orc):
    """The attention and its exact softmax sum over a context past 1024 positions (the benchmark's prompt
    length): KV seeded by a prompt the engine ingests itself, then greedy tokens against the checker."""
    from camelid_b200 import synth

    cfg = synth.engine_config("llama-8b", max_pos=1280, n_layers=2)
    pair = ModelPair(cfg, "q4_k_m", seed=7)
    prompt = orc.synth_tokens(7, 5, 1100, cfg.vocab)
    n_match, gap = _greedy(pair, orc, prompt, 34)
    assert n_match == 34, (n_match, gap)


def test_mixtral_shape_two_layers(cm, orc):
    """Config 5's shape (8 experts, top-2, ffn 14336, vocab 32000), two layers: the expert matvecs multiply
    the f32 activation with dequantised weights in index order, like the reference; bit identity again."""
    from camelid_b200 import synth

    cfg = synth.engine_config("mixtral-8x7b", max_pos=128, n_layers=2, max_seqs=2)
    pair = ModelPair(cfg, "q4_k_m", seed=20261125)
    prompt = orc.synth_tokens(20261125, 5, 6, cfg.vocab)
    eq_t, eq_l, total, worst, gate = _bit_identity(pair, orc, prompt, 3)
    print(f"mixtral x2: taps bit-identical at {eq_t}/{total} positions, logits {eq_l}/{total}, worst {worst:.2e}")
    assert gate == total and eq_t == total and eq_l == total, (eq_t, eq_l, total, worst)
    n_match, gap = _greedy(pair, orc, prompt, 34, seq=1)
    print(f"mixtral x2 layers: {n_match}/34 greedy tokens equal (gap {gap})")
    assert n_match == 34, (n_match, gap)
