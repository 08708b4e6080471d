"""Engine-level parity on a B200 through the C ABI: whole decode steps against the CPU
checker holding byte-identical weights.

The engine keeps every f32 operation in the CPU path's order, so for dense models the bar is
bit identity: residual stream after every layer, logits, KV rows and every greedy token equal the
checker's.  (Acceptance gates, for reference: per-layer hidden states and logits within max-abs
2e-2 and relative 1e-2; greedy token ids equal for at least the first 32 generated tokens.)
"""
import numpy as np
import pytest

from helpers import ModelPair, greedy_match, hidden_gate

pytestmark = pytest.mark.gpu


class Lcg:
    """The reference tests' generator (src/cuda_resident/tests.rs:3700-3717)."""

    def __init__(self, seed):
        self.s = seed

    def f32(self, n):
        out = np.empty(n, np.float32)
        for i in range(n):
            self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            out[i] = np.float32(np.float32(self.s >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
        return out


# full_forward_token_matches_cpu (src/cuda_resident/tests.rs:2962-3134): the reference's own
# tiny Llama (2 layers, hidden 64, 2 heads / 1 kv head, head_dim 32, ffn 128, vocab 96), Q8_0
# weights from its LCG, norm weights 1 +- 0.2, four positions fed as embeddings; token ids
# must be equal.
def test_reference_tiny_model_token_identity(cm, orc):
    L, hidden, heads, kv, hd, ffn, vocab, max_pos = 2, 64, 2, 1, 32, 128, 96, 16
    rng = Lcg(0xABCDEF)
    cfg = cm.EngineConfig(n_layers=L, n_heads=heads, n_kv_heads=kv, head_dim=hd, hidden=hidden, ffn_dim=ffn, max_pos=max_pos,
                          vocab=vocab, rope_dim=hd, eps=1e-5, rope_theta=10000.0)
    eng = cm.ResidentDecode(cfg)
    ref = orc.OracleModel(cfg.oracle_dict())
    shapes = {"q": (heads * hd, hidden), "k": (kv * hd, hidden), "v": (kv * hd, hidden), "o": (hidden, heads * hd),
              "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    for layer in range(L):
        projs = {n: (8, orc.quantize(8, rng.f32(r * c))) for n, (r, c) in shapes.items()}
        an = rng.f32(hidden) * np.float32(0.2) + np.float32(1.0)
        fn = rng.f32(hidden) * np.float32(0.2) + np.float32(1.0)
        eng.set_layer(layer, projs, an, fn)
        ref.set_layer(layer, projs, an, fn)
    fnorm = rng.f32(hidden) * np.float32(0.2) + np.float32(1.0)
    out_w = orc.quantize(8, rng.f32(vocab * hidden))
    eng.set_output(fnorm, (8, out_w))
    ref.set_output(fnorm, 8, out_w)
    assert eng.weights_ready() and eng.n_layers() == L and eng.max_pos() == max_pos
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    for position in range(4):
        emb = rng.f32(hidden)
        c, s = orc.rope_table(position, hd, 10000.0)
        logits, _, _ = ref.forward(emb, position)
        tok = eng.forward_token(emb, c, s, position, scale, True)
        assert tok == orc.argmax(logits), position
        eng.set_filled(position + 1)
    assert eng.filled() == 4


@pytest.fixture(scope="module", params=["q8_0", "q4_k_m"])
def pair(request, cm):
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny", max_pos=160, max_seqs=4)
    return ModelPair(cfg, request.param, seed=20261125)


def test_per_layer_hidden_logits_and_kv_are_bit_identical(pair, orc):
    eng, ref, cfg = pair.engine, pair.oracle, pair.cfg
    toks = orc.synth_tokens(1, 1, 12, cfg.vocab)
    for pos, t in enumerate(toks):
        emb = ref.embedding(int(t))
        c, s = pair.rope(pos)
        ref_logits, ref_hidden, ref_taps = ref.forward(emb, pos, want_taps=True)
        hidden, taps = eng.forward_token_hidden(emb, c, s, pos, pair.scale, taps=True)
        for layer in range(cfg.n_layers):
            assert np.array_equal(taps[layer].view(np.uint32), ref_taps[layer].view(np.uint32)), (pos, layer, hidden_gate(taps[layer], ref_taps[layer]))
        assert np.array_equal(hidden.view(np.uint32), ref_hidden.view(np.uint32))
        logits = eng.forward_token_logits(emb, c, s, pos, pair.scale)
        assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32)), (pos, hidden_gate(logits, ref_logits))
    for layer in range(cfg.n_layers):
        ck, cv = eng.read_kv_layer(layer, len(toks))
        rk, rv = ref.read_kv_layer(layer, len(toks))
        assert np.array_equal(ck, rk) and np.array_equal(cv, rv), layer


def test_greedy_tokens_match_checker(pair, orc):
    eng, ref, cfg = pair.engine, pair.oracle, pair.cfg
    n_gen = 48
    runs = []
    for prompt_seed in (2, 3, 4, 5):
        prompt = orc.synth_tokens(prompt_seed, 1, 9, cfg.vocab)
        ref_tokens, _, gaps = ref.generate(prompt, n_gen, want_gaps=True)
        first = eng.prefill_tokens(0, prompt, 0)
        out = eng.decode_greedy([0], [first], [len(prompt)], n_gen - 1)
        got = np.concatenate([[first], out[:, 0]])
        runs.append(greedy_match(got, ref_tokens, gaps))
    assert all(n == n_gen for n, _ in runs), runs  # every token of every prompt
    ms, launches = eng.last_timing()
    assert ms > 0 and launches > 0


def test_batched_rows_equal_serial_bitwise(pair, orc):
    """phase7_independent_paged_batch*_matches_*_serial_forwards and
    verify_batch_matches_sequential (src/cuda_resident/tests.rs:6267, :3947)."""
    eng, cfg = pair.engine, pair.cfg
    prompts = [orc.synth_tokens(3, s, 6 + s, cfg.vocab) for s in range(4)]
    firsts = [eng.prefill_tokens(s, prompts[s], 0) for s in range(4)]
    # serial: each sequence alone
    serial_logits = []
    for s in range(4):
        _, lg, _ = eng.step_batch([s], [firsts[s]], [len(prompts[s])], want_logits=True)
        serial_logits.append(lg[0])
    # batched: the same four rows in one step (KV rows are rewritten with identical values)
    toks, lg, _ = eng.step_batch([0, 1, 2, 3], firsts, [len(p) for p in prompts], want_logits=True)
    for s in range(4):
        assert np.array_equal(lg[s], serial_logits[s]), s
        assert toks[s] == int(np.argmax(serial_logits[s]))
    # verify_batch: k consecutive positions of one sequence in one pass == k serial forward_token calls
    ref = pair.oracle
    embs = np.stack([ref.embedding(int(t)) for t in prompts[0][:5]])
    cs = [pair.rope(p) for p in range(5)]
    cos_all, sin_all = np.stack([c for c, _ in cs]), np.stack([s for _, s in cs])
    serial = [eng.forward_token(embs[p], cos_all[p], sin_all[p], p, pair.scale, True) for p in range(5)]
    k0, v0 = eng.read_kv_layer(1, 5)
    batch = eng.verify_batch(embs, cos_all, sin_all, 0, 5, pair.scale)
    k1, v1 = eng.read_kv_layer(1, 5)
    assert list(batch) == serial
    assert np.array_equal(k0, k1) and np.array_equal(v0, v1)
    # prefill (embedding form) leaves the same KV as serial calls
    eng.prefill(embs, cos_all, sin_all, 5, pair.scale)
    k2, v2 = eng.read_kv_layer(1, 5)
    assert np.array_equal(k0, k2) and np.array_equal(v0, v2)


def test_seed_layer_round_trip_and_continue(pair, orc):
    eng, cfg = pair.engine, pair.cfg
    prompt = orc.synth_tokens(4, 1, 10, cfg.vocab)
    first = eng.prefill_tokens(0, prompt, 0)
    saved = [eng.read_kv_layer(l, len(prompt)) for l in range(cfg.n_layers)]
    cont = eng.decode_greedy([0], [first], [len(prompt)], 4)[:, 0]
    eng.prefill_tokens(0, orc.synth_tokens(5, 1, 10, cfg.vocab), 0)  # overwrite the cache
    for l, (ck, cv) in enumerate(saved):
        eng.seed_layer(l, ck, cv, len(prompt))
    again = eng.decode_greedy([0], [first], [len(prompt)], 4)[:, 0]
    assert np.array_equal(cont, again)


def test_error_paths_do_not_touch_the_device(pair, cm):
    eng, cfg = pair.engine, pair.cfg
    with pytest.raises(cm.CmldError) as ei:
        eng.decode_greedy([0], [0], [cfg.max_pos - 1], 5)
    assert ei.value.code == 7
    with pytest.raises(cm.CmldError):
        eng.step_batch([9], [0], [0])
    with pytest.raises(cm.CmldError):
        eng.step_batch([0], [cfg.vocab], [0])
    with pytest.raises(cm.CmldError):
        eng.set_layer(0, {"q": (8, np.zeros(10, np.uint8))}, np.ones(cfg.hidden), np.ones(cfg.hidden))
    with pytest.raises(cm.CmldError) as ei:
        eng.set_layer(0, {n: (2, np.zeros(18, np.uint8)) for n in ("q", "k", "v", "o", "gate", "up", "down")},
                      np.ones(cfg.hidden), np.ones(cfg.hidden))
    assert ei.value.code == 3  # Q4_0 is outside the path


def test_generic_and_staged_matvec_paths_agree(cm, orc):
    """The engine built with CMLD_FLAG_DIRECT_GEMV (separate quantise kernels + the generic matvec),
    the default engine (staged matvec with fused prologues), the engine with separate preparation
    kernels and no graphs, and the plain reference-order engine (CMLD_FLAG_EXACT_ORDER) all keep the
    CPU path's order of operations: identical logits."""
    from camelid_b200 import synth

    for shape, mix in (("tiny", "q8_0"), ("tiny", "q4_k_m"), ("small", "q4_k_m")):
        cfg = synth.engine_config(shape, max_pos=64)
        a = ModelPair(cfg, mix, seed=9)
        b = ModelPair(synth.engine_config(shape, max_pos=64, flags=2), mix, seed=9)
        c = ModelPair(synth.engine_config(shape, max_pos=64, flags=8 | 1 | 4), mix, seed=9)  # separate prep kernels, no graph, no PDL
        d = ModelPair(synth.engine_config(shape, max_pos=64, flags=16), mix, seed=9)
        prompt = orc.synth_tokens(8, 1, 8, cfg.vocab)
        fa, fb, fc, fd = (m.engine.prefill_tokens(0, prompt, 0) for m in (a, b, c, d))
        _, la, _ = a.engine.step_batch([0], [fa], [8], want_logits=True)
        _, lb, _ = b.engine.step_batch([0], [fb], [8], want_logits=True)
        _, lc, _ = c.engine.step_batch([0], [fc], [8], want_logits=True)
        _, ld, _ = d.engine.step_batch([0], [fd], [8], want_logits=True)
        assert fa == fb == fc == fd
        assert np.array_equal(la, lb) and np.array_equal(la, lc) and np.array_equal(la, ld)
        _, launches_a = a.engine.last_timing()
        _, launches_c = c.engine.last_timing()
        if shape == "small":  # wide enough for the staged kernel, whose fused prologues (the default) save kernels
            assert launches_a < launches_c
        for m in (a, b, c, d):
            m.engine.close()


def test_wire_upload_path_equals_device_generated(cm, orc):
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny", max_pos=64)
    a = ModelPair(cfg, "q4_k_m", seed=5, via="device")
    b = ModelPair(cfg, "q4_k_m", seed=5, via="wire")
    prompt = orc.synth_tokens(6, 1, 8, cfg.vocab)
    fa, fb = a.engine.prefill_tokens(0, prompt, 0), b.engine.prefill_tokens(0, prompt, 0)
    _, la, _ = a.engine.step_batch([0], [fa], [8], want_logits=True)
    _, lb, _ = b.engine.step_batch([0], [fb], [8], want_logits=True)
    assert fa == fb and np.array_equal(la, lb)


def test_mixtral_shaped_moe_parity(cm, orc):
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny-moe", max_pos=96, max_seqs=2)
    pair = ModelPair(cfg, "q4_k_m", seed=31)
    eng, ref = pair.engine, pair.oracle
    prompt = orc.synth_tokens(7, 1, 6, cfg.vocab)
    for pos, t in enumerate(prompt):
        emb = ref.embedding(int(t))
        c, s = pair.rope(pos)
        ref_logits, ref_hidden, ref_taps = ref.forward(emb, pos, want_taps=True)
        hidden, taps = eng.forward_token_hidden(emb, c, s, pos, pair.scale, taps=True)
        for layer in range(cfg.n_layers):
            assert np.array_equal(taps[layer].view(np.uint32), ref_taps[layer].view(np.uint32)), (pos, layer, hidden_gate(taps[layer], ref_taps[layer]))
        logits = eng.forward_token_logits(emb, c, s, pos, pair.scale)
        assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32)), hidden_gate(logits, ref_logits)
    ref_tokens, _, gaps = ref.generate(prompt, 40, want_gaps=True)
    first = eng.prefill_tokens(1, prompt, 0)
    got = np.concatenate([[first], eng.decode_greedy([1], [first], [len(prompt)], 39)[:, 0]])
    n_match, gap = greedy_match(got, ref_tokens, gaps)
    assert n_match == 40, (n_match, gap)


def test_tensor_batch_flag_moves_small_batches_to_the_tensor_core_kernel(cm, orc):
    """CMLD_FLAG_TENSOR_BATCH (64): steps of 5..32 rows use the int8 mma.sync matvec.  Same integers, f32 terms
    added in another order: logits within the acceptance gate of the default engine's, and the rows of such a
    step do not depend on their neighbours."""
    from camelid_b200 import synth
    from helpers import hidden_gate

    cfg = synth.engine_config("tiny", max_pos=64, max_seqs=6)
    base = synth.build_engine(cfg, "q4_k_m", 5)
    fast = synth.build_engine(synth.engine_config("tiny", max_pos=64, max_seqs=6, flags=64), "q4_k_m", 5)
    toks = [3, 7, 11, 19, 23, 29]
    seqs = list(range(6))
    _, l0, h0 = base.step_batch(seqs, toks, [0] * 6, want_logits=True, want_hidden=True)
    _, l1, h1 = fast.step_batch(seqs, toks, [0] * 6, want_logits=True, want_hidden=True)
    ok, max_abs, rel = hidden_gate(l1, l0)
    assert ok, (max_abs, rel)
    _, l2, _ = fast.step_batch(seqs[::-1], toks[::-1], [0] * 6, want_logits=True)
    assert np.array_equal(l2[::-1], l1)
    base.close()
    fast.close()


# Continuous batching (ContinuousBatch::run_round, src/api/continuous_batch.rs:86-104): a round is N
# independent serial token steps, so the oracle for a 16- or 32-row step is N single-sequence runs of
# the checker.  "small" is wide enough (hidden 4096) for every matvec to take the staged kernel.
@pytest.mark.parametrize("shape,mix,rows", [("small", "q4_k_m", 16), ("small", "q4_k_m", 32), ("small", "q8_0", 32),
                                             ("tiny-moe", "q4_k_m", 16), ("tiny-moe", "q4_k_m", 32)])
def test_steps_of_16_and_32_rows_equal_independent_sequences(cm, orc, shape, mix, rows):
    from camelid_b200 import synth

    cfg = synth.engine_config(shape, max_pos=48, max_seqs=rows)
    pair = ModelPair(cfg, mix, seed=77)
    eng, ref = pair.engine, pair.oracle
    prompts = [orc.synth_tokens(50 + s, 1, 3 + s % 5, cfg.vocab) for s in range(rows)]
    firsts = [eng.prefill_tokens(s, prompts[s], 0) for s in range(rows)]
    # the checker, one sequence at a time: prompt, then the logits of the step that follows it
    want_first, want_logits = [], []
    for s in range(rows):
        for pos, t in enumerate(prompts[s]):
            lg, _, _ = ref.forward(ref.embedding(int(t)), pos)
        want_first.append(orc.argmax(lg))
        lg, _, _ = ref.forward(ref.embedding(want_first[-1]), len(prompts[s]))
        want_logits.append(lg)
    assert firsts == want_first
    toks, lg, _ = eng.step_batch(list(range(rows)), firsts, [len(p) for p in prompts], want_logits=True)
    for s in range(rows):
        assert np.array_equal(lg[s].view(np.uint32), want_logits[s].view(np.uint32)), (s, hidden_gate(lg[s], want_logits[s]))
        assert toks[s] == orc.argmax(want_logits[s])
    # rows do not depend on their neighbours: the same rows in another order
    order = list(range(rows))[::-1]
    _, lg2, _ = eng.step_batch(order, [firsts[s] for s in order], [len(prompts[s]) for s in order], want_logits=True)
    assert np.array_equal(lg2[::-1], lg)


def test_prefill_chunk_of_32_rows_leaves_the_serial_kv(cm, orc):
    """prefill_then_decode_matches_sequential (src/cuda_resident/tests.rs:3143): a 40-token prompt ingested in
    chunks of 32 rows leaves the KV rows, and gives the next token, of token-by-token steps — which are the
    checker's."""
    from camelid_b200 import synth

    cfg = synth.engine_config("small", max_pos=64, max_seqs=2)
    pair = ModelPair(cfg, "q4_k_m", seed=78)
    eng, ref = pair.engine, pair.oracle
    prompt = orc.synth_tokens(9, 1, 40, cfg.vocab)
    first = eng.prefill_tokens(0, prompt, 0)
    tok = None
    for pos, t in enumerate(prompt):  # serial steps on the second sequence
        tok, _, _ = eng.step_batch([1], [int(t)], [pos])
        lg, _, _ = ref.forward(ref.embedding(int(t)), pos)
    assert first == int(tok[0]) == orc.argmax(lg)
    for layer in range(cfg.n_layers):
        rk, rv = ref.read_kv_layer(layer, len(prompt))
        k0, v0 = eng.read_kv_layer(layer, len(prompt))
        assert np.array_equal(k0, rk) and np.array_equal(v0, rv), layer


def test_verify_tree_predicts_what_a_linear_decode_of_each_path_predicts(cm, orc):
    """verify_tree (src/cuda_resident.rs:22944): every node of a draft tree in one batched pass.  The token predicted
    after node i equals the CPU checker's greedy token after prompt + the tokens on the path to node i (lossless
    speculation, :4343-4352); after compact_tree_kv_path the cache is that of a linear decode of the accepted path,
    so decoding on gives the checker's tokens."""
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny", max_pos=96)
    pair = ModelPair(cfg, "q4_k_m", seed=41)
    eng, ref = pair.engine, pair.oracle
    prompt = orc.synth_tokens(41, 5, 7, cfg.vocab)
    base = len(prompt)
    root = eng.prefill_tokens(0, prompt, 0)
    truth, _ = ref.generate(prompt, 8)  # the greedy continuation: truth[0] is the root token
    assert root == truth[0]
    # breadth-first tree: node 0 = root; one branch follows the greedy continuation for three steps, others do not
    parents = [-1, 0, 0, 0, 1, 1, 2, 4, 4, 7, 7, 9]
    rng = np.random.default_rng(9)
    tokens = [int(root)] + [int(t) for t in rng.integers(0, cfg.vocab, len(parents) - 1)]
    tokens[2] = int(truth[1])           # child of the root on the greedy path
    tokens[6] = int(truth[2])           # its child
    depth = [0] * len(parents)
    for i, par in enumerate(parents):
        if par >= 0:
            depth[i] = depth[par] + 1
    emb = np.stack([ref.embedding(t) for t in tokens])
    cs = [pair.rope(base + d) for d in depth]
    got = eng.verify_tree(emb, np.stack([c for c, _ in cs]), np.stack([s for _, s in cs]), parents, base, pair.scale)
    for i in range(len(parents)):
        path, j = [], i
        while j >= 0:
            path.append(tokens[j])
            j = parents[j]
        seq = np.concatenate([prompt, np.array(path[::-1], np.int32)])
        want, _ = ref.generate(seq, 1)
        assert got[i] == want[0], (i, got[i], want[0])
    # accept the longest path whose tokens are the model's own predictions: 0 -> 2 -> 6
    accepted = [0]
    while True:
        nxt = [j for j, par in enumerate(parents) if par == accepted[-1] and tokens[j] == got[accepted[-1]]]
        if not nxt:
            break
        accepted.append(nxt[0])
    assert accepted == [0, 2, 6]
    eng.compact_tree_kv_path(accepted, base)
    n_acc = len(accepted)
    cont = eng.decode_greedy([0], [int(got[accepted[-1]])], [base + n_acc], 4)[:, 0]
    assert int(got[accepted[-1]]) == truth[n_acc] and np.array_equal(cont, truth[n_acc + 1: n_acc + 5]), (cont, truth)
    # argument checks: a node may not name a later node, rows must be base + index
    with pytest.raises(cm.CmldError):
        eng.verify_tree(emb[:2], np.stack([cs[0][0], cs[1][0]]), np.stack([cs[0][1], cs[1][1]]), [-1, 0], cfg.max_pos - 1, pair.scale)


def test_forward_token_sample_draws_from_the_steps_own_logits(cm, orc):
    """forward_token_sample (src/cuda_resident.rs:20163): the token drawn on the device is the checker's draw over the
    logits of the very same forward pass (bit-identical to the CPU path's), with and without the min-p filter."""
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny", max_pos=64)
    pair = ModelPair(cfg, "q4_k_m", seed=3)
    eng, ref = pair.engine, pair.oracle
    tok = 5
    for pos in range(6):
        emb = ref.embedding(tok)
        c, s = pair.rope(pos)
        ref_logits, _, _ = ref.forward(emb, pos)
        if pos % 2 == 0:
            got = eng.forward_token_sample(emb, c, s, pos, pair.scale, 0.9, 1000 + pos)
            want, scores = orc.sample_gumbel(ref_logits, np.float32(1.0) / np.float32(0.9), 1000 + pos)
        else:
            got = eng.forward_token_sample(emb, c, s, pos, pair.scale, 0.9, 1000 + pos, min_p=0.05)
            want, scores = orc.sample_gumbel_filtered(ref_logits, 0.9, 0.05, 1000 + pos)
        if isinstance(got, tuple):  # the filter handed the row back: the logits come with it, bit for bit
            assert got[0] is None and np.array_equal(got[1].view(np.uint32), ref_logits.view(np.uint32))
            got = want if want >= 0 else int(np.argmax(ref_logits))
        else:
            assert want >= 0 and (got == want or abs(float(scores[got]) - float(scores[want])) <= 1e-5 * max(1.0, abs(float(scores[want]))))
        tok = int(got)


def test_q8_0_kv_cache_follows_the_cpu_lanes_scalar_arithmetic(cm, orc):
    """CMLD_FLAG_KV_Q8_0 (new_with_kv_quant, src/cuda_resident.rs:15748): K and V rows are kept as Q8_0 blocks
    (quantize_block_q8_0, src/tensor/kv_quant.rs:123) and attention runs over the blocks in the order of the CPU
    lane's scalar path (vec_dot_row_q8_0 :180, axpy_row_q8_0 :203).  Against the checker holding its cache the same
    way: residual stream, logits, cache rows and greedy tokens are bit-identical.  (The reference's AVX2 path adds in
    another order; its own test holds the two to 1e-5.)"""
    from camelid_b200 import synth

    cfg = synth.engine_config("tiny", max_pos=64, flags=256)
    pair = ModelPair(cfg, "q4_k_m", seed=19)
    eng, ref = pair.engine, pair.oracle
    ref.set_kv_q8(True)
    prompt = orc.synth_tokens(19, 5, 9, cfg.vocab)
    for pos in range(5):
        emb = ref.embedding(int(prompt[pos]))
        c, s = pair.rope(pos)
        ref_logits, _, ref_taps = ref.forward(emb, pos, want_taps=True)
        _, taps = eng.forward_token_hidden(emb, c, s, pos, pair.scale, taps=True)
        logits = eng.forward_token_logits(emb, c, s, pos, pair.scale)
        assert np.array_equal(taps.view(np.uint32), ref_taps.view(np.uint32)), pos
        assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32)), pos
    # the cache rows read back dequantised (code * d): what the blocks hold is what the checker's blocks hold
    ck, cv = eng.read_kv_layer(1, 5)
    nb = cfg.head_dim // 32
    kq, vq = ref.read_kv_layer(1, 5)          # the checker keeps codes (as floats) ...
    assert np.all(np.abs(kq) <= 127) and np.array_equal(kq, np.round(kq))
    ratio = np.where(kq != 0, ck / np.where(kq != 0, kq, 1), 0).reshape(cfg.n_kv_heads, 5, nb, 32)
    for blk in ratio.reshape(-1, 32):          # ... so every block's values are one scale times its codes
        nz = blk[blk != 0]
        assert nz.size == 0 or np.all(nz == nz[0])
    # a full generation: prompt through the 32-row chunks, then greedy steps
    ref2 = ModelPair(cfg, "q4_k_m", seed=19)
    ref2.oracle.set_kv_q8(True)
    want, _ = ref2.oracle.generate(prompt, 24)
    first = ref2.engine.prefill_tokens(0, prompt, 0)
    rest = ref2.engine.decode_greedy([0], [first], [len(prompt)], 23)[:, 0]
    assert np.array_equal(np.concatenate([[first], rest]), want)
    # seeding quantises rows exactly like an append does
    rows = np.random.default_rng(2).standard_normal((cfg.n_kv_heads, 3, cfg.head_dim)).astype(np.float32)
    eng.seed_layer(0, rows, rows * 0.5, 3)
    back_k, back_v = eng.read_kv_layer(0, 3)
    import ctypes as C
    for kh in range(cfg.n_kv_heads):
        for p in range(3):
            for b in range(nb):
                codes = np.empty(32, np.float32)
                blk = np.ascontiguousarray(rows[kh, p, 32 * b: 32 * b + 32])
                d = orc.lib().orc_kv_q8_0_quantize_block(blk.ctypes.data_as(C.c_void_p), codes.ctypes.data_as(C.c_void_p))
                assert np.array_equal(back_k[kh, p, 32 * b: 32 * b + 32], (codes * np.float32(d)).astype(np.float32))
