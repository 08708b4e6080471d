"""Pins for the CPU checker: the reference's golden vectors and known-answer tests.

Each case restates a test of the Camelid tree (cited per test) against ``oracle/``.
These run without a GPU.
"""
import json
import math

import numpy as np
import pytest

from conftest import GOLDEN

QT = {"Q8_0": 8, "Q4_K": 12, "Q6_K": 14}


def _fixture(name):
    fx = json.loads((GOLDEN / f"dequant_{name}.json").read_text())
    wire = np.frombuffer(bytes.fromhex(fx["quant_hex"]), dtype=np.uint8)
    ref_bits = np.array([int(s, 16) for s in fx["ref_f32_bits"]], dtype=np.uint32)
    return fx, wire, ref_bits


# tests/runnable_dequant.rs:82-159 — bit-exact dequantisation of the ggml fixtures.
@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "Q6_K"])
def test_dequant_matches_golden_bits(orc, name):
    fx, wire, ref_bits = _fixture(name)
    assert wire.size == fx["n_blocks"] * fx["block_bytes"]
    out = orc.dequant(QT[name], wire, fx["n_elements"])
    assert np.array_equal(out.view(np.uint32), ref_bits)


# src/inference/kv_f16.rs:181-373 — exhaustive f16 -> f32 -> f16 round trip, and
# src/tensor/mod.rs:8117 edge cases.
def test_f16_round_trip_exhaustive(orc):
    L = orc.lib()
    for h in range(1 << 16):
        exp = (h >> 10) & 0x1F
        if exp == 0x1F and (h & 0x3FF):
            continue  # NaN payloads are not preserved bit-for-bit
        f = L.orc_f16_bits_to_f32(h)
        assert L.orc_f32_to_f16_bits(f) == h, hex(h)
    # numpy agrees on every finite value
    hs = np.arange(1 << 16, dtype=np.uint16)
    finite = ((hs >> 10) & 0x1F) != 0x1F
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([L.orc_f16_bits_to_f32(int(h)) for h in hs[finite]], np.float32)
    assert np.array_equal(got.view(np.uint32), want[finite].view(np.uint32))


def test_f32_to_f16_rounding_edges(orc):
    L = orc.lib()
    rng = np.random.default_rng(7)
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(3.0),
        (rng.standard_normal(5000) * 1e-6).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5,
                  1.0009765625, 1.00048828125, 1.00146484375], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16_bits(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)
    # KV store canonicalises NaN (src/inference/kv_f16.rs:33-67)
    assert L.orc_kv_f32_to_f16_bits(float("nan")) & 0x7FFF == 0x7E00


# src/inference/tests.rs:17058-17074 — q8_k_quantizer_mirrors_reference_semantics.
def test_q8_k_quantizer_semantics(orc):
    row = np.zeros(256, np.float32)
    row[0], row[1] = -10.0, 4.0
    qs, d = orc.quantize_act_q8_k(row)
    assert abs(d[0] - 1.0 / 12.7) < 1e-6
    assert qs[0] == -127 and qs[1] == 51
    qs, d = orc.quantize_act_q8_k(np.zeros(256, np.float32))
    assert d[0] == 0.0 and not qs.any()
    # first max wins on |x| ties: +3 then -3 keeps the sign of the first
    row = np.zeros(256, np.float32)
    row[5], row[9] = 3.0, -3.0
    qs, d = orc.quantize_act_q8_k(row)
    assert qs[5] == -127 and qs[9] == 127 and d[0] < 0


# src/inference.rs:22510-22528 — Q8_0 activation quantiser: half-away rounding, scale
# rounded through f16, inverse from the unrounded scale.
def test_q8_0_activation_quantiser(orc):
    x = np.zeros(32, np.float32)
    x[0], x[1], x[2], x[3] = 127.0, 0.5, -0.5, 1.5
    qs, sc = orc.quantize_act_q8_0(x)
    assert sc[0] == 1.0
    assert list(qs[:4]) == [127, 1, -1, 2]  # ties away from zero
    rng = np.random.default_rng(3)
    x = rng.standard_normal(64).astype(np.float32)
    qs, sc = orc.quantize_act_q8_0(x)
    for b in range(2):
        blk = x[32 * b:32 * b + 32]
        du = np.float32(np.abs(blk).max()) / np.float32(127.0)
        assert sc[b] == np.float32(np.float16(du))
        inv = np.float32(1.0) / du
        want = np.clip(np.sign(blk * inv) * np.floor(np.abs(blk * inv) + np.float32(0.5)), -128, 127)
        assert np.array_equal(qs[32 * b:32 * b + 32], want.astype(np.int8))


# src/inference/tests.rs:16301-16349 — q6_k_wire_dot_consistent_with_dequant.
def test_q6_k_dot_consistent_with_dequant(orc):
    block = np.zeros(210, np.uint8)
    for i in range(128):
        block[i] = (i * 37 + 11) % 256
    for i in range(64):
        block[128 + i] = (i * 73 + 5) % 256
    for i in range(16):
        block[192 + i] = (i * 9 - 60) & 0xFF
    dbits = orc.lib().orc_f32_to_f16_bits(0.0375)
    block[208], block[209] = dbits & 0xFF, dbits >> 8
    act = (np.cos(np.arange(256, dtype=np.float32) * np.float32(0.21)) * np.float32(4.0)).astype(np.float32)
    xq, xd = orc.quantize_act_q8_k(act)
    dot = orc.matvec_quantised(14, block, 1, 256, xq, xd)[0]
    deq = orc.dequant(14, block, 256)
    d_back = orc.lib().orc_f16_bits_to_f32(dbits)
    aux = np.zeros(8, np.int64)
    for j in range(16):
        scale = int(np.int8(block[192 + j]))
        for l in range(16):
            w = deq[16 * j + l]
            q = 0 if scale == 0 else int(round(float(w) / (d_back * scale)))
            aux[l % 8] += scale * int(xq[16 * j + l]) * q
    reference = float(np.sum(np.float32(d_back) * xd[0] * aux.astype(np.float32), dtype=np.float32))
    assert abs(dot - reference) <= abs(reference) * 1e-5 + 1e-4


# src/inference/tests.rs:16400-16432 — q4_k_wire_dot_consistent_with_tensor_dequant.
def test_q4_k_dot_consistent_with_dequant(orc):
    blocks = 3
    wire = np.array([(i * 131 + 17) % 256 for i in range(blocks * 144)], np.uint8)
    L = orc.lib()
    for b in range(blocks):
        for off, val in ((0, 0.0173), (2, 0.0049)):
            bits = L.orc_f32_to_f16_bits(val)
            wire[b * 144 + off], wire[b * 144 + off + 1] = bits & 0xFF, bits >> 8
    act = (np.sin(np.arange(blocks * 256, dtype=np.float32) * np.float32(0.37)) * np.float32(3.0)).astype(np.float32)
    xq, xd = orc.quantize_act_q8_k(act)
    dot = float(orc.matvec_quantised(12, wire, 1, blocks * 256, xq, xd)[0])
    deq = orc.dequant(12, wire, blocks * 256).astype(np.float64)
    reference = float(np.sum(deq * (np.repeat(xd.astype(np.float64), 256) * xq.astype(np.float64))))
    assert abs(dot - reference) <= abs(reference) * 1e-4 + 1e-3


def test_q8_0_dot_matches_definition(orc):
    rng = np.random.default_rng(11)
    w = rng.standard_normal((5, 128)).astype(np.float32)
    wire = orc.quantize(8, w)
    x = rng.standard_normal(128).astype(np.float32)
    xq, xs = orc.quantize_act_q8_0(x)
    got = orc.matvec_quantised(8, wire, 5, 128, xq, xs)
    blk = wire.reshape(5, 4, 34)
    ws = blk[:, :, :2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    wq = blk[:, :, 2:].view(np.int8).astype(np.int32)
    for r in range(5):
        s = np.float32(0)
        for b in range(4):
            isum = int(np.dot(wq[r, b], xq[32 * b:32 * b + 32].astype(np.int32)))
            s = np.float32(s + np.float32(np.float32(np.float32(isum) * ws[r, b]) * xs[b]))
        assert got[r] == s


# src/quantize.rs:731-810 — quantiser accuracy / decoder-layout cases.
def test_weight_quantisers_round_trip(orc):
    x = ((np.arange(32, dtype=np.float32) - 16.0) * 0.125).astype(np.float32)
    rec = orc.dequant(8, orc.quantize(8, x), 32)
    assert np.abs(rec - x).max() < 0.05
    orig = np.zeros(256, np.float32)
    for g in range(8):
        off = 2.0 if g == 6 else (-2.0 if g == 7 else 0.0)
        orig[32 * g:32 * g + 32] = (np.arange(32, dtype=np.float32) - 15.5) * (g + 1.0) * 0.03125 + off
    rec = orc.dequant(12, orc.quantize(12, orig), 256)
    for g in range(8):
        assert np.abs(rec[32 * g:32 * g + 32] - orig[32 * g:32 * g + 32]).max() < 0.3
    # this project's Q6_K quantiser: relative error of a 6-bit code
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(1024) * 0.02).astype(np.float32)
    rec = orc.dequant(14, orc.quantize(14, x), 1024)
    assert np.abs(rec - x).max() < 0.02 * 4 / 31 * 1.2


# src/inference/tests.rs:12256-12303 and :12305-12360 — RoPE on each head / freq base.
def test_rope_known_answers(orc):
    c, s = orc.rope_table(1, 2, 10000.0)
    out = orc.rope_apply([1.0, 0.0, 0.0, 1.0], heads=2, head_dim=2, rope_dim=2, cosv=c, sinv=s)
    sin1, cos1 = math.sin(1.0), math.cos(1.0)
    assert np.allclose(out, [cos1, sin1, -sin1, cos1], atol=1e-6)
    c, s = orc.rope_table(3, 4, 500000.0)
    theta1 = np.float32(500000.0) ** np.float32(-0.5)
    assert abs(c[1] - math.cos(3.0 * float(theta1))) < 1e-6
    assert abs(s[0] - math.sin(3.0)) < 1e-6
    # split-half pairing (NeoX) rotates (i, i+half)
    c, s = orc.rope_table(1, 4, 10000.0)
    out = orc.rope_apply([1.0, 0.0, 0.0, 0.0], heads=1, head_dim=4, rope_dim=4, cosv=c, sinv=s, split_half=True)
    assert np.allclose(out, [cos1, 0.0, sin1, 0.0], atol=1e-6)


# src/inference/tests.rs:15494-15560 — causal_attention_context_attends_over_prior_and_current_positions.
def test_attention_known_answer(orc):
    k = np.array([[1.0, 0.0], [0.0, 1.0]], np.float32)
    v = np.array([[10.0, 0.0], [0.0, 20.0]], np.float32)
    out = orc.attention_head([1.0, 0.0], k, v, n_pos=2, head_dim=2, scale=1.0 / math.sqrt(2.0))
    first = math.exp(1.0 / math.sqrt(2.0))
    p = first / (first + 1.0)
    assert np.allclose(out, [p * 10.0, (1.0 - p) * 20.0], atol=1e-5)


# src/inference/tests.rs:15903-15922 — softmax_top_k renormalisation and tie-break.
def test_softmax_top_k(orc):
    top = orc.softmax_top_k([0.0, 1.0, 2.0], 2)
    assert [t[0] for t in top] == [2, 1]
    assert abs(sum(t[1] for t in top) - 1.0) < 1e-6
    assert abs(top[0][1] - math.exp(2.0) / (math.exp(2.0) + math.exp(1.0))) < 1e-6
    top = orc.softmax_top_k([1.0, 1.0, 1.0, 0.0], 2)
    assert [t[0] for t in top] == [0, 1]
    assert abs(top[0][1] - 0.5) < 1e-6 and abs(top[1][1] - 0.5) < 1e-6


# src/inference/tests.rs:15925-15961 — mixtral_moe_ffn_routes_top_k_experts.
def test_mixtral_moe_routes_top_k(orc):
    cfg = dict(n_layers=1, n_heads=1, n_kv_heads=1, head_dim=2, hidden=2, ffn_dim=2, max_pos=4, vocab=2,
               n_experts=2, n_experts_used=2)
    m = orc.OracleModel(cfg)
    eye_then_zero = np.array([1, 0, 0, 1, 0, 0, 0, 0], np.float32).view(np.uint8)
    zero_proj = np.zeros(4, np.float32).view(np.uint8)
    projs = {n: (0, zero_proj) for n in ("q", "k", "v", "o")}
    m.set_layer(0, projs, np.ones(2, np.float32), np.ones(2, np.float32))
    m.set_moe(0, np.array([10.0, 0.0, 0.0, 0.0], np.float32), (0, eye_then_zero), (0, eye_then_zero), (0, eye_then_zero))
    m.set_output(np.ones(2, np.float32), 0, np.eye(2, dtype=np.float32).view(np.uint8))
    # attention contributes zero (all-zero projections); feed x whose RMS-normed value is (1,1)
    _, hidden, _ = m.forward(np.array([1.0, 1.0], np.float32), 0, want_logits=False)
    expected = 1.0 / (1.0 + math.exp(-1.0))
    assert np.allclose(hidden - 1.0, expected, atol=1e-3)


# src/inference.rs:8904-8917 — strict '>' keeps the first of equal maxima.
def test_argmax_first_wins(orc):
    assert orc.argmax([1.0, 3.0, 3.0, 2.0]) == 1
    assert orc.argmax([-1.0, -1.0]) == 0


def test_rms_norm_sequential(orc):
    rng = np.random.default_rng(2)
    x = rng.standard_normal(64).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    got = orc.rms_norm(x, w, 1e-5)
    ss = np.float32(0)
    for v in x:
        ss = np.float32(ss + np.float32(v * v))
    scale = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(64)) + np.float32(1e-5), dtype=np.float32)
    want = (x * scale) * w
    assert np.array_equal(got, want.astype(np.float32))


def test_synthetic_generator_is_standard_normal_and_pure(orc):
    a = orc.synth_normal(1234, 7, 0, 200000, 1.0)
    b = orc.synth_normal(1234, 7, 1000, 1000, 1.0)
    assert np.array_equal(a[1000:2000], b)
    assert abs(float(a.mean())) < 0.01 and abs(float(a.std()) - 1.0) < 0.01
    assert abs(float((np.abs(a) < 1.0).mean()) - 0.6827) < 0.01
    assert not np.array_equal(a[:100], orc.synth_normal(1234, 8, 0, 100, 1.0))
    golden = json.loads((GOLDEN / "synth_vectors.json").read_text())
    for case in golden["cases"]:
        x = orc.synth_normal(case["seed"], case["stream"], case["start"], case["n"], case["sigma"])
        assert [format(int(v), "08x") for v in x.view(np.uint32)[:8]] == case["first_bits"]
        for name, qt in QT.items():
            assert orc.quantize(qt, x).tobytes().hex() == case["wire_hex"][name]


# The CUDA library's expf restates glibc's algorithm (camelid_b200/csrc/expf_exact.cuh); its C twin
# must agree with this machine's libm expf bit for bit on the ranges SwiGLU and the softmax use.
def test_expf_twin_matches_libm(orc):
    L = orc.lib()
    assert L.orc_expf_twin_mismatches(-110.0, 0.0, 3_000_001) == 0      # softmax: exp(score - max)
    assert L.orc_expf_twin_mismatches(-30.0, 30.0, 3_000_001) == 0       # SwiGLU: exp(-g)
    assert L.orc_expf_twin_mismatches(80.0, 95.0, 200_001) == 0          # overflow edge
    assert L.orc_expf_twin_mismatches(-1e-3, 1e-3, 200_001) == 0
    assert L.orc_expf_twin(float("-inf")) == 0.0 and L.orc_expf_twin(0.0) == 1.0


def test_kv_prefix_written_to_the_model_reads_back_rounded_to_f16():
    """write_kv_layer plants a KV prefix (the reference's seed_layer, src/cuda_resident.rs:17355) and
    read_kv_layer returns it rounded to f16; a forward pass then attends over it."""
    from oracle import oracle as orc

    cfg = dict(n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, hidden=256, ffn_dim=512, rope_dim=64, max_pos=16, vocab=64,
               eps=1e-5, rope_theta=10000.0)
    m = orc.OracleModel(cfg)
    rng = np.random.default_rng(3)
    ck = rng.standard_normal((2, 5, 64)).astype(np.float32)
    cv = rng.standard_normal((2, 5, 64)).astype(np.float32)
    m.write_kv_layer(1, ck, cv)
    rk, rv = m.read_kv_layer(1, 5)
    assert np.array_equal(rk, ck.astype(np.float16).astype(np.float32))
    assert np.array_equal(rv, cv.astype(np.float16).astype(np.float32))
    zk, _ = m.read_kv_layer(0, 5)
    assert not zk.any()


def test_sampling_math_of_the_checker():
    """The checker's restatement of src/cuda_resident/sampling.cuh: the uniform's clamp changes exactly one of the 2^24
    mantissas (the reference's host test prints "uniform 16777216 changed 1", src/inference/cuda_min_p_host_tests.rs:228),
    uniforms lie in (0, 1), a cold temperature collapses the Gumbel draw to the greedy argmax, and the min-p classifier
    keeps exactly the tokens whose probability ratio to the best token exceeds min_p wherever it decides."""
    from oracle import oracle as orc

    assert orc.lib().orc_sample_uniform_clamped_count() == 1
    us = np.array([orc.lib().orc_sample_uniform(12345, i) for i in range(2000)], np.float32)
    assert us.min() > 0.0 and us.max() < 1.0 and abs(float(us.mean()) - 0.5) < 0.03
    assert len(set(us.view(np.uint32).tolist())) > 1990
    rng = np.random.default_rng(2)
    logits = (rng.standard_normal(5000) * 3).astype(np.float32)
    idx, _ = orc.sample_gumbel(logits, 1.0e6, 7)
    assert idx == int(np.argmax(logits))
    draws = [orc.sample_gumbel(logits, 1.0, seed)[0] for seed in range(200)]
    assert len(set(draws)) > 20  # a warm temperature does spread the draws
    mx = float(logits.max())
    decided = 0
    for i in range(0, 5000, 7):
        k = orc.lib().orc_min_p_candidate(float(logits[i]), mx, 0.05, 5000)
        ratio = math.exp(float(logits[i]) - mx)
        if k >= 0:
            decided += 1
            assert k == (1 if ratio > 0.05 else 0)
        else:
            assert abs(ratio - 0.05) < 1e-5
    assert decided > 700
    assert orc.lib().orc_min_p_candidate(1.0, 2.0, 1.0, 10) == -1 and orc.lib().orc_min_p_candidate(float("nan"), 2.0, 0.1, 10) == -1
    tok, scores = orc.sample_gumbel_filtered(logits, 0.8, 0.05, 3)
    kept = np.isfinite(scores)
    assert tok >= 0 and kept[tok] and scores[tok] == scores[kept].max() and 1 <= kept.sum() < 5000


def test_q8_0_kv_block_functions_of_the_checker():
    """The checker's restatement of src/tensor/kv_quant.rs (scalar path) on the values of the reference's own unit test
    (q8_0_roundtrip_and_dot_match_dequantized_values, :905-933): round trip within 0.05, the block dot equals the dot
    with the dequantised values within 1e-5, and the fused accumulation equals prob * value + out within 1e-5."""
    import ctypes as C

    from oracle import oracle as orc

    original = ((np.arange(32, dtype=np.float32) - 16.0) * 0.25).astype(np.float32)
    codes = np.empty(32, np.float32)
    d = np.float32(orc.lib().orc_kv_q8_0_quantize_block(original.ctypes.data_as(C.c_void_p), codes.ctypes.data_as(C.c_void_p)))
    rec = (codes * d).astype(np.float32)
    assert np.abs(original - rec).max() < 0.05 and np.abs(codes).max() == 127
    assert d == np.float16(np.float32(4.0) / np.float32(127.0)).astype(np.float32)
    query = ((np.arange(32, dtype=np.float32) - 7.0) * 0.125).astype(np.float32)
    # one position, one block: the attention helper's score is (sum q*code)*d*scale and its output prob*d*code
    out, scores = np.empty(32, np.float32), np.empty(1, np.float32)
    sc = np.array([d], np.float32)
    rc = orc.lib().orc_attention_head_q8(query.ctypes.data_as(C.c_void_p), codes.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p),
                                         codes.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p), 32, 1, 1, 32, 1.0,
                                         out.ctypes.data_as(C.c_void_p), scores.ctypes.data_as(C.c_void_p))
    assert rc == 0 and scores[0] == 1.0           # a single position has probability one
    assert np.abs(out - rec).max() < 1e-5         # ... and the context is its dequantised value row
    zero = np.zeros(32, np.float32)
    assert orc.lib().orc_kv_q8_0_quantize_block(zero.ctypes.data_as(C.c_void_p), codes.ctypes.data_as(C.c_void_p)) == 0.0 and not codes.any()
