"""Kernel-level parity on a B200: every CUDA kernel of the path, called through the C ABI,
against the CPU checker on the same seeded inputs.  Integer/byte results are compared
bit-for-bit; f32 results within the tolerance written beside each check.
"""
import json

import numpy as np
import pytest

from conftest import GOLDEN
from helpers import close_enough

pytestmark = pytest.mark.gpu

QT = {"Q8_0": 8, "Q4_K": 12, "Q6_K": 14}


def lcg_bytes(seed, n):
    """The reference tests' 64-bit LCG (src/cuda_resident/tests.rs:3700-3717), byte stream."""
    out = np.empty(n, np.uint8)
    s = seed
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = s >> 56
    return out


# tests/runnable_dequant.rs:82-159 — bit-exact, through upload, re-layout and the dequant kernel.
@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "Q6_K"])
def test_dequant_matches_golden_bits(cm, name):
    fx = json.loads((GOLDEN / f"dequant_{name}.json").read_text())
    wire = np.frombuffer(bytes.fromhex(fx["quant_hex"]), dtype=np.uint8)
    ref_bits = np.array([int(s, 16) for s in fx["ref_f32_bits"]], dtype=np.uint32)
    w = cm.Weight.from_wire(QT[name], 1, fx["n_elements"], wire)
    assert np.array_equal(w.dequant().view(np.uint32).ravel(), ref_bits)
    assert np.array_equal(w.export_wire(), wire)


@pytest.mark.parametrize("name,rows,cols", [("Q8_0", 7, 96), ("Q4_K", 5, 768), ("Q6_K", 3, 768), ("Q6_K", 4, 2048)])
def test_random_wire_roundtrip_and_dequant(cm, orc, name, rows, cols):
    qt = QT[name]
    rng = np.random.default_rng(rows * cols)
    wire = rng.integers(0, 256, rows * orc.row_bytes(qt, cols), dtype=np.uint8)
    # keep f16 scale fields finite
    blk = {8: 34, 12: 144, 14: 210}[qt]
    v = wire.reshape(-1, blk)
    for off in {8: [0], 12: [0, 2], 14: [208]}[qt]:
        v[:, off + 1] &= 0x3B
    w = cm.Weight.from_wire(qt, rows, cols, wire)
    assert np.array_equal(w.export_wire(), wire)
    ref = orc.dequant(qt, wire, rows * cols)
    assert np.array_equal(w.dequant().view(np.uint32).ravel(), ref.view(np.uint32))


def test_q8_0_host_block_form(cm, orc):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((6, 128)).astype(np.float32)
    wire = orc.quantize(8, x)
    b = wire.reshape(-1, 34)
    host = np.zeros((b.shape[0], 36), np.uint8)
    host[:, :4] = b[:, :2].copy().view(np.float16).astype(np.float32).view(np.uint8).reshape(-1, 4)
    host[:, 4:] = b[:, 2:]
    w = cm.Weight.from_wire(cm.Q8_0_HOST36, 6, 128, host)
    assert np.array_equal(w.export_wire(), wire)


# The device generator + quantisers reproduce the CPU checker's bytes.
@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "Q6_K", "F32"])
def test_synthetic_weights_match_checker(cm, orc, name):
    qt = {"F32": 0, **QT}[name]
    w = cm.Weight.synth(qt, 20261125, 77, 9, 512, 0.02, row0=3)
    ref = orc.synth_tensor(qt, 20261125, 77, 9, 512, 0.02, row0=3)
    assert np.array_equal(w.export_wire(), ref)
    golden = json.loads((GOLDEN / "synth_vectors.json").read_text())["cases"][0]
    g = cm.Weight.synth(0, golden["seed"], golden["stream"], 1, golden["n"], golden["sigma"])
    bits = g.export_wire().view(np.uint32)[:8]
    assert [format(int(v), "08x") for v in bits] == golden["first_bits"]


@pytest.mark.parametrize("cols,batch", [(64, 1), (256, 3), (4096, 2), (14336, 1)])
def test_activation_quantisers_bit_exact(cm, orc, cols, batch):
    from camelid_b200.engine import quantize_activation, export_activation

    rng = np.random.default_rng(cols + batch)
    x = (rng.standard_normal((batch, cols)) * 1.7).astype(np.float32)
    x[0, :32] = 0.0                       # an all-zero Q8_0 block
    x[0, 40] = 2.5
    x[0, 41] = -2.5                       # |x| tie: the first keeps the sign
    if cols >= 512:
        x[-1, 256:512] = 0.0              # an all-zero Q8_K superblock
    x[0, 33] = 0.5 * np.abs(x[0, 32:64]).max() / 127 * 3  # near a .5 rounding boundary
    act = quantize_activation(cm.ACT_Q8_0, x)
    codes, scales = export_activation(cm.ACT_Q8_0, act, cols, batch)
    for b in range(batch):
        rq, rs = orc.quantize_act_q8_0(x[b])
        assert np.array_equal(codes[b], rq) and np.array_equal(scales[b].view(np.uint32), rs.view(np.uint32))
    if cols % 256 == 0:
        act = quantize_activation(cm.ACT_Q8_K, x)
        codes, scales = export_activation(cm.ACT_Q8_K, act, cols, batch)
        for b in range(batch):
            rq, rd = orc.quantize_act_q8_k(x[b])
            assert np.array_equal(codes[b], rq) and np.array_equal(scales[b].view(np.uint32), rd.view(np.uint32))


# q4k_gemv_matches_oracle / q6k_gemv_matches_oracle / q8 (src/cuda_resident/tests.rs:7749,
# :10302): same wire bytes, same quantised activation, CPU row dot as the oracle.
@pytest.mark.parametrize("name,rows,cols", [
    ("Q8_0", 96, 64), ("Q8_0", 515, 2048), ("Q8_0", 64, 8192),
    ("Q4_K", 37, 256), ("Q4_K", 512, 4096), ("Q4_K", 130, 3072), ("Q4_K", 64, 14336),
    ("Q6_K", 33, 256), ("Q6_K", 512, 4096), ("Q6_K", 130, 3072), ("Q6_K", 64, 14336),
    # column shards of an eight-way tensor-parallel split: rows of two and seven superblocks
    ("Q4_K", 300, 512), ("Q4_K", 300, 1792), ("Q6_K", 300, 512), ("Q6_K", 300, 1792)])
@pytest.mark.parametrize("batch", [1, 2, 3, 8])
@pytest.mark.parametrize("kernel", ["staged", "generic", "tcgen05"])
def test_gemv_matches_checker(cm, orc, name, rows, cols, batch, kernel):
    """All matvec kernels add a row's f32 terms in the CPU dot's order: every output equals the
    checker's bit for bit (the staged kernel takes the shapes it supports, the generic one the rest;
    the tcgen05 kernel, forced here from one row, computes the integer parts on the tensor cores)."""
    from camelid_b200.engine import quantize_activation, export_activation, DeviceBuffer
    from camelid_b200._lib import check

    check(cm.lib().cmld_gemv_select_kernel({"generic": 1, "staged": 16, "tcgen05": 32}[kernel]))
    qt = QT[name]
    wire = orc.synth_tensor(qt, 11, rows * 7 + cols, rows, cols, 0.02)
    w = cm.Weight.from_wire(qt, rows, cols, wire)
    rng = np.random.default_rng(rows + cols + batch)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    kind = cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K
    act = quantize_activation(kind, x)
    codes, scales = export_activation(kind, act, cols, batch)
    y = w.gemv(act, batch)
    res = rng.standard_normal((batch, rows)).astype(np.float32)
    res_d = DeviceBuffer.from_numpy(res)
    y_res = w.gemv(act, batch, res_d)
    try:
        for b in range(batch):
            ref = orc.matvec_quantised(qt, wire, rows, cols, codes[b], scales[b])
            bad = np.nonzero(y[b].view(np.uint32) != ref.view(np.uint32))[0]
            assert bad.size == 0, (name, rows, cols, b, bad[:5], y[b][bad[:5]], ref[bad[:5]])
            assert np.array_equal(y_res[b], (res[b] + y[b]).astype(np.float32))
    finally:
        check(cm.lib().cmld_gemv_select_kernel(0))


# The staged kernel's fused prologues: RMSNorm / plain / SwiGLU + quantiser + matvec in one launch
# equals the three separate steps (same quantised codes, so the same result bit for bit).
@pytest.mark.parametrize("name,rows,cols", [("Q8_0", 200, 2048), ("Q4_K", 200, 4096), ("Q6_K", 200, 4096), ("Q4_K", 72, 14336),
                                            ("Q6_K", 100, 3072)])
@pytest.mark.parametrize("mode", [1, 2, 3])
@pytest.mark.parametrize("batch", [1, 3])
def test_fused_prologue_equals_separate_steps(cm, orc, name, rows, cols, mode, batch):
    from camelid_b200.engine import quantize_activation, DeviceBuffer
    from camelid_b200._lib import check

    qt = QT[name]
    w = cm.Weight.from_wire(qt, rows, cols, orc.synth_tensor(qt, 3, cols + rows, rows, cols, 0.02))
    rng = np.random.default_rng(cols + mode)
    x = rng.standard_normal((batch, cols)).astype(np.float32) * 1.5
    x2 = rng.standard_normal((batch, cols)).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    res = rng.standard_normal((batch, rows)).astype(np.float32)
    xd, x2d, nwd, resd = (DeviceBuffer.from_numpy(a) for a in (x, x2, nw, res))
    y = DeviceBuffer(batch * rows * 4)
    check(cm.lib().cmld_gemv_fused(w._h, mode, xd.ptr, x2d.ptr, nwd.ptr, 1e-5, batch, y.ptr, resd.ptr))
    got = y.to_numpy(np.float32).reshape(batch, rows)
    # separate steps on the device: f(x) as f32, then quantise, then matvec + residual
    fx = DeviceBuffer(x.nbytes)
    if mode == 1:
        check(cm.lib().cmld_rms_norm(xd.ptr, nwd.ptr, cols, batch, 1e-5, fx.ptr, 0, None))
    elif mode == 3:
        check(cm.lib().cmld_silu_mul(xd.ptr, x2d.ptr, cols, batch, fx.ptr, 0, None))
    f = fx.to_numpy(np.float32).reshape(batch, cols) if mode != 2 else x
    act = quantize_activation(cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K, f)
    want = w.gemv(act, batch, resd)
    assert np.array_equal(got, want)


# More than 8 activation rows.  By default they take the tcgen05 kernel: the weights are read once for up to
# 32 rows, the integer parts come from the tensor cores and the f32 terms are added in the CPU dot's order
# (the checker's bits).  The older int8 mma.sync kernel adds the superblocks' f32 terms as a tree, so it is
# opt-in and held to a tolerance.
@pytest.mark.parametrize("name,rows,cols", [
    ("Q8_0", 96, 256), ("Q8_0", 515, 2048), ("Q8_0", 70, 1792),
    ("Q4_K", 37, 256), ("Q4_K", 512, 4096), ("Q4_K", 130, 1792), ("Q4_K", 64, 14336),
    ("Q6_K", 33, 256), ("Q6_K", 512, 4096), ("Q6_K", 130, 1792), ("Q6_K", 64, 14336)])
@pytest.mark.parametrize("batch", [9, 16, 27, 32])
def test_gemv_batched_tensor_core_kernel_matches_checker(cm, orc, name, rows, cols, batch):
    from camelid_b200.engine import quantize_activation, export_activation, DeviceBuffer
    from camelid_b200._lib import check

    qt = QT[name]
    wire = orc.synth_tensor(qt, 13, rows * 5 + cols, rows, cols, 0.02)
    w = cm.Weight.from_wire(qt, rows, cols, wire)
    rng = np.random.default_rng(rows + cols + batch)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    kind = cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K
    act = quantize_activation(kind, x)
    codes, scales = export_activation(kind, act, cols, batch)
    res = rng.standard_normal((batch, rows)).astype(np.float32)
    res_d = DeviceBuffer.from_numpy(res)
    # default: one pass over the weights on the tcgen05 tensor cores (when the columns are a multiple of 256, else
    # passes of the ordered kernels) -> the checker's bits, whatever the batch
    y = w.gemv(act, batch)
    y_res = w.gemv(act, batch, res_d)
    for b in range(batch):
        ref = orc.matvec_quantised(qt, wire, rows, cols, codes[b], scales[b])
        bad = np.nonzero(y[b].view(np.uint32) != ref.view(np.uint32))[0]
        assert bad.size == 0, (name, rows, cols, b, bad.size, bad[:5], y[b][bad[:5]], ref[bad[:5]])
        assert np.array_equal(y_res[b], (res[b] + y[b]).astype(np.float32))
    # the very same bits whatever the row's neighbours are, and from the staged kernel
    y_rev = w.gemv(quantize_activation(kind, x[::-1].copy()), batch)
    assert np.array_equal(y_rev[::-1].view(np.uint32), y.view(np.uint32))
    check(cm.lib().cmld_gemv_select_kernel(16))
    try:
        assert np.array_equal(w.gemv(act, batch).view(np.uint32), y.view(np.uint32))
    finally:
        check(cm.lib().cmld_gemv_select_kernel(0))
    # opt-in: the int8 mma.sync kernel (kernel choice 8), one pass over the weights, tree sums
    check(cm.lib().cmld_gemv_select_kernel(8))
    try:
        ym = w.gemv(act, batch)
        ym_res = w.gemv(act, batch, res_d)
        for b in range(batch):
            ref = orc.matvec_quantised(qt, wire, rows, cols, codes[b], scales[b])
            # tolerance: 1e-4 relative + 1e-5 of the largest output (f32 reassociation of <= 448 terms)
            ok, max_abs, n_bad = close_enough(ym[b], ref, rel=1e-4, floor=1e-5)
            assert ok, (name, rows, cols, b, max_abs, n_bad)
            assert np.array_equal(ym_res[b], (res[b] + ym[b]).astype(np.float32))
        # the very same bits whatever the row's neighbours are
        y_again = w.gemv(quantize_activation(kind, x[::-1].copy()), batch)
        assert np.array_equal(y_again[::-1], ym)
    finally:
        check(cm.lib().cmld_gemv_select_kernel(0))


@pytest.mark.parametrize("name,rows,cols,batch", [
    ("Q4_K", 128 * 40 + 17, 512, 32), ("Q4_K", 128 * 170, 256, 32), ("Q4_K", 128 * 170, 256, 16),
    ("Q6_K", 128 * 90 + 5, 512, 32), ("Q6_K", 128 * 170, 256, 11), ("Q8_0", 128 * 40, 768, 24), ("Q8_0", 128 * 170 + 64, 256, 32)])
def test_gemv_tcgen05_many_tiles(cm, orc, name, rows, cols, batch):
    """Launches with more tiles than SMs: a CTA walks several tiles, takes 16 or 32 activation rows at once
    (two epilogue warp groups, two groups of columns each) and the last tile is ragged.  Bits of the checker."""
    from camelid_b200.engine import quantize_activation, export_activation

    qt = QT[name]
    wire = orc.synth_tensor(qt, 17, rows + cols, rows, cols, 0.02)
    w = cm.Weight.from_wire(qt, rows, cols, wire)
    x = np.random.default_rng(rows + batch).standard_normal((batch, cols)).astype(np.float32)
    kind = cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K
    act = quantize_activation(kind, x)
    codes, scales = export_activation(kind, act, cols, batch)
    for rep in range(3):  # repeated: the pipeline's hand-offs are timing dependent
        y = w.gemv(act, batch)
        for b in range(batch):
            ref = orc.matvec_quantised(qt, wire, rows, cols, codes[b], scales[b])
            bad = np.nonzero(y[b].view(np.uint32) != ref.view(np.uint32))[0]
            assert bad.size == 0, (name, rows, cols, b, rep, bad.size, bad[:5])


def test_gemv_end_to_end_against_f32_activation_path(cm, orc):
    """orc.matvec quantises the f32 activation itself: checks quantise+gemv as one unit."""
    from camelid_b200.engine import quantize_activation

    for name, cols in (("Q8_0", 2048), ("Q4_K", 4096), ("Q6_K", 4096)):
        qt = QT[name]
        wire = orc.synth_tensor(qt, 5, cols, 256, cols, 0.02)
        x = np.random.default_rng(cols).standard_normal(cols).astype(np.float32)
        y = cm.Weight.from_wire(qt, 256, cols, wire).gemv(quantize_activation(cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K, x), 1)[0]
        ok, max_abs, n_bad = close_enough(y, orc.matvec(qt, wire, 256, cols, x))
        assert ok, (name, max_abs, n_bad)


@pytest.mark.parametrize("cols,batch", [(64, 1), (2048, 2), (4096, 1), (14336, 3)])
def test_rms_norm_and_swiglu(cm, orc, cols, batch):
    from camelid_b200.engine import DeviceBuffer, export_activation
    from camelid_b200._lib import check

    rng = np.random.default_rng(cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32) * 2.0
    wgt = (1.0 + 0.2 * rng.standard_normal(cols)).astype(np.float32)
    xd, wd, od = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(wgt), DeviceBuffer(x.nbytes)
    act = DeviceBuffer(batch * cm.act_row_bytes(cols))
    kind = cm.ACT_Q8_K if cols % 256 == 0 else cm.ACT_Q8_0
    check(cm.lib().cmld_rms_norm(xd.ptr, wd.ptr, cols, batch, 1e-5, od.ptr, kind, act.ptr))
    out = od.to_numpy(np.float32).reshape(batch, cols)
    codes, scales = export_activation(kind, act, cols, batch)
    for b in range(batch):
        ref = orc.rms_norm(x[b], wgt, 1e-5)
        # the mean square has the bits of the CPU's sequential sum, so the normalised row is the CPU's
        assert np.array_equal(out[b].view(np.uint32), ref.view(np.uint32))
        # the fused quantiser is the standalone quantiser applied to the kernel's own f32 output
        rq, rs = (orc.quantize_act_q8_k if kind == cm.ACT_Q8_K else orc.quantize_act_q8_0)(out[b])
        assert np.array_equal(codes[b], rq) and np.array_equal(scales[b], rs)
    g = rng.standard_normal((batch, cols)).astype(np.float32) * 3.0
    gd = DeviceBuffer.from_numpy(g)
    check(cm.lib().cmld_silu_mul(gd.ptr, xd.ptr, cols, batch, od.ptr, 0, None))
    out = od.to_numpy(np.float32).reshape(batch, cols)
    ref = np.stack([orc.silu_mul(g[b], x[b]) for b in range(batch)])
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))  # expf restated from glibc: the same bits


# The sum of squares is evaluated in parallel with the sequential sum's bits (runs of additions inside one binade
# applied as integer steps, ties and binade crossings replayed): rows built to hit the replay paths.
@pytest.mark.parametrize("cols", [4096, 8192, 1024])
def test_rms_norm_sum_of_squares_is_the_sequential_sum(cm, orc, cols):
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check

    rng = np.random.default_rng(cols + 5)
    rows = []
    for mode in range(12):
        sigma = 10.0 ** rng.integers(-6, 7)
        x = rng.standard_normal(cols).astype(np.float32) * np.float32(sigma)
        if mode == 1:
            x[rng.random(cols) < 0.01] *= 100.0                      # outliers
        if mode == 2:
            x = (rng.integers(0, 64, cols) / 8.0).astype(np.float32)  # few mantissa bits: many ties
        if mode == 3:
            x[rng.random(cols) < 0.66] = 0.0                          # zeros
        if mode == 4:
            x = np.ldexp(rng.integers(1, 5, cols).astype(np.float32), rng.integers(-10, 10, cols)).astype(np.float32)
        if mode == 5:
            x[:100] = 0.0                                             # leading zeros
        if mode == 6:
            x[700] = 1e4                                              # one giant
        if mode == 7:
            x[:] = 1.0                                                # constant
        if mode == 8:
            x = (0.5 + rng.integers(0, 2, cols)).astype(np.float32)   # ties everywhere
        if mode == 9:
            x = (rng.standard_normal(cols) * 1e-18).astype(np.float32)  # squares in the subnormal range
        if mode == 10:
            x = (rng.standard_normal(cols) * 1e15).astype(np.float32)
        if mode == 11:
            x = np.sqrt((rng.integers(1, 1025, cols) * 0.5)).astype(np.float32)
        rows.append(x.astype(np.float32))
    x = np.stack(rows)
    wgt = np.ones(cols, np.float32)
    xd, wd, od = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(wgt), DeviceBuffer(x.nbytes)
    check(cm.lib().cmld_rms_norm(xd.ptr, wd.ptr, cols, len(rows), 1e-5, od.ptr, 0, None))
    out = od.to_numpy(np.float32).reshape(len(rows), cols)
    for b in range(len(rows)):
        ref = orc.rms_norm(x[b], wgt, 1e-5)
        assert np.array_equal(out[b].view(np.uint32), ref.view(np.uint32)), b


# The exact sum's two walks on the device: the usual one (integer steps, unchecked, verified on the side) and the
# fallback (every step checked; here every second run is forced to fail its check and is replayed term by term).
@pytest.mark.parametrize("n", [256, 1280, 4096, 8192])
def test_exact_sum_walks_agree_with_the_sequential_sum(cm, n):
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check

    rng = np.random.default_rng(n)
    cases = []
    g = rng.standard_normal(n).astype(np.float32)
    cases.append((g * g).astype(np.float32))                                   # squares of N(0, 1)
    cases.append(np.exp(g - 3.2).astype(np.float32))                           # softmax weights
    cases.append((rng.integers(0, 64, n) / 8.0).astype(np.float32))            # ties
    cases.append(np.full(n, 0.99999994, np.float32))                           # crossings at item boundaries
    cases.append((1.0 + (rng.integers(0, 3, n) - 1) * 5.9604645e-8).astype(np.float32))
    big = (g * g).astype(np.float32)
    big[n // 3] = 1e4                                                          # one giant term
    cases.append(big)
    cases.append(np.zeros(n, np.float32))
    for k, terms in enumerate(cases):
        seq = np.float32(0.0)
        for t in terms:
            seq = np.float32(seq + t)
        td = DeviceBuffer.from_numpy(terms)
        out = np.zeros(2, np.float32)
        check(cm.lib().cmld_exact_sum_selftest(td.ptr, n, out.ctypes.data))
        assert out.view(np.uint32)[0] == np.float32(seq).view(np.uint32), (k, out[0], seq)
        assert out.view(np.uint32)[1] == np.float32(seq).view(np.uint32), (k, out[1], seq)


def test_argmax_lowest_index_wins(cm, orc):
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check

    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 128256)).astype(np.float32)
    x[0, 70000] = x[0, 100] = 9.0
    x[1, 128255] = 11.0
    x[2, :] = -1.0
    out = np.zeros(3, np.uint32)
    xd = DeviceBuffer.from_numpy(x)  # keep the device buffer alive across the call
    check(cm.lib().cmld_argmax(xd.ptr, 128256, 3, out.ctypes.data))
    assert list(out) == [orc.argmax(x[0]), orc.argmax(x[1]), orc.argmax(x[2])] == [100, 128255, 0]


# attention_decode_matches_cpu (src/cuda_resident/tests.rs:5066) with GQA and split ranges.
@pytest.mark.parametrize("n_heads,n_kv,hd,n_pos", [(2, 1, 32, 1), (2, 1, 32, 4), (32, 8, 64, 33), (24, 8, 128, 300),
                                                    (32, 8, 128, 1153), (8, 8, 128, 70), (8, 1, 64, 515),
                                                    (32, 8, 128, 2048), (32, 8, 128, 2049), (16, 4, 64, 3000)])
def test_attention_matches_checker(cm, orc, n_heads, n_kv, hd, n_pos):
    """Up to 2048 positions the ranges are merged inside a thread-block cluster; beyond that through global
    memory by the CTA that finishes last: both forms are covered."""
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check

    max_pos = 2048 if n_pos <= 2048 else 4096
    rng = np.random.default_rng(n_heads * n_pos)
    q = rng.standard_normal((n_heads, hd)).astype(np.float32)
    k = np.zeros((n_kv, max_pos, hd), np.float16)
    v = np.zeros((n_kv, max_pos, hd), np.float16)
    k[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    v[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    out_d = DeviceBuffer(n_heads * hd * 4)
    qd, kd, vd = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(k), DeviceBuffer.from_numpy(v)
    check(cm.lib().cmld_attention_decode(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, n_pos, scale, out_d.ptr))
    out = out_d.to_numpy(np.float32).reshape(n_heads, hd)
    kf, vf = k.astype(np.float32), v.astype(np.float32)
    g = n_heads // n_kv
    for h in range(n_heads):
        ref = orc.attention_head(q[h], kf[h // g, :n_pos], vf[h // g, :n_pos], n_pos, hd, scale)
        # tolerance 2e-5 of the largest output: split ranges + online softmax reassociate the sums
        assert np.abs(out[h] - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max()), (h, np.abs(out[h] - ref).max())


# The attention the engine runs by default: every sum in the CPU's order, so the CPU's bits.
@pytest.mark.parametrize("n_heads,n_kv,hd,n_pos", [(2, 1, 32, 4), (32, 8, 64, 1), (32, 8, 64, 33), (24, 8, 128, 300),
                                                    (32, 8, 128, 1153), (8, 8, 128, 70), (8, 1, 64, 515), (16, 8, 128, 256),
                                                    (32, 8, 128, 2049), (16, 4, 64, 3000), (32, 8, 128, 8192),
                                                    (8, 8, 64, 9), (24, 8, 64, 700), (4, 4, 128, 1025)])
def test_attention_reference_order_is_bit_identical(cm, orc, n_heads, n_kv, hd, n_pos):
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check

    max_pos = max(256, n_pos)
    rng = np.random.default_rng(n_heads * n_pos + 1)
    q = rng.standard_normal((n_heads, hd)).astype(np.float32)
    k = np.zeros((n_kv, max_pos, hd), np.float16)
    v = np.zeros((n_kv, max_pos, hd), np.float16)
    k[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    v[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    out_d = DeviceBuffer(n_heads * hd * 4)
    qd, kd, vd = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(k), DeviceBuffer.from_numpy(v)
    check(cm.lib().cmld_attention_decode_ordered(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, n_pos, scale, out_d.ptr))
    out = out_d.to_numpy(np.float32).reshape(n_heads, hd)
    kf, vf = k.astype(np.float32), v.astype(np.float32)
    g = n_heads // n_kv
    for h in range(n_heads):
        ref = orc.attention_head(q[h], kf[h // g, :n_pos], vf[h // g, :n_pos], n_pos, hd, scale)
        bad = np.nonzero(out[h].view(np.uint32) != ref.view(np.uint32))[0]
        assert bad.size == 0, (h, bad[:4], out[h][bad[:4]], ref[bad[:4]])


# ---- on-device sampling (src/cuda_resident/sampling.cuh): the uniforms are integer arithmetic and must equal the
# checker's bit for bit; the Gumbel scores go through the device's logf / expf, so a draw may differ from the
# checker's only where the two best scores lie within 1e-5 (relative) of each other — the tolerance of this test.
def _draw_ok(tok, ref_tok, scores):
    if tok == ref_tok:
        return True
    best = float(scores[ref_tok])
    return abs(float(scores[tok]) - best) <= 1e-5 * max(1.0, abs(best))


def test_sampling_kernels_match_the_checker(cm, orc):
    from camelid_b200.engine import DeviceBuffer
    from camelid_b200._lib import check
    import ctypes as C

    n = 32000
    for seed in (0, 1, 0x915E55A9DA3C1891):
        got = np.empty(4096, np.float32)
        check(cm.lib().cmld_sample_uniforms(seed, 4096, got.ctypes.data_as(C.c_void_p)))
        ref = np.array([orc.lib().orc_sample_uniform(seed, i) for i in range(4096)], np.float32)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal(n) * 4).astype(np.float32)
    dev = DeviceBuffer.from_numpy(logits)
    tok = C.c_uint32(0)
    same = 0
    for seed in range(60):
        for inv_temp in (1.0, 1.0 / 0.7):
            check(cm.lib().cmld_sample_gumbel(dev.ptr, n, inv_temp, seed, C.byref(tok)))
            ref_tok, scores = orc.sample_gumbel(logits, inv_temp, seed)
            assert _draw_ok(tok.value, ref_tok, scores), (seed, inv_temp, tok.value, ref_tok)
            same += int(tok.value == ref_tok)
    assert same >= 115  # practically always the very same token
    check(cm.lib().cmld_sample_gumbel(dev.ptr, n, 1.0e6, 3, C.byref(tok)))
    assert tok.value == int(np.argmax(logits))  # a cold temperature is the greedy argmax
    # min-p mask and filtered draw
    mask = np.empty(n, np.int32)
    for min_p in (0.02, 0.2):
        check(cm.lib().cmld_sample_min_p_mask(dev.ptr, n, min_p, mask.ctypes.data_as(C.c_void_p)))
        mx = float(logits.max())
        ref_mask = np.array([orc.lib().orc_min_p_candidate(float(x), mx, min_p, n) for x in logits], np.int32)
        diff = np.nonzero(mask != ref_mask)[0]
        ratio = np.exp(logits[diff].astype(np.float64) - mx)
        assert np.all(np.abs(ratio - min_p) <= 2 * 64 * 1.1920929e-7 * min_p), (min_p, diff[:5])
        for seed in range(20):
            check(cm.lib().cmld_sample_gumbel_filtered(dev.ptr, n, 0.8, min_p, seed, C.byref(tok)))
            ref_tok, scores = orc.sample_gumbel_filtered(logits, 0.8, min_p, seed)
            if tok.value == 0xFFFFFFFF or ref_tok < 0:
                # a token within the margin of the cutoff sends the row to the CPU on one side or both
                assert (mask == -1).any() or (ref_mask == -1).any()
                continue
            assert _draw_ok(tok.value, ref_tok, scores), (min_p, seed, tok.value, ref_tok)
    # a non-finite logit hands the row back
    bad = logits.copy()
    bad[17] = np.inf
    check(cm.lib().cmld_sample_gumbel_filtered(DeviceBuffer.from_numpy(bad).ptr, n, 0.8, 0.1, 1, C.byref(tok)))
    assert tok.value == 0xFFFFFFFF
