"""Quantised-matvec microbenchmark (benchmark configuration 2): weights M x K in
{4096x4096, 14336x4096, 4096x14336, 128256x4096} x {Q8_0, Q4_K, Q6_K}, seeded N(0, 0.02);
activations f32 N(0,1) at batch 1, 4, 8; outputs f32.  Prints one JSON line per case with the
achieved HBM GB/s (algorithmic bytes = weight wire bytes + int8 activation codes + f32 outputs,
over the mean launch time from CUDA events; weight copies rotate so that they exceed the L2).

    python -m camelid_b200.microbench [--qt Q4_K] [--rows 14336 --cols 4096] [--batch 1] [--iters 200]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
from pathlib import Path

import numpy as np

SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
BPW = {"Q8_0": 34 / 32, "Q4_K": 144 / 256, "Q6_K": 210 / 256}


def peak_gbs() -> tuple[float, str]:
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def run_case(qt_name: str, rows: int, cols: int, batch: int, iters: int, warmup: int, l2_bytes: float = 400e6) -> dict:
    import camelid_b200 as cm
    from camelid_b200._lib import check
    from camelid_b200.engine import QT_NAMES, DeviceBuffer, quantize_activation

    qt = QT_NAMES[qt_name]
    wbytes = rows * cols * BPW[qt_name]
    n_copies = max(1, int(np.ceil(l2_bytes / wbytes))) if iters > 3 else 1
    copies = [cm.Weight.synth(qt, 20261125, 5000 + i, rows, cols, 0.02) for i in range(n_copies)]
    x = np.random.default_rng(0).standard_normal((batch, cols)).astype(np.float32)
    act = quantize_activation(cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K, x)
    y = DeviceBuffer(batch * rows * 4)
    arr = (C.c_void_p * n_copies)(*[w._h for w in copies])
    ms = C.c_float(0)
    check(cm.lib().cmld_gemv_time(arr, n_copies, act.ptr, batch, y.ptr, warmup, iters, C.byref(ms)))
    alg = wbytes + cols * batch + rows * 4 * batch
    gbs = alg / (ms.value * 1e-3) / 1e9
    peak, kind = peak_gbs()
    return {"qt": qt_name, "rows": rows, "cols": cols, "batch": batch, "us_per_launch": ms.value * 1e3, "algorithmic_bytes": alg,
            "achieved_gbs": gbs, "frac_of_copy_peak": gbs / peak, "peak_kind": kind, "frac_of_8tbs_nominal": gbs / 8000.0,
            "weight_copies": n_copies, "iters": iters}


def run_attention(ctx: int, iters: int) -> dict:
    """The reference-order decode attention at the Llama-3-8B shape (32 query heads, 8 KV heads, head_dim 128) over
    `ctx` cached positions of seeded f16 K/V: wall time per call of the operator entry point (launch and
    synchronisation included), and the KV bytes one call reads."""
    import time

    import camelid_b200 as cm
    from camelid_b200._lib import check
    from camelid_b200.engine import DeviceBuffer

    n_heads, n_kv, hd = 32, 8, 128
    max_pos = max(2048, 1 << (ctx - 1).bit_length())
    rng = np.random.default_rng(1)
    q = rng.standard_normal((n_heads, hd)).astype(np.float32)
    k = rng.standard_normal((n_kv, max_pos, hd)).astype(np.float16)
    v = rng.standard_normal((n_kv, max_pos, hd)).astype(np.float16)
    out_d = DeviceBuffer(n_heads * hd * 4)
    qd, kd, vd = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(k), DeviceBuffer.from_numpy(v)
    scale = float(1 / np.sqrt(hd))
    for _ in range(3):
        check(cm.lib().cmld_attention_decode_ordered(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, ctx, scale, out_d.ptr))
    t0 = time.perf_counter()
    for _ in range(iters):
        check(cm.lib().cmld_attention_decode_ordered(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, ctx, scale, out_d.ptr))
    dt = (time.perf_counter() - t0) / iters
    return {"op": "attention_decode_ordered", "n_heads": n_heads, "n_kv_heads": n_kv, "head_dim": hd, "context": ctx,
            "wall_us_per_call": dt * 1e6, "kv_bytes": 2 * n_kv * ctx * hd * 2, "iters": iters}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--attention", type=int, default=0, metavar="CTX",
                    help="run the reference-order decode attention at the 8B shape over CTX positions instead of the matvec cases")
    ap.add_argument("--qt", default=None, choices=sorted(BPW))
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--cols", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--kernel", default="staged", choices=["staged", "direct", "mma", "tcgen05"],
                    help="staged = bulk-copy pipelined kernel when the shape fits (default); direct = direct-load kernel")
    ap.add_argument("--pdl", action="store_true", help="chain the timed launches with programmatic dependent launch")
    a = ap.parse_args()
    if a.attention:
        print(json.dumps(run_attention(a.attention, max(1, a.iters))), flush=True)
        return
    import camelid_b200 as cm
    from camelid_b200._lib import check

    sel = {"direct": 1, "mma": 4, "tcgen05": 32}.get(a.kernel, 0)
    check(cm.lib().cmld_gemv_select_kernel(sel))
    if a.pdl:
        check(cm.lib().cmld_gemv_select_kernel(sel | 2))
    qts = [a.qt] if a.qt else sorted(BPW)
    shapes = [(a.rows, a.cols)] if a.rows and a.cols else SHAPES
    batches = [a.batch] if a.batch else [1, 4, 8]
    for qt in qts:
        for rows, cols in shapes:
            for b in batches:
                res = run_case(qt, rows, cols, b, a.iters, a.warmup)
                res["kernel"] = a.kernel
                res["pdl"] = bool(a.pdl)
                print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
