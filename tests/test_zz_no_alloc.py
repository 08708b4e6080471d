"""The allocation-free attention entry point, for callers that cannot call cudaMalloc on their
hot path (a host whose memory pool owns the whole device, or one whose CUDA binding offers
launches and copies but no allocator).  It must return exactly what the allocating entry point
returns, call after call, although every call reuses the same fixed scratch array and finds the
previous call's bytes in it.  This file sorts last so a failure here cannot hide other tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(seed, n_heads, n_kv, hd, n_pos, max_pos):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n_heads, hd)).astype(np.float32)
    k = np.zeros((n_kv, max_pos, hd), np.float16)
    v = np.zeros((n_kv, max_pos, hd), np.float16)
    k[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    v[:, :n_pos] = rng.standard_normal((n_kv, n_pos, hd)).astype(np.float16)
    return q, k, v


def test_noalloc_attention_matches_allocating_entry_point_twice_in_a_row(cm):
    from camelid_b200._lib import check
    from camelid_b200.engine import DeviceBuffer

    # Calls in a row with different shapes.  Contexts past 2048 positions go through the fixed array (split-range
    # partials and the per-head arrival counters): the second such call finds the first one's partials and
    # counters there and must not be disturbed by them.  Then two short-context calls, which merge their
    # ranges inside a thread-block cluster and use the array for the position word only.
    for seed, (n_heads, n_kv, hd, n_pos, max_pos) in enumerate([(32, 8, 128, 2500, 4096), (24, 8, 64, 2100, 4096),
                                                                 (32, 8, 128, 1153, 2048), (24, 8, 64, 77, 2048)]):
        q, k, v = _case(seed, n_heads, n_kv, hd, n_pos, max_pos)
        qd, kd, vd = DeviceBuffer.from_numpy(q), DeviceBuffer.from_numpy(k), DeviceBuffer.from_numpy(v)
        out_a, out_b = DeviceBuffer(q.nbytes), DeviceBuffer(q.nbytes)
        scale = float(1.0 / np.sqrt(np.float32(hd)))
        check(cm.lib().cmld_attention_decode(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, n_pos, scale, out_a.ptr))
        check(cm.lib().cmld_attention_decode_noalloc(qd.ptr, kd.ptr, vd.ptr, n_heads, n_kv, hd, max_pos, n_pos, scale, out_b.ptr))
        a, b = out_a.to_numpy(np.float32), out_b.to_numpy(np.float32)
        # same kernel, same split count: the tolerance is zero
        assert np.isfinite(b).all() and np.array_equal(a, b)


def test_noalloc_attention_rejects_sizes_beyond_its_array(cm):
    from camelid_b200.engine import DeviceBuffer

    buf = DeviceBuffer(1 << 20)
    rc = cm.lib().cmld_attention_decode_noalloc(buf.ptr, buf.ptr, buf.ptr, 128, 8, 128, 2048, 10, 0.1, buf.ptr)
    assert rc == 2 and b"at most 64 query heads" in cm.lib().cmld_last_error()
