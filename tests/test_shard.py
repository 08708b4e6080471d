"""Host-side sharding logic, on CPU: which rows/columns a rank holds, that the ranks' partial
results add up to the unsharded result, and the packed argmax key; the exchange itself runs as
two gloo ranks."""
import os
import socket
import struct

import numpy as np
import pytest

from camelid_b200 import shard, synth


def _cfg(shape="llama-8b", **kw):
    return synth.engine_config(shape, max_pos=64, **kw)


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_tp_slices_tile_every_matrix(size):
    cfg = _cfg()
    shapes = dict(synth.proj_shapes(cfg), output=(cfg.vocab, cfg.hidden))
    for role, (rows, cols) in shapes.items():
        seen = np.zeros((rows, cols // 256), np.int32)  # at 256-column granularity
        for r in range(size):
            sl = shard.tp_slices(cfg, r, size)[role]
            assert sl.col0 % 256 == 0 and sl.n_cols % 256 == 0
            seen[np.ix_(sl.row_index(), np.arange(sl.col0 // 256, (sl.col0 + sl.n_cols) // 256))] += 1
        assert (seen == 1).all(), role


def test_tp_keeps_query_heads_with_their_kv_head():
    cfg = _cfg()
    g = cfg.n_heads // cfg.n_kv_heads
    for size in (2, 4, 8):
        for r in range(size):
            s = shard.tp_slices(cfg, r, size)
            q_heads = set(s["q"].row_index() // cfg.head_dim)
            kv_heads = set(s["k"].row_index() // cfg.head_dim)
            assert {h // g for h in q_heads} == kv_heads
            assert set(s["v"].row_index() // cfg.head_dim) == kv_heads


def test_tp_rejects_shapes_that_do_not_split():
    with pytest.raises(ValueError):
        shard.tp_slices(_cfg(), 0, 3)
    with pytest.raises(ValueError):
        shard.tp_slices(_cfg("llama-3b"), 0, 16)
    with pytest.raises(ValueError):
        shard.tp_slices(_cfg("mixtral-8x7b"), 0, 2)


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_ep_experts_partition(size):
    got = sorted(e for r in range(size) for e in shard.ep_experts(r, size, 8))
    assert got == list(range(8))
    cfg = _cfg("mixtral-8x7b")
    for r in range(size):
        sl = shard.ep_slices(cfg, r, size)["gate_exps"]
        experts = sorted(set(sl.row_index() // cfg.ffn_dim))
        assert experts == shard.ep_experts(r, size, 8)


def test_rank_config_marks_the_right_axis():
    assert shard.rank_config(_cfg(), 3, 4).tp_size == 4 and shard.rank_config(_cfg(), 3, 4).tp_rank == 3
    c = shard.rank_config(_cfg("mixtral-8x7b"), 1, 2)
    assert (c.ep_rank, c.ep_size, c.tp_size) == (1, 2, 1)
    assert shard.rank_config(_cfg(), 0, 1) == _cfg()


def test_argmax_key_orders_like_strict_greater_scan():
    rng = np.random.default_rng(5)
    vals = rng.normal(size=4096).astype(np.float32)
    vals[100] = vals[3000] = vals.max() + 1  # a tie: the lower index must win
    vals[7] = -np.inf
    keys = [shard.pack_argmax_key(float(v), i) for i, v in enumerate(vals)]
    assert shard.unpack_argmax_index(max(keys)) == 100 == int(np.argmax(vals))
    # monotone in the value for negatives, zeros and positives
    probe = np.array([-np.inf, -3.5, -1e-30, -0.0, 0.0, 1e-30, 2.0, np.inf], np.float32)
    k = [shard.pack_argmax_key(float(v), 0) >> 32 for v in probe]
    assert all(a <= b for a, b in zip(k, k[1:])) and k[0] < k[1] < k[2] and k[5] < k[6] < k[7]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank, world, port, shape, out_dir):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = synth.engine_config(shape, max_pos=16)
        rng = np.random.default_rng(11)  # same stream on every rank: the "replicated" tensors
        shapes = dict(synth.proj_shapes(cfg), output=(cfg.vocab, cfg.hidden))
        full = {k: rng.normal(0, 0.05, v).astype(np.float32) for k, v in shapes.items()}
        h = rng.normal(size=cfg.hidden).astype(np.float32)
        sl = shard.tp_slices(cfg, rank, world)
        w = {k: sl[k].take(full[k]) for k in full}
        # attention stand-in: per head, out = v of its kv head scaled by sum(q_head) (keeps the head pairing visible)
        hd, g = cfg.head_dim, cfg.n_heads // cfg.n_kv_heads
        q, v = w["q"] @ h, w["v"] @ h
        attn = np.concatenate([v[(i // g) * hd:(i // g + 1) * hd] * np.tanh(q[i * hd:(i + 1) * hd].sum()) for i in range(q.size // hd)])
        part = w["o"] @ attn + (h if rank == 0 else 0)  # rank 0 carries the residual
        t = torch.from_numpy(part.astype(np.float32))
        dist.all_reduce(t)
        h1 = t.numpy().copy()
        act = np.maximum(w["gate"] @ h1, 0) * (w["up"] @ h1)
        part = w["down"] @ act + (h1 if rank == 0 else 0)
        t = torch.from_numpy(part.astype(np.float32))
        dist.all_reduce(t)
        h2 = t.numpy().copy()
        logits = w["output"] @ h2
        i = int(np.argmax(logits))
        key = shard.pack_argmax_key(float(logits[i]), i + sl["output"].row0)
        kt = torch.tensor([key - (1 << 63)], dtype=torch.int64)  # gloo has no u64: shift keeps the order
        dist.all_reduce(kt, op=dist.ReduceOp.MAX)
        token = shard.unpack_argmax_index(int(kt.item()) + (1 << 63))
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), h2=h2, token=token)
        if rank == 0:
            # unsharded statement of the same sublayers
            q, v = full["q"] @ h, full["v"] @ h
            attn = np.concatenate([v[(i // g) * hd:(i // g + 1) * hd] * np.tanh(q[i * hd:(i + 1) * hd].sum()) for i in range(cfg.n_heads)])
            r1 = full["o"] @ attn + h
            r2 = full["down"] @ (np.maximum(full["gate"] @ r1, 0) * (full["up"] @ r1)) + r1
            np.savez(os.path.join(out_dir, "full.npz"), h2=r2, token=int(np.argmax(full["output"] @ r2)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_gloo_ranks_reproduce_the_unsharded_layer(tmp_path, world):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_gloo_rank, args=(world, port, "tiny-tp", str(tmp_path)), nprocs=world, join=True)
    full = np.load(tmp_path / "full.npz")
    for r in range(world):
        got = np.load(tmp_path / f"r{r}.npz")
        np.testing.assert_allclose(got["h2"], full["h2"], rtol=2e-5, atol=2e-5)
        assert int(got["token"]) == int(full["token"])
    a, b = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    assert np.array_equal(a["h2"], b["h2"])  # every rank ends with the very same residual stream
