"""Which part of each tensor a rank of a sharded engine holds.

Camelid itself has no tensor or expert parallelism (its multi-node mode is a two-stage TCP
pipeline, src/distributed.rs in the Camelid tree), so the split is this library's own:

* dense model, ``tp_size`` ranks: q/k/v/gate/up by rows (q and k/v by whole kv groups, so a query
  head and its kv head share a rank), o/down by columns on 256-value boundaries, the output
  matrix by vocabulary rows; token embeddings, norms and the residual stream are replicated.
  Each sublayer ends in one all-reduce(sum) of ``[rows][hidden]`` f32; greedy argmax is one
  all-reduce(max) of a packed (value, index) key per row.
* Mixtral-shaped model, ``ep_size`` ranks: attention and router replicated, expert ``e`` on rank
  ``e % ep_size``; one all-reduce(sum) per MoE layer.

Everything here is plain integer logic (no device), so it is tested on CPU.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, replace

PROJ_NAMES = ("q", "k", "v", "o", "gate", "up", "down")


@dataclass(frozen=True)
class Slice:
    """Rows ``(first_block + j*block_step) * block_rows + [0, block_rows)`` for ``j < n_blocks``,
    columns ``[col0, col0 + n_cols)`` of a ``rows x cols`` matrix."""
    block_rows: int
    first_block: int
    block_step: int
    n_blocks: int
    col0: int
    n_cols: int

    @property
    def rows(self) -> int:
        return self.block_rows * self.n_blocks

    @property
    def contiguous_rows(self) -> bool:
        return self.n_blocks == 1 or self.block_step == 1

    @property
    def row0(self) -> int:
        return self.first_block * self.block_rows

    def row_index(self):
        import numpy as np
        blocks = self.first_block + np.arange(self.n_blocks) * self.block_step
        return (blocks[:, None] * self.block_rows + np.arange(self.block_rows)[None, :]).reshape(-1)

    def take(self, full):
        """The slice of a numpy matrix (used by CPU tests as the statement of what the device copy does)."""
        return full[self.row_index()][:, self.col0:self.col0 + self.n_cols]


def _rows(rows: int, cols: int, rank: int, size: int) -> Slice:
    if rows % size:
        raise ValueError(f"{rows} rows do not split over {size} ranks")
    return Slice(rows // size, rank, 1, 1, 0, cols)


def _cols(rows: int, cols: int, rank: int, size: int, quantum: int = 256) -> Slice:
    if cols % (size * quantum):
        raise ValueError(f"{cols} columns do not split over {size} ranks in multiples of {quantum}")
    return Slice(rows, 0, 1, 1, rank * (cols // size), cols // size)


def check_tp(cfg, size: int):
    if cfg.n_experts > 0:
        raise ValueError("a Mixtral-shaped model shards by experts, not tensor-parallel")
    if cfg.n_kv_heads % size or cfg.vocab % size or cfg.ffn_dim % (size * 256) or (cfg.n_heads // size * cfg.head_dim) % 256:
        raise ValueError(f"tp_size {size} does not divide this model")


def tp_slices(cfg, rank: int, size: int) -> dict:
    """role -> Slice for a dense model; roles are q,k,v,o,gate,up,down,output."""
    check_tp(cfg, size)
    qw, kvw = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    return {
        "q": _rows(qw, cfg.hidden, rank, size), "k": _rows(kvw, cfg.hidden, rank, size), "v": _rows(kvw, cfg.hidden, rank, size),
        "o": _cols(cfg.hidden, qw, rank, size),
        "gate": _rows(cfg.ffn_dim, cfg.hidden, rank, size), "up": _rows(cfg.ffn_dim, cfg.hidden, rank, size),
        "down": _cols(cfg.hidden, cfg.ffn_dim, rank, size),
        "output": _rows(cfg.vocab, cfg.hidden, rank, size),
    }


def ep_experts(rank: int, size: int, n_experts: int) -> list[int]:
    if n_experts % size:
        raise ValueError(f"{n_experts} experts do not split over {size} ranks")
    return list(range(rank, n_experts, size))


def ep_slices(cfg, rank: int, size: int) -> dict:
    """role -> Slice of the stacked expert slabs ([n_experts * rows_per_expert][cols])."""
    n_local = len(ep_experts(rank, size, cfg.n_experts))
    return {
        "gate_exps": Slice(cfg.ffn_dim, rank, size, n_local, 0, cfg.hidden),
        "up_exps": Slice(cfg.ffn_dim, rank, size, n_local, 0, cfg.hidden),
        "down_exps": Slice(cfg.hidden, rank, size, n_local, 0, cfg.ffn_dim),
    }


def rank_config(cfg, rank: int, size: int):
    """The EngineConfig rank ``rank`` of ``size`` passes to the engine (global dimensions plus its shard)."""
    if size <= 1:
        return cfg
    if cfg.n_experts > 0:
        ep_experts(rank, size, cfg.n_experts)
        return replace(cfg, ep_rank=rank, ep_size=size)
    check_tp(cfg, size)
    return replace(cfg, tp_rank=rank, tp_size=size)


def pack_argmax_key(value: float, index: int) -> int:
    """The 64-bit key whose unsigned maximum over shards is the greedy token: order-preserving bits
    of the f32 value above, the inverted global index below (so equal values keep the lowest index,
    as the reference's strict ``>`` scan does)."""
    (u,) = struct.unpack("<I", struct.pack("<f", value))
    u = (~u & 0xFFFFFFFF) if u & 0x80000000 else (u | 0x80000000)
    return (u << 32) | (0xFFFFFFFF - index)


def unpack_argmax_index(key: int) -> int:
    return 0xFFFFFFFF - (key & 0xFFFFFFFF)
