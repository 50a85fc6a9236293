"""Row-sharded tensor parallelism for the projection path (one process per GPU).

The reference is single-GPU; sharding is this build's addition.  Output rows are independent, so rank r owns
rows ``[r * N / g, (r + 1) * N / g)`` of every matrix (whole rows: blocks are never split and ``row_bytes`` is
unchanged), the activations are replicated, and the partial outputs ``[m, N / g]`` of all ranks are gathered
into ``[m, N]``.  Only byte slicing and index arithmetic live here; the collective is ``torch.distributed``.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

BLOCK = {8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210), 20: (32, 18), 23: (256, 136)}  # GGML type id -> (elements, bytes)


def shard_range(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """First row and row count of ``rank``'s shard; rows must divide evenly (they do for every 27B shape at g <= 8)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    per = rows // world
    return rank * per, per


def shard_packed(packed: np.ndarray, fmt: int, rows: int, cols: int, rank: int, world: int, experts: int = 1) -> np.ndarray:
    """The GGUF bytes of ``rank``'s rows.  With stacked experts every expert's rows are sharded alike, so the
    shard is again ``experts`` stacked slices of ``rows / world`` rows."""
    el, bb = BLOCK[fmt]
    if cols % el:
        raise ValueError("row width is not a whole number of blocks")
    row_bytes = cols // el * bb
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    if packed.size != row_bytes * rows * experts:
        raise ValueError("byte length differs from geometry")
    first, per = shard_range(rows, rank, world)
    view = packed.reshape(experts, rows, row_bytes)
    return np.ascontiguousarray(view[:, first:first + per, :]).reshape(-1)


def expert_range(experts: int, rank: int, world: int) -> Tuple[int, int]:
    """First expert and expert count of ``rank`` under expert parallelism (``experts`` must divide evenly)."""
    return shard_range(experts, rank, world)


def shard_experts(packed: np.ndarray, fmt: int, rows_e: int, cols: int, experts: int, rank: int, world: int) -> np.ndarray:
    """The GGUF bytes of ``rank``'s experts of a stacked ``[experts, rows_e, cols]`` matrix: one contiguous slice
    (`expert_matrix`, src/quantization.rs:136-139)."""
    el, bb = BLOCK[fmt]
    if cols % el:
        raise ValueError("row width is not a whole number of blocks")
    per_expert = cols // el * bb * rows_e
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    if packed.size != per_expert * experts:
        raise ValueError("byte length differs from geometry")
    first, count = expert_range(experts, rank, world)
    return packed[first * per_expert:(first + count) * per_expert]


def token_owner_range(tokens: int, rank: int, world: int) -> Tuple[int, int, int]:
    """Expert parallelism at wide inputs combines every token on one rank: ``ceil(tokens / world)`` rounded up to a
    multiple of 4 tokens per rank, contiguous.  Returns (tokens per rank, first token of ``rank``, its token count)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    per = ((tokens + world - 1) // world + 3) // 4 * 4
    first = rank * per
    return per, first, max(0, min(per, tokens - first))


def token_owner(token: int, per_rank: int, world: int) -> int:
    """The rank that combines ``token``."""
    return min(token // per_rank, world - 1)


def gathered_to_rows(gathered, m: int, rows: int, world: int):
    """``all_gather_into_tensor`` concatenates rank outputs ``[world][m][rows / world]``; the projection's
    output is ``[m][rows]``.  Works on torch tensors and numpy arrays (a view plus one transposing copy)."""
    per = rows // world
    g = gathered.reshape(world, m, per)
    if hasattr(g, "permute"):
        return g.permute(1, 0, 2).reshape(m, rows)
    return g.transpose(1, 0, 2).reshape(m, rows)
