"""Tile and path choices of the inference plan.

Two kinds of tables live here.  The reference's own policy tables, which its callers import
and its tests pin value for value (``lightmoe/inference.py:26-50``): they are restated because
the numbers are part of the drop-in surface, not because this build's kernels follow them.  And
the choices this build's kernels are actually launched with, which come from measurements on
B200 (``pick_tiles``).
"""

from __future__ import annotations

import math

DECODE_ROWS_PER_EXPERT = 16  # a step with at most this many rows per expert on average is a decode step
FAST_DECODE_ROWS = 64
FUSED_PREPARE_MAX_ROWS = 1024  # dispatch + quantize in one launch up to this many routes
# Decode steps of up to this many routes run on the decode-shaped GEMM (weights on the 128-row
# side of the MMA, work dealt in quarter blocks); larger ones on 128 x 256 tiles.  Measured on
# hidden 6144 / intermediate 2048 / 256 experts / top-8: 8 tokens 205 vs 220 us, 32 tokens 542 vs
# 523 us, 64 tokens 739 vs 710 us: once every SM has several whole tiles, the wide tile streams
# the weights a little faster, and the balance the decode-shaped kernel buys no longer matters.
SWAPPED_MAX_ROWS = 128


# ---- the reference's tables (pinned by tests/test_imports.py:36-40, tests/test_inference.py:310-323)
def _use_swapped_fc2(tokens: int) -> bool:
    return tokens <= 8


def _decode_tile_rows(tokens: int, hidden: int, intermediate: int, experts: int) -> int:
    wide = hidden >= 4096 and intermediate >= 2048 and experts >= 48
    if wide and tokens >= 64:
        return 32
    if wide and tokens >= 16:
        return 16
    return 8


def _tile_m(token_expert_assignments: int, experts: int, hidden: int, intermediate: int):
    dense_rows = token_expert_assignments >= 256 * experts
    first = 256 if dense_rows else 128
    second = 256 if (dense_rows and hidden > 2048 and intermediate > 1024) else 128
    return first, second


# ---- what this build launches
def expected_padded_rows(mean_rows: float, tile: int) -> float:
    """Rows an expert occupies once padded to whole ``tile``-row tiles, averaged over a
    per-expert row count drawn from N(mean, mean) (uniform routing)."""
    sigma = max(math.sqrt(mean_rows), 1.0)

    def below(v: float) -> float:
        return 0.5 * (1.0 + math.erf((v - mean_rows) / (sigma * math.sqrt(2.0))))

    lowest = max(0, int((mean_rows - 5.0 * sigma) // tile))
    highest = int((mean_rows + 5.0 * sigma) // tile) + 1
    return sum((below((t + 1) * tile) - below(t * tile)) * (t + 1) * tile for t in range(lowest, highest + 1))


def pick_tiles(rows: int, experts: int, n: int, k: int, *, nvfp4_out: bool) -> tuple[int, int]:
    """(tile_m, tile_n) of a prefill GEMM with ``rows`` rows over ``experts`` experts.

    128 x 256 tiles pull a quarter less data into the SM per FLOP than 128 x 128 tiles and
    were 1.25x to 1.7x faster on every prefill shape measured (K from 512 to 4096), so the wide
    tile is taken whenever N is two or more whole 128-column blocks (with an odd count the last
    tile is half empty: N = 1920 as 7.5 wide tiles ran 1.9x faster than as 15 narrow ones).  256 x 256 tiles on CTA pairs move another 30 %
    fewer bytes through each SM's shared memory and issue half as many MMAs: about 1.25x
    faster per padded row on a first projection with K >= 4096, about 1.1x elsewhere -- but they
    pad every expert to 256 rows, so they are taken only when that padding costs less than the
    pair wins (with about 256 rows per expert the taller tile pads 20 % more and loses; with
    192, or with 512 and more, it wins).
    """
    if n % 128 or n < 256:
        return 128, 128
    if rows < 128 * experts:
        return 128, 256
    mean_rows = rows / experts
    gain = 1.22 if (nvfp4_out and k >= 4096) else 1.10
    pays = expected_padded_rows(mean_rows, 256) <= gain * expected_padded_rows(mean_rows, 128)
    return (256 if pays else 128), 256


__all__ = ["DECODE_ROWS_PER_EXPERT", "FAST_DECODE_ROWS", "FUSED_PREPARE_MAX_ROWS", "SWAPPED_MAX_ROWS",
           "expected_padded_rows",
           "pick_tiles"]
