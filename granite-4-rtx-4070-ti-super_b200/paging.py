"""Host side of the paged KV write: position -> pool-row tables for 16-token pages.

The device kernels only ever see integer pool rows; how pages are allocated is the
serving loop's business. These helpers restate the one rule the reference's pool uses
(``engine/src/kv_pool.cc:285-298``, ``engine/src/kv_pool.h:137-151``): logical position p of
a sequence lives in physical row ``block_table[p // B] * B + p % B`` with B tokens per page
(``engine/src/kv_pool.h:83``: 16). Pure numpy, no device work.
"""
from __future__ import annotations

import numpy as np

TOKENS_PER_PAGE = 16


def row_table(block_table, n_positions: int, tokens_per_page: int = TOKENS_PER_PAGE) -> np.ndarray:
    """Physical row of each logical position [0, n_positions) of one sequence."""
    block_table = np.asarray(block_table, dtype=np.int64)
    need = (n_positions + tokens_per_page - 1) // tokens_per_page
    if need > block_table.size:
        raise ValueError(f"{n_positions} positions need {need} pages, the sequence has "
                         f"{block_table.size}")
    p = np.arange(n_positions, dtype=np.int64)
    return (block_table[p // tokens_per_page] * tokens_per_page + p % tokens_per_page).astype(np.int32)


def validate_rows(kv_rows, pool_rows: int) -> None:
    """The reference checks a table for range and distinctness before handing it to the device
    (``engine/src/forward_gpu.cu:3570-3586``); two tokens must never share a pool row."""
    kv_rows = np.asarray(kv_rows)
    if kv_rows.size and (kv_rows.min() < 0 or kv_rows.max() >= pool_rows):
        raise ValueError("pool row out of range")
    if np.unique(kv_rows).size != kv_rows.size:
        raise ValueError("pool rows are not distinct")


def permuted_block_tables(n_sequences: int, pages_per_sequence: int, pool_pages: int, seed: int):
    """Disjoint block tables drawn from one random permutation of the pool's pages."""
    if n_sequences * pages_per_sequence > pool_pages:
        raise ValueError("pool too small")
    perm = np.random.default_rng(seed).permutation(pool_pages)
    return [perm[s * pages_per_sequence:(s + 1) * pages_per_sequence] for s in range(n_sequences)]


def batch_rows(block_tables, first_positions, tokens_per_sequence: int,
               tokens_per_page: int = TOKENS_PER_PAGE):
    """Per-row (RoPE position, pool row) arrays for a batch of sequences, sequence-major.

    Sequence s contributes tokens at RoPE positions first_positions[s] + [0, tokens_per_sequence)
    and stores token i in the page block_tables[s][i // B] at slot (first_positions[s] + i) % B
    when that stays inside the page run, i.e. its pages hold this chunk from slot 0 of the
    first page on: logical index within the chunk decides the page, as in row_table().
    """
    pos, rows = [], []
    for bt, p0 in zip(block_tables, first_positions):
        pos.append(np.arange(p0, p0 + tokens_per_sequence, dtype=np.int32))
        rows.append(row_table(bt, tokens_per_sequence, tokens_per_page))
    return np.concatenate(pos), np.concatenate(rows)
