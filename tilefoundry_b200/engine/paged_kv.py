"""Paged bf16 KV cache bookkeeping (host side).

Layout follows the reference's paged fixture
(``tests/fixtures/placed/mha_decode_paged.py:46-80``): a pool viewed
``(pages, page_size, heads, dim)``; the logical cache of a sequence is
``index_select(pool, block_table)`` flattened over ``(page, slot)``.  Allocation is
deterministic -- page ``i`` of sequence ``b`` is pool page ``b * pages_per_seq + i``
-- so the table can be checked bit for bit against a host reference.
"""
from __future__ import annotations

import torch

PAGE_SIZE = 64


def pages_for(max_ctx: int, page_size: int = PAGE_SIZE) -> int:
    return (max_ctx + page_size - 1) // page_size


def block_table(batch: int, max_ctx: int, page_size: int = PAGE_SIZE, device="cpu") -> torch.Tensor:
    per = pages_for(max_ctx, page_size)
    return torch.arange(batch * per, dtype=torch.int32, device=device).reshape(batch, per)


def new_pool(batch: int, max_ctx: int, heads: int, dim: int, page_size: int = PAGE_SIZE,
             device="cuda", dtype=torch.bfloat16) -> torch.Tensor:
    return torch.zeros(batch * pages_for(max_ctx, page_size), page_size, heads, dim, device=device, dtype=dtype)


def logical_view(pool: torch.Tensor, table_row: torch.Tensor, length: int) -> torch.Tensor:
    """``[1, length, heads, dim]``: the cache as the authored functions see it."""
    pages = torch.index_select(pool, 0, table_row.to(pool.device).long())
    return pages.reshape(1, -1, pool.shape[2], pool.shape[3])[:, :length]


def fill_from_logical(pool: torch.Tensor, table_row: torch.Tensor, cache: torch.Tensor) -> None:
    """Scatter a ``[1, C, heads, dim]`` cache into the pages the table names."""
    c = cache.shape[1]
    page_size = pool.shape[1]
    n_pages = pages_for(max(c, 1), page_size)
    if c == 0:
        return
    staged = torch.zeros(n_pages * page_size, pool.shape[2], pool.shape[3], device=pool.device, dtype=pool.dtype)
    staged[:c] = cache[0].to(pool.device)
    pool[table_row[:n_pages].to(pool.device).long()] = staged.reshape(n_pages, page_size, pool.shape[2], pool.shape[3])
