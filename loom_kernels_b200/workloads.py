"""Seeded synthetic inputs with the shapes of the benchmark configurations.

The reference measures on no public dataset: its inputs are seeded synthetic fixtures, and so
are these (N(0,1) values rounded to BF16, scattered page tables drawn from a shuffled pool).
Everything is generated with numpy's PCG64 from the given seed, so the same call reproduces the
same bytes on any machine; device copies are made by the caller.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

HEAD_DIM = 128
PAGE_SIZE = 16


def _bf16_bits(values: np.ndarray) -> np.ndarray:
    """F32 -> BF16 bit patterns with round-to-nearest-even (inputs are finite)."""
    x = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((x + 0x7FFF + ((x >> 16) & 1)) >> 16).astype(np.uint16)


def normal_bf16(rng: np.random.Generator, size: int, chunk: int = 1 << 24) -> np.ndarray:
    out = np.empty(size, dtype=np.uint16)
    for start in range(0, size, chunk):
        stop = min(size, start + chunk)
        out[start:stop] = _bf16_bits(rng.standard_normal(stop - start, dtype=np.float32))
    return out


@dataclass
class DecodeWorkload:
    """One paged-decode call: spec dimensions, host inputs (BF16 bits / I32) and its bytes."""
    name: str
    batch: int
    max_pages: int
    qh: int
    kvh: int
    kv_lens: np.ndarray
    indptr: np.ndarray
    indices: np.ndarray
    last: np.ndarray
    partitions: int = 0          # 0 = plan heuristic
    query: Optional[np.ndarray] = None
    key_pages: Optional[np.ndarray] = None
    value_pages: Optional[np.ndarray] = None
    notes: dict = field(default_factory=dict)

    def algorithmic_bytes(self, partitions: int = 1) -> int:
        """KV bytes read once + Q + O + LSE + page table (+ the split-K workspace round trip)."""
        kv = int(self.kv_lens.sum()) * self.kvh * HEAD_DIM * 2 * 2
        qo = 2 * self.batch * self.qh * HEAD_DIM * 2
        lse = self.batch * self.qh * 4
        table = (len(self.indices) + 2 * self.batch + 1) * 4
        workspace = 2 * self.batch * self.qh * partitions * 130 * 4 if partitions > 1 else 0
        return kv + qo + lse + table + workspace


def page_table(rng, kv_lens, pool_pages):
    pages = (np.asarray(kv_lens, dtype=np.int64) + PAGE_SIZE - 1) // PAGE_SIZE
    total = int(pages.sum())
    if total > pool_pages:
        raise ValueError(f"{total} pages do not fit a pool of {pool_pages}")
    indices = rng.permutation(pool_pages)[:total].astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    last = ((np.asarray(kv_lens, dtype=np.int64) - 1) % PAGE_SIZE + 1).astype(np.int32)
    return indptr, indices, last


def decode_workload(name, batch, qh, kvh, kv_lens, pool_pages, seed, partitions=0,
                    with_values=True, outlier_scale=None) -> DecodeWorkload:
    rng = np.random.default_rng(seed)
    kv_lens = np.asarray(kv_lens, dtype=np.int64)
    indptr, indices, last = page_table(rng, kv_lens, pool_pages)
    w = DecodeWorkload(name, batch, pool_pages, qh, kvh, kv_lens, indptr, indices, last, partitions)
    if with_values:
        pool = pool_pages * PAGE_SIZE * kvh * HEAD_DIM
        w.query = normal_bf16(rng, batch * qh * HEAD_DIM)
        if outlier_scale is None:
            w.key_pages = normal_bf16(rng, pool)
            w.value_pages = normal_bf16(rng, pool)
        else:
            k = rng.standard_normal(pool, dtype=np.float32).reshape(pool_pages, PAGE_SIZE, -1)
            v = rng.standard_normal(pool, dtype=np.float32).reshape(pool_pages, PAGE_SIZE, -1)
            tokens = []
            for r in range(batch):
                token = int(rng.integers(0, kv_lens[r]))
                page = indices[indptr[r] + token // PAGE_SIZE]
                k[page, token % PAGE_SIZE] *= outlier_scale
                v[page, token % PAGE_SIZE] *= outlier_scale
                tokens.append(token)
            w.key_pages, w.value_pages = _bf16_bits(k.ravel()), _bf16_bits(v.ravel())
            w.notes["outlier_tokens"] = tokens
    return w


def c1(with_values=True):
    """MHA, batch 1, 32/32 heads, context 1024 (64 pages of a 256-page pool)."""
    return decode_workload("C1 paged decode MHA b1 32/32 ctx1024 pool256", 1, 32, 32, [1024],
                           256, 0xC1, with_values=with_values)


def c3(batch=64, with_values=True, seed=0xC3):
    """GQA4, batch 64, 32/8 heads, every context 4096, pages scattered in a 20000-page pool."""
    pool = 20000 * batch // 64 if batch >= 64 else max(20000 * batch // 64, batch * 256 + 64)
    return decode_workload(f"C3 paged decode GQA4 b{batch} 32/8 ctx4096 pool{pool} direct", batch,
                           32, 8, [4096] * batch, pool, seed, partitions=1,
                           with_values=with_values)


def c4(with_values=True):
    """GQA8 64/8, batch 8, context 32768, 16 K-chunks, one x8 outlier token per sequence."""
    return decode_workload("C4 paged decode GQA8 b8 64/8 ctx32768 pool20000 split16", 8, 64, 8,
                           [32768] * 8, 20000, 0xC4, partitions=16, with_values=with_values,
                           outlier_scale=8.0)


def c5_lengths(requests=512, seed=0xC5):
    rng = np.random.default_rng(seed)
    return np.floor(np.exp(rng.uniform(np.log(128.0), np.log(16384.0), size=requests))).astype(
        np.int64)


@dataclass
class AppendWorkload:
    name: str
    batch: int
    max_pages: int
    qh: int
    kvh: int
    tokens: int
    batch_indices: np.ndarray
    positions: np.ndarray
    indptr: np.ndarray
    indices: np.ndarray
    last: np.ndarray
    query: Optional[np.ndarray] = None
    key: Optional[np.ndarray] = None
    value: Optional[np.ndarray] = None
    key_pages: Optional[np.ndarray] = None
    value_pages: Optional[np.ndarray] = None

    def algorithmic_bytes(self) -> int:
        per_token = (self.qh * HEAD_DIM * 2 * 2) + (self.kvh * HEAD_DIM * 2 * 2) * 2
        metadata = (2 * self.tokens + len(self.indices) + 2 * self.batch + 1) * 4
        return self.tokens * per_token + metadata


def c2(with_values=True, seed=0xC2):
    """Fused RoPE + append: 32 requests x uniform 1-64 new tokens, 32/8 heads, prior lengths
    uniform 0-2048, shuffled 8192-page pool, positions = prior + offset, request-major order."""
    rng = np.random.default_rng(seed)
    batch, pool_pages, qh, kvh = 32, 8192, 32, 8
    new = rng.integers(1, 65, size=batch)
    prior = rng.integers(0, 2049, size=batch)
    indptr, indices, last = page_table(rng, prior + new, pool_pages)
    batch_indices = np.repeat(np.arange(batch), new).astype(np.int32)
    positions = np.concatenate([prior[r] + np.arange(new[r]) for r in range(batch)]).astype(
        np.int32)
    tokens = int(new.sum())
    w = AppendWorkload(f"C2 RoPE+append b32 32/8 tokens{tokens} pool8192", batch, pool_pages, qh,
                       kvh, tokens, batch_indices, positions, indptr, indices, last)
    if with_values:
        pool = pool_pages * PAGE_SIZE * kvh * HEAD_DIM
        w.query = normal_bf16(rng, tokens * qh * HEAD_DIM)
        w.key = normal_bf16(rng, tokens * kvh * HEAD_DIM)
        w.value = normal_bf16(rng, tokens * kvh * HEAD_DIM)
        w.key_pages = normal_bf16(rng, pool)
        w.value_pages = normal_bf16(rng, pool)
    return w


def append_small(name, new, prior, qh, kvh, pool_pages, seed=0xA9):
    """A small explicit-token append call: request r appends new[r] tokens after prior[r]."""
    rng = np.random.default_rng(seed)
    new, prior = np.asarray(new, dtype=np.int64), np.asarray(prior, dtype=np.int64)
    batch = len(new)
    indptr, indices, last = page_table(rng, prior + new, pool_pages)
    batch_indices = np.repeat(np.arange(batch), new).astype(np.int32)
    positions = np.concatenate([prior[r] + np.arange(new[r]) for r in range(batch)]).astype(
        np.int32)
    tokens = int(new.sum())
    w = AppendWorkload(name, batch, pool_pages, qh, kvh, tokens, batch_indices, positions, indptr,
                       indices, last)
    pool = pool_pages * PAGE_SIZE * kvh * HEAD_DIM
    w.query = normal_bf16(rng, tokens * qh * HEAD_DIM)
    w.key = normal_bf16(rng, tokens * kvh * HEAD_DIM)
    w.value = normal_bf16(rng, tokens * kvh * HEAD_DIM)
    w.key_pages = normal_bf16(rng, pool)
    w.value_pages = normal_bf16(rng, pool)
    return w
