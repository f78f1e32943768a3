"""Partition of the attention path over the GPUs of one box.

A kv head and the query heads that read it form an independent group, so ranks
first divide the kv heads.  When there are more ranks than kv heads, the ranks
of one group also divide the sequence: position p of the cache lives on part
p % seq_parts of its group, every rank attends over the rows it holds, and the
partial results (output and log-sum-exp per head) are merged after the gather.
The reference has no multi-device code; this is new design on top of its
per-kv-head cache layout (src/shainet/native/cuda_kernels.cu:689-694).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class ShardPlan:
    world: int
    rank: int
    groups: int          # head groups = ranks that hold different kv heads
    seq_parts: int       # ranks per group, each holding every seq_parts-th position
    group: int           # this rank's head group
    seq_part: int        # this rank's part of the sequence within the group
    kv_begin: int
    kv_count: int
    head_begin: int
    head_count: int

    def owns_position(self, pos: int) -> bool:
        return pos % self.seq_parts == self.seq_part

    def local_rows(self, length: int) -> int:
        """How many of the positions 0..length-1 this rank holds."""
        return (length - self.seq_part + self.seq_parts - 1) // self.seq_parts if length > self.seq_part else 0


def plan(world: int, rank: int, num_heads: int, num_kv_heads: int) -> ShardPlan:
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    if num_heads % num_kv_heads:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    g = num_heads // num_kv_heads
    if world <= num_kv_heads:
        if num_kv_heads % world:
            raise ValueError(f"{world} ranks do not divide {num_kv_heads} kv heads")
        groups, seq_parts = world, 1
    else:
        if world % num_kv_heads:
            raise ValueError(f"{world} ranks are not a multiple of {num_kv_heads} kv heads")
        groups, seq_parts = num_kv_heads, world // num_kv_heads
    kv_count = num_kv_heads // groups
    group, seq_part = rank // seq_parts, rank % seq_parts
    return ShardPlan(world, rank, groups, seq_parts, group, seq_part, group * kv_count, kv_count,
                     group * kv_count * g, kv_count * g)


def merge_parts_host(outs: np.ndarray, lses: np.ndarray) -> np.ndarray:
    """Host mirror of the library's part merge: outs [parts, heads, head_dim] are the
    normalised results over disjoint row sets, lses [parts, heads] their max + ln(sum)."""
    outs = np.asarray(outs, np.float64)
    lses = np.asarray(lses, np.float64)
    mx = lses.max(axis=0, keepdims=True)
    w = np.where(np.isneginf(lses), 0.0, np.exp(lses - mx))
    return ((w[:, :, None] * outs).sum(axis=0) / w.sum(axis=0)[:, None]).astype(np.float32)
