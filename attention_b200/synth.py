"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five benchmark
configurations (C1..C5).  No dataset is involved: everything is a pure function of a seed.

  C1  FlashAttention fwd FP32 non-causal  B=2 S=512   H=8  D=64,  N(0,1)
  C2  FlashAttention fwd BF16 causal      B=4 S=4096  H=32 D=128, N(0,1)*0.5
  C3  paged decode FP16  batch 64  H=32 D=128 page 16, context ~ U[512, 8192], pages dealt from a
      seeded random permutation
  C4  FlashAttention fwd BF16 causal      B=1 S=32768 H=16 D=128, N(0,1)
  C5  paged decode FP16  batch 256 H=32 D=128 page 16, context ~ logU[1024, 32768], ~10 % of the
      logical page references shared between sequences (groups of 4 share a prefix)
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np

SEED_BASE = 1000


@dataclasses.dataclass(frozen=True)
class FaConfig:
    name: str
    batch: int
    seq: int
    heads: int
    head_dim: int
    dtype: str          # "f32" | "f16" | "bf16"
    causal: bool
    input_scale: float
    seed: int

    @property
    def flops(self) -> float:
        """Algorithmic FLOPs: 4*B*H*S^2*D, halved when causal (softmax excluded)."""
        f = 4.0 * self.batch * self.heads * self.seq * self.seq * self.head_dim
        return f / 2 if self.causal else f


@dataclasses.dataclass(frozen=True)
class DecodeConfig:
    name: str
    batch: int
    heads: int
    head_dim: int
    page_size: int
    dtype: str
    ctx_lo: int
    ctx_hi: int
    log_uniform: bool
    share_fraction: float   # target fraction of logical page references that are shared
    seed: int


C1 = FaConfig("C1", 2, 512, 8, 64, "f32", False, 1.0, SEED_BASE + 0)
C2 = FaConfig("C2", 4, 4096, 32, 128, "bf16", True, 0.5, SEED_BASE + 1)
C3 = DecodeConfig("C3", 64, 32, 128, 16, "f16", 512, 8192, False, 0.0, SEED_BASE + 2)
C4 = FaConfig("C4", 1, 32768, 16, 128, "bf16", True, 1.0, SEED_BASE + 3)
C5 = DecodeConfig("C5", 256, 32, 128, 16, "f16", 1024, 32768, True, 0.10, SEED_BASE + 4)


def context_lengths(cfg: DecodeConfig, batch: int | None = None) -> np.ndarray:
    """Per-sequence context lengths: uniform integers in [lo, hi], or floor(exp(U[ln lo, ln hi]))."""
    n = cfg.batch if batch is None else batch
    rng = np.random.default_rng(cfg.seed)
    u = rng.random(n)
    if cfg.log_uniform:
        ctx = np.floor(np.exp(math.log(cfg.ctx_lo) + u * math.log(cfg.ctx_hi / cfg.ctx_lo))).astype(np.int64)
    else:
        ctx = cfg.ctx_lo + np.floor(u * (cfg.ctx_hi - cfg.ctx_lo + 1)).astype(np.int64)
    return np.clip(ctx, cfg.ctx_lo, cfg.ctx_hi).astype(np.int32)


def page_permutation(num_pages: int, seed: int) -> np.ndarray:
    """Seeded Fisher-Yates permutation of [0, num_pages): the initial order of the free ring, so
    that pages dealt to sequences in order are scattered over the pool."""
    return np.random.default_rng(seed + 7919).permutation(num_pages).astype(np.int32)


@dataclasses.dataclass
class SharingPlan:
    """Which prefix each sequence shares.  Sequences come in groups of `group`; the first member
    of a group owns the prefix, the others fork it."""
    ctx: np.ndarray              # [batch] tokens per sequence
    group_leader: np.ndarray     # [batch] index of the sequence whose prefix is shared (itself for leaders)
    prefix_tokens: np.ndarray    # [batch] tokens shared with the leader (0 for leaders)
    logical_pages: int
    shared_refs: int             # logical page references that point at a page owned by another sequence

    @property
    def unique_pages(self) -> int:
        return self.logical_pages - self.shared_refs

    @property
    def shared_fraction(self) -> float:
        return self.shared_refs / max(1, self.logical_pages)


def sharing_plan(cfg: DecodeConfig, batch: int | None = None, group: int = 4) -> SharingPlan:
    """Groups of `group` consecutive sequences share a page-aligned prefix of the group's leader.
    The prefix length is the same fraction of the shortest member of every group, chosen so that
    shared references are about cfg.share_fraction of all logical page references."""
    ctx = context_lengths(cfg, batch)
    n = len(ctx)
    ps = cfg.page_size
    pages = (ctx.astype(np.int64) + ps - 1) // ps
    logical = int(pages.sum())
    leader = np.arange(n)
    prefix = np.zeros(n, dtype=np.int32)
    if cfg.share_fraction > 0:
        lo, hi = 0.0, 1.0
        for _ in range(40):                     # bisection on the prefix fraction
            frac = 0.5 * (lo + hi)
            refs = 0
            for g0 in range(0, n, group):
                members = range(g0, min(n, g0 + group))
                p = int(min(ctx[m] for m in members) * frac) // ps
                refs += p * (len(members) - 1)
            if refs / logical < cfg.share_fraction:
                lo = frac
            else:
                hi = frac
        frac = 0.5 * (lo + hi)
        for g0 in range(0, n, group):
            members = list(range(g0, min(n, g0 + group)))
            p = int(min(ctx[m] for m in members) * frac) // ps
            for m in members[1:]:
                leader[m] = g0
                prefix[m] = p * ps
    shared = int((prefix.astype(np.int64) // ps).sum())
    return SharingPlan(ctx, leader, prefix, logical, shared)


def kv_bytes_per_token(cfg: DecodeConfig) -> int:
    """K and V of one token slot over all heads, in the pool's storage type."""
    es = 4 if cfg.dtype == "f32" else 2
    return 2 * cfg.heads * cfg.head_dim * es


def decode_algorithmic_bytes(cfg: DecodeConfig, plan: SharingPlan) -> dict:
    """Bytes one decode step must move: unique KV token slots + Q + O + block table + lengths."""
    per_tok = kv_bytes_per_token(cfg)
    logical_tokens = int(plan.ctx.astype(np.int64).sum())
    shared_tokens = int(plan.prefix_tokens.astype(np.int64).sum())
    es = 4 if cfg.dtype == "f32" else 2
    n = len(plan.ctx)
    qo = 2 * n * cfg.heads * cfg.head_dim * es
    tables = plan.logical_pages * 4 + n * 4
    return {
        "kv_logical": logical_tokens * per_tok,
        "kv_unique": (logical_tokens - shared_tokens) * per_tok,
        "qo": qo,
        "tables": tables,
        "total_unique": (logical_tokens - shared_tokens) * per_tok + qo + tables,
        "total_logical": logical_tokens * per_tok + qo + tables,
    }
