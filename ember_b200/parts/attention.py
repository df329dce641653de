"""Grouped-query causal attention over a paged key/value cache.

Order of operations (src/backend/cpu/cpu_backend.cpp:141-200): fused q/k/v projection (+bias),
per-head RMSNorm of q and k, rotation of q and k, write of k and v to the request's pages,
attention of every new token over keys 0..pos (or the last ``window`` keys), output projection
added to the residual stream.  Sizes and constants come from ``AttentionSpec``.

Device layout of the weights is this part's own: q, k and v rows are concatenated into one
[q_dim + 2 kv_dim, hidden] matrix so the projection is one product.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .linear import Linear
from .registry import build_part, register_part


def plan_decode_splits(n_tokens: int, max_context: int, window: int, num_kv_heads: int, head_dim: int, sms: int,
                       cluster_splits: int, merge_kernel_us: float, cache_bytes_per_us: float):
    """How the key ranges of a decode step's single-token tiles are cut: ``(n_splits, split_keys, in_cluster)``.

    Splits are fixed ranges of ``split_keys`` keys (a multiple of 64) anchored at key 0 that cover ``max_context``;
    the number of *live* ones (those a window leaves non-empty) is chosen by a model of the kernel's time: the bytes
    of cache over the device's rate, stretched by idle SMs (blocks = tokens x key heads x splits against ``sms``)
    and by 4 % per further split.  ``in_cluster``: the splits of a tile are a thread-block cluster that merges in
    shared memory (at most ``cluster_splits``; 0 forbids it), chosen when the best such plan is estimated no slower
    than the best plan of up to 16 splits plus what the merge kernel costs."""
    live = max_context if window <= 0 else min(max_context, window + 64)
    blocks = max(1, n_tokens * num_kv_heads)
    stream_us = n_tokens * live * num_kv_heads * head_dim * 4 / cache_bytes_per_us         # keys and values, bf16

    def plan(most):
        splits, best = 1, None
        for cand in range(1, max(1, min(most, (live + 255) // 256)) + 1):
            cost = max(1.0, sms / float(blocks * cand)) * (1.0 + 0.04 * (cand - 1))
            if best is None or cost < best - 1e-9:
                splits, best = cand, cost
        return splits, best * stream_us

    live_splits, est = plan(16)
    in_cluster = False
    if cluster_splits > 1 and max_context <= live:          # (with a window the early splits are empty: too many)
        c_splits, c_est = plan(cluster_splits)
        if c_est <= est + merge_kernel_us:
            live_splits, in_cluster = c_splits, True
    split_keys = ((live + live_splits - 1) // live_splits + 63) // 64 * 64
    n_splits = (max_context + split_keys - 1) // split_keys
    return n_splits, split_keys, in_cluster and 1 < n_splits <= cluster_splits


class Attention(Mixer):
    graph_safe = True

    # keys per split and the most tokens in a step for which long key ranges are split
    SPLIT_KEYS = 256
    SPLIT_MAX_TOKENS = 256

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} heads do not divide into {s.num_kv_heads} key/value heads")
        if s.head_dim <= 0 or s.head_dim % 2 or s.head_dim > 256:
            raise ConfigError(f"head_dim {s.head_dim} must be even and at most 256")
        if s.window < 0:
            raise ConfigError("window must be >= 0")
        if s.group > ops.ATTENTION_MAX_GROUP:
            # refused when the model is built, not at its first step: the general attention kernel (the whole
            # float32 path, and bfloat16 geometries the tensor-core kernels do not take) holds one tile row per
            # query head of a group
            raise ConfigError(f"{s.group} query heads per key/value head: the attention kernels take at most "
                              f"{ops.ATTENTION_MAX_GROUP}")
        self.position = build_part("position", s.position)
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(s.head_dim)

    # ------------------------------------------------------------------ weights
    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        d = [WeightDecl(p + "q_proj.weight", (s.q_dim, s.hidden_size)),
             WeightDecl(p + "k_proj.weight", (s.kv_dim, s.hidden_size)),
             WeightDecl(p + "v_proj.weight", (s.kv_dim, s.hidden_size)),
             WeightDecl(p + "o_proj.weight", (s.hidden_size, s.q_dim))]
        if s.qk_norm:
            d += [WeightDecl(p + "q_norm.weight", (s.head_dim,), init="norm"),
                  WeightDecl(p + "k_norm.weight", (s.head_dim,), init="norm")]
        if s.bias:
            d += [WeightDecl(p + "q_proj.bias", (s.q_dim,), init="zeros"),
                  WeightDecl(p + "k_proj.bias", (s.kv_dim,), init="zeros"),
                  WeightDecl(p + "v_proj.bias", (s.kv_dim,), init="zeros")]
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        if any(v is None for v in got.values()):
            return  # the store reports what is missing
        q, k, v = (got[p + n + "_proj.weight"] for n in "qkv")
        wd = rt.weight_dtype(torch.result_type(q, k))
        qkv = torch.cat([rt.to_device(t, wd) for t in (q, k, v)], dim=0)
        bias = None
        if s.bias:
            bias = torch.cat([got[p + n + "_proj.bias"].float() for n in "qkv"]).to(rt.device)
        self.qkv = Linear(qkv, bias)
        self.o = Linear.from_host(got[p + "o_proj.weight"], rt)
        self.q_norm_w = rt.to_device(got[p + "q_norm.weight"], torch.float32) if s.qk_norm else None
        self.k_norm_w = rt.to_device(got[p + "k_norm.weight"], torch.float32) if s.qk_norm else None
        self.inv_freq, self.rotary = self.position.rotary_table(rt)

    # -------------------------------------------------------------------- cache
    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="window" if s.window > 0 else "full", num_kv_heads=s.num_kv_heads,
                         head_dim=s.head_dim, window=s.window)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, cache, owns_cache: bool = True) -> None:
        s, rt = self.spec, self.rt
        T, mt = ctx.T, ctx.max_tokens
        qkv = ctx.buf("attention.qkv", (mt, s.q_dim + 2 * s.kv_dim), rt.dtype)
        q = ctx.buf("attention.q", (mt, s.q_dim), rt.dtype)
        att = ctx.buf("attention.out", (mt, s.q_dim), rt.dtype)
        table = ctx.block_table(cache.group)
        rotates = self.inv_freq is not None and self.rotary > 0
        if (self.FUSE_QKV and (T >= ops.QKV_FUSE_MIN_TOKENS or T <= ops.QKV_FUSE_MAX_DECODE_TOKENS) and
                ops.gemm_tc_qkv_usable(x, self.qkv.weight, self.qkv.bias, T, s.num_heads, s.num_kv_heads, s.head_dim,
                                       self.rotary if rotates else 0)):
            # norm, rotation and the cache write happen in the product's epilogue: a prompt portion rotates with
            # the step's angle table, a decode step of a few tokens computes its angles itself
            cos_sin = self.position.cos_sin(ctx, rt) if rotates and T > 16 else None
            ops.gemm_tc_qkv(x, self.qkv.weight, T, s.num_heads, s.num_kv_heads, self.q_norm_w, self.k_norm_w,
                            s.qk_norm_eps, cos_sin, self.inv_freq if rotates and T <= 16 else None, ctx.positions,
                            ctx.seq_of, table, cache.page_tokens, cache.k, cache.v, q, write_kv=owns_cache, err=ctx.err,
                            stream=ctx.stream)
        elif (self.SUMS_TO_HEADS and 16 < T <= 128 and ops.gemm_tc_usable(x, self.qkv.weight, self.qkv.bias, ops.EPI_STORE)
              and ops.qk_norm_rope_store_sums_usable(s.head_dim, self.rotary if rotates else 0, self.qkv.n)):
            # 17 to 128 tokens: the product cuts K and adds its parts into a zeroed fp32 scratch; the head kernel
            # reads the sums there (and clears them) instead of a bf16 copy that a pass of its own would have to make
            sums = ops.gemm_tc(x, self.qkv.weight, None, T, ops.EPI_SUMS, err=ctx.err, stream=ctx.stream)
            ops.qk_norm_rope_store_sums(sums, T, s.num_heads, s.num_kv_heads, self.q_norm_w, self.k_norm_w, s.qk_norm_eps,
                                        self.inv_freq if rotates else None, ctx.positions, ctx.seq_of, table,
                                        cache.page_tokens, cache.k, cache.v, q, write_kv=owns_cache, err=ctx.err,
                                        stream=ctx.stream)
        else:
            self.qkv(ctx, x, qkv, T, ops.EPI_STORE)
            ops.qk_norm_rope_store(qkv, T, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm_w, self.k_norm_w,
                                   s.qk_norm_eps, self.inv_freq, self.rotary, ctx.positions, ctx.seq_of, table,
                                   cache.page_tokens, cache.k, cache.v, q, write_kv=owns_cache, err=ctx.err,
                                   stream=ctx.stream)
        self.attend(ctx, q, cache, table, att)
        self.o(ctx, att, residual, T, ops.EPI_ADD_F32)

    FUSE_QKV = True     # prompt portions: finish the heads in the epilogue of the q/k/v product
    SUMS_TO_HEADS = True     # 17 to 128 tokens: the head kernel reads the product's fp32 sums (tests switch it off)
    CLUSTER_MERGE = True            # tests switch it off to compare with the merge kernel
    MERGE_KERNEL_US = 3.0           # what the merge kernel costs a decode step per layer beyond the attention kernel
    CACHE_BYTES_PER_US = 6.4e6      # the rate at which the decode kernel streams the cache when the SMs are full

    def _tc_modes(self):
        """(prompt portions, single tokens): whether the tensor-core kernels take this geometry."""
        s, rt = self.spec, self.rt
        if rt.dtype != torch.bfloat16:
            return False, False
        return (ops.attention_tc_supported(s.head_dim, s.group, rt.page_tokens, 0),
                ops.attention_tc_supported(s.head_dim, s.group, rt.page_tokens, 1))

    def _fa(self) -> bool:
        """Whether prompt portions go to the tcgen05 kernel (needs the single-token kernel beside it)."""
        s, rt = self.spec, self.rt
        return (rt.dtype == torch.bfloat16 and ops.attention_fa_supported(s.head_dim, s.group, rt.page_tokens)
                and self._tc_modes()[1])

    def tile_requests(self):
        s = self.spec
        multi, single = self._tc_modes()
        if self._fa():
            return [(ops.attention_fa_tile_queries(s.group), "multi"), (1, "single")]
        if multi:
            tq = ops.attention_tc_tile_queries(s.group)
            return [(tq, "multi"), (1, "single")] if single else [(tq, "all")]
        return [(ops.attention_tile_queries(s.group), "all")]

    def attend(self, ctx, q: torch.Tensor, cache, table: torch.Tensor, out: torch.Tensor) -> None:
        """out[t, h, :] = softmax over the visible keys of (q . k * scale) times v."""
        s = self.spec
        multi, single = self._tc_modes()
        if multi and ops.TC_ENABLED:
            tq = ops.attention_tc_tile_queries(s.group)
            args = (s.num_heads, s.num_kv_heads, s.head_dim)
            if not single:
                tiles, n = ctx.attention_tiles(tq, "all")
                ops.attention_tc(q, cache.k, cache.v, out, 0, *args, tiles, n, table, cache.page_tokens, s.window,
                                 self.scale, err=ctx.err, stream=ctx.stream)
                return
            if self._fa():
                tiles, n = ctx.attention_tiles(ops.attention_fa_tile_queries(s.group), "multi")
                if n:
                    ops.attention_fa(q, cache.k, cache.v, out, *args, tiles, n, table, cache.page_tokens, s.window,
                                     self.scale, err=ctx.err, stream=ctx.stream)
            else:
                tiles, n = ctx.attention_tiles(tq, "multi")
                if n:
                    ops.attention_tc(q, cache.k, cache.v, out, 0, *args, tiles, n, table, cache.page_tokens, s.window,
                                     self.scale, err=ctx.err, stream=ctx.stream)
            tiles, n = ctx.attention_tiles(1, "single")
            if n:
                # Cut long key ranges only as far as it takes to keep the memory system busy: the kernel streams the
                # cache at the device's rate once about one block per SM is in flight, and every further split costs
                # (partial results written and read, the merge kernel).  Measured at 16/8 heads, context 3,200, us a
                # layer with 1 / 2 / 4 splits: 64 requests 122 / 130 / 134, 24 requests 52 / 60 / 58, 16 requests
                # 40 / 37 / 41, 8 requests - / 22.6 / 22.5, one request 19 (2) / 12.8 (4) / 10.1 (8).  Splits are
                # anchored at key 0, so with a window the early ones are empty.
                # Up to 8 splits of a tile can be a thread-block cluster that merges in shared memory; more go
                # through buffers and the merge kernel, which costs a step about MERGE_KERNEL_US a layer (batch 8,
                # 3 splits: 1.895 -> 1.805 ms a step; one request at 3,072: 12 splits through buffers 1.351 ms, 8 in a
                # cluster 1.305 ms; at 32,768 the 16 splits through buffers win, 28.5 against 42.9 us a layer).
                n_splits, split_keys, in_cluster = plan_decode_splits(
                    n, ctx.max_context, s.window, s.num_kv_heads, s.head_dim, ops.num_sms(q.device),
                    ops.ATTENTION_CLUSTER_SPLITS if self.CLUSTER_MERGE else 0, self.MERGE_KERNEL_US, self.CACHE_BYTES_PER_US)
                part_o = part_ml = None
                if n_splits > 1 and not in_cluster:
                    part_o = ctx.buf_dyn("attention.part_o", n * s.num_heads * n_splits * s.head_dim, torch.float32)
                    part_ml = ctx.buf_dyn("attention.part_ml", n * s.num_heads * n_splits * 2, torch.float32)
                ops.attention_tc(q, cache.k, cache.v, out, 1, *args, tiles, n, table, cache.page_tokens, s.window,
                                 self.scale, n_splits, split_keys, part_o, part_ml, err=ctx.err, stream=ctx.stream)
            return
        tile_q = ops.attention_tile_queries(s.group)
        tiles, n_tiles = ctx.attention_tiles(tile_q, "all")
        # long key ranges of a small step are cut into fixed splits so that more SMs share them
        span = ctx.max_context if s.window <= 0 else min(ctx.max_context, s.window + tile_q)
        n_splits, part_o, part_ml = 1, None, None
        if ctx.T <= self.SPLIT_MAX_TOKENS and span > 2 * self.SPLIT_KEYS:
            n_splits = (ctx.max_context + self.SPLIT_KEYS - 1) // self.SPLIT_KEYS
            part_o = ctx.buf_dyn("attention.part_o", ctx.T * s.num_heads * n_splits * s.head_dim, torch.float32)
            part_ml = ctx.buf_dyn("attention.part_ml", ctx.T * s.num_heads * n_splits * 2, torch.float32)
        ops.attention(q, cache.k, cache.v, out, ctx.T, s.num_heads, s.num_kv_heads, s.head_dim, tiles, n_tiles,
                      tile_q, table, cache.page_tokens, s.window, self.scale, n_splits, self.SPLIT_KEYS,
                      part_o, part_ml, err=ctx.err, stream=ctx.stream)


register_part("mixer", "attention", Attention)
