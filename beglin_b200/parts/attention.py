"""Grouped-query attention over the paged cache (the reference's attention, qwen_infer.c:1451-1548
for one token and :2075-2136 for a ragged batch).

Per step: one product for q, k and v together (the reference concatenates the three matrices and
their biases at load time too, qwen_infer.c:1316-1367), rotation of q and k fused with the append
of k and v to the pages, attention of every row over the pages of its own request, and the output
product.  All rows' keys and values are in the cache before any row's attention runs
(qwen_infer.c:2017-2023), which is what makes a prompt portion causal.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..csrc import ops
from .cache_need import PagedKVNeed, PagedKVView
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .rope import shared_position
from .spec import AttentionSpec, TensorRole
from .stream import ResidualStream


@register_mixer("gqa_attention")
class GQAAttention:
    @staticmethod
    def expected_tensors(spec: AttentionSpec) -> List[TensorRole]:
        qd, kvd = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        roles = [TensorRole("q_proj.weight", (qd, spec.hidden), True, True),
                 TensorRole("o_proj.weight", (spec.hidden, qd), True, True)]
        if spec.own_kv:
            roles += [TensorRole("k_proj.weight", (kvd, spec.hidden), True, True),
                      TensorRole("v_proj.weight", (kvd, spec.hidden), True, True)]
        if spec.qkv_bias:
            roles.append(TensorRole("q_proj.bias", (qd,), role="bias"))
            if spec.own_kv:
                roles += [TensorRole("k_proj.bias", (kvd,), role="bias"), TensorRole("v_proj.bias", (kvd,), role="bias")]
        if spec.out_bias:
            roles.append(TensorRole("o_proj.bias", (spec.hidden,), role="bias"))
        return roles

    @staticmethod
    def cache_need(spec: AttentionSpec) -> Optional[PagedKVNeed]:
        if not spec.own_kv:
            return None
        return PagedKVNeed(spec.n_kv_heads, spec.head_dim, spec.window)

    def __init__(self, spec: AttentionSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} kv heads")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim={spec.head_dim} must be even and at most 256")
        self.spec, self.ctx = spec, ctx
        self.nh, self.nkv, self.hd = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.qd, self.kvd = self.nh * self.hd, self.nkv * self.hd
        names = ["q_proj"] + (["k_proj", "v_proj"] if spec.own_kv else [])
        w = torch.cat([tensors[n + ".weight"] for n in names], dim=0)
        b = torch.cat([tensors[n + ".bias"].float() for n in names], dim=0) if spec.qkv_bias else None
        self.qkv = Linear(w, b, ctx, label="proj_qkv")
        self.o_proj = Linear(tensors["o_proj.weight"], tensors.get("o_proj.bias") if spec.out_bias else None, ctx,
                             label="proj_o")
        self.position = shared_position(spec.position, ctx)
        scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.hd))
        self.scale = float(np.float32(scale))
        self.plans = {d: ops.attention_plan(self.nh // self.nkv, self.hd, ctx.cache_dtype, d, ctx.attention,
                                            ctx.page_size) for d in (False, True)}
        self.window = int(spec.window) if spec.window else 0
        # the fused q/k/v product can rotate and append itself: whole heads rotated in halves, a cache of its own
        # in bfloat16
        self.rope_in_product = (spec.own_kv and self.position.rotary_dim == self.hd and not self.position.interleaved
                                and ctx.compute_dtype == torch.bfloat16 and ctx.cache_dtype == torch.bfloat16)

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: PagedKVView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to
        it) and None is returned; without, the addend is returned."""
        T = batch.n_rows
        if self.rope_in_product and self.qkv.rope_fuses(T, self.hd):
            # a step of few tokens: rotation and cache append inside the q/k/v product
            q = torch.empty((T, self.qd), dtype=self.ctx.compute_dtype, device=self.ctx.device)
            self.qkv.of_rope(h, q, (self.position.table(batch), batch.positions, batch.row_req, cache.block_table,
                                    cache.pool, cache.page_size, self.nh, self.nkv, self.hd))
        else:
            qkv = self.qkv.of(h)
            q = torch.empty((T, self.qd), dtype=self.ctx.compute_dtype, device=qkv.device)
            ops.rope_kv_append(qkv, q, T, self.nh, self.nkv, self.hd, self.position.rotary_dim, self.position.interleaved,
                               self.position.table(batch), batch.positions, batch.row_req, cache.block_table,
                               cache.pool if self.spec.own_kv else None, cache.page_size, self.ctx.status)
        kernel, bq, tile = self.plans[bool(getattr(batch, "decode_only", False))]
        qblk, n_qblk = batch.query_blocks(bq)
        if qblk is None and kernel != "mma_keys":
            batch.implicit_blocks = False              # this kernel wants the list
            qblk, n_qblk = batch.query_blocks(bq)
        out = torch.empty((T, self.qd), dtype=self.ctx.compute_dtype, device=q.device)
        ops.attention(q, q.stride(0), cache.pool, cache.block_table, batch.positions, qblk, n_qblk,
                      batch.max_position, T, self.nh, self.nkv, self.hd, self.window, self.ctx.kv_split, tile, bq,
                      self.scale, out, self.ctx.status, kernel)
        if stream is None:
            return self.o_proj.partial(out)
        self.o_proj.into(out, stream)
        return None
