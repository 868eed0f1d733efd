"""A decoder put together from a `ModelSpec`: embedding, the layers' blocks in the spec's run order,
final norm and head.  The class knows no architecture; which parts run and with which sizes is the
spec's business, and which tensors they get is decided by name.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..parts import registry
from ..parts.context import BuildContext
from ..parts.linear import Linear
from ..parts.spec import ModelSpec
from ..parts.stream import ResidualStream


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        """`tensors` maps checkpoint names to tensors (any device) in their stored types."""
        import beglin_b200.parts  # noqa: F401
        self.spec, self.ctx = spec, ctx
        if ctx.status is None:
            ctx.status = ops.new_status(ctx.device)
        self.embed = ctx.matrix(tensors[spec.embed_name])
        self.blocks = []
        for layer in spec.layers:
            parts = {}
            for slot, _, cls, pspec in registry.layer_slots(layer):
                mine = {}
                for role in cls.expected_tensors(pspec):
                    name = layer.names[f"{slot}.{role.name}"]
                    if name in tensors:
                        mine[role.name] = tensors[name]
                parts[slot] = cls(pspec, mine, ctx)
            self.blocks.append(registry.block_class(layer.block)(**parts))
        self.final_norm = registry.norm_class(spec.final_norm.kind)(
            spec.final_norm, {"weight": tensors[spec.final_norm_name]}, ctx)
        head_bias = None if spec.head_bias_name is None else tensors[spec.head_bias_name]
        if spec.head_name is None:
            self.head = Linear(self.embed, head_bias, ctx, label="head_gemv")     # ctx.matrix is a no-op on the table: one copy
        else:
            self.head = Linear(tensors[spec.head_name], head_bias, ctx, label="head_gemv")

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[Optional[object]]:
        """The cache need of every stage of the run order (None for a stage that reads another's)."""
        needs = []
        for stage in self.spec.order:
            need = None
            if stage.cache is None:
                for _, family, cls, pspec in registry.layer_slots(self.spec.layers[stage.layer]):
                    if family == "mixer":
                        need = cls.cache_need(pspec)
            needs.append(need)
        return needs

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (the tied head counted once)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        def walk(obj, depth=0):
            if isinstance(obj, torch.Tensor):
                add(obj)
            elif depth < 3 and hasattr(obj, "__dict__"):
                for k, v in vars(obj).items():
                    if k in ("ctx", "spec", "bias_c", "embed"):
                        continue
                    walk(v, depth + 1)

        for b in self.blocks:
            for part in vars(b).values():
                walk(part)
        walk(self.final_norm)
        walk(self.head)
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        """Run the batch's rows through every stage, from and into `cache`; return float logits
        [wanted rows, vocab], or None when no row's logits are wanted (the head is skipped then, as
        qwen_infer.c:2145 skips it)."""
        x = torch.empty((batch.n_rows, self.spec.hidden), dtype=torch.float32, device=self.ctx.device)
        ops.embed_gather(self.embed, batch.token_ids, x, self.ctx.status, scale=self.spec.embed_scale)
        stream = ResidualStream(x)
        for si, stage in enumerate(self.spec.order):
            owner = si if stage.cache is None else stage.cache
            view = cache.view(owner, batch) if owner in cache.stage_group else None
            self.blocks[stage.layer].forward(stream, batch, view)
        if batch.n_logit_rows == 0:
            return None
        h = self.final_norm.add_norm(stream.x, stream.pending, rows=batch.logit_rows, update=False)
        logits = self.head(h, out_dtype=torch.float32)
        if self.spec.logit_softcap > 0.0:
            ops.softcap(logits, self.spec.logit_softcap)
        return logits
