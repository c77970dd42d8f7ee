"""A decoder put together from a :class:`~ginfer_b200.parts.plan.ModelPlan`.

The reference's forward pass (``ginfer/model/model.cc:152-166,180-228``): embedding, the layers
in order, final norm over all rows, row selection, LM head.  Here the layers run in the order of
the plan's run list, each run with the cache binding the plan names for it, and the final norm
is computed only at the rows whose logits are wanted.
"""
from __future__ import annotations

import torch

from .base import StepContext, Summed, TensorSpec, make_part
from .plan import ModelPlan


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = make_part("embedding", plan.embedding)
        self.blocks = [make_part("block", ls.block, layer_spec=ls) for ls in plan.layers]
        self.final_norm = make_part("norm", plan.final_norm)
        self.head = make_part("head", plan.head)
        self.dtype: torch.dtype | None = None
        self.device: torch.device | None = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> list[TensorSpec]:
        """Every tensor of the model under its full name."""
        out = list(self.embedding.tensor_specs())
        for ls, blk in zip(self.plan.layers, self.blocks):
            pre = ls.prefix + "." if ls.prefix else ""
            out += [TensorSpec(pre + s.name, s.shape, s.role, s.int_high)
                    for s in blk.tensor_specs()]
        out += self.final_norm.tensor_specs()
        out += self.head.tensor_specs()
        names = [s.name for s in out]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"the plan names these tensors more than once: {dup}")
        return out

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        self.embedding.load(tensors, dtype, device)
        for ls, blk in zip(self.plan.layers, self.blocks):
            pre = ls.prefix + "." if ls.prefix else ""
            local = {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}
            blk.load(local, dtype, device)
        self.final_norm.load(tensors, dtype, device)
        self.head.load(tensors, dtype, device)

    # ------------------------------------------------------------------ caches
    def cache_specs(self) -> dict[int, object]:
        """Cache id -> spec, taken from the layer whose run writes that cache."""
        out: dict[int, object] = {}
        for e in self.plan.run:
            if e.write_cache:
                out[e.cache] = self.blocks[e.layer].mixer.cache_spec()
        for e in self.plan.run:
            if not e.write_cache:
                mine = self.blocks[e.layer].mixer.cache_spec()
                if mine != out[e.cache]:
                    raise ValueError(f"layer {e.layer} cannot read cache {e.cache}: it holds "
                                     f"{out[e.cache]} but the layer expects {mine}")
        return out

    # ------------------------------------------------------------------ one step
    def forward(self, ctx: StepContext, bind_cache) -> torch.Tensor:
        """Run the step's tokens; ``bind_cache(run_entry)`` gives the cache binding of a run.
        Returns fp32 logits ``[R, vocab]`` at ``ctx.logit_rows``."""
        delta = None
        x = self.embedding.forward(ctx.token_ids, ctx)
        run = self.plan.run
        for i, e in enumerate(run):
            blk = self.blocks[e.layer]
            if blk.takes_next_norm and i + 1 < len(run):
                # the block may prepare the input of the norm that the next run starts with
                x, delta = blk.forward(x, delta, ctx, bind_cache(e),
                                       then=self.blocks[run[i + 1].layer].first_norm())
            else:
                x, delta = blk.forward(x, delta, ctx, bind_cache(e))
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=ctx.device)
        if isinstance(x, Summed):
            _, n = self.final_norm.forward(x.tensor, None, rows=ctx.logit_rows, want_sum=False,
                                           out_dtype=ctx.dtype)
        else:
            _, n = self.final_norm.forward(x, delta, rows=ctx.logit_rows, want_sum=False)
        return self.head.forward(n, ctx)
