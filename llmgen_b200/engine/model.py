"""A decoder assembled from a `ModelSpec`: embedding, blocks in run order, final norm on the
wanted rows, output projection.

The forward pass is a plain sequence of kernel launches on the current stream (no DAG, no
placement: one model on one GPU needs neither; the reference builds a graph and a liveness plan
for the same fixed node list, src/graph/scheduler.zig:313-317).  Only the rows whose logits
are wanted reach the final norm and the output projection; the reference norms all rows, then
gathers (src/models/qwen3.zig:321-330), which gives the same values since the norm is
row-wise.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import build as kernel_build
from ..kernels import ops
from ..parts.base import LayerCache
from ..parts.linear import linear
from ..parts.reentry import Reentry
from ..parts.registry import build_block, build_norm, model_kernel_modules
from ..parts.spec import ModelSpec
from .context import StepContext


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        # the kernels this model's parts need, and the host runtime (cache manager, scheduler) beside them
        kernel_build.ensure_built(list(model_kernel_modules(spec)) + ["runtime"])
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.embedding = weights.device_tensor(spec.embedding, dtype, device)
        self.layers = [build_block(ls, weights, dtype, device) for ls in spec.layers]
        # what a run item does to the residual stream before its layer runs (items with equal specs share one object)
        made = {}
        self.before = []
        for item in spec.run_order:
            if item.before is not None and item.before not in made:
                made[item.before] = Reentry(item.before, weights, dtype, device)
            self.before.append(made.get(item.before))
        self.embedding_norm = build_norm(spec.embedding_norm, weights, dtype, device) if spec.embedding_norm is not None else None
        self.final_norm = build_norm(spec.final_norm, weights, dtype, device)
        self.lm_head = weights.device_tensor(spec.lm_head, dtype, device)   # the embedding itself when tied
        weights.release()
        for item in spec.run_order:
            if not 0 <= item.layer < len(self.layers):
                raise ValueError(f"run list names layer {item.layer}, the model has {len(self.layers)}")
        self.bad_token_flag = ops.bad_token_flag(device)      # read by the engine with every step's results

    # -- what the engine needs to size caches and limits
    def mixers(self):
        return [getattr(layer, "mixer", None) for layer in self.layers]

    def max_positions(self) -> int:
        limit = self.spec.max_positions
        for m in self.mixers():
            mp = m.max_positions() if m is not None and hasattr(m, "max_positions") else None
            if mp is not None:
                limit = min(limit, mp)
        return limit

    def weight_bytes(self) -> int:
        """Bytes of device memory held by the model's tensors (shared storage counted once)."""
        storages: Dict[int, int] = {}
        seen = set()

        def collect(obj):
            if isinstance(obj, torch.Tensor):
                if obj.is_cuda:
                    st = obj.untyped_storage()
                    storages[st.data_ptr()] = st.nbytes()
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    collect(v)
            elif hasattr(obj, "__dict__") and id(obj) not in seen:
                seen.add(id(obj))
                for v in vars(obj).values():
                    collect(v)

        collect(self)
        return sum(storages.values())

    # -- one pass
    def hidden_states(self, ctx: StepContext, caches: List[LayerCache]):
        """Run embedding and all run items; returns (residual float32 [T, H], pending delta)."""
        T, H = ctx.n_tokens, self.spec.hidden_size
        resid = ctx.workspace.buffer("residual", T, H, torch.float32)
        rows = resid if self.embedding_norm is None else ctx.workspace.buffer("embedding_rows", T, H, torch.float32)
        ops.embed_rows(rows, self.embedding, ctx.ids, self.bad_token_flag, ids_from=ctx.ids_from, sampled=ctx.prev_sampled,
                       scale=float(self.spec.embedding_scale))
        if self.embedding_norm is not None:
            # the table's rows pass a norm before they become the residual stream (float32 in, float32 out)
            self.embedding_norm.add_norm(rows, None, resid)
        x0 = None
        if any(b is not None for b in self.before):
            # the embedding's output, for the run items that mix it back into the stream
            x0 = ctx.workspace.buffer("embedding_out", T, H, torch.float32)
            ops.widen(x0, resid)
        delta = None
        ctx.normed_for = None
        stream = resid
        n_streams = int(getattr(self.spec, "residual_streams", 0) or 0)
        if n_streams > 0:
            # layers that keep several residual streams: every stream starts as the embedding's output
            resid = ctx.workspace.buffer("residual_streams", T, n_streams * H, torch.float32)
            ops.stream_spread(resid.view(T, n_streams, H), stream)
        order = self.spec.run_order
        for n, (item, cache, before) in enumerate(zip(order, caches, self.before)):
            if before is not None:
                before.forward(ctx, resid, delta, x0)
                delta = None
            # blocks that prepare the next block's input are told which block that is (none behind a re-entry step)
            ctx.next_block = (self.layers[order[n + 1].layer] if n + 1 < len(order) and self.before[n + 1] is None else None)
            delta = self.layers[item.layer].forward(ctx, resid, delta, cache)
        ctx.next_block = None
        if n_streams > 0:
            if delta is not None:
                raise ValueError("a model with residual streams is made of blocks that finish their own sums")
            ops.stream_spread(resid.view(T, n_streams, H), stream, collapse=True)     # the stream is the sum of the streams
            resid = stream
        return resid, delta

    def logits(self, ctx: StepContext, resid: torch.Tensor, delta: Optional[torch.Tensor],
               rows: torch.Tensor, n_rows: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """float32 logits [n_rows, vocab] of the token rows listed in `rows` (int32, device)."""
        H, V = self.spec.hidden_size, self.spec.vocab_size
        ws = ctx.workspace
        normed = ws.buffer("final_normed", n_rows, H, self.dtype, capacity_rows=max(n_rows, 64))
        self.final_norm.add_norm(resid, delta, normed, rows=rows)
        if out is None:
            out = torch.empty((n_rows, V), dtype=torch.float32, device=self.device)
        out = linear(normed, self.lm_head, out)
        if self.spec.logit_cap > 0 or self.spec.logit_scale != 1.0:
            ops.logit_cap(out, float(self.spec.logit_cap), float(self.spec.logit_scale))
        return out

    def forward(self, ctx: StepContext, caches: List[LayerCache], rows: torch.Tensor, n_rows: int,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        resid, delta = self.hidden_states(ctx, caches)
        return self.logits(ctx, resid, delta, rows, n_rows, out)
