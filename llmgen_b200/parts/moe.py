"""Feed-forwards of layers other than the gated dense one: a dense one without a gate, and a mixture of experts."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import register_feed_forward
from .spec import VECTOR, ClampedExpertSpec, DenseMLPSpec, GatedExpertSpec, GatedMLPSpec, RoutedMLPSpec, WeightDecl


class DenseMLP(FeedForward):
    """down( act(x Wup^T) ), act = relu(.)^2 or the tanh form of gelu: two products and one row-wise kernel between them, which also adds up the
    float32 slices when the first product was cut along K."""

    @staticmethod
    def weight_decls(spec: DenseMLPSpec):
        return [WeightDecl(spec.up_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.down_proj, (spec.hidden_size, spec.intermediate_size))]

    @staticmethod
    def kernel_modules(spec):
        return ("rowwise",) + GEMM_MODULES

    def __init__(self, spec: DenseMLPSpec, weights, dtype, device):
        if spec.activation not in ("relu2", "gelu_tanh"):
            raise ValueError(f"dense feed-forward: activation {spec.activation!r} is not supported")
        self.spec, self.dtype = spec, dtype
        self.w_up = weights.device_tensor(spec.up_proj, dtype, device)
        self.w_down = weights.device_tensor(spec.down_proj, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (2 * self.spec.intermediate_size + self.spec.hidden_size) * elem + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x):
        T, F = x.shape[0], self.spec.intermediate_size
        ws = ctx.workspace
        up = linear_sliced(ws, "ffn_up", x, self.w_up, self.dtype)
        act = ws.buffer("ffn_act", T, F, self.dtype)
        ops.act_rows(act, up, self.spec.activation)
        return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype)


def _expert_form(e):
    """(activation of `act_rows`, alpha, limit, plain gated unit?) of an expert's spec."""
    if isinstance(e, GatedExpertSpec):
        if e.activation != "silu":
            raise ValueError(f"routed feed-forward: expert activation {e.activation!r} is not supported")
        return "silu_glu", 1.0, 0.0, True
    return "clamped_glu", float(e.alpha), float(e.limit), False


def _expert_decls(e, hidden: int):
    return [WeightDecl(e.gate_proj, (e.intermediate_size, hidden)), WeightDecl(e.up_proj, (e.intermediate_size, hidden)),
            WeightDecl(e.down_proj, (hidden, e.intermediate_size))]


class RoutedMLP(FeedForward):
    """Mixture of experts whose every launch has a shape that follows from (tokens, experts, top) alone: no result is
    read back on the host, so a step holding it is recorded into a CUDA graph like any other.

    `moe_route` scores each token in float32 against the float32 router and keeps its `top` experts; `moe_plan` groups
    the (token, choice) slots by expert into tiles (a list of fixed length, padded); `moe_combine` adds a token's rows
    in slot order to the shared expert's output.  The experts' matrices are stacked [experts, ...] at load.  Between
    plan and sum:

      bfloat16   tiles of 128 rows, every expert's rows starting on a tile: `moe_gather` copies the rows (times their
                 weights, where the weight is on the expert's input; else `moe_combine` applies it) into that order, and the grouped tensor-core product (`gemm_tc_grouped`: TMA, tcgen05.mma,
                 the expert of each tile read from the device) runs gate/up of all experts in one launch, the clamped
                 gated activation follows row-wise, and a second grouped launch runs down
      float32    (and operands TMA refuses) tiles of 16 rows through `moe_experts`, float32 sums on the CUDA cores

    The shared expert is two of the framework's own products with the same activation between them; a plain
    silu-gated one is the dense gated feed-forward's first half (`GatedMLP.hidden`: the activation in the product's
    epilogue) and one more product."""

    step_arrays_follow_shapes = True

    @staticmethod
    def weight_decls(spec: RoutedMLPSpec):
        decls = [WeightDecl(spec.router, (len(spec.experts), spec.hidden_size))]
        if spec.router_bias:
            decls.append(WeightDecl(spec.router_bias, (len(spec.experts),), VECTOR))
        for e in spec.experts:
            decls += _expert_decls(e, spec.hidden_size)
        if spec.shared is not None:
            decls += _expert_decls(spec.shared, spec.hidden_size)
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("moe", "rowwise", "elementwise") + GEMM_MODULES

    def __init__(self, spec: RoutedMLPSpec, weights, dtype, device):
        first = spec.experts[0]
        if any((type(e), e.intermediate_size, _expert_form(e)) != (type(first), first.intermediate_size, _expert_form(first))
               for e in spec.experts):
            raise ValueError("routed feed-forward: all routed experts share one kind, size and constants")
        if not 0 < spec.top_k <= len(spec.experts):
            raise ValueError(f"routed feed-forward: top {spec.top_k} of {len(spec.experts)} experts")
        if spec.scoring not in ops.ROUTER_SCORINGS:
            raise ValueError(f"routed feed-forward: scoring {spec.scoring!r} is not supported")
        self.spec, self.dtype = spec, dtype
        self.E, self.top, self.F = len(spec.experts), spec.top_k, first.intermediate_size
        self.router = weights.device_tensor(spec.router, torch.float32, device)      # routing is float32 in both dtypes
        self.router_bias = weights.device_tensor(spec.router_bias, dtype, device).contiguous() if spec.router_bias else None
        self.act, self.alpha, self.limit, self.plain = _expert_form(first)
        self.shared_form = _expert_form(spec.shared) if spec.shared is not None else None
        stack = lambda names: torch.stack([weights.device_tensor(n, dtype, device, keep=False) for n in names]).contiguous()
        self.w_gate = stack([e.gate_proj for e in spec.experts])     # [E, F, H]
        self.w_up = stack([e.up_proj for e in spec.experts])         # [E, F, H]
        self.w_down = stack([e.down_proj for e in spec.experts])     # [E, H, F]
        # the tensor-core path reads gate and up as one matrix per expert, [E, 2F, H]: gate rows, then up rows
        H = spec.hidden_size
        self.grouped = dtype == torch.bfloat16 and H % 8 == 0 and self.F % 8 == 0
        if self.grouped:
            self.w_gate_up = torch.cat([self.w_gate, self.w_up], dim=1).contiguous()
            self.w_gate = self.w_up = None
        self.shared_gate_up = self.shared_down = self.shared_mlp = None
        if isinstance(spec.shared, GatedExpertSpec):
            from .mlp import GatedMLP
            sh = spec.shared
            self.shared_mlp = GatedMLP(GatedMLPSpec(H, sh.intermediate_size, sh.gate_proj, sh.up_proj, sh.down_proj, sh.activation),
                                       weights, dtype, device)
        elif spec.shared is not None:
            self.shared_gate_up = torch.cat([weights.device_tensor(spec.shared.gate_proj, dtype, device, keep=False),
                                             weights.device_tensor(spec.shared.up_proj, dtype, device, keep=False)], dim=0).contiguous()
            self.shared_down = weights.device_tensor(spec.shared.down_proj, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        H = self.spec.hidden_size
        slots = tokens * self.top
        shared = tokens * (3 * self.spec.shared.intermediate_size + H) * elem if self.spec.shared is not None else 0
        if self.shared_mlp is not None:
            shared += self.shared_mlp.workspace_bytes(tokens)
        rows = slots + ops.MOE_GROUPED_TILE * min(self.E, slots) if self.grouped else slots
        return rows * (3 * self.F + 2 * H) * 4 + tokens * H * 4 + shared + 16 * (rows + self.E) + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x):
        T, H = x.shape
        ws = ctx.workspace
        spec, top = self.spec, self.top
        n_slots = T * top
        tile = ops.MOE_GROUPED_TILE if self.grouped else 0
        tiles = ops.moe_max_tiles(n_slots, self.E, tile)
        n_rows = tiles * tile if self.grouped else n_slots          # rows of the sorted (and, grouped, padded) order
        ints = ws.flat("moe_ints", 2 * n_slots + n_rows + 3 * tiles, torch.int32)
        slot_expert, pos_of_slot, order = ints[:n_slots], ints[n_slots:2 * n_slots], ints[2 * n_slots:2 * n_slots + n_rows]
        tile_expert, tile_start, tile_rows = (ints[2 * n_slots + n_rows + i * tiles:2 * n_slots + n_rows + (i + 1) * tiles] for i in range(3))
        slot_weight = ws.flat("moe_weights", n_slots, torch.float32)
        ops.moe_route(x, self.router, slot_expert, slot_weight, top, spec.scoring, spec.renormalize, bias=self.router_bias)
        ops.moe_plan(slot_expert, n_slots, self.E, order, pos_of_slot, tile_expert, tile_start, tile_rows, tile=tile, padded=self.grouped)
        cap = (ws.default_rows * top // 128 + self.E) * 128 if self.grouped else ws.default_rows * top
        rows = ws.buffer("moe_rows", n_rows, H, torch.float32, capacity_rows=cap)
        if self.grouped:
            xs = ws.buffer("moe_in", n_rows, H, self.dtype, capacity_rows=cap)
            ops.moe_gather(xs, x, order, slot_weight, top, scale_rows=spec.weight_on_input)
            gate_up = ws.buffer("moe_gate_up", n_rows, 2 * self.F, self.dtype, capacity_rows=cap)
            ops.gemm_tc_grouped(gate_up, xs, self.w_gate_up, tile_expert, real_rows=n_slots)
            y = ws.buffer("moe_act", n_rows, self.F, self.dtype, capacity_rows=cap)
            ops.act_rows(y, gate_up, self.act, alpha=self.alpha, limit=self.limit)
            ops.gemm_tc_grouped(rows, y, self.w_down, tile_expert, real_rows=n_slots)
        else:
            y = ws.buffer("moe_act", n_rows, self.F, torch.float32, capacity_rows=cap)
            ops.moe_experts(y, x, self.w_gate, self.w_up, order, slot_weight, tile_expert, tile_start, tile_rows, n_slots, top,
                            first=True, weight_on_input=spec.weight_on_input, alpha=self.alpha, limit=self.limit, plain=self.plain)
            ops.moe_experts(rows, y, self.w_down, None, order, slot_weight, tile_expert, tile_start, tile_rows, n_slots, top,
                            first=False, weight_on_input=spec.weight_on_input)
        shared_out = None
        if self.shared_mlp is not None:
            shared_out = linear(self.shared_mlp.hidden(ctx, x), self.shared_mlp.w_down, ws.buffer("moe_shared_out", T, H, self.dtype))
        elif spec.shared is not None:
            Fs = spec.shared.intermediate_size
            gate_up = linear_sliced(ws, "moe_shared_gate_up", x, self.shared_gate_up, self.dtype)
            act = ws.buffer("moe_shared_act", T, Fs, self.dtype)
            ops.act_rows(act, gate_up, self.shared_form[0], alpha=self.shared_form[1], limit=self.shared_form[2])
            shared_out = linear(act, self.shared_down, ws.buffer("moe_shared_out", T, H, self.dtype))
        out = ws.flat("moe_out", T * H, torch.float32).view(1, T, H)
        # the grouped products leave an expert's plain output: a weight on the output is applied as the rows are added
        ops.moe_combine(out[0], rows, pos_of_slot, shared_out, top,
                        slot_weight=slot_weight if self.grouped and not spec.weight_on_input else None)
        return ops.Partials(out)


register_feed_forward("dense_mlp", DenseMLP)
register_feed_forward("routed_mlp", RoutedMLP)
