"""Recurrent mixers on `csrc/memory_scan.cu`: a gated recurrence per channel whose gates read the current token only, and two
matrix memories (exponential gates under a running maximum; the delta rule with a decay per key channel and a removal rate of
its own).  Their states live in the cache manager's slots."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import register_mixer
from .spec import VECTOR, GeneralDeltaSpec, MinGRUSpec, MLSTMSpec, WeightDecl

MODULES = ("memory_scan", "rowwise") + GEMM_MODULES


class MinGRU(Mixer):
    """One packed projection [z | u | gate] that leaves in float32 (what enters the recurrence is 32-bit arithmetic) -> one
    kernel: the gates, S_t = (1 - z) S_(t-1) + z candidate over each sequence's new tokens, times silu(gate) -> output
    projection.  State of a request: S [width] float32.  Lengths and slots are read from the step's device arrays; any step
    may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: MinGRUSpec):
        C, W = spec.width, spec.hidden_size
        decls = [WeightDecl(spec.z_proj, (C, W)), WeightDecl(spec.x_proj, (C, W)), WeightDecl(spec.gate_proj, (C, W)),
                 WeightDecl(spec.o_proj, (W, C))]
        return decls + [WeightDecl(n, (C,), VECTOR) for n in (spec.z_bias, spec.x_bias) if n]

    @staticmethod
    def kernel_modules(spec):
        return MODULES

    def __init__(self, spec: MinGRUSpec, weights, dtype, device):
        self.spec, self.dtype, self.C = spec, dtype, spec.width
        names = (spec.z_proj, spec.x_proj, spec.gate_proj)
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.b_z = weights.device_tensor(spec.z_bias, dtype, device).contiguous() if spec.z_bias else None
        self.b_x = weights.device_tensor(spec.x_bias, dtype, device).contiguous() if spec.x_bias else None

    def state_request(self) -> StateRequest:
        return StateRequest((self.C,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (self.C * (12 + elem) + self.spec.hidden_size * elem) + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T, C, ws = ctx.n_tokens, self.C, ctx.workspace
        zxg = linear(x, self.w_in, ws.buffer("mingru_in", T, 3 * C, torch.float32))
        out = ws.buffer("mingru_out", T, C, self.dtype)
        ops.min_gru(out, zxg, self.b_z, self.b_x, cache.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs)
        return linear_sliced(ws, "mingru_proj", out, self.w_o, self.dtype)


class MLSTM(Mixer):
    """One packed projection [q | k | v | gate | i | f] -> the log gates per token and head and the running maximum along each
    sequence (two launches) -> the memory's walk, which also divides by max(|n . q|, exp(-m)) + den_eps -> each head's row
    divided by its root mean square, times the gains and sigmoid(gate), one kernel -> output projection.

    State of a request, one float32 row of the cache manager's slots: [S (heads x key_dim x value_dim) | n (heads x key_dim) |
    m (heads)].  Lengths and slots are read from the step's device arrays; any step may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: MLSTMSpec):
        H, D, E, W = spec.num_heads, spec.key_dim, spec.value_dim, spec.hidden_size
        decls = [WeightDecl(spec.q_proj, (H * D, W)), WeightDecl(spec.k_proj, (H * D, W)), WeightDecl(spec.v_proj, (H * E, W)),
                 WeightDecl(spec.gate_proj, (H * E, W)), WeightDecl(spec.i_proj, (H, W)), WeightDecl(spec.f_proj, (H, W)),
                 WeightDecl(spec.o_proj, (W, H * E)), WeightDecl(spec.out_gain, (H * E,), VECTOR)]
        return decls + [WeightDecl(n, (H,), VECTOR) for n in (spec.i_bias, spec.f_bias) if n]

    @staticmethod
    def kernel_modules(spec):
        return MODULES

    def __init__(self, spec: MLSTMSpec, weights, dtype, device):
        H, D, E = spec.num_heads, spec.key_dim, spec.value_dim
        if D > 256:
            raise ValueError(f"mlstm: key width {D} exceeds 256")
        if not spec.gate_cap > 0:
            raise ValueError(f"mlstm: the gates' bound {spec.gate_cap} must be positive")
        self.spec, self.dtype = spec, dtype
        self.H, self.D, self.E = H, D, E
        names = (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.i_proj, spec.f_proj)
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.k_off, self.v_off = H * D, 2 * H * D
        self.g_off = self.v_off + H * E
        self.i_off = self.g_off + H * E
        self.f_off = self.i_off + H
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.out_gain = weights.device_tensor(spec.out_gain, dtype, device).contiguous()
        self.b_i = weights.device_tensor(spec.i_bias, dtype, device).contiguous() if spec.i_bias else None
        self.b_f = weights.device_tensor(spec.f_bias, dtype, device).contiguous() if spec.f_bias else None
        self.m_off = H * D * E + H * D

    def state_request(self) -> StateRequest:
        return StateRequest((self.m_off + self.H,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (self.w_in.shape[0] * elem + self.H * 16 + self.H * self.E * (4 + elem) + self.spec.hidden_size * elem) \
            + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T, ws = ctx.n_tokens, ctx.workspace
        H, D, E = self.H, self.D, self.E
        packed = linear(x, self.w_in, ws.buffer("mlstm_in", T, self.w_in.shape[0], self.dtype))
        q, k, v = packed[:, :self.k_off], packed[:, self.k_off:self.v_off], packed[:, self.v_off:self.g_off]
        gates = ws.buffer("mlstm_gates", T, 4 * H, torch.float32)
        scale = float(D) ** -0.5
        ops.mlstm_gates(gates, q, k, packed[:, self.i_off:self.f_off], packed[:, self.f_off:], self.b_i, self.b_f,
                        cache.state[:, self.m_off:], ctx.cu_q, ctx.state_slots, ctx.n_seqs, H, D, float(self.spec.gate_cap), scale)
        o = ws.buffer("mlstm_o", T, H * E, torch.float32)
        ops.memory_scan(o, q, k, v, None, gates, cache.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs, H, D, E, "mlstm",
                        r_scale=scale, den_eps=float(self.spec.den_eps))
        y = ws.buffer("mlstm_y", T, H * E, self.dtype)
        ops.gated_rmsnorm(y.view(T * H, E), o.view(T * H, E), packed[:, self.g_off:self.i_off], self.out_gain, float(self.spec.eps),
                          heads=H, gains_per_head=True)
        return linear_sliced(ws, "mlstm_out", y, self.w_o, self.dtype)


class GeneralDelta(Mixer):
    """One packed projection [r | k | v | gate | removal | decay's low rank] -> tanh and the decay's up-projection into float32 ->
    a pass over the tokens that makes the decays, the unit keys, the removal vectors and the tokens' own dots -> the memory's
    walk S_t = diag(w) S - (a u)(u^T S) + k v^T, o = S_t^T r -> each head's row divided by its root mean square, times the gains and
    sigmoid(gate), one kernel -> output projection.

    State of a request: S [heads, head_dim, head_dim] float32 in the cache manager's slots.  Lengths and slots are read from the
    step's device arrays; any step may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: GeneralDeltaSpec):
        H, D, W, R = spec.num_heads, spec.head_dim, spec.hidden_size, spec.decay_rank
        decls = [WeightDecl(n, (H * D, W)) for n in (spec.r_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.removal_proj)]
        decls += [WeightDecl(spec.decay_down, (R, W)), WeightDecl(spec.decay_up, (H * D, R)), WeightDecl(spec.o_proj, (W, H * D))]
        decls += [WeightDecl(n, (H * D,), VECTOR) for n in (spec.removal_bias, spec.decay_bias, spec.out_gain)]
        return decls

    @staticmethod
    def kernel_modules(spec):
        return MODULES

    def __init__(self, spec: GeneralDeltaSpec, weights, dtype, device):
        H, D = spec.num_heads, spec.head_dim
        if D > 256:
            raise ValueError(f"general delta rule: head width {D} exceeds 256")
        self.spec, self.dtype, self.H, self.D = spec, dtype, H, D
        names = (spec.r_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.removal_proj, spec.decay_down)
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.w_up = weights.device_tensor(spec.decay_up, dtype, device)
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.a_bias = weights.device_tensor(spec.removal_bias, dtype, device).contiguous()
        self.w_bias = weights.device_tensor(spec.decay_bias, dtype, device).contiguous()
        self.out_gain = weights.device_tensor(spec.out_gain, dtype, device).contiguous()

    def state_request(self) -> StateRequest:
        return StateRequest((self.H * self.D * self.D,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        hd = self.H * self.D
        return tokens * (self.w_in.shape[0] * elem + self.spec.decay_rank * elem + hd * (20 + elem) + 8 * self.H
                         + self.spec.hidden_size * elem) + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T, ws = ctx.n_tokens, ctx.workspace
        H, D, R = self.H, self.D, self.spec.decay_rank
        hd = H * D
        packed = linear(x, self.w_in, ws.buffer("gdelta_in", T, self.w_in.shape[0], self.dtype))
        r, k, v, gate, a = (packed[:, i * hd:(i + 1) * hd] for i in range(5))
        low = ws.buffer("gdelta_low", T, R, self.dtype)
        ops.act_rows(low, packed[:, 5 * hd:], "tanh")
        # the decays' up-projection leaves in float32: what follows it (sigmoid, exponential) is 32-bit arithmetic
        decay = linear(low, self.w_up, ws.buffer("gdelta_decay", T, hd, torch.float32))
        aux = ws.buffer("gdelta_aux", T, 3 * hd, torch.float32)
        dots = ws.buffer("gdelta_dots", T, 2 * H, torch.float32)
        ops.delta_rule_prep(aux, dots, r, k, a, decay, self.a_bias, self.w_bias, ctx.cu_q, ctx.n_seqs, H, D,
                            float(self.spec.decay_scale), float(self.spec.unit_eps))
        o = ws.buffer("gdelta_o", T, hd, torch.float32)
        ops.memory_scan(o, r, k, v, aux, dots, cache.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs, H, D, D, "delta")
        y = ws.buffer("gdelta_y", T, hd, self.dtype)
        ops.gated_rmsnorm(y.view(T * H, D), o.view(T * H, D), gate, self.out_gain, float(self.spec.eps), heads=H, gains_per_head=True)
        return linear_sliced(ws, "gdelta_out", y, self.w_o, self.dtype)


register_mixer("min_gru", MinGRU)
register_mixer("mlstm", MLSTM)
register_mixer("general_delta", GeneralDelta)
