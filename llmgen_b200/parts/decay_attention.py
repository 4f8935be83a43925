"""Linear attention with a decay per head and key channel that each token decides: two recurrent mixers whose state
lives in the cache manager's slots, both on the recurrence kernel `decay_scan` (csrc/recurrent.cu)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import norm_class, register_mixer
from .spec import VECTOR, ChannelDecayAttentionSpec, TokenShiftDecaySpec, WeightDecl


def _scan_buffers(ws, T: int, H: int, D: int, E: int):
    """The recurrence kernel's scratch: a float32 row [q | k | v] per token, two numbers per token and head, and the
    states of the segments in which long sequences are walked."""
    return (ws.buffer("decay_scan_qkv", T, 2 * H * D + H * E, torch.float32),
            ws.buffer("decay_scan_dots", T, 2 * H, torch.float32),
            ws.flat("decay_scan_segments", ops.decay_scan_segment_floats(H, D, E), torch.float32))


class ChannelDecayAttention(Mixer):
    """One packed projection [q | k | v | gate | decay's low rank] -> the decay's up-projection into float32 -> the
    recurrence S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over each sequence's new tokens with
    a = sigmoid(z + b)^(1 / tau) (the preparation pass leaves 1 - a and scales q; both float32) -> RMSNorm of each
    head's output times silu(gate), one kernel -> output projection.

    State of a request: S [heads, key_dim, value_dim] float32 in the cache manager's slots.  Lengths and slots are read
    from the step's device arrays; any step may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: ChannelDecayAttentionSpec):
        H, D, E, W, R = spec.num_heads, spec.key_dim, spec.value_dim, spec.hidden_size, spec.decay_rank
        return [WeightDecl(spec.q_proj, (H * D, W)), WeightDecl(spec.k_proj, (H * D, W)), WeightDecl(spec.v_proj, (H * E, W)),
                WeightDecl(spec.gate_proj, (H * E, W)), WeightDecl(spec.o_proj, (W, H * E)), WeightDecl(spec.decay_down, (R, W)),
                WeightDecl(spec.decay_up, (H * D, R)), WeightDecl(spec.decay_bias, (H * D,), VECTOR)] \
            + norm_class(spec.out_norm).weight_decls(spec.out_norm)

    @staticmethod
    def kernel_modules(spec):
        return ("recurrent", "rowwise") + GEMM_MODULES

    def __init__(self, spec: ChannelDecayAttentionSpec, weights, dtype, device):
        H, D, E = spec.num_heads, spec.key_dim, spec.value_dim
        if D > 256:
            raise ValueError(f"channel-decay attention: key width {D} exceeds 256")
        if not spec.tau > 0:
            raise ValueError(f"channel-decay attention: tau {spec.tau} must be positive")
        if spec.out_norm.kind != "rmsnorm" or spec.out_norm.dim != E or spec.out_norm.weight_offset != 0.0:
            raise ValueError("channel-decay attention: the output norm is a plain RMSNorm over a head's values")
        self.spec, self.dtype = spec, dtype
        self.H, self.D, self.E = H, D, E
        names = (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.decay_down)
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.k_off, self.v_off = H * D, 2 * H * D
        self.g_off = self.v_off + H * E
        self.a_off = self.g_off + H * E
        self.w_decay = weights.device_tensor(spec.decay_up, dtype, device)
        self.decay_bias = weights.device_tensor(spec.decay_bias, dtype, device).contiguous()
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.norm_gain = weights.device_tensor(spec.out_norm.weight, dtype, device)
        self.norm_eps = float(spec.out_norm.eps)

    def state_request(self) -> StateRequest:
        return StateRequest((self.H * self.D * self.E,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        hd, he = self.H * self.D, self.H * self.E
        return tokens * (self.w_in.shape[0] * elem + (3 * hd + 2 * he + 2 * self.H) * 4 + he * elem + self.spec.hidden_size * elem) \
            + ops.SLICED_PRODUCT_BYTES + 4 * ops.decay_scan_segment_floats(self.H, self.D, self.E)

    def forward(self, ctx, x, cache: LayerCache):
        T, ws = ctx.n_tokens, ctx.workspace
        H, D, E = self.H, self.D, self.E
        packed = linear(x, self.w_in, ws.buffer("cda_in", T, self.w_in.shape[0], self.dtype))
        # the decays' up-projection leaves in float32: what follows it (sigmoid, logarithm, power) is 32-bit arithmetic
        decay = linear(packed[:, self.a_off:], self.w_decay, ws.buffer("cda_decay", T, H * D, torch.float32))
        o = ws.buffer("cda_o", T, H * E, torch.float32)
        qkv_buf, dots, segments = _scan_buffers(ws, T, H, D, E)
        ops.decay_scan(o, packed[:, :self.k_off], packed[:, self.k_off:self.v_off], packed[:, self.v_off:self.g_off], decay,
                       self.decay_bias, None, cache.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs, H, D, E, "sigmoid_pow",
                       float(self.spec.tau), float(D) ** -0.5, False, qkv_buf, dots, segments)
        # one gain vector for all heads: every (token, head) is a row of the norm; the gate's rows lie in the packed product
        y = ws.buffer("cda_y", T, H * E, self.dtype)
        ops.gated_rmsnorm(y.view(T * H, E), o.view(T * H, E), packed[:, self.g_off:self.a_off], self.norm_gain, self.norm_eps,
                          gate_form="silu", heads=H)
        return linear_sliced(ws, "cda_out", y, self.w_o, self.dtype)


class TokenShiftDecay(Mixer):
    """`token_shift_mix` makes the five blends of every token with the one before it (the step's first token of a
    sequence reads the request's state) -> r, k, v, gate and the decay's low rank, one product each, each on its own
    blend -> tanh and the decay's up-projection into float32 -> the recurrence
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_(t-1) + k_t v_t^T with w = exp(-exp(z + w0)) -> each head's
    o divided by its root mean square, times the gains of its head and silu(gate), one kernel -> output projection.

    State of a request, one float32 row of the cache manager's slots: [S (heads x head_dim x head_dim) | the last input
    row].  Lengths and slots are read from the step's device arrays; any step may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: TokenShiftDecaySpec):
        H, D, W, R = spec.num_heads, spec.head_dim, spec.hidden_size, spec.decay_rank
        decls = [WeightDecl(n, (W,), VECTOR) for n in spec.mix]
        decls += [WeightDecl(n, (H * D, W)) for n in (spec.r_proj, spec.k_proj, spec.v_proj, spec.gate_proj)]
        decls += [WeightDecl(spec.decay_down, (R, W)), WeightDecl(spec.decay_up, (H * D, R)), WeightDecl(spec.decay_bias, (H * D,), VECTOR),
                  WeightDecl(spec.bonus, (H, D), VECTOR), WeightDecl(spec.out_gain, (H * D,), VECTOR), WeightDecl(spec.o_proj, (W, H * D))]
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("recurrent", "rowwise") + GEMM_MODULES

    def __init__(self, spec: TokenShiftDecaySpec, weights, dtype, device):
        H, D = spec.num_heads, spec.head_dim
        if D > 256:
            raise ValueError(f"token-shift mixer: head width {D} exceeds 256")
        if len(spec.mix) != 5:
            raise ValueError("token-shift mixer: five blends (r, k, v, gate, decay)")
        self.spec, self.dtype = spec, dtype
        self.H, self.D = H, D
        self.mu = torch.stack([weights.device_tensor(n, dtype, device, keep=False) for n in spec.mix]).contiguous()   # float32 [5, W]
        self.w_r, self.w_k, self.w_v, self.w_g = (weights.device_tensor(n, dtype, device)
                                                  for n in (spec.r_proj, spec.k_proj, spec.v_proj, spec.gate_proj))
        self.w_down = weights.device_tensor(spec.decay_down, dtype, device)
        self.w_up = weights.device_tensor(spec.decay_up, dtype, device)
        self.decay_bias = weights.device_tensor(spec.decay_bias, dtype, device).contiguous()
        self.bonus = weights.device_tensor(spec.bonus, dtype, device).contiguous()
        self.out_gain = weights.device_tensor(spec.out_gain, dtype, device).contiguous()
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.s_size = H * D * D

    def state_request(self) -> StateRequest:
        return StateRequest((self.s_size + self.spec.hidden_size,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        hd, W = self.H * self.D, self.spec.hidden_size
        return tokens * ((5 * W + 5 * hd + 2 * self.spec.decay_rank + W) * elem + (5 * hd + 2 * self.H) * 4) + ops.SLICED_PRODUCT_BYTES \
            + 4 * ops.decay_scan_segment_floats(self.H, self.D, self.D)

    def forward(self, ctx, x, cache: LayerCache):
        T, ws = ctx.n_tokens, ctx.workspace
        H, D, W, R = self.H, self.D, self.spec.hidden_size, self.spec.decay_rank
        mixed = ws.flat("tsd_mixed", 5 * ws.default_rows * W, self.dtype)[:5 * T * W].view(5, T, W)
        ops.token_shift_mix(mixed, x, self.mu, cache.state[:, self.s_size:], ctx.cu_q, ctx.state_slots, ctx.n_seqs)
        r = linear(mixed[0], self.w_r, ws.buffer("tsd_r", T, H * D, self.dtype))
        k = linear(mixed[1], self.w_k, ws.buffer("tsd_k", T, H * D, self.dtype))
        v = linear(mixed[2], self.w_v, ws.buffer("tsd_v", T, H * D, self.dtype))
        gate = linear(mixed[3], self.w_g, ws.buffer("tsd_gate", T, H * D, self.dtype))
        low = linear_sliced(ws, "tsd_low", mixed[4], self.w_down, self.dtype)
        low_act = ws.buffer("tsd_low_act", T, R, self.dtype)
        ops.act_rows(low_act, low, "tanh")
        # the decays' up-projection leaves in float32: what follows it (two exponentials) is 32-bit arithmetic
        decay = linear(low_act, self.w_up, ws.buffer("tsd_decay", T, H * D, torch.float32))
        o = ws.buffer("tsd_o", T, H * D, torch.float32)
        qkv_buf, dots, segments = _scan_buffers(ws, T, H, D, D)
        ops.decay_scan(o, r, k, v, decay, self.decay_bias, self.bonus, cache.state, ctx.cu_q, ctx.state_slots, ctx.n_seqs, H, D, D,
                       "exp_exp", 1.0, 1.0, True, qkv_buf, dots, segments)
        y = ws.buffer("tsd_y", T, H * D, self.dtype)
        ops.gated_rmsnorm(y.view(T * H, D), o.view(T * H, D), gate, self.out_gain, float(self.spec.eps), gate_form="silu", heads=H,
                          gains_per_head=True)
        return linear_sliced(ws, "tsd_out", y, self.w_o, self.dtype)


register_mixer("channel_decay_attention", ChannelDecayAttention)
register_mixer("token_shift_decay", TokenShiftDecay)
