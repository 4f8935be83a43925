"""The gated delta rule with a decay per key channel: a recurrent mixer whose state lives in the cache manager's slots."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import norm_class, register_mixer
from .spec import VECTOR, GatedDeltaSpec, WeightDecl


class GatedDelta(Mixer):
    """One packed projection [q | k | v | beta | decay's low rank | gate's low rank] -> the short convolution and silu
    of q, k, v (float32 out) -> the two low-rank up-projections (the decay's into float32) -> a pass over the tokens that
    makes q and k unit vectors, exponentiates the decays and takes beta through its sigmoid, and the recurrence over each
    sequence's new tokens (csrc/recurrent.cu: `delta_scan`, two launches) -> RMSNorm of each head's output times sigmoid(gate), one kernel ->
    output projection.

    State of a request, one float32 row of the cache manager's slots: [S (heads x key_dim x value_dim) | the
    convolution's last taps - 1 inputs over the channels of q, k, v side by side, oldest first].  Lengths and slots
    are read from the step's device arrays; any step may be replayed from the graph of its shape."""

    step_arrays_follow_shapes = True
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: GatedDeltaSpec):
        H, G, D, E, W = spec.num_heads, spec.num_kv_heads, spec.key_dim, spec.value_dim, spec.hidden_size
        widths = (G * D, G * D, H * E)
        decls = [WeightDecl(spec.q_proj, (G * D, W)), WeightDecl(spec.k_proj, (G * D, W)), WeightDecl(spec.v_proj, (H * E, W)),
                 WeightDecl(spec.beta_proj, (H, W)), WeightDecl(spec.decay_down, (spec.decay_rank, W)),
                 WeightDecl(spec.decay_up, (H * D, spec.decay_rank)), WeightDecl(spec.decay_bias, (H * D,), VECTOR),
                 WeightDecl(spec.decay_log, (H,), VECTOR), WeightDecl(spec.gate_down, (spec.gate_rank, W)),
                 WeightDecl(spec.gate_up, (H * E, spec.gate_rank)), WeightDecl(spec.o_proj, (W, H * E))]
        decls += [WeightDecl(n, (w, spec.conv.taps), VECTOR) for n, w in zip(spec.conv_weights, widths)]
        return decls + norm_class(spec.out_norm).weight_decls(spec.out_norm)

    @staticmethod
    def kernel_modules(spec):
        return ("recurrent", "rowwise") + GEMM_MODULES

    def __init__(self, spec: GatedDeltaSpec, weights, dtype, device):
        H, G, D, E = spec.num_heads, spec.num_kv_heads, spec.key_dim, spec.value_dim
        if H % G != 0:
            raise ValueError(f"gated delta rule: {H} heads are not a multiple of {G} key heads")
        if D > 256:
            raise ValueError(f"gated delta rule: key width {D} exceeds 256")
        if spec.conv.channels != 2 * G * D + H * E or not 1 <= spec.conv.taps <= 8 or len(spec.conv_weights) != 3:
            raise ValueError("gated delta rule: one convolution of 1 to 8 taps over the channels of q, k and v")
        if spec.out_norm.kind != "rmsnorm" or spec.out_norm.dim != E or spec.out_norm.weight_offset != 0.0:
            raise ValueError("gated delta rule: the output norm is a plain RMSNorm over a head's values")
        self.spec, self.dtype = spec, dtype
        self.H, self.G, self.D, self.E = H, G, D, E
        self.qkv = spec.conv.channels
        names = (spec.q_proj, spec.k_proj, spec.v_proj, spec.beta_proj, spec.decay_down, spec.gate_down)
        self.w_in = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.beta_off = self.qkv
        self.decay_off = self.beta_off + H
        self.gate_off = self.decay_off + spec.decay_rank
        self.w_decay = weights.device_tensor(spec.decay_up, dtype, device)
        self.w_gate = weights.device_tensor(spec.gate_up, dtype, device)
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.conv_w = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in spec.conv_weights], dim=0).contiguous()
        self.dt_bias = weights.device_tensor(spec.decay_bias, dtype, device).contiguous()
        self.a_log = weights.device_tensor(spec.decay_log, dtype, device).contiguous()
        self.norm_gain = weights.device_tensor(spec.out_norm.weight, dtype, device)
        self.norm_eps = float(spec.out_norm.eps)
        self.s_size = H * D * E

    def state_request(self) -> StateRequest:
        return StateRequest((self.s_size + (self.spec.conv.taps - 1) * self.qkv,), torch.float32)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        he = self.H * self.E
        return tokens * (self.w_in.shape[0] * elem + self.qkv * 4 + self.H * self.D * 4 + he * (4 + 2 * elem)
                         + self.spec.hidden_size * elem) + ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T, ws = ctx.n_tokens, ctx.workspace
        H, G, D, E = self.H, self.G, self.D, self.E
        packed = linear(x, self.w_in, ws.buffer("delta_in", T, self.w_in.shape[0], self.dtype))
        qkv = ws.buffer("delta_qkv", T, self.qkv, torch.float32)
        ops.short_conv(qkv, packed[:, :self.qkv], self.conv_w, cache.state[:, self.s_size:], ctx.cu_q, ctx.state_slots, ctx.n_seqs,
                       activation="silu")
        # the decays' up-projection leaves in float32: what follows it (softplus, exponentials) is 32-bit arithmetic
        decay = linear(packed[:, self.decay_off:self.gate_off], self.w_decay, ws.buffer("delta_decay", T, H * D, torch.float32))
        gate = linear(packed[:, self.gate_off:], self.w_gate, ws.buffer("delta_gate", T, H * E, self.dtype))
        o = ws.buffer("delta_o", T, H * E, torch.float32)
        ops.delta_scan(o, qkv, packed[:, self.beta_off:self.decay_off], decay, self.dt_bias, self.a_log, cache.state, ctx.cu_q,
                       ctx.state_slots, ctx.n_seqs, H, G, D, E, float(self.spec.unit_eps), float(D) ** -0.5,
                       beta_buf=ws.buffer("delta_beta", T, H + G, torch.float32))
        y = ws.buffer("delta_y", T, H * E, self.dtype)
        ops.gated_rmsnorm(y.view(T * H, E), o.view(T * H, E), gate, self.norm_gain, self.norm_eps, heads=H)
        return linear_sliced(ws, "mixer_out", y, self.w_o, self.dtype)


register_mixer("gated_delta", GatedDelta)
