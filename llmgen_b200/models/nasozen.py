"""Nasozen: from its typed configuration to a `ModelSpec`.

A pre-norm decoder over several residual streams per token (`MultiStreamBlockSpec`: hyper-connections with a multiplier on
every sublayer's output), whose table of embeddings is also its output matrix, whose layers pick one of three mixers, and
which may run a stretch of its layers several times:

    mixer "parallel"        `ParallelMixerSpec` of two branches on the same input, added with a scale each:
                            left   `AttentionSpec`: grouped-query attention without biases whose q, k and v pass a short causal
                                   convolution, whose q and k are normed over their whole projections, with the first
                                   `rot.dims` values of a head turned in half-split pairs, values turned by their position
                                   (and the output turned back), a sliding window, a learned sink score per head, and a gate
                                   per head
                            right  `MinGRUSpec`: a gated recurrence per channel whose gates read the current token only
    mixer "mlstm"           `MLSTMSpec`: a matrix memory with exponential gates under a running maximum
    mixer "general_delta"   `GeneralDeltaSpec`: the delta rule with a decay per key channel and a removal rate of its own
    mlp null | dense | moe  none | `DenseMLPSpec` with the tanh form of gelu | `RoutedMLPSpec`: softmax over all experts, the
                            `top` largest choose, their scores divided by their sum weigh the outputs of plain silu-gated experts
    loop                    layers [start, stop) appear `times` times in the run list, every appearance with a cache (or
                            state) number of its own

Tensor names of a model folder (layer i):

    embed [vocab, width]; final.norm [width]
    l<i>.norm1, l<i>.norm2 [width]; l<i>.hc1.{in,out} [streams], l<i>.hc1.mix [streams, streams], l<i>.hc2.* the same
    l<i>.mix.left.{q,k,v,o}, .{q,k,v}.conv, .{q,k}.norm, .sink, .g; l<i>.mix.right.{z,x,g,o}, .{z,x}.b          parallel
    l<i>.mix.{q,k,v,g,o,norm,i,f}, .{i,f}.b                                                                    mlstm
    l<i>.mix.{r,k,v,g,o,norm,a,w1,w2}, .a.b, .w0                                                               general_delta
    l<i>.mlp.{up,down} | l<i>.mlp.router, l<i>.mlp.e<j>.{gate,up,down}

Fixed by the architecture, not by its config.json: the delta rule's decay scale exp(-1/2) and its unit keys' 1e-6, the
memory's 1e-6 in its denominator, the weights' 1e-20.  The rank of the delta rule's low-rank projection is a size that a
model folder gives by the shape of `w1` (`NasozenConfig.fill_from_tensor_shapes`).
"""
from __future__ import annotations

import math

from ..config.nasozen import DENSE, MLSTM, PARALLEL, NasozenConfig
from ..parts.spec import (AttentionSpec, DenseMLPSpec, GatedExpertSpec, GeneralDeltaSpec, MinGRUSpec, MLSTMSpec, ModelSpec,
                          MultiStreamBlockSpec, ParallelMixerSpec, RMSNormSpec, RopeSpec, RoutedMLPSpec, ShortConvSpec,
                          StreamCoefficients)
from ..registry import register_architecture
from .sarulix import sarulix_run_order

DELTA_DECAY_SCALE = math.exp(-0.5)
UNIT_EPS = 1e-6
MEMORY_DEN_EPS = 1e-6


def build_nasozen_spec(cfg: NasozenConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    ignorable = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", layer.mixer
        if layer.type == PARALLEL:
            a = m.left
            rope = RopeSpec(rotary_dim=a.rot_dims, theta=a.rot_base, max_positions=cfg.max_positions, pairing="half") \
                if a.rot_dims else None
            channels = (a.heads + a.kv_heads) * a.dim + a.kv_heads * a.vdim
            left = AttentionSpec(
                hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
                q_proj=p + "left.q", k_proj=p + "left.k", v_proj=p + "left.v", o_proj=p + "left.o",
                q_norm=RMSNormSpec(a.heads * a.dim, eps, p + "left.q.norm"), k_norm=RMSNormSpec(a.kv_heads * a.dim, eps, p + "left.k.norm"),
                position=rope, window=a.window or None, v_head_dim=a.vdim, sink=True, sink_scores=p + "left.sink",
                gate_proj=p + "left.g", gate_per_head=True, row_norms=True, rotate_values=rope is not None,
                conv=ShortConvSpec(channels, a.conv, p + "left.qkv.conv"),
                conv_weights=(p + "left.q.conv", p + "left.k.conv", p + "left.v.conv"))
            right = MinGRUSpec(hidden_size=W, width=m.right_width, z_proj=p + "right.z", x_proj=p + "right.x", gate_proj=p + "right.g",
                               o_proj=p + "right.o", z_bias=p + "right.z.b", x_bias=p + "right.x.b")
            mixer = ParallelMixerSpec(branches=(left, right), scales=(m.left_scale, m.right_scale))
        elif layer.type == MLSTM:
            mixer = MLSTMSpec(hidden_size=W, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, gate_cap=m.gate_cap, eps=eps,
                              q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", i_proj=p + "i", f_proj=p + "f", gate_proj=p + "g",
                              o_proj=p + "o", out_gain=p + "norm", i_bias=p + "i.b", f_bias=p + "f.b", den_eps=MEMORY_DEN_EPS)
        else:
            mixer = GeneralDeltaSpec(hidden_size=W, num_heads=m.heads, head_dim=m.dim, eps=eps, r_proj=p + "r", k_proj=p + "k",
                                     v_proj=p + "v", gate_proj=p + "g", o_proj=p + "o", removal_proj=p + "a", removal_bias=p + "a.b",
                                     decay_down=p + "w1", decay_up=p + "w2", decay_bias=p + "w0", out_gain=p + "norm",
                                     decay_rank=m.decay_rank, decay_scale=DELTA_DECAY_SCALE, unit_eps=UNIT_EPS)
        ffn = None
        if layer.mlp is not None:
            q, f = f"l{i}.mlp.", layer.mlp
            if f.kind == DENSE:
                ffn = DenseMLPSpec(W, f.ff, q + "up", q + "down", activation="gelu_tanh")
            else:
                ffn = RoutedMLPSpec(
                    hidden_size=W, router=q + "router", top_k=f.top, scoring="softmax", renormalize=True, weight_on_input=False,
                    experts=tuple(GatedExpertSpec(f.ff, f"{q}e{j}.gate", f"{q}e{j}.up", f"{q}e{j}.down") for j in range(f.experts)))
        else:
            # a layer without a feed-forward has no use for its second norm and coefficients; a folder may carry them
            ignorable += [f"l{i}.norm2", f"l{i}.hc2.*"]
        coefficients = (lambda n: StreamCoefficients(f"l{i}.hc{n}.in", f"l{i}.hc{n}.out", f"l{i}.hc{n}.mix")) if cfg.streams else (lambda n: None)
        layers.append(MultiStreamBlockSpec(
            mixer_norm=RMSNormSpec(W, eps, f"l{i}.norm1"), mixer=mixer,
            ffn_norm=RMSNormSpec(W, eps, f"l{i}.norm2") if ffn is not None else None, ffn=ffn, streams=cfg.streams or 1,
            residual_mult=cfg.residual_mult, mixer_streams=coefficients(1), ffn_streams=coefficients(2) if ffn is not None else None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding="embed", layers=tuple(layers),
        run_order=sarulix_run_order(len(layers), cfg.loop, reentry=False), final_norm=RMSNormSpec(W, eps, "final.norm"),
        lm_head="embed", max_positions=cfg.max_positions, residual_streams=cfg.streams or 1, ignorable_tensors=tuple(ignorable))


register_architecture("Nasozen", NasozenConfig, build_nasozen_spec, aliases=("nasozen",))
