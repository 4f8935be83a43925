"""Fonuvik: from its typed configuration to a `ModelSpec`.

A decoder whose table of embeddings is also its output matrix, whose embedding rows pass a norm before they become the
residual stream, and whose layers norm every sublayer's input and output (`SandwichBlockSpec`).  Layer by layer:

    mixer "parallel"   `ParallelMixerSpec` of two branches on the same input, added with a scale each:
                       left   `AttentionSpec`: grouped-query attention without biases, values of their own width, the first
                              `rot.dims` values of a head turned in pairs (2i, 2i + 1) by frequencies scaled by wavelength,
                              heads of q and k divided by their root mean square after the rotation, a scale of its own,
                              and a mask in blocks of `mask.size` positions
                       right  `ChannelDecayAttentionSpec`: linear attention with a decay per head and key channel
    mixer "wkv"        `TokenShiftDecaySpec`: time mixing over blends of a token with the one before it
    mlp null | moe     none | `RoutedMLPSpec`: the `top` largest router logits (with a bias) choose, the weights are the
                       softmax over the chosen logits and multiply the experts' outputs; plain silu-gated experts; a
                       shared expert for every token

Tensor names of a model folder (layer i):

    embed [vocab, width]; embed.norm, final.norm [width]
    l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b [width]
    l<i>.mix.left.{q,k,v,o}; l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b}                          parallel
    l<i>.mix.mu.{r,k,v,g,w}, l<i>.mix.{r,k,v,g,o,w1,w2,w0,u,norm}                                 wkv
    l<i>.mlp.router, l<i>.mlp.router.b, l<i>.mlp.e<j>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down}

The ranks of the decays' low-rank projections are sizes that a model folder gives by the shapes of `a1` and `w1`
(`FonuvikConfig.fill_from_tensor_shapes`).
"""
from __future__ import annotations

from ..config.fonuvik import PARALLEL, FonuvikConfig
from ..parts.spec import (AttentionSpec, ChannelDecayAttentionSpec, GatedExpertSpec, ModelSpec, ParallelMixerSpec, RMSNormSpec,
                          RopeSpec, RoutedMLPSpec, RunItem, SandwichBlockSpec, TokenShiftDecaySpec)
from ..registry import register_architecture


def build_fonuvik_spec(cfg: FonuvikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    ignorable = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", layer.mixer
        if layer.type == PARALLEL:
            a, b = m.left, m.right
            rope = RopeSpec(rotary_dim=a.rot_dims, theta=a.rot_base, max_positions=cfg.max_positions, pairing="interleaved",
                            scaling=a.rot_scaling) if a.rot_dims else None
            left = AttentionSpec(
                hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
                q_proj=p + "left.q", k_proj=p + "left.k", v_proj=p + "left.v", o_proj=p + "left.o", position=rope,
                v_head_dim=a.vdim, unit_norm_eps=eps, chunk=a.chunk)
            right = ChannelDecayAttentionSpec(
                hidden_size=W, num_heads=b.heads, key_dim=b.dim, value_dim=b.vdim, tau=b.tau,
                q_proj=p + "right.q", k_proj=p + "right.k", v_proj=p + "right.v", gate_proj=p + "right.g", o_proj=p + "right.o",
                decay_down=p + "right.a1", decay_up=p + "right.a2", decay_bias=p + "right.a2.b",
                out_norm=RMSNormSpec(b.vdim, eps, p + "right.norm"), decay_rank=b.decay_rank)
            mixer = ParallelMixerSpec(branches=(left, right), scales=(m.left_scale, m.right_scale))
        else:
            mixer = TokenShiftDecaySpec(
                hidden_size=W, num_heads=m.heads, head_dim=m.dim, eps=eps, mix=tuple(p + "mu." + s for s in "rkvgw"),
                r_proj=p + "r", k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g", o_proj=p + "o", decay_down=p + "w1",
                decay_up=p + "w2", decay_bias=p + "w0", bonus=p + "u", out_gain=p + "norm", decay_rank=m.decay_rank)
        ffn = None
        if layer.mlp is not None:
            q, f = f"l{i}.mlp.", layer.mlp
            expert = lambda name, ff: GatedExpertSpec(ff, q + name + ".gate", q + name + ".up", q + name + ".down")
            ffn = RoutedMLPSpec(
                hidden_size=W, router=q + "router", experts=tuple(expert(f"e{j}", f.ff) for j in range(f.experts)), top_k=f.top,
                shared=expert("shared", f.shared_ff) if f.shared_ff else None, scoring="softmax_top", weight_on_input=False,
                router_bias=q + "router.b")
        else:
            ignorable += [f"l{i}.norm2", f"l{i}.norm2b"]
        layers.append(SandwichBlockSpec(
            mixer_norm=RMSNormSpec(W, eps, f"l{i}.norm1"), mixer=mixer, mixer_out_norm=RMSNormSpec(W, eps, f"l{i}.norm1b"),
            ffn_norm=RMSNormSpec(W, eps, f"l{i}.norm2") if ffn is not None else None, ffn=ffn,
            ffn_out_norm=RMSNormSpec(W, eps, f"l{i}.norm2b") if ffn is not None else None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding="embed", layers=tuple(layers),
        run_order=tuple(RunItem(layer=i, cache=i) for i in range(len(layers))), final_norm=RMSNormSpec(W, eps, "final.norm"),
        lm_head="embed", max_positions=cfg.max_positions, embedding_norm=RMSNormSpec(W, eps, "embed.norm"),
        # a layer without a feed-forward has no use for its second pair of norms; a folder may carry them all the same
        ignorable_tensors=tuple(ignorable))


register_architecture("Fonuvik", FonuvikConfig, build_fonuvik_spec, aliases=("fonuvik",))
