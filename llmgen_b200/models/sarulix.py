"""Sarulix: from its typed configuration to a `ModelSpec`.

A pre-norm decoder (`PreNormBlockSpec`, gains stored around zero) whose layers pick one of three mixers, and which may
run a stretch of its layers several times:

    mixer "attention"       `AttentionSpec` with its variations on: biases on q, k, v and the output, per-head norms of q
                            and k, rotation of the first `rot.dims` values of a head (half-split pairs), a bound on
                            the scores (softcap), a sink in the softmax's denominator, an output gate, values of their
                            own width
    mixer "rglru"           `RGLRUSpec`: a recurrent block around a real-gated linear recurrent unit
    mixer "channel_delta"   `GatedDeltaSpec`: the gated delta rule with a decay per head and key channel
    mlp null | dense        none | `GatedMLPSpec` with the tanh form of gelu
    loop                    layers [start, stop) appear `times` times in the run list, every appearance with a cache
                            (or state) number of its own; the first layer of every pass is preceded by a `ReentrySpec`
                            (the stream mixed with the embedding's output through `loop.in`, plus row t of `loop.step`)

Tensor names of a model folder (layer i):

    embed [vocab, width]; final.norm [width]; head [vocab, width]; loop.in [width, 2 width]; loop.step [times, width]
    l<i>.norm1, l<i>.norm2 [width]
    l<i>.mix.{q,k,v,o}(.b), l<i>.mix.{q,k}.norm, l<i>.mix.g                                         attention
    l<i>.mix.{y,x}(.b), l<i>.mix.conv(.b), l<i>.mix.{ra,ri}(.b), l<i>.mix.lam, l<i>.mix.o             rglru
    l<i>.mix.{q,k,v}(.conv), l<i>.mix.{b,a1,a2,dt_bias,A_log,g1,g2,norm,o}                          channel_delta
    l<i>.mlp.{gate,up,down}

Fixed by the architecture, not by its config.json: the recurrent unit's decay scale 8, the unit vectors' 1e-6, the
sink, causal attention without a window, an untied output matrix.  The ranks of the delta rule's low-rank projections
are sizes that a model folder gives by the shapes of `a1` and `g1` (`SarulixConfig.fill_from_tensor_shapes`).
"""
from __future__ import annotations

from ..config.sarulix import ATTENTION, RGLRU, SarulixConfig
from ..parts.spec import (AttentionSpec, GatedDeltaSpec, GatedMLPSpec, ModelSpec, PreNormBlockSpec, ReentrySpec, RGLRUSpec,
                          RMSNormSpec, RopeSpec, RunItem, ShortConvSpec)
from ..registry import register_architecture

RGLRU_DECAY_SCALE = 8.0
UNIT_EPS = 1e-6


def sarulix_run_order(n_layers: int, loop, reentry: bool = True):
    """The run list: layers before the loop, the loop's layers `times` times (each appearance with a cache number of
    its own, the first of a pass behind a `ReentrySpec` unless `reentry` is off), the rest."""
    if loop is None:
        return tuple(RunItem(layer=i, cache=i) for i in range(n_layers))
    items, cache = [], 0
    for i in range(loop.start):
        items.append(RunItem(layer=i, cache=cache))
        cache += 1
    for t in range(loop.times):
        for i in range(loop.start, loop.stop):
            before = ReentrySpec("loop.in", "loop.step", t, loop.times) if reentry and i == loop.start else None
            items.append(RunItem(layer=i, cache=cache, before=before))
            cache += 1
    for i in range(loop.stop, n_layers):
        items.append(RunItem(layer=i, cache=cache))
        cache += 1
    return tuple(items)


def build_sarulix_spec(cfg: SarulixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", layer.mixer
        if layer.type == ATTENTION:
            rope = RopeSpec(rotary_dim=m.rot_dims, theta=m.rot_base, max_positions=cfg.max_positions, pairing="half") \
                if m.rot_dims else None
            mixer = AttentionSpec(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
                q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", o_proj=p + "o",
                q_norm=RMSNormSpec(m.dim, eps, p + "q.norm"), k_norm=RMSNormSpec(m.dim, eps, p + "k.norm"), position=rope,
                v_head_dim=m.vdim, q_bias=p + "q.b", k_bias=p + "k.b", v_bias=p + "v.b", o_bias=p + "o.b",
                softcap=m.softcap, sink=True, gate_proj=p + "g")
        elif layer.type == RGLRU:
            mixer = RGLRUSpec(
                hidden_size=W, width=m.width, blocks=m.blocks, conv=ShortConvSpec(m.width, m.conv, p + "conv", p + "conv.b"),
                y_proj=p + "y", x_proj=p + "x", o_proj=p + "o", a_gate=p + "ra", i_gate=p + "ri", lam=p + "lam",
                y_bias=p + "y.b", x_bias=p + "x.b", a_gate_bias=p + "ra.b", i_gate_bias=p + "ri.b",
                decay_scale=RGLRU_DECAY_SCALE)
        else:
            channels = 2 * m.kv_heads * m.dim + m.heads * m.vdim
            mixer = GatedDeltaSpec(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                conv=ShortConvSpec(channels, m.conv, p + "qkv.conv"), conv_weights=(p + "q.conv", p + "k.conv", p + "v.conv"),
                q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", beta_proj=p + "b", decay_down=p + "a1", decay_up=p + "a2",
                decay_bias=p + "dt_bias", decay_log=p + "A_log", gate_down=p + "g1", gate_up=p + "g2", o_proj=p + "o",
                out_norm=RMSNormSpec(m.vdim, eps, p + "norm"),
                decay_rank=m.decay_rank, gate_rank=m.gate_rank, unit_eps=UNIT_EPS)
        ffn = None
        if layer.mlp is not None:
            q = f"l{i}.mlp."
            ffn = GatedMLPSpec(W, layer.mlp.ff, q + "gate", q + "up", q + "down", activation="gelu_tanh")
        layers.append(PreNormBlockSpec(
            mixer_norm=RMSNormSpec(W, eps, f"l{i}.norm1", weight_offset=1.0), mixer=mixer,
            ffn_norm=RMSNormSpec(W, eps, f"l{i}.norm2", weight_offset=1.0) if ffn is not None else None, ffn=ffn))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding="embed", layers=tuple(layers),
        run_order=sarulix_run_order(len(layers), cfg.loop), final_norm=RMSNormSpec(W, eps, "final.norm", weight_offset=1.0),
        lm_head="head", max_positions=cfg.max_positions, embedding_scale=cfg.embedding_scale, logit_scale=cfg.logit_scale,
        # a layer without a feed-forward has no use for a second norm; a folder may carry one all the same
        ignorable_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None))


register_architecture("Sarulix", SarulixConfig, build_sarulix_spec, aliases=("sarulix",))
