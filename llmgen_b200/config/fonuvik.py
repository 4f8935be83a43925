"""Typed configuration of the Fonuvik decoder, read from its config.json.

    architecture      "Fonuvik"
    vocab, width      sizes of the table of embeddings and of the residual stream
    norm.eps          eps of every norm
    layers[i]         type: "parallel" | "wkv"; mixer: that mixer's sizes and constants; mlp: null or
                      {kind: "moe", router: {experts, top}, expert: {ff}, shared: {ff} (optional)}
    parallel mixer    left_scale, right_scale;
                      left: heads, kv_heads, dim, vdim, scale, mask: {size}, rot: {base, dims, scaling: {factor, low, high,
                      original} (optional)} (optional);
                      right: heads, dim, vdim, tau
    wkv mixer         heads, dim

Every size and constant comes from the file.  The ranks of the decays' low-rank projections are sizes that a model folder
gives by the shapes of its tensors alone (`l<i>.mix.right.a1`, `l<i>.mix.w1`, both [rank, width]):
`fill_from_tensor_shapes` puts them into the mixer's object as `decay_rank`, which a configuration written by hand (the
random-weights mode) may name itself (default 16).  `max_positions` (rows of the rotary tables) is optional.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .derupel import _sub

PARALLEL = "parallel"
WKV = "wkv"
MOE = "moe"
DEFAULT_MAX_POSITIONS = 1 << 17
DEFAULT_LOW_RANK = 16


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int
    rot_base: float
    rot_dims: int                                   # 0: no rotation
    rot_scaling: Optional[Tuple[float, float, float, float]]    # (factor, low, high, original)


@dataclass(frozen=True)
class ChannelDecayConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkedAttentionConfig
    right: ChannelDecayConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class WkvMixerConfig:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int          # 0: no shared expert


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: Optional[MoeConfig]


def _left(m: ConfigReader, r: ConfigReader, where: str) -> Optional[ChunkedAttentionConfig]:
    heads, kv_heads = m.integer("heads"), m.integer("kv_heads")
    dim, vdim, scale = m.integer("dim"), m.integer("vdim"), m.number("scale")
    mask = _sub(m, "mask", m.where)
    chunk = mask.integer("size") if mask is not None else None
    rot = _sub(m, "rot", m.where, required=False)
    base = rot.number("base") if rot is not None else 1.0
    dims = rot.integer("dims", minimum=0) if rot is not None else 0
    scaling = None
    sc = _sub(rot, "scaling", rot.where, required=False) if rot is not None else None
    if sc is not None:
        vals = (sc.number("factor"), sc.number("low"), sc.number("high"), sc.number("original"))
        if None not in vals:
            r.check(vals[2] > vals[1], f"{where}.rot.scaling: high {vals[2]} must exceed low {vals[1]}")
            scaling = vals
        else:
            return None
    if None in (heads, kv_heads, dim, vdim, scale, chunk, base, dims):
        return None
    r.check(heads % kv_heads == 0, f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    r.check(dims % 2 == 0 and dims <= dim, f"{where}.rot.dims {dims} must be even and at most dim {dim}")
    r.check(dim % 2 == 0, f"{where}.dim {dim} must be even")
    return ChunkedAttentionConfig(heads, kv_heads, dim, vdim, scale, chunk, base, dims, scaling)


def _layer(data, i: int, r: ConfigReader, where: str) -> Optional[LayerConfig]:
    if not isinstance(data, dict):
        r.problem(f"layers[{i}] must be an object")
        return None
    n0 = len(r.problems)
    lr = ConfigReader(data, f"{where}.layers[{i}]")
    lr.problems = r.problems
    kind = lr.string("type", choices=(PARALLEL, WKV))
    m = _sub(lr, "mixer", lr.where)
    mixer = None
    if m is not None and kind == PARALLEL:
        ls, rs = m.number("left_scale", positive=False), m.number("right_scale", positive=False)
        lm, rm = _sub(m, "left", m.where), _sub(m, "right", m.where)
        left = _left(lm, r, f"layers[{i}].mixer.left") if lm is not None else None
        right = None
        if rm is not None:
            heads, dim, vdim, tau = rm.integer("heads"), rm.integer("dim"), rm.integer("vdim"), rm.number("tau")
            rank = rm.integer("decay_rank", default=DEFAULT_LOW_RANK)
            if None not in (heads, dim, vdim, tau, rank):
                right = ChannelDecayConfig(heads, dim, vdim, tau, rank)
        if None not in (ls, rs, left, right):
            mixer = ParallelMixerConfig(left, right, ls, rs)
    elif m is not None and kind == WKV:
        heads, dim = m.integer("heads"), m.integer("dim")
        rank = m.integer("decay_rank", default=DEFAULT_LOW_RANK)
        if None not in (heads, dim, rank):
            mixer = WkvMixerConfig(heads, dim, rank)
    mlp = None
    if data.get("mlp") is not None:
        f = _sub(lr, "mlp", lr.where)
        if f is not None:
            f.string("kind", choices=(MOE,))
            router, expert = _sub(f, "router", f.where), _sub(f, "expert", f.where)
            shared = _sub(f, "shared", f.where, required=False)
            experts = router.integer("experts") if router is not None else None
            top = router.integer("top") if router is not None else None
            ff = expert.integer("ff") if expert is not None else None
            shared_ff = shared.integer("ff") if shared is not None else 0
            if None not in (experts, top, ff, shared_ff):
                r.check(top <= experts, f"layers[{i}].mlp.router: top {top} of {experts} experts")
                mlp = MoeConfig(experts, top, ff, shared_ff)
    if len(r.problems) > n0 or kind is None or mixer is None:
        return None
    return LayerConfig(kind, mixer, mlp)


@dataclass(frozen=True)
class FonuvikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LayerConfig, ...]
    max_positions: int
    raw: dict

    architecture = "Fonuvik"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "FonuvikConfig":
        r = ConfigReader(data, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        norm = _sub(r, "norm", where)
        eps = norm.number("eps") if norm is not None else None
        max_positions = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS)
        layers = r.raw("layers")
        parsed = []
        if not isinstance(layers, list) or not layers:
            r.problem("'layers' must be a non-empty list")
        else:
            parsed = [_layer(d, i, r, where) for i, d in enumerate(layers)]
        r.finish()
        return cls(vocab, width, eps, tuple(parsed), max_positions, dict(data))

    def to_dict(self) -> dict:
        return dict(self.raw)

    @staticmethod
    def fill_from_tensor_shapes(data: dict, shapes: dict) -> dict:
        """`data` with `decay_rank` added to every mixer with a low-rank decay that does not name it, from the shapes of
        the folder's tensors `l<i>.mix.right.a1` / `l<i>.mix.w1` ([rank, width])."""
        import copy
        layers = data.get("layers")
        if not isinstance(layers, list):
            return data
        out = copy.deepcopy(data)
        for i, layer in enumerate(out["layers"]):
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                continue
            if layer.get("type") == PARALLEL:
                target, tensor = layer["mixer"].get("right"), f"l{i}.mix.right.a1"
            elif layer.get("type") == WKV:
                target, tensor = layer["mixer"], f"l{i}.mix.w1"
            else:
                continue
            if isinstance(target, dict) and "decay_rank" not in target and tensor in shapes and len(shapes[tensor]) == 2:
                target["decay_rank"] = int(shapes[tensor][0])
        return out
