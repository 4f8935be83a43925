"""Typed configuration of the Nasozen decoder, read from its config.json.

    architecture      "Nasozen"
    vocab, width      sizes of the table of embeddings (which is also the output matrix) and of the residual stream
    norm.eps          eps of every RMSNorm
    residual_mult     factor on every sublayer's output as it joins the stream (optional, 1)
    streams           number of residual streams per token (optional; absent: one plain stream)
    loop              optional {start, stop, times}: layers [start, stop) run `times` times in a row with the same weights
    layers[i]         type: "parallel" | "mlstm" | "general_delta"; mixer: that mixer's sizes and constants;
                      mlp: null, {kind: "dense", ff} or {kind: "moe", expert: {ff}, router: {experts, top}}
    parallel          left: {heads, kv_heads, dim, vdim, scale, conv (taps), mask: {size} (optional), rot: {base, dims}
                      (optional)}, right: {width}, left_scale, right_scale
    mlstm             heads, dim, vdim, gate_cap
    general_delta     heads, dim; optional decay_rank

Every size and constant comes from the file.  The rank of the delta rule's low-rank decay projection is a size that a
model folder gives by the shape of its tensor `l<i>.mix.w1` alone: `fill_from_tensor_shapes` puts it into the mixer's object
as `decay_rank`, which a configuration written by hand (the random-weights mode) may name itself (default 16).
`max_positions` (rows of the rotary tables) is optional.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .derupel import _sub
from .sarulix import LoopConfig

PARALLEL = "parallel"
MLSTM = "mlstm"
GENERAL_DELTA = "general_delta"
DENSE = "dense"
MOE = "moe"
DEFAULT_MAX_POSITIONS = 1 << 16
DEFAULT_LOW_RANK = 16


@dataclass(frozen=True)
class LeftConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int               # taps
    window: int             # 0: every earlier key
    rot_base: float
    rot_dims: int           # 0: no rotation (of q, k or v)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: LeftConfig
    right_width: int
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class MLSTMMixerConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class GeneralDeltaMixerConfig:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


def _left(m: ConfigReader, r: ConfigReader, i: int) -> Optional[LeftConfig]:
    a = _sub(m, "left", m.where)
    if a is None:
        return None
    heads, kv_heads = a.integer("heads"), a.integer("kv_heads")
    dim, vdim, scale, conv = a.integer("dim"), a.integer("vdim"), a.number("scale"), a.integer("conv")
    mask = _sub(a, "mask", a.where, required=False)
    window = mask.integer("size") if mask is not None else 0
    rot = _sub(a, "rot", a.where, required=False)
    base = rot.number("base") if rot is not None else 1.0
    dims = rot.integer("dims", minimum=0) if rot is not None else 0
    if None in (heads, kv_heads, dim, vdim, scale, conv, window, base, dims):
        return None
    r.check(heads % kv_heads == 0, f"layers[{i}].mixer.left: {heads} heads are not a multiple of {kv_heads} kv_heads")
    r.check(dims % 2 == 0 and dims <= dim, f"layers[{i}].mixer.left.rot.dims {dims} must be even and at most dim {dim}")
    r.check(dims == 0 or vdim % 2 == 0, f"layers[{i}].mixer.left.vdim {vdim} must be even for rotated values")
    r.check(conv <= 8, f"layers[{i}].mixer.left.conv {conv} taps: at most 8")
    return LeftConfig(heads, kv_heads, dim, vdim, scale, conv, window, base, dims)


def _layer(data, i: int, r: ConfigReader, where: str) -> Optional[LayerConfig]:
    if not isinstance(data, dict):
        r.problem(f"layers[{i}] must be an object")
        return None
    n0 = len(r.problems)
    lr = ConfigReader(data, f"{where}.layers[{i}]")
    lr.problems = r.problems
    kind = lr.string("type", choices=(PARALLEL, MLSTM, GENERAL_DELTA))
    m = _sub(lr, "mixer", lr.where)
    mixer = None
    if m is not None and kind == PARALLEL:
        left = _left(m, r, i)
        right = _sub(m, "right", m.where)
        width = right.integer("width") if right is not None else None
        ls, rs = m.number("left_scale", default=1.0, positive=False), m.number("right_scale", default=1.0, positive=False)
        if None not in (left, width, ls, rs):
            mixer = ParallelMixerConfig(left, width, ls, rs)
    elif m is not None and kind == MLSTM:
        heads, dim, vdim, cap = m.integer("heads"), m.integer("dim"), m.integer("vdim"), m.number("gate_cap")
        if None not in (heads, dim, vdim, cap):
            mixer = MLSTMMixerConfig(heads, dim, vdim, cap)
    elif m is not None and kind == GENERAL_DELTA:
        heads, dim = m.integer("heads"), m.integer("dim")
        rank = m.integer("decay_rank", default=DEFAULT_LOW_RANK)
        if None not in (heads, dim, rank):
            mixer = GeneralDeltaMixerConfig(heads, dim, rank)
    mlp = None
    if data.get("mlp") is not None:
        f = _sub(lr, "mlp", lr.where)
        if f is not None:
            fk = f.string("kind", choices=(DENSE, MOE))
            if fk == DENSE:
                ff = f.integer("ff")
                mlp = MlpConfig(fk, ff) if ff is not None else None
            elif fk == MOE:
                e, ro = _sub(f, "expert", f.where), _sub(f, "router", f.where)
                ff = e.integer("ff") if e is not None else None
                experts = ro.integer("experts") if ro is not None else None
                top = ro.integer("top") if ro is not None else None
                if None not in (ff, experts, top):
                    r.check(top <= experts, f"layers[{i}].mlp.router: top {top} of {experts} experts")
                    mlp = MlpConfig(fk, ff, experts, top)
    if len(r.problems) > n0 or kind is None or mixer is None:
        return None
    return LayerConfig(kind, mixer, mlp)


@dataclass(frozen=True)
class NasozenConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    streams: int            # 0: the key is absent, one plain stream without coefficients
    layers: Tuple[LayerConfig, ...]
    loop: Optional[LoopConfig]
    max_positions: int
    raw: dict

    architecture = "Nasozen"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "NasozenConfig":
        r = ConfigReader(data, where)
        vocab, width = r.integer("vocab"), r.integer("width")
        norm = _sub(r, "norm", where)
        eps = norm.number("eps") if norm is not None else None
        mult = r.number("residual_mult", default=1.0, positive=False)
        streams = r.integer("streams", default=0, minimum=0)
        max_positions = r.integer("max_positions", default=DEFAULT_MAX_POSITIONS)
        layers = r.raw("layers")
        parsed = []
        if not isinstance(layers, list) or not layers:
            r.problem("'layers' must be a non-empty list")
        else:
            parsed = [_layer(d, i, r, where) for i, d in enumerate(layers)]
        loop = None
        if data.get("loop") is not None:
            lp = _sub(r, "loop", where)
            if lp is not None:
                start, stop, times = lp.integer("start", minimum=0), lp.integer("stop"), lp.integer("times")
                if None not in (start, stop, times):
                    r.check(start < stop <= len(parsed), f"loop [{start}, {stop}) does not lie within the {len(parsed)} layers")
                    loop = LoopConfig(start, stop, times)
        if streams is not None:
            r.check(streams <= 16, f"streams {streams}: at most 16")
        r.finish()
        return cls(vocab, width, eps, mult, streams, tuple(parsed), loop, max_positions, dict(data))

    def to_dict(self) -> dict:
        return dict(self.raw)

    @staticmethod
    def fill_from_tensor_shapes(data: dict, shapes: dict) -> dict:
        """`data` with `decay_rank` added to every general_delta mixer that does not name it, from the shape of the folder's
        tensor `l<i>.mix.w1` ([rank, width])."""
        import copy
        layers = data.get("layers")
        if not isinstance(layers, list):
            return data
        out = copy.deepcopy(data)
        for i, layer in enumerate(out["layers"]):
            if isinstance(layer, dict) and layer.get("type") == GENERAL_DELTA and isinstance(layer.get("mixer"), dict):
                tensor = f"l{i}.mix.w1"
                if "decay_rank" not in layer["mixer"] and tensor in shapes and len(shapes[tensor]) == 2:
                    layer["mixer"]["decay_rank"] = int(shapes[tensor][0])
        return out
