"""Small Nasozen configurations with random weights, for the tests: the engine's model and the tensors the plain
implementation reads, made from one seed."""
from __future__ import annotations

import copy
from typing import Dict, List, Sequence

import torch

from tests.derupel_util import TOL, driver, ids_for, relative_error, row_errors, run_in_portions  # noqa: F401


def left(heads, kv_heads, dim, vdim, scale, conv, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def parallel(left_m, width, mlp, scales=(0.7, 1.2)):
    return {"type": "parallel", "mixer": {"left": left_m, "right": {"width": width}, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


def mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def gdelta(heads, dim, mlp, decay_rank=5):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def config(layers, width=48, vocab=97, eps=1e-5, streams=3, mult=0.8, loop=None) -> dict:
    cfg = {"architecture": "Nasozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": copy.deepcopy(list(layers))}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# Every kind of layer, sizes that differ from one another wherever they can: key width != value width, grouped heads, half
# a head rotated, a window that is no multiple of a page (16), three streams, a loop over the two middle layers, a dense
# feed-forward, two routed ones and a layer without one.
MIXED = config([
    gdelta(2, 16, dense(40)),
    parallel(left(4, 2, 16, 24, 0.3, 3, window=24, rot=(300.0, 8)), 40, moe(6, 2, 24)),
    mlstm(3, 8, 12, 10.0, moe(5, 3, 16)),
    gdelta(4, 8, None, decay_rank=3),
], width=48, loop=(1, 3, 2))
# Sizes that are multiples of little, and values that a usual model makes equal or one: one stream (with coefficients of its
# own), a multiplier of one, one head, as many key heads as heads, every expert chosen, one expert chosen of one, a
# convolution of one tap, no window, no rotation, both scales 1, widths that are no multiples of 4.
ODD = config([
    parallel(left(3, 3, 10, 6, 0.4, 1), 7, moe(3, 3, 20), scales=(1.0, 1.0)),
    mlstm(1, 6, 10, 4.0, moe(1, 1, 30)),
    gdelta(1, 10, dense(18), decay_rank=2),
    parallel(left(1, 1, 12, 20, 0.2, 2, window=4096, rot=(77.0, 12)), 21, None),
], width=36, vocab=50, eps=1e-4, streams=1, mult=1.0)
# No streams at all (a plain pre-norm layer with a multiplier), a loop from layer 0 that runs three times, a whole head
# rotated, a window of one position (every token sees itself and the sink), a window of two, four taps.
PLAIN = config([
    parallel(left(2, 1, 8, 8, 0.35, 4, window=1, rot=(50.0, 8)), 16, dense(24), scales=(1.3, 0.4)),
    mlstm(2, 12, 6, 15.0, None),
    parallel(left(2, 2, 12, 10, 0.3, 2, window=2, rot=(1000.0, 4)), 9, moe(4, 1, 12)),
], width=24, vocab=61, streams=None, mult=0.6, loop=(0, 2, 3))
# Eight query heads on one key head; key widths beyond 64 and 128 in the memories (the kernel's wider forms), more value
# columns than one of its blocks takes, widths that are no multiples of 8 or 16, five streams.
WIDE = config([
    mlstm(2, 72, 40, 15.0, None),
    parallel(left(8, 1, 32, 16, 0.18, 3, window=33, rot=(100.0, 32)), 72, moe(4, 2, 48)),
    gdelta(1, 136, None),
    mlstm(1, 20, 72, 6.0, dense(32)),
], width=48, vocab=61, eps=1e-6, streams=5, mult=1.1)
# Key and value widths that the tensor-core attention of the bfloat16 engine takes (64 and 128, equal and not), with windows
# that are no multiple of its tiles of 64 keys; prompts of a few hundred tokens cross several tiles of keys and of queries.
TENSOR = config([
    parallel(left(6, 3, 64, 64, 0.11, 3, window=96, rot=(10000.0, 32)), 32, moe(4, 2, 64)),
    parallel(left(2, 1, 128, 64, 0.09, 2, window=40, rot=(500.0, 128)), 16, None),
    parallel(left(2, 2, 64, 128, 0.125, 4, window=130, rot=(200000.0, 16)), 24, None),
], width=64, vocab=97, streams=2)
# One parallel layer whose weights `plant_needle` rewrites so that one token's query finds one other token's key.
NEEDLE_WINDOW = 40
NEEDLE = config([parallel(left(2, 1, 64, 16, 0.25, 3, window=NEEDLE_WINDOW, rot=(30.0, 8)), 8, moe(3, 1, 32), scales=(1.0, 0.2))],
                width=32, vocab=53, streams=2, mult=1.0)
NEEDLE_ID, PROBE_ID, FILLER_ID = 5, 9, 11
# States that keep (nearly) everything and nothing else to carry information over more than one token: losing a state, or a
# token of it, shows at every later position.
KEEPING_GRU = config([parallel(left(1, 1, 8, 8, 0.3, 1, window=1), 16, None, scales=(0.1, 1.0))], width=32, vocab=53, streams=2)
KEEPING_MLSTM = config([mlstm(2, 8, 8, 15.0, None)], width=32, vocab=53, streams=2)
KEEPING_DELTA = config([gdelta(2, 8, None)], width=32, vocab=53, streams=2)


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what="") -> None:
    """float32: every row within TOL.  bfloat16: nine rows in ten within TOL and the median within half of it; a router
    score that bfloat16 rounding moves across another sends one token to another expert, which is a large difference at that
    row and says nothing about a kernel."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, float(e.max()))
    else:
        assert float(e.quantile(0.9)) < TOL[dtype] and float(e.median()) < TOL[dtype] / 2, (what, float(e.quantile(0.9)), float(e.median()))


def draw(cfg: dict, seed: int, sigma: float = 0.1, sigma_norm: float = 0.2):
    from llmgen_b200.parts.registry import model_weight_decls
    from llmgen_b200.registry import config_from_dict
    from llmgen_b200.weights import random_tensors
    arch, typed = config_from_dict(cfg)
    spec = arch.build_spec(typed)
    decls = model_weight_decls(spec)
    return spec, decls, random_tensors(decls, seed, sigma, sigma_norm, torch.bfloat16)     # stored as a model folder stores them


def build(cfg: dict, seed: int, dtype: str = "float32", sigma: float = 0.1, sigma_norm: float = 0.2, prepare=None):
    """(the engine's model on the GPU, tensors by name on the CPU)."""
    from llmgen_b200.engine.api import require_cuda, resolve_dtype
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.weights import weights_from_dict
    spec, decls, tensors = draw(cfg, seed, sigma, sigma_norm)
    if prepare is not None:
        prepare(cfg, tensors)
    model = DecoderModel(spec, weights_from_dict(tensors, decls), resolve_dtype(dtype), require_cuda())
    return model, tensors


def keep_long(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Makes the one-layer KEEPING models remember: update gates near zero, forget gates near one, decays near one and
    hardly any removal, with writes small enough for hundreds of tokens."""
    if "l0.mix.right.z.b" in tensors:
        tensors["l0.mix.right.z.b"].fill_(-7.0)
        tensors["l0.mix.right.z"].mul_(0.1)
    if "l0.mix.f.b" in tensors:
        tensors["l0.mix.f.b"].fill_(7.0)
        tensors["l0.mix.i.b"].fill_(-2.0)
    if "l0.mix.w0" in tensors:
        tensors["l0.mix.w0"].fill_(-7.0)
        tensors["l0.mix.a.b"].fill_(-7.0)
        tensors["l0.mix.w2"].mul_(0.1)


def plant_needle(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Rewrites the tensors of the one-layer NEEDLE model in place so that the query of token PROBE_ID points where the key
    of token NEEDLE_ID points: queries read the first half of the normed row, keys the second half, through the same matrix
    rows; the probe's first half is the needle's second half; the convolutions pass the current token alone, the gains are
    one, and the norms over whole projections remove the lengths.  The rows of the rotated values of a head are small, so
    the position decides little.  The score of that pair is then about scale * dim = 16 against about 2 for random
    directions and a sink score of zero: where the window lets the probe see the needle, the probe's output is nearly the
    needle's value (turned by their distance), and a key or value that is not the one written for the needle shows far
    beyond rounding."""
    m = cfg["layers"][0]["mixer"]["left"]
    heads, kv, dim, width = m["heads"], m["kv_heads"], m["dim"], cfg["width"]
    half = width // 2
    wq, wk = tensors["l0.mix.left.q"], tensors["l0.mix.left.k"]
    wk[:, :half] = 0
    rot = m["rot"]["dims"]
    for g in range(kv):
        wk[g * dim:g * dim + rot] *= 0.1
    for h in range(heads):
        g = h // (heads // kv)
        wq[h * dim:(h + 1) * dim, :half] = wk[g * dim:(g + 1) * dim, half:]
    wq[:, half:] = 0
    for n in ("l0.mix.left.q.conv", "l0.mix.left.k.conv", "l0.mix.left.v.conv"):
        tensors[n].zero_()
        tensors[n][:, -1] = 1.0
    for n in ("l0.norm1", "l0.mix.left.q.norm", "l0.mix.left.k.norm"):
        tensors[n].fill_(1.0)
    tensors["l0.mix.left.sink"].zero_()
    emb = tensors["embed"]
    emb[PROBE_ID, :half] = emb[NEEDLE_ID, half:]


def needle_ids(cfg: dict, n: int, needle_at: int, seed: int) -> List[int]:
    """`n` random ids with the needle token at `needle_at` only and the probe token last only."""
    ids = [t if t not in (NEEDLE_ID, PROBE_ID) else FILLER_ID for t in ids_for(cfg, n, seed)]
    ids[needle_at] = NEEDLE_ID
    ids[-1] = PROBE_ID
    return ids


def plain_logits(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    from tests.plain import nasozen_plain
    return nasozen_plain.forward(cfg, tensors, ids)
