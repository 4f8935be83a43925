"""Small Fonuvik configurations with random weights, for the tests: the engine's model and the tensors the plain
implementation reads, made from one seed."""
from __future__ import annotations

import copy
from typing import Dict, List, Sequence

import torch

from tests.derupel_util import TOL, driver, ids_for, relative_error, row_errors, run_in_portions  # noqa: F401


def left(heads, kv_heads, dim, vdim, scale, chunk, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def right(heads, dim, vdim, tau, decay_rank=4):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}


def parallel(left_m, right_m, mlp, scales=(1.2, 0.7)):
    return {"type": "parallel", "mixer": {"left": left_m, "right": right_m, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


def wkv(heads, dim, mlp, decay_rank=5):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": mlp}


def moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def config(layers, width=48, vocab=97, eps=1e-5) -> dict:
    return {"architecture": "Fonuvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(list(layers))}


# Both kinds of layer twice, sizes that differ from one another wherever they can: heads x dim of the token-shift mixer
# wider and narrower than the stream, key width != value width in both branches, grouped heads, half a head rotated with
# frequencies in all three ranges of the wavelength rule (short waves kept, long ones divided, some blended), a block of
# the mask that is no multiple of a page (16) or of anything else, a layer without a feed-forward, one without a shared
# expert, and scales of the two branches that differ.
MIXED = config([
    wkv(4, 16, moe(6, 2, 40, 56)),
    parallel(left(4, 2, 16, 24, 0.3, 24, rot=(300.0, 8), scaling=(4.0, 1.0, 4.0, 64)), right(2, 8, 12, 8.0), moe(5, 3, 24, 32)),
    wkv(2, 16, None, decay_rank=3),
    parallel(left(2, 1, 24, 8, 0.21, 10, rot=(5000.0, 24)), right(3, 12, 8, 2.5, decay_rank=6), moe(4, 1, 32), scales=(0.6, 1.5)),
], width=48)
# Sizes that are multiples of little (the products fall back from the TMA-fed kernels, vector loads to scalar ones), and
# values that a usual model makes equal or one: one head, as many key heads as heads, every expert chosen, one expert
# chosen of one, tau = 1, both scales 1, no rotation at all, a block of one position (every token sees itself alone), a
# block longer than any prompt here (plain causal attention), key and value widths that are no multiples of 4.
ODD = config([
    parallel(left(3, 3, 10, 6, 0.4, 1), right(1, 6, 10, 1.0, decay_rank=3), moe(3, 3, 20, 12), scales=(1.0, 1.0)),
    wkv(1, 10, moe(1, 1, 30), decay_rank=2),
    parallel(left(1, 1, 12, 20, 0.2, 4096, rot=(77.0, 12)), right(2, 10, 6, 3.0, decay_rank=1), None),
    wkv(3, 6, moe(7, 2, 10, 22)),
], width=36, vocab=50, eps=1e-4)
# Eight query heads on one key head; key widths beyond 64 and 128 in the recurrences (the kernel's wider forms), more
# value columns than one of its blocks takes (72), a key width that is no multiple of 8 (40).
WIDE = config([
    wkv(2, 72, None),
    parallel(left(8, 1, 32, 16, 0.18, 33, rot=(100.0, 32), scaling=(8.0, 1.0, 2.0, 32)), right(2, 40, 72, 16.0), moe(4, 2, 48, 24)),
    parallel(left(2, 2, 16, 16, 0.25, 7), right(1, 136, 8, 4.0), None, scales=(0.9, 1.1)),
], width=48, vocab=61, eps=1e-6)
# Key and value widths that the tensor-core attention of the bfloat16 engine takes (64 and 128, equal and not), with
# blocks of the mask that are no multiple of its tiles of 64 keys; prompts of a few hundred tokens then cross several
# tiles of keys and of queries, and several blocks of the mask begin inside a tile.
TENSOR = config([
    parallel(left(6, 3, 64, 64, 0.11, 96, rot=(10000.0, 32)), right(2, 16, 16, 8.0), moe(4, 2, 64, 64)),
    wkv(2, 32, None),
    parallel(left(2, 1, 128, 64, 0.09, 40, rot=(500.0, 128), scaling=(8.0, 1.0, 4.0, 128)), right(1, 16, 32, 4.0), None),
    parallel(left(2, 2, 64, 128, 0.125, 130), right(1, 8, 16, 2.0), None),
], width=64, vocab=97)
# One parallel layer whose weights `plant_needle` rewrites so that one token's query finds one other token's key.
NEEDLE_CHUNK = 48
NEEDLE = config([parallel(left(2, 1, 64, 16, 0.25, NEEDLE_CHUNK, rot=(30.0, 8)), right(1, 8, 8, 4.0), moe(3, 1, 32, 32), scales=(1.0, 0.2))],
                width=32, vocab=53)
NEEDLE_ID, PROBE_ID, FILLER_ID = 5, 9, 11
# States that keep (nearly) everything and nothing else to carry information over more than one token: losing a state,
# or a token of it, shows at every later position.
KEEPING_DECAY = config([parallel(left(1, 1, 8, 8, 0.3, 1), right(2, 8, 8, 4.0), None, scales=(0.1, 1.0))], width=32, vocab=53)
KEEPING_WKV = config([wkv(2, 8, None)], width=32, vocab=53)


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what="") -> None:
    """float32: every row within TOL.  bfloat16: four rows in five within TOL and the median within two thirds of it.
    A layer of this design norms what every sublayer returns, so the rounding of a sublayer's last product reaches the
    stream at full size whatever the sublayer's output was, eight times in four layers of width 48: the medians
    measured on requests alone, whole or token by token, lie between 0.016 and 0.032 (the highest on requests of under twenty tokens).  That noise on a router's input
    moves a logit across its neighbour for a few tokens in a hundred at each of three routed layers (a steeper router
    changes nothing: gap and noise grow together); such a token goes to another expert, which is a difference of some
    tenths at its row that no kernel caused, and it differs with the cut of the prompt.  What a fault costs is far more
    (the needle tests measure it), and the float32 engine is held to 2e-5 at every row."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, float(e.max()))
    else:
        assert float(e.quantile(0.8)) < TOL[dtype] and float(e.median()) < TOL[dtype] * 2 / 3, (what, float(e.quantile(0.8)), float(e.median()))


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
    """Makes the one-layer KEEPING models remember: the decays lie just below one (the sigmoid's bias far above zero,
    the double exponential's far below), and the writes stay small enough for hundreds of tokens."""
    if "l0.mix.right.a2.b" in tensors:
        tensors["l0.mix.right.a2.b"].fill_(9.0)
        tensors["l0.mix.right.a2"].mul_(0.1)
    if "l0.mix.w0" in tensors:
        tensors["l0.mix.w0"].fill_(-8.0)
        tensors["l0.mix.w2"].mul_(0.1)


def plant_needle(cfg: dict, tensors: Dict[str, torch.Tensor]) -> None:
    """Rewrites the tensors of the one-layer NEEDLE model in place so that the query of token PROBE_ID points where the
    key of token NEEDLE_ID points: queries read the first half of the normed residual row, keys the second half, through
    the same matrix rows; the gains of the two norms before the mixer are one, so the two halves differ by a factor that
    the per-head unit norm removes; the probe's first half is the needle's second half.  The matrix rows of the rotated
    values are small, so the position decides little.  The score of that pair is then about scale * dim = 16 against
    about 2 for random directions: where the mask lets the probe see the needle, the probe's output is nearly the
    needle's value, and a key or value that is not the one written for the needle shows far beyond rounding."""
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
    for n in ("l0.norm1", "embed.norm"):
        tensors[n].fill_(1.0)
    emb = tensors["embed"]
    emb[PROBE_ID, :half] = emb[NEEDLE_ID, half:]


def needle_ids(cfg: dict, n: int, needle_at: int, seed: int) -> List[int]:
    """`n` random ids with the needle token at `needle_at` only and the probe token last only."""
    ids = [t if t not in (NEEDLE_ID, PROBE_ID) else FILLER_ID for t in ids_for(cfg, n, seed)]
    ids[needle_at] = NEEDLE_ID
    ids[-1] = PROBE_ID
    return ids


def plain_logits(cfg: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    from tests.plain import fonuvik_plain
    return fonuvik_plain.forward(cfg, tensors, ids)
