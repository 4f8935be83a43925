"""Fonuvik on the CPU: its typed configuration, the parts the registry makes of it, the tensors it declares, and the
plain implementation's own consistency (the recurrences against closed forms, the mask and the frequencies by hand)."""
import copy
import math

import pytest
import torch

from llmgen_b200.config.base import ConfigError
from llmgen_b200.parts.registry import model_weight_decls
from llmgen_b200.registry import config_from_dict
from tests import fonuvik_util as fu
from tests.plain import fonuvik_plain as plain


def spec_of(cfg):
    arch, typed = config_from_dict(cfg)
    return arch.build_spec(typed)


def test_the_registry_finds_the_architecture_and_the_parts_it_is_made_of():
    spec = spec_of(fu.MIXED)
    assert spec.architecture == "Fonuvik" and spec.lm_head == spec.embedding == "embed"
    assert spec.embedding_norm is not None and spec.embedding_norm.weight == "embed.norm"
    assert [layer.mixer.kind for layer in spec.layers] == ["token_shift_decay", "parallel", "token_shift_decay", "parallel"]
    assert [layer.ffn is not None for layer in spec.layers] == [True, True, False, True]
    assert [item.layer for item in spec.run_order] == [0, 1, 2, 3]
    par = spec.layers[1].mixer
    assert par.scales == (1.2, 0.7) and [b.kind for b in par.branches] == ["attention", "channel_decay_attention"]
    att, lin = par.branches
    assert att.chunk == 24 and att.v_head_dim == 24 and att.num_kv_heads == 2 and att.scale == 0.3 and att.unit_norm_eps == 1e-5
    assert att.position.rotary_dim == 8 and att.position.pairing == "interleaved" and att.position.scaling == (4.0, 1.0, 4.0, 64.0)
    assert (lin.num_heads, lin.key_dim, lin.value_dim, lin.tau, lin.decay_rank) == (2, 8, 12, 8.0, 4)
    assert spec.layers[3].mixer.branches[0].position.scaling is None
    ffn = spec.layers[1].ffn
    assert ffn.top_k == 3 and len(ffn.experts) == 5 and ffn.shared.intermediate_size == 32 and ffn.scoring == "softmax_top" and ffn.router_bias == "l1.mlp.router.b"
    assert spec.layers[3].ffn.shared is None
    assert spec_of(fu.ODD).layers[0].mixer.branches[0].position is None       # no rotation at all


def test_declared_tensors_have_the_design_s_names_and_shapes():
    shapes = {d.name: tuple(d.shape) for d in model_weight_decls(spec_of(fu.MIXED))}
    assert shapes["embed"] == (97, 48) and shapes["embed.norm"] == (48,) and shapes["final.norm"] == (48,)
    assert shapes["l0.mix.mu.w"] == (48,) and shapes["l0.mix.r"] == (64, 48) and shapes["l0.mix.o"] == (48, 64)
    assert shapes["l0.mix.w1"] == (5, 48) and shapes["l0.mix.w2"] == (64, 5) and shapes["l0.mix.w0"] == (64,)
    assert shapes["l0.mix.u"] == (4, 16) and shapes["l0.mix.norm"] == (64,)
    assert shapes["l1.mix.left.q"] == (64, 48) and shapes["l1.mix.left.k"] == (32, 48) and shapes["l1.mix.left.v"] == (48, 48)
    assert shapes["l1.mix.left.o"] == (48, 96)
    assert shapes["l1.mix.right.q"] == (16, 48) and shapes["l1.mix.right.v"] == (24, 48) and shapes["l1.mix.right.g"] == (24, 48)
    assert shapes["l1.mix.right.a1"] == (4, 48) and shapes["l1.mix.right.a2"] == (16, 4) and shapes["l1.mix.right.a2.b"] == (16,)
    assert shapes["l1.mix.right.norm"] == (12,) and shapes["l1.mix.right.o"] == (48, 24)
    assert shapes["l1.mlp.router"] == (5, 48) and shapes["l1.mlp.router.b"] == (5,) and shapes["l1.mlp.e4.down"] == (48, 24)
    assert shapes["l1.mlp.shared.gate"] == (32, 48) and "l3.mlp.shared.gate" not in shapes
    assert "l2.norm2" not in shapes and "l2.norm2b" not in shapes and shapes["l2.norm1b"] == (48,) and shapes["l3.norm2b"] == (48,)


def test_low_ranks_come_from_the_folder_s_tensor_shapes_when_the_file_does_not_name_them():
    from llmgen_b200.config.fonuvik import FonuvikConfig
    cfg = copy.deepcopy(fu.MIXED)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    del cfg["layers"][1]["mixer"]["right"]["decay_rank"]
    filled = FonuvikConfig.fill_from_tensor_shapes(cfg, {"l0.mix.w1": (7, 48), "l1.mix.right.a1": (9, 48)})
    spec = spec_of(filled)
    assert spec.layers[0].mixer.decay_rank == 7 and spec.layers[1].mixer.branches[1].decay_rank == 9
    assert spec.layers[2].mixer.decay_rank == 3                             # a rank the file names stays
    assert "decay_rank" not in cfg["layers"][0]["mixer"]                    # the caller's dict is left alone


def test_every_problem_of_a_configuration_is_listed_at_once():
    bad = copy.deepcopy(fu.MIXED)
    del bad["norm"]
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    bad["layers"][3]["mixer"]["left"]["rot"]["dims"] = 7
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["type"] = "conv"
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    assert "norm" in text and "kv_heads" in text and "rot.dims" in text and "top" in text and "type" in text


def test_the_plain_recurrences_agree_with_their_closed_forms():
    torch.manual_seed(0)
    T, W = 7, 6
    m = {"heads": 2, "dim": 3, "vdim": 2, "tau": 3.0}
    w = {n: torch.randn(s, dtype=torch.float64) * 0.5 for n, s in (("q", (6, W)), ("k", (6, W)), ("v", (4, W)), ("g", (4, W)), ("o", (W, 4)),
                                                                     ("a1", (2, W)), ("a2", (6, 2)), ("a2.b", (6,)), ("norm", (2,)))}
    h = torch.randn(T, W, dtype=torch.float64)
    out, S = plain.channel_decay_attention(h, w, m, 1e-5)
    a = torch.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"]).pow(1 / 3.0).view(T, 2, 3)
    k, v = (h @ w["k"].T).view(T, 2, 3), (h @ w["v"].T).view(T, 2, 2)
    want = sum(a[j + 1:].prod(dim=0)[:, :, None] * k[j][:, :, None] * v[j][:, None, :] for j in range(T))
    assert torch.allclose(S, want, atol=1e-12)
    # carried state: two halves give what the whole gives
    first, S1 = plain.channel_decay_attention(h[:3], w, m, 1e-5)
    second, S2 = plain.channel_decay_attention(h[3:], w, m, 1e-5, state=S1)
    assert torch.allclose(torch.cat([first, second]), out, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # the token-shift mixer: with all blends 0 nothing of the token before enters the projections, and the first
    # token's read-out is the bonus term alone: o_0 = (r_0 . (u * k_0)) v_0
    m2 = {"heads": 1, "dim": 3}
    w2 = {n: torch.randn(s, dtype=torch.float64) * 0.5 for n, s in (("r", (3, W)), ("k", (3, W)), ("v", (3, W)), ("g", (3, W)), ("o", (W, 3)),
                                                                      ("w1", (2, W)), ("w2", (3, 2)), ("w0", (3,)), ("u", (1, 3)), ("norm", (3,)))}
    for s in "rkvgw":
        w2["mu." + s] = torch.zeros(W, dtype=torch.float64)
    out2, last, S3 = plain.token_shift_decay(h, w2, m2, 1e-5)
    r0, k0, v0 = w2["r"] @ h[0], w2["k"] @ h[0], w2["v"] @ h[0]
    o0 = (r0 * w2["u"][0] * k0).sum() * v0
    want0 = (plain.rms_norm(o0, None, 1e-5) * w2["norm"] * plain.silu(w2["g"] @ h[0])) @ w2["o"].T
    assert torch.allclose(out2[0], want0, atol=1e-12) and torch.equal(last, h[-1])
    decay = torch.exp(-torch.exp(torch.tanh(h @ w2["w1"].T) @ w2["w2"].T + w2["w0"]))
    kk, vv = h @ w2["k"].T, h @ w2["v"].T
    want3 = sum(decay[j + 1:].prod(dim=0)[:, None] * kk[j][:, None] * vv[j][None, :] for j in range(T))
    assert torch.allclose(S3[0], want3, atol=1e-12)
    # with blends of one, every projection reads the token before
    for s in "rkvgw":
        w2["mu." + s] = torch.ones(W, dtype=torch.float64)
    shifted, _, _ = plain.token_shift_decay(h[1:], w2, m2, 1e-5, prev=h[0])
    for s in "rkvgw":
        w2["mu." + s] = torch.zeros(W, dtype=torch.float64)
    unshifted, _, _ = plain.token_shift_decay(h[:-1], w2, m2, 1e-5)
    assert torch.allclose(shifted, unshifted, atol=1e-12)


def test_the_plain_mask_and_frequencies_by_hand():
    # a block of 3: position 3 sees itself alone, position 5 sees 3, 4, 5; the weights are a softmax over those
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": 3}}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "o": eye}
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [2.0, 0.0], [0.0, 3.0], [1.0, 0.0]], dtype=torch.float64)
    out = plain.chunked_attention(h, w, m, 0.0)
    assert torch.allclose(out[3], h[3]) and torch.allclose(out[0], h[0])
    unit = h / h.pow(2).mean(dim=-1, keepdim=True).sqrt()
    p = torch.softmax(unit[3:6] @ unit[5], dim=0)
    assert torch.allclose(out[5], p @ h[3:6])
    # the wavelength rule: dims 8, base 100, original 32, low 1, high 4 -> waves below 8 stay, beyond 32 are divided
    f = plain.scaled_frequencies(100.0, 8, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32})
    raw = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    waves = [2 * math.pi / x for x in raw]
    assert waves[0] < 8 < waves[1] < 32 < waves[2]
    assert f[0] == raw[0] and f[2] == raw[2] / 8 and f[3] == raw[3] / 8
    s = (32 / waves[1] - 1.0) / 3.0
    assert abs(f[1] - ((1 - s) * raw[1] / 8 + s * raw[1])) < 1e-15 and raw[1] / 8 < f[1] < raw[1]
    # pairs (2i, 2i + 1) turn together; the values beyond the rotated ones pass
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0]]], dtype=torch.float64)
    y = plain.rotate_interleaved(x, [3], [0.5, 0.25])
    assert torch.allclose(y[0, 0], torch.tensor([math.cos(1.5), math.sin(1.5), -2 * math.sin(0.75), 2 * math.cos(0.75), 5.0], dtype=torch.float64))
    # the router: the largest logits choose, the weights are a softmax over them alone
    mlp = {"router": {"experts": 3, "top": 2}}
    wr = {"router": torch.tensor([[1.0], [3.0], [2.0]], dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 1.5], dtype=torch.float64)}
    for e in range(3):
        wr[f"e{e}.gate"] = torch.full((1, 1), 10.0, dtype=torch.float64)
        wr[f"e{e}.up"] = torch.full((1, 1), float(e + 1), dtype=torch.float64)
        wr[f"e{e}.down"] = torch.ones(1, 1, dtype=torch.float64)
    got = plain.routed_ff(torch.ones(1, 1, dtype=torch.float64), wr, mlp)
    pw = torch.softmax(torch.tensor([3.5, 3.0], dtype=torch.float64), dim=0)      # experts 2 and 1
    silu10 = 10.0 / (1.0 + math.exp(-10.0))
    assert torch.allclose(got, (pw[0] * 3.0 + pw[1] * 2.0) * silu10 * torch.ones(1, 1, dtype=torch.float64))
