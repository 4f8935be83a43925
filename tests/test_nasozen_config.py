"""Nasozen on the CPU: its typed configuration, the parts the registry makes of it, the tensors it declares, and the plain
implementation's own consistency (the memories against other forms of the same sums, the window and the rotation by hand)."""
import copy
import math

import pytest
import torch

from llmgen_b200.config.base import ConfigError
from llmgen_b200.parts.registry import model_weight_decls
from llmgen_b200.registry import config_from_dict
from tests import nasozen_util as nu
from tests.plain import nasozen_plain as plain


def spec_of(cfg):
    arch, typed = config_from_dict(cfg)
    return arch.build_spec(typed)


def test_the_registry_finds_the_architecture_and_the_parts_it_is_made_of():
    spec = spec_of(nu.MIXED)
    assert spec.architecture == "Nasozen" and spec.lm_head == spec.embedding == "embed" and spec.residual_streams == 3
    assert [layer.kind for layer in spec.layers] == ["multi_stream"] * 4
    assert [layer.mixer.kind for layer in spec.layers] == ["general_delta", "parallel", "mlstm", "general_delta"]
    assert [layer.ffn.kind if layer.ffn is not None else None for layer in spec.layers] == ["dense_mlp", "routed_mlp", "routed_mlp", None]
    assert [item.layer for item in spec.run_order] == [0, 1, 2, 1, 2, 3]
    assert [item.cache for item in spec.run_order] == [0, 1, 2, 3, 4, 5] and all(item.before is None for item in spec.run_order)
    assert all(layer.streams == 3 and layer.residual_mult == 0.8 for layer in spec.layers)
    assert spec.layers[1].mixer_streams.mix == "l1.hc1.mix" and spec.layers[1].ffn_streams.read == "l1.hc2.in" and spec.layers[3].ffn_streams is None
    par = spec.layers[1].mixer
    assert par.scales == (0.7, 1.2) and [b.kind for b in par.branches] == ["attention", "min_gru"]
    att, gru = par.branches
    assert att.window == 24 and att.v_head_dim == 24 and att.num_kv_heads == 2 and att.scale == 0.3 and att.conv.taps == 3
    assert att.conv.channels == 4 * 16 + 2 * 16 + 2 * 24 and att.row_norms and att.rotate_values and att.gate_per_head and att.sink
    assert att.q_norm.dim == 64 and att.k_norm.dim == 32 and att.sink_scores == "l1.mix.left.sink"
    assert att.position.rotary_dim == 8 and att.position.pairing == "half" and att.position.theta == 300.0
    assert gru.width == 40
    mem = spec.layers[2].mixer
    assert (mem.num_heads, mem.key_dim, mem.value_dim, mem.gate_cap, mem.den_eps) == (3, 8, 12, 10.0, 1e-6)
    rule = spec.layers[3].mixer
    assert (rule.num_heads, rule.head_dim, rule.decay_rank) == (4, 8, 3) and abs(rule.decay_scale - math.exp(-0.5)) < 1e-15
    ffn = spec.layers[1].ffn
    assert ffn.top_k == 2 and len(ffn.experts) == 6 and ffn.scoring == "softmax" and ffn.renormalize and not ffn.weight_on_input
    assert spec.layers[0].ffn.activation == "gelu_tanh"
    odd = spec_of(nu.ODD)
    assert odd.layers[0].mixer.branches[0].position is None and not odd.layers[0].mixer.branches[0].rotate_values
    assert odd.layers[0].mixer.branches[0].window is None and odd.residual_streams == 1 and odd.layers[0].mixer_streams is not None
    bare = spec_of(nu.PLAIN)
    assert bare.layers[0].mixer_streams is None and bare.layers[0].streams == 1 and bare.residual_streams == 1
    assert [item.layer for item in bare.run_order] == [0, 1, 0, 1, 0, 1, 2]


def test_declared_tensors_have_the_design_s_names_and_shapes():
    shapes = {d.name: tuple(d.shape) for d in model_weight_decls(spec_of(nu.MIXED))}
    assert shapes["embed"] == (97, 48) and shapes["final.norm"] == (48,) and "head" not in shapes
    assert shapes["l0.hc1.in"] == (3,) and shapes["l0.hc2.out"] == (3,) and shapes["l0.hc1.mix"] == (3, 3)
    assert shapes["l0.mix.r"] == (32, 48) and shapes["l0.mix.a"] == (32, 48) and shapes["l0.mix.a.b"] == (32,)
    assert shapes["l0.mix.w1"] == (5, 48) and shapes["l0.mix.w2"] == (32, 5) and shapes["l0.mix.w0"] == (32,) and shapes["l0.mix.norm"] == (32,)
    assert shapes["l0.mlp.up"] == (40, 48) and shapes["l0.mlp.down"] == (48, 40)
    assert shapes["l1.mix.left.q"] == (64, 48) and shapes["l1.mix.left.k"] == (32, 48) and shapes["l1.mix.left.v"] == (48, 48)
    assert shapes["l1.mix.left.q.norm"] == (64,) and shapes["l1.mix.left.k.norm"] == (32,) and shapes["l1.mix.left.sink"] == (4,)
    assert shapes["l1.mix.left.q.conv"] == (64, 3) and shapes["l1.mix.left.v.conv"] == (48, 3) and shapes["l1.mix.left.g"] == (4, 48)
    assert shapes["l1.mix.left.o"] == (48, 96)
    assert shapes["l1.mix.right.z"] == (40, 48) and shapes["l1.mix.right.x.b"] == (40,) and shapes["l1.mix.right.o"] == (48, 40)
    assert shapes["l2.mix.q"] == (24, 48) and shapes["l2.mix.v"] == (36, 48) and shapes["l2.mix.i"] == (3, 48) and shapes["l2.mix.f.b"] == (3,)
    assert shapes["l2.mix.norm"] == (36,) and shapes["l2.mix.o"] == (48, 36)
    assert shapes["l1.mlp.router"] == (6, 48) and shapes["l1.mlp.e5.down"] == (48, 24) and shapes["l2.mlp.e4.gate"] == (16, 48)
    assert "l3.norm2" not in shapes and "l3.hc2.in" not in shapes and shapes["l3.hc1.mix"] == (3, 3)
    assert not any(n.startswith("l0.hc") for n in {d.name for d in model_weight_decls(spec_of(nu.PLAIN))})


def test_the_low_rank_comes_from_the_folder_s_tensor_shapes_when_the_file_does_not_name_it():
    from llmgen_b200.config.nasozen import NasozenConfig
    cfg = copy.deepcopy(nu.MIXED)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    filled = NasozenConfig.fill_from_tensor_shapes(cfg, {"l0.mix.w1": (7, 48), "l3.mix.w1": (9, 48)})
    assert filled["layers"][0]["mixer"]["decay_rank"] == 7 and filled["layers"][3]["mixer"]["decay_rank"] == 3
    assert "decay_rank" not in cfg["layers"][0]["mixer"]


def test_every_problem_of_a_configuration_is_listed_at_once():
    cfg = copy.deepcopy(nu.MIXED)
    cfg["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    cfg["layers"][1]["mixer"]["left"]["rot"]["dims"] = 7
    cfg["layers"][2]["mixer"].pop("gate_cap")
    cfg["layers"][1]["mlp"]["router"]["top"] = 9
    cfg["loop"]["stop"] = 11
    cfg["streams"] = 20
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    text = str(e.value)
    for piece in ("kv_heads", "rot.dims", "gate_cap", "top 9", "loop", "streams"):
        assert piece in text, piece
    bad = copy.deepcopy(nu.MIXED)
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_the_plain_memories_agree_with_other_forms_of_the_same_sums():
    """mLSTM: with gates that never need the maximum (small inputs), the memory is a plain weighted sum of k v^T; the delta
    rule: with no removal and decays of one it is the sum of k v^T."""
    torch.manual_seed(0)
    T, W, H, D, E = 9, 12, 2, 4, 6
    h = torch.randn(T, W, dtype=torch.float64)
    p = {n: torch.randn(s, dtype=torch.float64) * 0.3 for n, s in (("q", (H * D, W)), ("k", (H * D, W)), ("v", (H * E, W)), ("g", (H * E, W)),
                                                                  ("o", (W, H * E)), ("i", (H, W)), ("f", (H, W)), ("i.b", (H,)), ("f.b", (H,)))}
    p["norm"] = torch.ones(H * E, dtype=torch.float64)
    m = {"heads": H, "dim": D, "vdim": E, "gate_cap": 15.0}
    got = plain.mlstm(h, p, m, 1e-5)
    q = (h @ p["q"].T).view(T, H, D) * D ** -0.5
    k, v = (h @ p["k"].T).view(T, H, D), (h @ p["v"].T).view(T, H, E)
    li = 15.0 * torch.tanh((h @ p["i"].T + p["i.b"]) / 15.0)
    lf = torch.nn.functional.logsigmoid(15.0 * torch.tanh((h @ p["f"].T + p["f.b"]) / 15.0))
    o = torch.zeros(T, H, E, dtype=torch.float64)
    for t in range(T):
        for hh in range(H):
            # unnormalised: weights exp(i_s + sum of f after s); the design's maximum only rescales numerator and denominator
            logw = torch.stack([li[s, hh] + lf[s + 1:t + 1, hh].sum() for s in range(t + 1)])
            mx = max(float(logw.max()), float(lf[:t + 1, hh].sum()))     # the running maximum started at zero, decayed
            w = torch.exp(logw - mx)
            S = sum(w[s] * torch.outer(k[s, hh], v[s, hh]) for s in range(t + 1))
            n = sum(w[s] * k[s, hh] for s in range(t + 1))
            o[t, hh] = (S.T @ q[t, hh]) / (max(abs(float(n @ q[t, hh])), math.exp(-mx)) + 1e-6)
    want = plain.heads_out(o, h, p, 1e-5)
    # the running maximum of the design equals max over s of (log weight) and of the decayed start: same numbers
    assert float((got - want).abs().max()) < 1e-9
    Dd = 4
    pd = {n: torch.randn(s, dtype=torch.float64) * 0.3 for n, s in (("r", (H * Dd, W)), ("k", (H * Dd, W)), ("v", (H * Dd, W)), ("g", (H * Dd, W)),
                                                                    ("o", (W, H * Dd)), ("a", (H * Dd, W)), ("w1", (3, W)), ("w2", (H * Dd, 3)))}
    pd["norm"] = torch.ones(H * Dd, dtype=torch.float64)
    pd["a.b"] = torch.full((H * Dd,), -60.0, dtype=torch.float64)       # no removal
    pd["w0"] = torch.full((H * Dd,), -60.0, dtype=torch.float64)        # decays of one
    got = plain.general_delta(h, pd, {"heads": H, "dim": Dd}, 1e-5)
    r, k, v = ((h @ pd[n].T).view(T, H, Dd) for n in "rkv")
    o = torch.stack([torch.stack([sum(torch.outer(k[s, hh], v[s, hh]) for s in range(t + 1)).T @ r[t, hh] for hh in range(H)]) for t in range(T)])
    assert float((got - plain.heads_out(o, h, pd, 1e-5)).abs().max()) < 1e-9


def test_the_plain_attention_s_window_sink_and_rotations_by_hand():
    """Two tokens, one head, no convolution beyond the current token: the weights are exp(s) / (sum + exp(sink)); a window of
    one leaves the token itself; the value turned by j and the output turned back by i leave a rotation by j - i."""
    torch.manual_seed(1)
    W, D, E = 6, 4, 4
    h = torch.randn(2, W, dtype=torch.float64)
    p = {"q": torch.randn(D, W, dtype=torch.float64), "k": torch.randn(D, W, dtype=torch.float64), "v": torch.randn(E, W, dtype=torch.float64),
         "g": torch.zeros(1, W, dtype=torch.float64), "o": torch.eye(E, dtype=torch.float64), "sink": torch.tensor([0.3], dtype=torch.float64),
         "q.norm": torch.ones(D, dtype=torch.float64), "k.norm": torch.ones(D, dtype=torch.float64)}
    for n in "qkv":
        p[n + ".conv"] = torch.tensor([[0.0, 1.0]] * p[n].shape[0], dtype=torch.float64)
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": E, "scale": 0.5, "conv": 2, "rot": {"base": 10.0, "dims": 2}}
    got = plain.windowed_sink_attention(h, p, m, 1e-5)
    q = plain.rms_unit(h @ p["q"].T, 1e-5)
    k = plain.rms_unit(h @ p["k"].T, 1e-5)
    v = h @ p["v"].T

    def turn(x, a):      # dims 2: values 0 and 1 of the head are one pair
        out = x.clone()
        out[0], out[1] = x[0] * math.cos(a) - x[1] * math.sin(a), x[1] * math.cos(a) + x[0] * math.sin(a)
        return out

    q1, k0, k1 = turn(q[1], 1.0), turn(k[0], 0.0), turn(k[1], 1.0)
    s = torch.stack([q1 @ k0, q1 @ k1]) * 0.5
    w = torch.exp(s) / (torch.exp(s).sum() + math.exp(0.3))

    def turn_value(x, pos):   # pairs (0, 2) and (1, 3), frequencies 10^(-2m/4)
        out = x.clone()
        for mm in range(2):
            a = pos * 10.0 ** (-2.0 * mm / 4)
            out[mm], out[mm + 2] = x[mm] * math.cos(a) - x[mm + 2] * math.sin(a), x[mm + 2] * math.cos(a) + x[mm] * math.sin(a)
        return out

    want1 = 0.5 * (w[0] * turn_value(v[0], -1.0) + w[1] * v[1])           # gate sigmoid(0) = 1/2
    assert float((got[1] - want1).abs().max()) < 1e-12
    m1 = dict(m, mask={"size": 1})
    alone = plain.windowed_sink_attention(h, p, m1, 1e-5)
    w_self = math.exp(float(s[1])) / (math.exp(float(s[1])) + math.exp(0.3))
    assert float((alone[1] - 0.5 * w_self * v[1]).abs().max()) < 1e-12
