"""Nasozen in plain, slow torch (float64 on the CPU): the oracle of the Nasozen tests.

One function per mechanism, written from the design's equations; it shares no code with the package.  A model is a
configuration dict (the keys of the architecture's config.json) and a dict of tensors by the names of a model folder.
Everything walks a sequence token by token where the design is a recurrence, and key by key where it is attention.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# --------------------------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rmsnorm(x, gain, eps):
    return rms_unit(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, taps):
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the first token."""
    T, C = u.shape
    K = taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def turn_halves(x, pos, dims, base, sign=1.0):
    """x [..., d]: the first `dims` values turned, value i with value i + dims/2, by sign * pos * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = sign * pos * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        lo, hi = x[..., i], x[..., i + half]
        out[..., i] = lo * c - hi * s
        out[..., i + half] = hi * c + lo * s
    return out


# --------------------------------------------------------------------------------------------- mixers
def windowed_sink_attention(h, p, m, eps):
    """The left branch of the parallel mixer.  h [T, W]; p: the branch's tensors by their last name."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if "conv" in m:
        q, k, v = short_conv(q, p["q.conv"]), short_conv(k, p["k.conv"]), short_conv(v, p["v.conv"])
    q = rmsnorm(q, p["q.norm"], eps).view(T, H, D)
    k = rmsnorm(k, p["k.norm"], eps).view(T, G, D)
    v = v.view(T, G, E)
    rot = m.get("rot")
    if rot is not None:
        q = torch.stack([turn_halves(q[t], t, rot["dims"], rot["base"]) for t in range(T)])
        k = torch.stack([turn_halves(k[t], t, rot["dims"], rot["base"]) for t in range(T)])
        v = torch.stack([turn_halves(v[t], t, E, rot["base"]) for t in range(T)])
    gate = torch.sigmoid(h @ p["g"].T)                       # [T, H]
    window = m["mask"]["size"] if m.get("mask") else None
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[first:i + 1, g] @ q[i, hh]) * m["scale"]
            top = max(float(s.max()), float(p["sink"][hh]))
            e = torch.exp(s - top)
            w = e / (e.sum() + math.exp(float(p["sink"][hh]) - top))
            o = (w[:, None] * v[first:i + 1, g]).sum(dim=0)
            if rot is not None:
                o = turn_halves(o, i, E, rot["base"], sign=-1.0)
            out[i, hh] = o * gate[i, hh]
    return out.reshape(T, H * E) @ p["o"].T


def min_gru(h, p):
    """The right branch of the parallel mixer."""
    T = h.shape[0]
    z = torch.sigmoid(h @ p["z"].T + p["z.b"])
    u = h @ p["x"].T + p["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = silu(h @ p["g"].T)
    return (min_gru_scan(z, cand)[0] * gate) @ p["o"].T


def min_gru_scan(z, cand, S=None):
    """S_t = (1 - z_t) S_(t-1) + z_t cand_t from S (zeros): every S_t, and the last one."""
    S = torch.zeros(z.shape[1], dtype=z.dtype) if S is None else S
    rows = []
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return torch.stack(rows), S


def parallel_mixer(h, p, m, eps):
    left = {n[len("left."):]: t for n, t in p.items() if n.startswith("left.")}
    right = {n[len("right."):]: t for n, t in p.items() if n.startswith("right.")}
    return m["left_scale"] * windowed_sink_attention(h, left, m["left"], eps) + m["right_scale"] * min_gru(h, right)


def heads_out(o, h, p, eps):
    """Each head's row divided by its root mean square, the heads side by side times the gains and the gate, W_o."""
    T = o.shape[0]
    y = rms_unit(o, eps).reshape(T, -1) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return y @ p["o"].T


def mlstm(h, p, m, eps):
    T = h.shape[0]
    H, D, E, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ p["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, E)
    gi = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    return heads_out(mlstm_memory(q, k, v, gi, gf)[0], h, p, eps)


def mlstm_memory(q, k, v, gi, gf, state=None):
    """q, k [T, H, D], v [T, H, E], log gates [T, H]; state (S, n, m) or None for zeros: every o_t and the last state."""
    T, H, D = q.shape
    E = v.shape[2]
    S, n, mx = state if state is not None else (torch.zeros(H, D, E, dtype=q.dtype), torch.zeros(H, D, dtype=q.dtype), torch.zeros(H, dtype=q.dtype))
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hde,hd->he", S, q[t]) / den[:, None]
    return o, (S, n, mx)


def general_delta(h, p, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ p["r"].T).view(T, H, D)
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, D)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ p["w1"].T) @ p["w2"].T + p["w0"])).view(T, H, D)
    a = torch.sigmoid(h @ p["a"].T + p["a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    return heads_out(delta_memory(r, k, v, w, a, u)[0], h, p, eps)


def delta_memory(r, k, v, w, a, u, S=None):
    """All [T, H, D]; S [H, D, D] or None for zeros: S_t = diag(w) S - (a u)(u^T S) + k v^T, o_t = S_t^T r; every o_t and the last S."""
    T, H, D = r.shape
    S = torch.zeros(H, D, v.shape[2], dtype=r.dtype) if S is None else S
    o = torch.zeros(T, H, v.shape[2], dtype=r.dtype)
    for t in range(T):
        seen = torch.einsum("hd,hde->he", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, r[t])
    return o, S


# --------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, p):
    return gelu_tanh(h @ p["up"].T) @ p["down"].T


def routed_ff(h, p, f):
    scores = torch.softmax(h @ p["router"].T, dim=-1)
    top = f["router"]["top"]
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        best = torch.topk(scores[t], top).indices
        total = scores[t][best].sum() + 1e-20
        for e in best.tolist():
            y = (silu(h[t] @ p[f"e{e}.gate"].T) * (h[t] @ p[f"e{e}.up"].T)) @ p[f"e{e}.down"].T
            out[t] += scores[t][e] / total * y
    return out


# --------------------------------------------------------------------------------------------- the model
def sub(tensors, prefix):
    return {n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)}


def run_mixer(kind, h, p, m, eps):
    if kind == "parallel":
        return parallel_mixer(h, p, m, eps)
    if kind == "mlstm":
        return mlstm(h, p, m, eps)
    if kind == "general_delta":
        return general_delta(h, p, m, eps)
    raise ValueError(kind)


def run_ff(h, p, f):
    return dense_ff(h, p) if f["kind"] == "dense" else routed_ff(h, p, f)


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    inside = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + inside * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token (float64), and, asked for, the stream (the sum of the
    streams) after every layer run."""
    tensors = {n: t.to(F64) for n, t in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x0 = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    n_streams = cfg.get("streams")
    xs = [x0.clone() for _ in range(n_streams or 1)]
    after = []
    for li in layer_order(cfg):
        layer, t = cfg["layers"][li], sub(tensors, f"l{li}.")
        subs = [(1, lambda h: run_mixer(layer["type"], h, sub(t, "mix."), layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda h: run_ff(h, sub(t, "mlp."), layer["mlp"])))
        for q, fn in subs:
            if n_streams is None:
                xs[0] = xs[0] + mult * fn(rmsnorm(xs[0], t[f"norm{q}"], eps))
                continue
            a_in, a_out, a_mix = t[f"hc{q}.in"], t[f"hc{q}.out"], t[f"hc{q}.mix"]
            u = sum(a_in[s] * xs[s] for s in range(n_streams))
            y = fn(rmsnorm(u, t[f"norm{q}"], eps))
            xs = [sum(a_mix[s, d] * xs[s] for s in range(n_streams)) + mult * a_out[d] * y for d in range(n_streams)]
        after.append(sum(xs))
    x = rmsnorm(sum(xs), tensors["final.norm"], eps)
    logits = x @ tensors["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
