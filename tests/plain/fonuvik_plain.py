"""A plain, slow implementation of the Fonuvik decoder: whole sequences, no cache, no state carried between calls,
one function per mechanism, float64 (or float32) on the CPU.  It shares no code with `llmgen_b200`: tensors come in
as a dict, the configuration as the parsed config.json.

Notation: h is a sublayer's input [T, width]; W_x is the tensor `<layer>.mix.x` or `<layer>.mlp.x`, stored [out, in]
and applied as h W^T.  N(x, g) = x / sqrt(mean(x^2) + eps) * g;  U(x) = N(x, 1).

    embedding      x = N(embed[id], g_embed)
    layer          x <- x + N(mixer(N(x, g1)), g1b);  x <- x + N(ff(N(x, g2)), g2b)  (the second only with a ff)
    parallel       a_left * chunked_attention(h) + a_right * channel_decay_attention(h)
    chunked_attention
                   q, k, v = h W^T; the first `dims` values of a head turned in pairs (2i, 2i+1) by pos * f_i, f_i the
                   scaled frequencies; then U(q), U(k) per head; s = q.k * scale; softmax over the keys j <= i of the
                   same block of `size` positions; concat heads, Wo
    channel_decay_attention
                   q = h Wq^T / sqrt(dim), k, v; a = sigmoid(W_a2 W_a1 h + b)^(1/tau) [heads, dim];
                   S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t; (N_head(o, g) * silu(h Wg^T)) Wo^T
    token_shift_decay
                   m_s = h + (h_prev - h) * mu_s for s in r, k, v, g, w; r, k, v = W m; gate = silu(Wg m_g);
                   w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0)); o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;
                   S_t = diag(w_t) S_(t-1) + k_t v_t^T; (U_head(o) * g_norm * gate) Wo^T
    routed ff      z = Wr h + b; the `top` largest z choose; weights softmax over the chosen z; expert
                   Wd (silu(Wg h) * Wu h); plus the shared expert
    logits         N(x, g_final) embed^T
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def rms_norm(x: torch.Tensor, gain, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


def scaled_frequencies(base: float, dims: int, scaling: Optional[dict]) -> List[float]:
    """f_i = base^(-2i/dims), then the wavelength rule: short waves stay, long waves are divided by `factor`, and
    the ones between are blended."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_interleaved(x: torch.Tensor, positions: Sequence[int], freqs: Sequence[float]) -> torch.Tensor:
    """x [T, heads, >= 2 len(freqs)]: values 2i and 2i + 1 of a head turned by position * freqs[i]."""
    out = x.clone()
    pos = torch.tensor(list(positions), dtype=x.dtype)
    for i, f in enumerate(freqs):
        ang = pos * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def chunked_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int = 0) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = (h @ w["v"].T).view(T, G, E)
    positions = list(range(pos0, pos0 + T))
    rot = m.get("rot")
    if rot is not None:
        freqs = scaled_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q = rotate_interleaved(q, positions, freqs)
        k = rotate_interleaved(k, positions, freqs)
    q = rms_norm(q, None, eps)
    k = rms_norm(k, None, eps)
    size = int(m["mask"]["size"])
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for i in range(T):
        first = (positions[i] // size) * size - pos0
        lo = max(first, 0)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * float(m["scale"])
            p = torch.softmax(s, dim=0)
            out[i, hh] = p @ v[lo:i + 1, g]
    return out.reshape(T, H * E) @ w["o"].T


def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, state: Optional[torch.Tensor] = None,
                     bonus: Optional[torch.Tensor] = None):
    """q, k, a [T, heads, dim], v [T, heads, vdim]; S [heads, dim, vdim] starts at `state` or zero.
    Without `bonus`: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.
    With `bonus` u [heads, dim]: o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t, then the same update.
    Returns (o [T, heads, vdim], the last S)."""
    T, H, D = q.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        if bonus is not None:
            o[t] = torch.einsum("hde,hd->he", S + bonus[:, :, None] * kv, q[t])
        S = a[t][:, :, None] * S + kv
        if bonus is None:
            o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o, S


def channel_decay_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                            state: Optional[torch.Tensor] = None):
    """Returns (output [T, width], final state [heads, dim, vdim])."""
    T = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, E)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    a = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).view(T, H, D)
    o, S = decay_recurrence(q, k, v, a, state)
    o = rms_norm(o, w["norm"], eps).reshape(T, H * E)
    return (o * silu(h @ w["g"].T)) @ w["o"].T, S


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    left = chunked_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right, _ = channel_decay_attention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def token_shift_decay(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, prev: Optional[torch.Tensor] = None,
                      state: Optional[torch.Tensor] = None):
    """Returns (output [T, width], last input row, final state [heads, dim, dim])."""
    T, W = h.shape
    H, D = m["heads"], m["dim"]
    first = torch.zeros(1, W, dtype=h.dtype) if prev is None else prev.view(1, W)
    hp = torch.cat([first, h[:-1]], dim=0)
    mix = {s: h + (hp - h) * w["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].T).view(T, H, D)
    k = (mix["k"] @ w["k"].T).view(T, H, D)
    v = (mix["v"] @ w["v"].T).view(T, H, D)
    gate = silu(mix["g"] @ w["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).view(T, H, D)
    u = w["u"].view(H, D)
    o, S = decay_recurrence(r, k, v, decay, state, bonus=u)
    o = rms_norm(o, None, eps).reshape(T, H * D) * w["norm"]
    return (o * gate) @ w["o"].T, h[-1].clone(), S


def gated_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict, route_on: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`route_on`: the rows the router sees, where they differ from the experts' input (a rounded copy)."""
    T = h.shape[0]
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = (h if route_on is None else route_on) @ w["router"].T + w["router.b"]
    out = torch.zeros_like(h)
    for t in range(T):
        order = sorted(range(n), key=lambda e: (-float(z[t, e]), e))[:top]
        p = torch.softmax(z[t, order], dim=0)
        for c, e in enumerate(order):
            out[t] += p[c] * gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence from position 0.  `layers_out`: a list that receives the residual stream
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = rms_norm(w["embed"][torch.tensor(list(ids), dtype=torch.long)], w["embed.norm"], eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            y = parallel_mixer(h, sub(w, p + "mix."), layer["mixer"], eps)
        elif layer["type"] == "wkv":
            y, _, _ = token_shift_decay(h, sub(w, p + "mix."), layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + rms_norm(routed_ff(h, sub(w, p + "mlp."), layer["mlp"]), w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
