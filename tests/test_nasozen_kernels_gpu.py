"""The kernels that Nasozen added, each by itself against the plain functions of tests/plain/nasozen_plain.py (float64 on the
CPU): the step between two sublayers of a layer with several residual streams, the norms over whole projections with both
rotations, the turn back with the gate per head, learned sink scores in the attention kernel, the gated recurrence, and the two
matrix memories with their preparation, state carried from step to step."""
import math

import pytest
import torch

from tests.plain import nasozen_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"


def rnd(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
    assert err < tol, err


def steps_of(*lens_of_steps):
    """Three sequences in slots 2, 0, 3 and, in the middle of the list, one without tokens and without a slot."""
    for step, lens in enumerate(lens_of_steps):
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        cu = cu[:2] + cu[1:2] + cu[2:]
        yield step, lens, torch.tensor(cu, dtype=torch.int32, device=DEV), torch.tensor([2, -1, 0, 3], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,H", [(1, 40), (3, 36), (4, 260), (8, 48), (12, 20)])
def test_stream_step_rewrites_every_stream_from_the_old_ones_and_reads_for_the_next_sublayer(S, H, dtype):
    from llmgen_b200.kernels import ops
    dt, n = DT[dtype], 7
    xs = rnd((n, S, H), 1)
    mix, out, read, gain = rnd((S, S), 2, 0.5), rnd((S,), 3), rnd((S,), 4), 1 + rnd((H,), 5, 0.2)
    y1, y2 = rnd((n, H), 6, 1.0, dt), rnd((3, n, H), 7)
    forms = [("array", y1, y1.double()), ("slices", ops.Partials(y2.to(DEV)), y2.double().sum(0)),
             ("pair", ops.WeightedPair(y1.to(DEV), 0.6, ops.Partials(y2.to(DEV)), 1.1), 0.6 * y1.double() + 1.1 * y2.double().sum(0))]
    for name, y, y64 in forms:
        streams = xs.clone().to(DEV)
        normed = torch.zeros(n, H, dtype=dt, device=DEV)
        ops.stream_step(streams, y.to(DEV) if isinstance(y, torch.Tensor) else y, mix.to(DEV), out.to(DEV), read.to(DEV), gain.to(DEV), 1e-5, normed, dt)
        x64 = xs.double()
        new = torch.einsum("st,nsh->nth", mix.double(), x64) + out.double()[None, :, None] * y64[:, None, :]
        close(streams, new, 1e-6)
        want = plain.rmsnorm(torch.einsum("t,nth->nh", read.double(), new), gain.double(), 1e-5)
        close(normed, want, 1e-5 if dtype == "float32" else 1e-2)
    # either half alone: a read without a write leaves the streams; a write without a read touches nothing else
    streams = xs.clone().to(DEV)
    normed = torch.zeros(n, H, dtype=dt, device=DEV)
    ops.stream_step(streams, None, None, None, read.to(DEV), gain.to(DEV), 1e-5, normed, dt)
    assert torch.equal(streams.cpu(), xs)
    close(normed, plain.rmsnorm(torch.einsum("t,nth->nh", read.double(), xs.double()), gain.double(), 1e-5), 1e-5 if dtype == "float32" else 1e-2)
    ops.stream_step(streams, y1.to(DEV), mix.to(DEV), out.to(DEV), None, None, 0.0, None, dt)
    close(streams, torch.einsum("st,nsh->nth", mix.double(), xs.double()) + out.double()[None, :, None] * y1.double()[:, None, :], 1e-6)
    row = rnd((n, H), 9).to(DEV)
    ops.stream_spread(streams, row)
    assert all(torch.equal(streams[:, s], row) for s in range(S))
    streams.copy_(xs)
    ops.stream_spread(streams, row, collapse=True)
    close(row, xs.double().sum(1), 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nk,hd,vd,rot", [(4, 2, 16, 24, 8), (3, 3, 10, 6, 0), (8, 1, 32, 16, 32), (1, 1, 12, 20, 12)])
def test_norms_over_whole_projections_both_rotations_and_the_turn_back(nq, nk, hd, vd, rot, dtype):
    """q and k are normed over all heads at once; the first `rot` values of a head are turned; v is turned over all of its
    width and stored at the token's slot (shuffled pages); `unrotate_gate` turns a row back and applies one gate per head."""
    from llmgen_b200.kernels import ops
    dt, n, page, pages, base = DT[dtype], 9, 4, 6, 50.0
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    C = nq * hd + nk * (hd + vd)
    x = rnd((n, C + 3), 1)
    qg, kg = 1 + rnd((nq * hd,), 2, 0.3), 1 + rnd((nk * hd,), 3, 0.3)
    pos = torch.tensor([0, 1, 2, 40, 41, 7, 8, 9, 300], dtype=torch.int32)
    slots = torch.tensor([20, 21, 22, 3, -1, 9, 10, 11, 0], dtype=torch.int32)

    def table(dims):
        ang = torch.arange(512, dtype=torch.float64)[:, None] * base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        return ang.cos().float().to(DEV), ang.sin().float().to(DEV)

    cos, sin = table(rot) if rot else (None, None)
    vcos, vsin = table(vd) if rot else (None, None)
    kc = torch.full((pages, nk, page, hd), 7.0, dtype=dt, device=DEV)
    vc = torch.full((pages, nk, page, vd), 7.0, dtype=dt, device=DEV)
    q = torch.zeros(n, nq * hd, dtype=dt, device=DEV)
    ops.attn_prep_rows(x.to(DEV), q, kc, vc, pos.to(DEV), slots.to(DEV), cos, sin, vcos, vsin, qg.to(DEV), kg.to(DEV), nq, nk, hd, vd, rot, page, 1e-5)
    x64 = x.double()
    q64 = plain.rmsnorm(x64[:, :nq * hd], qg.double(), 1e-5).view(n, nq, hd)
    k64 = plain.rmsnorm(x64[:, nq * hd:(nq + nk) * hd], kg.double(), 1e-5).view(n, nk, hd)
    v64 = x64[:, (nq + nk) * hd:C].reshape(n, nk, vd)
    for t in range(n):
        p = int(pos[t])
        qt = plain.turn_halves(q64[t], p, rot, base) if rot else q64[t]
        close(q[t], qt.reshape(-1), tol)
        s = int(slots[t])
        if s < 0:
            continue
        kt = plain.turn_halves(k64[t], p, rot, base) if rot else k64[t]
        vt = plain.turn_halves(v64[t], p, vd, base) if rot else v64[t]
        close(kc[s // page, :, s % page], kt, tol)
        close(vc[s // page, :, s % page], vt, tol)
    used = {int(s) for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in used:
            assert float(kc[s // page, :, s % page].float().min()) == 7.0 and float(vc[s // page, :, s % page].float().max()) == 7.0
    o = rnd((n, nq * vd), 5, 1.0, dt)
    gate = rnd((n, nq + 2), 6, 1.0, dt)
    o_dev = o.clone().to(DEV)
    ops.unrotate_gate(o_dev, gate.to(DEV)[:, 1:nq + 1], pos.to(DEV), vcos, vsin, nq, vd)
    for t in range(n):
        back = plain.turn_halves(o[t].double().view(nq, vd), int(pos[t]), vd, base, sign=-1.0) if rot else o[t].double().view(nq, vd)
        close(o_dev[t], (back * torch.sigmoid(gate[t, 1:nq + 1].double())[:, None]).reshape(-1), tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_learned_sink_scores_enter_the_softmax_once_also_when_the_keys_come_in_parts(dtype):
    from llmgen_b200.kernels import ops
    dt, nq, nkv, hd, vd, page, n_keys = DT[dtype], 4, 2, 16, 8, 16, 300
    tol = 2e-5 if dtype == "float32" else 2e-2
    k = rnd((n_keys, nkv, hd), 1, 1.0, dt)
    v = rnd((n_keys, nkv, vd), 2, 1.0, dt)
    q = rnd((1, nq * hd), 3, 1.0, dt)
    sinks = torch.tensor([-2.0, 0.0, 1.5, 6.0])
    pages = (n_keys + page - 1) // page
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(4))
    kc = torch.zeros(pages, nkv, page, hd, dtype=dt)
    vc = torch.zeros(pages, nkv, page, vd, dtype=dt)
    for j in range(n_keys):
        kc[order[j // page], :, j % page], vc[order[j // page], :, j % page] = k[j], v[j]
    bt = order.to(torch.int32).to(DEV)
    ctx_len = torch.tensor([n_keys], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    tile_seq, tile_q0 = torch.tensor([0], dtype=torch.int32, device=DEV), torch.tensor([0], dtype=torch.int32, device=DEV)
    for window in (0, 70):
        first = max(0, n_keys - window) if window else 0
        want = torch.zeros(nq, vd, dtype=torch.float64)
        for h in range(nq):
            s = (k[first:, h // 2].double() @ q[0, h * hd:(h + 1) * hd].double()) * 0.25
            e = torch.exp(s - s.max())
            w = e / (e.sum() + math.exp(float(sinks[h]) - float(s.max())))
            want[h] = w @ v[first:, h // 2].double()
        for parts in (1, 3):
            out = torch.zeros(1, nq * vd, dtype=dt, device=DEV)
            scratch = torch.zeros(ops.attention_scratch_floats(1, nq, vd, parts), device=DEV) if parts > 1 else None
            ops.paged_attention(out, q.to(DEV), nq * hd, kc.to(DEV), vc.to(DEV), bt, pages, ctx_len, cu, tile_seq, tile_q0, 1, 1, nq, nkv, hd, page,
                                window, 0.25, parts, 0, scratch, vd=vd, sink=True, sink_values=sinks.to(DEV))
            close(out.view(nq, vd), want, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C", [7, 40, 300])
def test_the_gated_recurrence_carries_its_state_from_step_to_step(C, dtype):
    from llmgen_b200.kernels import ops
    dt = DT[dtype]
    bz, bx = rnd((C,), 1), rnd((C,), 2)
    state = torch.zeros(5, C + 2, device=DEV)
    state[1] = 7.0
    S = {i: None for i in range(3)}
    for step, lens, cu, slots in steps_of([5, 1, 9], [1, 2, 70], [2, 2, 1]):
        n = sum(lens)
        zxg = rnd((n + 2, 3 * C), 10 + step, 1.5)
        out = torch.full((n + 2, C), 3.0, dtype=dt, device=DEV)
        ops.min_gru(out, zxg.to(DEV), bz.to(DEV), bx.to(DEV), state, cu, slots, 4)
        at = 0
        for i, m in enumerate(lens):
            rows = zxg[at:at + m].double()
            z = torch.sigmoid(rows[:, :C] + bz.double())
            u = rows[:, C:2 * C] + bx.double()
            cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            all_s, S[i] = plain.min_gru_scan(z, cand, S[i])
            close(out[at:at + m], all_s * plain.silu(rows[:, 2 * C:]), 1e-5 if dtype == "float32" else 1e-2)
            at += m
        assert float(out[n:].float().min()) == 3.0                      # rows beyond the sequences
    for i, slot in enumerate((2, 0, 3)):
        close(state[slot, :C], S[i], 1e-5)
    assert float(state[1].min()) == 7.0 and float(state[:, C:].abs().sum()) == 14.0      # a slot nobody owns; columns beyond the state


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,E", [(3, 8, 12), (1, 6, 10), (2, 72, 40), (1, 20, 72), (2, 136, 8)])
def test_the_memory_under_a_running_maximum_step_by_step(H, D, E, dtype):
    from llmgen_b200.kernels import ops
    dt, cap = DT[dtype], 6.0
    # inputs are the same rounded values on both sides.  The largest outputs are those whose denominator |n . q| is what a
    # cancellation left, which float32 holds to fewer digits than the sums it came from
    tol = 1e-4
    bi, bf = rnd((H,), 1), rnd((H,), 2) + 2.0
    size = H * D * E + H * D + H
    state = torch.zeros(5, size + 1, device=DEV)
    state[1] = 7.0
    st = {i: None for i in range(3)}
    for step, lens, cu, slots in steps_of([5, 1, 9], [1, 2, 40], [2, 2, 1]):
        n = sum(lens)
        packed = rnd((n + 2, 2 * H * D + H * E + 2 * H), 20 + step, 1.0, dt)
        packed[:, -2 * H:] *= 4
        dev = packed.to(DEV)
        q, k, v = dev[:, :H * D], dev[:, H * D:2 * H * D], dev[:, 2 * H * D:2 * H * D + H * E]
        gi, gf = dev[:, -2 * H:-H], dev[:, -H:]
        gates = torch.zeros(n + 2, 4 * H, device=DEV)
        ops.mlstm_gates(gates, q, k, gi, gf, bi.to(DEV), bf.to(DEV), state[:, H * D * E + H * D:], cu, slots, 4, H, D, cap, D ** -0.5)
        o = torch.full((n + 2, H * E), 3.0, device=DEV)
        ops.memory_scan(o, q, k, v, None, gates, state, cu, slots, 4, H, D, E, "mlstm", r_scale=D ** -0.5, den_eps=1e-6)
        p64 = packed.double()
        at = 0
        for i, m in enumerate(lens):
            rows = p64[at:at + m]
            li = cap * torch.tanh((rows[:, -2 * H:-H] + bi.double()) / cap)
            lf = torch.nn.functional.logsigmoid(cap * torch.tanh((rows[:, -H:] + bf.double()) / cap))
            want, st[i] = plain.mlstm_memory(rows[:, :H * D].view(m, H, D) * D ** -0.5, rows[:, H * D:2 * H * D].view(m, H, D),
                                             rows[:, 2 * H * D:2 * H * D + H * E].view(m, H, E), li, lf, st[i])
            close(o[at:at + m], want.reshape(m, -1), tol)
            at += m
        assert float(o[n:].min()) == 3.0
    for i, slot in enumerate((2, 0, 3)):
        S, nn, mx = st[i]
        close(state[slot, :H * D * E], S.reshape(-1), tol)
        close(state[slot, H * D * E:H * D * E + H * D], nn.reshape(-1), tol)
        close(state[slot, H * D * E + H * D:size], mx, tol)
    assert float(state[1].min()) == 7.0 and float(state[:, size].abs().sum()) == 7.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D", [(2, 16), (1, 10), (4, 8), (1, 136), (2, 72)])
def test_the_generalized_delta_rule_step_by_step(H, D, dtype):
    from llmgen_b200.kernels import ops
    dt = DT[dtype]
    tol = 2e-5 if dtype == "float32" else 1e-4
    hd = H * D
    a_bias, w_bias = rnd((hd,), 1), rnd((hd,), 2) - 2.0
    scale = math.exp(-0.5)
    state = torch.zeros(5, hd * D + 1, device=DEV)
    state[1] = 7.0
    st = {i: None for i in range(3)}
    for step, lens, cu, slots in steps_of([5, 1, 9], [1, 2, 40], [2, 2, 1]):
        n = sum(lens)
        packed = rnd((n + 2, 4 * hd), 30 + step, 1.0, dt)
        decay = rnd((n + 2, hd), 40 + step, 2.0)
        dev = packed.to(DEV)
        r, k, v, a = (dev[:, i * hd:(i + 1) * hd] for i in range(4))
        aux, dots = torch.zeros(n + 2, 3 * hd, device=DEV), torch.zeros(n + 2, 2 * H, device=DEV)
        ops.delta_rule_prep(aux, dots, r, k, a, decay.to(DEV), a_bias.to(DEV), w_bias.to(DEV), cu, 4, H, D, scale, 1e-6)
        o = torch.full((n + 2, hd), 3.0, device=DEV)
        ops.memory_scan(o, r, k, v, aux, dots, state, cu, slots, 4, H, D, D, "delta")
        p64 = packed.double()
        at = 0
        for i, m in enumerate(lens):
            rows = p64[at:at + m]
            r64, k64, v64 = (rows[:, j * hd:(j + 1) * hd].view(m, H, D) for j in range(3))
            a64 = torch.sigmoid(rows[:, 3 * hd:] + a_bias.double()).view(m, H, D)
            w64 = torch.exp(-scale * torch.sigmoid(decay[at:at + m].double() + w_bias.double())).view(m, H, D)
            u64 = k64 / torch.sqrt((k64 * k64).sum(-1, keepdim=True) + 1e-6)
            want, st[i] = plain.delta_memory(r64, k64, v64, w64, a64, u64, st[i])
            close(o[at:at + m], want.reshape(m, -1), tol)
            at += m
        assert float(o[n:].min()) == 3.0
    for i, slot in enumerate((2, 0, 3)):
        close(state[slot, :hd * D], st[i].reshape(-1), tol)
    assert float(state[1].min()) == 7.0 and float(state[:, hd * D].abs().sum()) == 7.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vd", [64, 128])
def test_the_attention_kernel_turns_a_row_back_and_applies_the_gate_of_its_head(vd, dtype):
    """Value widths that the kernels finish themselves: the weighted sum of a head is turned back by minus the query's position
    and multiplied by one gate per head, in one part and when key parts are merged."""
    from llmgen_b200.kernels import ops
    dt, nq, nkv, hd, page, n_keys, base = DT[dtype], 4, 2, 16, 16, 200, 40.0
    tol = 2e-5 if dtype == "float32" else 2e-2
    k, v = rnd((n_keys, nkv, hd), 1, 1.0, dt), rnd((n_keys, nkv, vd), 2, 1.0, dt)
    q, gate = rnd((1, nq * hd), 3, 1.0, dt), rnd((1, nq), 4, 1.0, dt)
    sinks = torch.tensor([-1.0, 0.5, 2.0, 0.0])
    pages = (n_keys + page - 1) // page
    kc, vc = torch.zeros(pages, nkv, page, hd, dtype=dt), torch.zeros(pages, nkv, page, vd, dtype=dt)
    for j in range(n_keys):
        kc[j // page, :, j % page], vc[j // page, :, j % page] = k[j], v[j]
    ang = torch.arange(256, dtype=torch.float64)[:, None] * base ** (-2.0 * torch.arange(vd // 2, dtype=torch.float64) / vd)
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    bt = torch.arange(pages, dtype=torch.int32, device=DEV)
    ctx_len = torch.tensor([n_keys], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    one = torch.tensor([0], dtype=torch.int32, device=DEV)
    pos = torch.tensor([n_keys - 1], dtype=torch.int32, device=DEV)
    want = torch.zeros(nq, vd, dtype=torch.float64)
    for h in range(nq):
        s = (k[:, h // 2].double() @ q[0, h * hd:(h + 1) * hd].double()) * 0.25
        e = torch.exp(s - s.max())
        w = e / (e.sum() + math.exp(float(sinks[h]) - float(s.max())))
        row = plain.turn_halves(w @ v[:, h // 2].double(), n_keys - 1, vd, base, sign=-1.0)
        want[h] = row * torch.sigmoid(gate[0, h].double())
    for parts in (1, 2):
        out = torch.zeros(1, nq * vd, dtype=dt, device=DEV)
        scratch = torch.zeros(ops.attention_scratch_floats(1, nq, vd, parts), device=DEV) if parts > 1 else None
        ops.paged_attention(out, q.to(DEV), nq * hd, kc.to(DEV), vc.to(DEV), bt, pages, ctx_len, cu, one, one, 1, 1, nq, nkv, hd, page, 0, 0.25,
                            parts, 0, scratch, vd=vd, sink=True, sink_values=sinks.to(DEV), gate=gate.to(DEV), gate_per_head=True,
                            turn_back=(cos, sin), positions=pos)
        close(out.view(nq, vd), want, tol)
