"""The kernels that Fonuvik added, each by itself against the plain functions of tests/plain/fonuvik_plain.py (float64 on
the CPU): the blends of a token with the one before it, the recurrence with a decay per key channel in both orders of a
token's steps (whole sequences and segments side by side), and the sum of two mixers inside the norm that follows."""
import pytest
import torch

from tests.plain import fonuvik_plain as plain

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
@pytest.mark.parametrize("W,n_mix", [(48, 5), (36, 1), (260, 3)])
def test_token_shift_reads_the_last_row_of_the_step_before(W, n_mix, dtype):
    """A sequence's first token of a step is blended with the state's row (zeros for a new request), every other one
    with the row above; the sequence's last row is left in the state; slots nobody owns and rows beyond the sequences
    stay as they were."""
    from llmgen_b200.kernels import ops
    dt = DT[dtype]
    mu = rnd((n_mix, W), 1, 0.5)
    state = torch.zeros(5, W + 3, device=DEV)
    state[1] = 7.0
    prev = {i: torch.zeros(W, dtype=torch.float64) for i in range(3)}
    for step, lens, cu, slots in steps_of([5, 1, 9], [1, 2, 30], [2, 2, 1]):
        n = sum(lens)
        x = rnd((n + 2, W), 10 + step, 1.0, dt)
        out = torch.full((n_mix, n + 2, W), 3.0, dtype=dt, device=DEV)
        ops.token_shift_mix(out, x.to(DEV), mu.to(DEV), state, cu, slots, 4)
        at = 0
        for i, m in enumerate(lens):
            rows = x[at:at + m].double()
            before = torch.cat([prev[i].view(1, W), rows[:-1]])
            for j in range(n_mix):
                close(out[j, at:at + m], rows + (before - rows) * mu[j].double(), 1e-6 if dtype == "float32" else 1e-2)
            prev[i] = rows[-1]
            at += m
        assert bool((out[:, n:] == 3.0).all())
        for i, slot in enumerate((2, 0, 3)):
            close(state[slot, :W], prev[i], 1e-7)
        assert bool((state[1] == 7.0).all()) and bool((state[:, W:] == (torch.arange(5, device=DEV) == 1)[:, None] * 7.0).all())


def decay_inputs(n, H, D, E, seed, dtype, z_scale=1.0):
    dt = DT[dtype]
    q, k, v = rnd((n, H * D), seed, 1.0, dt), rnd((n, H * D), seed + 1, 1.0, dt), rnd((n, H * E), seed + 2, 1.0, dt)
    z = rnd((n, H * D), seed + 3, z_scale)
    return q, k, v, z


def plain_decays(z, bias, form, tau):
    x = z.double() + bias.double()
    return torch.exp(torch.nn.functional.logsigmoid(x) / tau) if form == "sigmoid_pow" else torch.exp(-torch.exp(x))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("form,read_first", [("sigmoid_pow", False), ("exp_exp", True)])
@pytest.mark.parametrize("H,D,E", [(2, 8, 12), (3, 40, 72), (1, 136, 8), (2, 64, 64), (1, 6, 10)])
def test_decay_scan_carries_its_state_between_calls(H, D, E, form, read_first, dtype):
    """Both orders of a token's steps, key widths of every register layout, value widths beyond a block's columns and no
    multiples of four; steps after the first, of a few rows (one launch that prepares and walks) and of more (two); a
    sequence without tokens or slot in the list."""
    from llmgen_b200.kernels import ops
    tau, q_scale = 3.0, 0.7
    bias = rnd((H * D,), 5, 0.5) + (2.0 if form == "sigmoid_pow" else -2.0)
    bonus = rnd((H * D,), 6, 1.0) if read_first else None
    state = torch.zeros(5, H * D * E + 5, device=DEV)
    state[1] = 7.0
    S = {i: torch.zeros(H, D, E, dtype=torch.float64) for i in range(3)}
    segments = torch.empty(ops.decay_scan_segment_floats(H, D, E), device=DEV)
    for step, lens, cu, slots in steps_of([5, 1, 19], [1, 2, 33], [17, 16, 1], [1, 1, 1], [3, 1, 2]):
        n = sum(lens)
        q, k, v, z = decay_inputs(n + 2, H, D, E, 20 + 10 * step, dtype)
        out = torch.full((n + 2, H * E), 3.0, device=DEV)
        zz = z.clone().to(DEV)
        ops.decay_scan(out, q.to(DEV), k.to(DEV), v.to(DEV), zz, bias.to(DEV), bonus.to(DEV) if read_first else None, state, cu, slots,
                       4, H, D, E, form, tau, q_scale, read_first, torch.empty(n + 2, 2 * H * D + H * E, device=DEV),
                       torch.empty(n + 2, 2 * H, device=DEV), segments)
        a = plain_decays(z, bias, form, tau)
        at = 0
        for i, m in enumerate(lens):
            rows = slice(at, at + m)
            want, S[i] = plain.decay_recurrence(q[rows].double().view(m, H, D) * q_scale, k[rows].double().view(m, H, D),
                                                v[rows].double().view(m, H, E), a[rows].view(m, H, D), S[i],
                                                bonus.double().view(H, D) if read_first else None)
            close(out[rows], want.reshape(m, H * E), 3e-6)
            at += m
        assert bool((out[n:] == 3.0).all())
        for i, slot in enumerate((2, 0, 3)):
            close(state[slot, :H * D * E], S[i].reshape(-1), 3e-6)
        assert bool((state[1] == 7.0).all())


@pytest.mark.parametrize("form,read_first", [("sigmoid_pow", False), ("exp_exp", True)])
@pytest.mark.parametrize("H,D,E,lens", [(2, 16, 24, [300, 0, 41]), (1, 72, 40, [64, 65, 400]), (2, 128, 16, [1, 700, 257])])
def test_decay_scan_in_segments_is_the_walk_from_first_to_last(H, D, E, lens, form, read_first):
    """Steps long enough for segments (a sequence of one segment beside sequences of several, the last segment of one
    token, of a whole segment, and ragged), after a step that left a state: outputs and states as the plain walk's, with
    decays close to one so that the first segment still counts in the last."""
    from llmgen_b200.kernels import ops
    tau, q_scale = 8.0, 0.5
    bias = rnd((H * D,), 5, 0.3) + (4.0 if form == "sigmoid_pow" else -6.0)
    bonus = rnd((H * D,), 6, 1.0) if read_first else None
    state = torch.zeros(4, H * D * E, device=DEV)
    S = {i: torch.zeros(H, D, E, dtype=torch.float64) for i in range(3)}
    segments = torch.empty(ops.decay_scan_segment_floats(H, D, E), device=DEV)
    for step, step_lens in enumerate(([3, 2, 5], lens)):
        n = sum(step_lens)
        cu = torch.tensor([0] + [sum(step_lens[:i + 1]) for i in range(3)], dtype=torch.int32, device=DEV)
        slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
        q, k, v, z = decay_inputs(n, H, D, E, 40 + step, "float32", 0.5)
        k = k * 0.2
        out = torch.full((n, H * E), 3.0, device=DEV)
        ops.decay_scan(out, q.to(DEV), k.to(DEV), v.to(DEV), z.clone().to(DEV), bias.to(DEV), bonus.to(DEV) if read_first else None, state,
                       cu, slots, 3, H, D, E, form, tau, q_scale, read_first, torch.empty(n, 2 * H * D + H * E, device=DEV),
                       torch.empty(n, 2 * H, device=DEV), segments)
        a = plain_decays(z, bias, form, tau)
        at = 0
        for i, m in enumerate(step_lens):
            if m:
                rows = slice(at, at + m)
                want, S[i] = plain.decay_recurrence(q[rows].double().view(m, H, D) * q_scale, k[rows].double().view(m, H, D),
                                                    v[rows].double().view(m, H, E), a[rows].view(m, H, D), S[i],
                                                    bonus.double().view(H, D) if read_first else None)
                close(out[rows], want.reshape(m, H * E), 5e-6)
            at += m
        for i, slot in enumerate((2, 0, 3)):
            close(state[slot], S[i].reshape(-1), 5e-6)
    assert float(a.min()) > 0.9          # the long sequences' first tokens still count at their end


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_mixers_are_added_inside_the_norm_that_follows(dtype):
    """resid += N(a y1 + b y2) * w, and the next sublayer's input N(resid) * w' beside it; `scaled_sum` adds the pair up
    for consumers that take one array."""
    from llmgen_b200.kernels import ops
    dt = DT[dtype]
    n, W, eps = 37, 52, 1e-5
    y1, y2 = rnd((n, W), 1, 1.0, dt), rnd((n, W), 2, 2.0, dt)
    resid = rnd((n, W), 3)
    w, w_next = rnd((W,), 4) + 1.0, rnd((W,), 5) + 1.0
    pair = ops.WeightedPair(y1.to(DEV), 1.3, y2.to(DEV), -0.4)
    r = resid.clone().to(DEV)
    copy = torch.empty(n, W, dtype=dt, device=DEV)
    ops.norm_add(r, pair, w.to(DEV), eps, copy, dt, next_gain=w_next.to(DEV), next_eps=eps)
    total = 1.3 * y1.double() - 0.4 * y2.double()
    want = resid.double() + plain.rms_norm(total, w.double(), eps)
    close(r, want, 2e-6)
    close(copy, plain.rms_norm(want, w_next.double(), eps), 2e-6 if dtype == "float32" else 1e-2)
    out = torch.empty(1, n, W, device=DEV)
    got = ops.scaled_sum(out, pair, dt)
    close(got.tensor[0], total, 2e-6)
