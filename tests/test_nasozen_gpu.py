"""Nasozen through the engine against the plain implementation (tests/plain/nasozen_plain.py, float64 on the CPU):
whole prompts, portions, token by token, batches, pages and state slots used again, graphs replayed, generation."""
import copy

import pytest
import torch

from tests import nasozen_util as nu

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "WIDE", "ODD", "PLAIN"])
def test_whole_prompt_and_portions_match_the_plain_model(name, dtype):
    cfg = getattr(nu, name)
    model, tensors = nu.build(cfg, seed=3, dtype=dtype)
    ids = nu.ids_for(cfg, 75, seed=1)
    want = nu.plain_logits(cfg, tensors, ids)
    drv = nu.driver(model, dtype)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [len(ids)]), want, dtype)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [33, 2, 1, 17, 1]), want, dtype)


def one_mechanism(which: str) -> dict:
    """One layer of MIXED alone, or its parallel layer with one branch silenced (a scale of zero)."""
    if which in ("delta", "dense"):
        layer = copy.deepcopy(nu.MIXED["layers"][0])
        if which == "delta":
            layer["mlp"] = None
        return nu.config([layer])
    if which == "mlstm":
        layer = copy.deepcopy(nu.MIXED["layers"][2])
        layer["mlp"] = None
        return nu.config([layer], streams=2)
    layer = copy.deepcopy(nu.MIXED["layers"][1])
    if which == "routed":
        return nu.config([layer])
    layer["mlp"] = None
    layer["mixer"]["left_scale"], layer["mixer"]["right_scale"] = (1.3, 0.0) if which == "left" else (0.0, 0.8)
    return nu.config([layer], streams=4 if which == "left" else None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["left", "right", "mlstm", "delta", "dense", "routed"])
def test_each_mechanism_in_a_layer_of_its_own(which, dtype):
    cfg = one_mechanism(which)
    model, tensors = nu.build(cfg, seed=21, dtype=dtype, sigma=0.2)
    ids = nu.ids_for(cfg, 90, seed=8)
    want = nu.plain_logits(cfg, tensors, ids)
    drv = nu.driver(model, dtype)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [90]), want, dtype, which)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [40, 1, 1, 7, 2]), want, dtype, which)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_any_size_and_single_tokens_give_the_whole_prompts_logits(dtype):
    cfg = nu.MIXED
    model, tensors = nu.build(cfg, seed=4, dtype=dtype)
    ids = nu.ids_for(cfg, 101, seed=2)
    want = nu.plain_logits(cfg, tensors, ids)
    drv = nu.driver(model, dtype)
    for portions in ([1], [2], [3, 2, 33, 31, 1, 16, 2], [32, 32, 5, 1], [47, 1, 1, 2], [24, 24, 10, 10, 1]):
        got = nu.run_in_portions(drv, "a", ids, portions)
        nu.assert_close(got, want, dtype, portions)
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_that_cross_tiles_of_the_tensor_core_attention(dtype, eager):
    """300 tokens whole, in portions whose tiles of queries begin anywhere among the keys' tiles and the windows' edges, and
    beside another request; launched and replayed."""
    cfg = nu.TENSOR
    model, tensors = nu.build(cfg, seed=15, dtype=dtype)
    ids, other = nu.ids_for(cfg, 300, seed=5), nu.ids_for(cfg, 90, seed=6)
    want, want_other = nu.plain_logits(cfg, tensors, ids), nu.plain_logits(cfg, tensors, other)
    drv = nu.driver(model, dtype, pool_tokens=448, eager=eager)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [300]), want, dtype)
    nu.assert_close(nu.run_in_portions(drv, "a", ids, [130, 70, 1, 2, 97]), want, dtype)
    got_a = [drv.step([("a", ids[:200], list(range(200)))])]
    out = drv.step([("a", ids[200:], list(range(100))), ("b", other, list(range(90)))], end=["a", "b"])
    nu.assert_close(torch.cat([got_a[0], out[:100]]), want, dtype)
    nu.assert_close(out[100:], want_other, dtype)


def test_the_logits_do_not_depend_on_the_cut_beyond_rounding():
    """float32: token by token, in twos and whole agree far inside the tolerance against the plain model."""
    cfg = nu.WIDE
    model, _ = nu.build(cfg, seed=14, dtype="float32")
    ids = nu.ids_for(cfg, 80, seed=3)
    drv = nu.driver(model, "float32")
    whole = nu.run_in_portions(drv, "a", ids, [80])
    for portions in ([1], [2], [17, 3], [33, 33, 1]):
        assert nu.relative_error(nu.run_in_portions(drv, "a", ids, portions), whole) < 2e-6, portions


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_match_each_alone(dtype, eager):
    """Three requests of different lengths, portions of some beside single tokens of others; launched kernel by kernel and
    replayed from the graphs of the steps' shapes."""
    cfg = nu.MIXED
    model, tensors = nu.build(cfg, seed=5, dtype=dtype)
    ids = {"a": nu.ids_for(cfg, 70, 11), "b": nu.ids_for(cfg, 19, 12), "c": nu.ids_for(cfg, 41, 13)}
    want = {r: nu.plain_logits(cfg, tensors, t) for r, t in ids.items()}
    drv = nu.driver(model, dtype, eager=eager)
    plan = {"a": [33, 1, 1, 2, 30, 1, 1, 1], "b": [2, 1, 1, 1, 14], "c": [1, 1, 17, 2, 20]}
    pos = {r: 0 for r in ids}
    got = {r: [] for r in ids}
    k = 0
    while any(pos[r] < len(ids[r]) for r in ids):
        entries, owners, end = [], [], []
        for r in ids:
            if pos[r] >= len(ids[r]) or (r == "b" and k == 2):          # b sits one step out
                continue
            n = min(plan[r][min(k, len(plan[r]) - 1)], len(ids[r]) - pos[r])
            entries.append((r, ids[r][pos[r]:pos[r] + n], list(range(n))))
            owners.append((r, n))
            pos[r] += n
            if pos[r] == len(ids[r]):
                end.append(r)
        out = drv.step(entries, end=end)
        at = 0
        for r, n in owners:
            got[r].append(out[at:at + n])
            at += n
        k += 1
    for r in ids:
        nu.assert_close(torch.cat(got[r]), want[r], dtype, r)
    if not eager:
        assert drv.executor.n_shaped_steps > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_state_slots_are_used_again(dtype):
    """A pool of 6 pages and 2 state slots, five requests one after and beside another: every page and slot serves several
    requests, and a request that starts in a used slot starts from empty states and no token before its first."""
    cfg = nu.MIXED
    model, tensors = nu.build(cfg, seed=6, dtype=dtype)
    drv = nu.driver(model, dtype, pool_tokens=96, page_size=16, max_num_seqs=2)
    lengths = [40, 50, 33, 17, 48]
    all_ids = [nu.ids_for(cfg, n, 20 + i) for i, n in enumerate(lengths)]
    want = [nu.plain_logits(cfg, tensors, t) for t in all_ids]
    slots_seen = set()
    got0 = nu.run_in_portions(drv, 0, all_ids[0], [13, 27])
    nu.assert_close(got0, want[0], dtype)
    for a, b in ((1, 2), (3, 4)):
        ga, gb = [], []
        pa = pb = 0
        while pa < lengths[a] or pb < lengths[b]:
            entries = []
            na = min(11, lengths[a] - pa)
            nb = min(20 if pb == 0 else 1, lengths[b] - pb)
            if na:
                entries.append((a, all_ids[a][pa:pa + na], list(range(na))))
            if nb:
                entries.append((b, all_ids[b][pb:pb + nb], list(range(nb))))
            pa, pb = pa + na, pb + nb
            end = [r for r, p, n in ((a, pa, na), (b, pb, nb)) if n and p == lengths[r]]
            out = drv.step(entries, end=[])
            slots_seen |= {drv.executor.cache.state.slot(r) for r, _, _ in entries}
            for r in end:
                drv.executor.release(r)
                del drv.positions[r]
            if na:
                ga.append(out[:na])
            if nb:
                gb.append(out[na:na + nb])
        nu.assert_close(torch.cat(ga), want[a], dtype, a)
        nu.assert_close(torch.cat(gb), want[b], dtype, b)
    assert slots_seen == {0, 1}
    assert drv.executor.cache.all_free()


def plain_with_window(cfg, tensors, ids, size):
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["left"]["mask"]["size"] = size
    return nu.plain_logits(other, tensors, ids)


# (tokens, the needle's place, pages of): the probe is the last token and sees the NEEDLE_WINDOW = 40 positions up to itself
EDGES = [
    (300, 260, 16),     # the oldest key of the window: just inside
    (300, 259, 16),     # the key before it: just outside
    (300, 298, 16),     # the newest but one
    (300, 0, 16),       # far away
    (289, 249, 32),     # just inside, the window's edge inside a page
    (289, 248, 32),     # just outside
    (273, 233, 16),     # the probe opens a page; just inside
    (272, 232, 16),     # the probe closes a page; just inside
    (272, 231, 16),     # just outside, the last key of the page before the window's first
    (41, 0, 16),        # the first key of all, just outside
    (40, 0, 16),        # and just inside
    (30, 0, 16),        # a prompt shorter than the window
]


@pytest.mark.parametrize("n,needle_at,page", EDGES)
def test_one_key_decides_inside_the_window_and_not_outside(n, needle_at, page):
    """The last token's query finds the key of one token only (`plant_needle`).  Where that key lies in the probe's window,
    the probe's logits follow the needle's value; where it lies outside (one position is enough), they must not: the plain
    model with a wider window then differs by hundreds of tolerances, as it does without the needle when the needle is
    inside.  Whole, in portions cut at and beside the needle and the window's edge, and with the probe decoded alone after
    single tokens."""
    cfg = nu.NEEDLE
    model, tensors = nu.build(cfg, seed=7, dtype="float32", sigma=0.3, prepare=nu.plant_needle)
    ids = nu.needle_ids(cfg, n, needle_at, 31)
    want = nu.plain_logits(cfg, tensors, ids)
    inside = (n - 1) - needle_at < nu.NEEDLE_WINDOW
    if inside:
        without = list(ids)
        without[needle_at] = nu.FILLER_ID
        assert nu.relative_error(nu.plain_logits(cfg, tensors, without)[-1:], want[-1:]) > 100 * nu.TOL["float32"]
    else:
        assert nu.relative_error(plain_with_window(cfg, tensors, ids, 4096)[-1:], want[-1:]) > 100 * nu.TOL["float32"]
    drv = nu.driver(model, "float32", pool_tokens=320, page_size=page)
    edge = max(n - nu.NEEDLE_WINDOW, 0)
    cuts = {(n,), (max(needle_at, 1), 1, 2, n), (needle_at + 1, 1, n), (max(n - 10, 1),) + (1,) * 10, (max(n - 45, 1),) + (1,) * 45}
    if edge > 1:
        cuts |= {(edge, n), (edge - 1, 2, n), (edge + 1, n)}
    for portions in sorted(cuts):
        got = nu.run_in_portions(drv, "a", ids, list(portions))
        assert nu.relative_error(got, want) < nu.TOL["float32"], portions
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("eager", [True, False])
def test_the_needle_in_the_bfloat16_engine_and_beside_other_requests(eager):
    """The tensor-core attention of the bfloat16 engine takes this layer's widths: the needle just inside and just outside
    the probe's window, two requests in one step; launched and replayed."""
    cfg = nu.NEEDLE
    model, tensors = nu.build(cfg, seed=7, dtype="bfloat16", sigma=0.3, prepare=nu.plant_needle)
    n = 300
    ids_in, ids_out = nu.needle_ids(cfg, n, 260, 31), nu.needle_ids(cfg, n, 259, 32)
    want_in, want_out = nu.plain_logits(cfg, tensors, ids_in), nu.plain_logits(cfg, tensors, ids_out)
    # what a fault would cost at the probe, against which the bfloat16 engine's error is small
    cost = min(nu.relative_error(plain_with_window(cfg, tensors, ids_out, 4096)[-1:], want_out[-1:]),
               nu.relative_error(plain_with_window(cfg, tensors, ids_in, 39)[-1:], want_in[-1:]))
    assert cost > 5 * nu.TOL["bfloat16"]
    drv = nu.driver(model, "bfloat16", pool_tokens=640, eager=eager)
    for first in (n, 290, 280):
        a = [drv.step([("a", ids_in[:first], list(range(first))), ("b", ids_out[:first], list(range(first)))],
                      end=["a", "b"] if first == n else [])]
        for t in range(first, n):
            a.append(drv.step([("a", ids_in[t:t + 1], [0]), ("b", ids_out[t:t + 1], [0])], end=["a", "b"] if t == n - 1 else []))
        got_in = torch.cat([a[0][:first]] + [x[:1] for x in a[1:]])
        got_out = torch.cat([a[0][first:]] + [x[1:] for x in a[1:]])
        nu.assert_close(got_in, want_in, "bfloat16", first)
        nu.assert_close(got_out, want_out, "bfloat16", first)
        assert nu.relative_error(got_in[-1:], want_in[-1:]) < nu.TOL["bfloat16"]
        assert nu.relative_error(got_out[-1:], want_out[-1:]) < nu.TOL["bfloat16"]


@pytest.mark.parametrize("name", ["KEEPING_GRU", "KEEPING_MLSTM", "KEEPING_DELTA"])
def test_a_state_that_forgets_little_is_carried_through_portions_and_long_decoding(name):
    cfg = getattr(nu, name)
    model, tensors = nu.build(cfg, seed=8, dtype="float32", prepare=nu.keep_long)
    ids = nu.ids_for(cfg, 400, 41)
    want = nu.plain_logits(cfg, tensors, ids)
    drv = nu.driver(model, "float32", pool_tokens=448)
    for portions in ([400], [31, 33, 32, 1, 2, 64, 1], [100] + [1] * 300):
        got = nu.run_in_portions(drv, "a", ids, portions)
        assert nu.relative_error(got, want) < nu.TOL["float32"], portions[:3]
    # a state lost where a portion was cut would show at the next token: the plain model started there differs
    for cut in (31, 100, 398):
        restarted = nu.plain_logits(cfg, tensors, ids[cut:cut + 2])
        assert nu.relative_error(restarted[:1], want[cut:cut + 1]) > 100 * nu.TOL["float32"], cut
    # and the first token still counts at the end: without it the last logits differ
    shifted = nu.plain_logits(cfg, tensors, ids[1:])
    assert nu.relative_error(shifted[-1:], want[-1:]) > 5 * nu.TOL["float32"]


@pytest.mark.parametrize("name", ["MIXED", "ODD", "PLAIN"])
def test_the_first_tokens_of_a_sequence(name):
    """One, two and three tokens: zeros before the start of a convolution, memories and maxima that start from nothing, a
    lone key against the sink."""
    cfg = getattr(nu, name)
    model, tensors = nu.build(cfg, seed=9, dtype="float32")
    drv = nu.driver(model, "float32")
    for n in (1, 2, 3, 6):
        ids = nu.ids_for(cfg, n, 50 + n)
        for portions in ([1], [n]):
            got = nu.run_in_portions(drv, "a", ids, portions)
            assert nu.relative_error(got, nu.plain_logits(cfg, tensors, ids)) < nu.TOL["float32"], (n, portions)


@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine_and_its_scheduler(eager):
    """`LLM.generate` (scheduler, chunked prompts, decode graphs, sampling kernel) against greedy decoding with the plain
    model."""
    from llmgen_b200.engine.api import LLM
    from llmgen_b200.sampling.params import SamplingParams
    cfg = nu.MIXED
    model, tensors = nu.build(cfg, seed=10, dtype="float32")
    prompts = [nu.ids_for(cfg, n, 60 + n) for n in (9, 21, 4)]
    new = 10
    ref = []
    for p in prompts:
        seq = list(p)
        for _ in range(new):
            seq.append(int(nu.plain_logits(cfg, tensors, seq)[-1].argmax()))
        ref.append(seq[len(p):])
    llm = LLM(model, dtype="float32", max_model_len=64, max_num_seqs=2, max_batched_tokens=64, pass_tokens=64, block_size=16,
              kv_blocks=8, policy="chunked", chunk=8, eager=eager, capture_at_start=False)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o["token_ids"] for o in outs] == ref
    assert llm.executor.cache.all_free()
    if not eager:
        assert llm.executor.n_graph_steps > 0


def test_a_model_folder_through_the_replay_program_and_the_command_line(tmp_path):
    """A Nasozen folder written by the random-weights mode, with the low rank left to the tensors' shapes: `bin/trace_run`
    replays a trace of five requests on four state slots and a pool smaller than their sum (float32 logits against the
    plain model), and `python -m llmgen_b200 chat` generates the plain model's greedy tokens."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors.torch import load_file

    from llmgen_b200.engine.api import write_random_model
    from tests.util import ROOT
    cfg = nu.MIXED
    folder = write_random_model(str(tmp_path / "model"), cfg, seed=13, sigma=0.1, sigma_norm=0.2)
    path = os.path.join(folder, "config.json")
    with open(path) as f:
        written = json.load(f)
    assert written["architecture"] == "Nasozen"
    for layer in written["layers"]:          # as a folder from elsewhere has it: the shapes say the low rank
        layer["mixer"].pop("decay_rank", None)
    with open(path, "w") as f:
        json.dump(written, f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    lengths = [70, 40, 23, 64, 51]
    ids = [nu.ids_for(cfg, n, 70 + i) for i, n in enumerate(lengths)]
    want = [nu.plain_logits(cfg, tensors, t) for t in ids]
    steps, pos, live, waiting = [], [0] * 5, [0, 1, 2, 3], [4]
    portions = [17, 2, 1, 30, 1, 1, 64]
    k = 0
    while live:
        entries, ended = [], []
        for r in live:
            n = min(portions[(k + r) % len(portions)], lengths[r] - pos[r])
            entries.append((r, pos[r], pos[r] + n))
            pos[r] += n
            if pos[r] == lengths[r]:
                ended.append(r)
        steps.append((entries, ended))
        live = [r for r in live if r not in ended]
        if ended and waiting:
            live.append(waiting.pop(0))
        k += 1
    lines = [json.dumps({"step": i, "entries": [{"id": f"r{r}", "tokens": ids[r][lo:hi], "want": list(range(hi - lo))} for r, lo, hi in entries],
                         "end": [f"r{r}" for r in ended]}) for i, (entries, ended) in enumerate(steps)]
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
                           "--max-tokens", "256"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    for i, (entries, _) in enumerate(steps):
        got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
        ref = torch.cat([want[r][lo:hi] for r, lo, hi in entries])
        assert nu.relative_error(got, ref) < nu.TOL["float32"], i
    prompt, new = ids[2][:9], 8
    seq = list(prompt)
    for _ in range(new):
        seq.append(int(nu.plain_logits(cfg, tensors, seq)[-1].argmax()))
    proc = subprocess.run([sys.executable, "-m", "llmgen_b200", "chat", ",".join(map(str, prompt)), str(new), "--model", folder, "--dtype", "float32",
                           "--max-model-len", "64", "--max-num-seqs", "2", "--max-batched-tokens", "64", "--kv-blocks", "8"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    printed = [l.split() for l in proc.stdout.splitlines() if l.split() and all(t.lstrip("-").isdigit() for t in l.split())]
    assert printed and [int(t) for t in printed[-1]] == seq[len(prompt):], proc.stdout[-2000:]
