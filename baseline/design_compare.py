"""`bench.py --designs`: Derupel (or, with `--designs-family sarulix`, `fonuvik` or `nasozen`, that design) beside Qwen3 at equal
layer sizes, random weights, one B200; `--designs-beside` names another design to stand beside it (Nasozen stands beside
Fonuvik, the closest model, unless told otherwise).

For each size two models are built: a Derupel whose layers alternate its two mixers and its two feed-forwards (a Sarulix
whose four layers are a recurrent unit, the delta rule, attention and a recurrent unit again, each with a feed-forward,
entered once through its loop's mixing step; a Fonuvik whose layers alternate the parallel mixer and the token-shift
mixer, each with a routed feed-forward whose chosen and shared experts together are as wide as the dense one; a Nasozen of
four residual streams whose layers are the parallel mixer, the generalized delta rule, the parallel mixer and the matrix
memory under a running maximum, three with a routed feed-forward and one with a dense one), and the
Qwen3 of the same width, depth, feed-forward width and vocabulary.
Measured for both:

  prefill   one prompt of 2,048 tokens through one step (the graph of its shape replayed), tokens/s and ms
  decode    steps of 8 single tokens at contexts from 512 upward through the decode graphs, tokens/s and ms a step
  kernels   every kernel binding's device time, GFLOP/s and GB/s in an eager prompt step and eager decode steps
            (`engine.profiler.OpProfiler`: launches serialised by the marks between them), with the fraction of the
            measured peaks (MEASURED_PEAKS.json; the recipe's fallback when the file is absent)

Inputs: the weights (hundreds of MB) exceed L2, so nothing is flushed between timed iterations.  Prints one JSON line.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

SIZES = {
    # width, layers, heads, head width, feed-forward width, experts, top, expert width, q_rank, kv_rank, rotated width
    "w1024": dict(width=1024, layers=4, heads=8, hd=128, ff=3072, experts=16, top=2, expert_ff=768, q_rank=384, kv_rank=256, rot=64),
    "w2048": dict(width=2048, layers=4, heads=16, hd=128, ff=6144, experts=32, top=4, expert_ff=1024, q_rank=768, kv_rank=512, rot=64),
}
VOCAB = 32000
PROMPT = 2048
CONTEXT = 4096


def derupel_config(s: dict) -> dict:
    decay = [1.0 - 2.0 ** (-3 - 5 * h / max(s["heads"] - 1, 1)) for h in range(s["heads"])]
    lightning = {"heads": s["heads"], "dim": s["hd"], "vdim": s["hd"], "decay": decay}
    latent = {"heads": s["heads"], "dim": s["hd"], "rot_dim": s["rot"], "vdim": s["hd"], "q_rank": s["q_rank"], "kv_rank": s["kv_rank"],
              "scale": (s["hd"] + s["rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": s["rot"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"], "limit": 7.0},
           "shared": {"ff": s["expert_ff"], "limit": 7.0}}
    layers = []
    for i in range(s["layers"]):
        layers.append({"type": "lightning" if i % 2 == 0 else "latent_attention", "mixer": lightning if i % 2 == 0 else latent,
                       "mlp": dense if (i // 2) % 2 == 0 else moe})
    return {"architecture": "Derupel", "vocab": VOCAB, "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": layers, "max_positions": CONTEXT}


def sarulix_config(s: dict) -> dict:
    W, heads, hd = s["width"], s["heads"], s["hd"]
    dense = {"kind": "dense", "ff": s["ff"]}
    lru = {"type": "rglru", "mixer": {"width": W, "blocks": heads, "conv": 4}, "mlp": dense}
    delta = {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": hd, "vdim": hd, "conv": 4,
                                                "decay_rank": 64, "gate_rank": 64}, "mlp": dense}
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                                          "softcap": 30.0, "rot": {"base": 10000.0, "dims": hd // 2}}, "mlp": dense}
    layers = [lru, delta, att, lru][: s["layers"]] + [lru] * max(0, s["layers"] - 4)
    return {"architecture": "Sarulix", "vocab": VOCAB, "width": W, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_scale": 1.0, "loop": {"start": 0, "stop": len(layers), "times": 1}, "layers": layers, "max_positions": CONTEXT}


def fonuvik_config(s: dict) -> dict:
    W, heads, hd = s["width"], s["heads"], s["hd"]
    routed = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]},
              "shared": {"ff": s["ff"] - s["top"] * s["expert_ff"]}}
    left = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": 1024},
            "rot": {"base": 500000.0, "dims": hd // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": max(1, heads // 2), "dim": hd, "vdim": hd, "tau": 16.0, "decay_rank": 64}
    par = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.5}, "mlp": routed}
    shift = {"type": "wkv", "mixer": {"heads": W // 64, "dim": 64, "decay_rank": 64}, "mlp": routed}
    layers = [par if i % 2 == 0 else shift for i in range(s["layers"])]
    return {"architecture": "Fonuvik", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6}, "layers": layers, "max_positions": CONTEXT}


def nasozen_config(s: dict) -> dict:
    W, heads, hd = s["width"], s["heads"], s["hd"]
    routed = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    left = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": hd, "vdim": hd, "scale": hd ** -0.5, "conv": 4, "mask": {"size": 1024},
            "rot": {"base": 500000.0, "dims": hd // 2}}
    par = {"type": "parallel", "mixer": {"left": left, "right": {"width": W}, "left_scale": 1.0, "right_scale": 0.5}, "mlp": routed}
    rule = {"type": "general_delta", "mixer": {"heads": W // 64, "dim": 64, "decay_rank": 64}, "mlp": routed}
    memory = {"type": "mlstm", "mixer": {"heads": max(1, heads // 2), "dim": hd, "vdim": hd, "gate_cap": 12.0}, "mlp": dense}
    layers = ([par, rule, par, memory] * s["layers"])[: s["layers"]]
    return {"architecture": "Nasozen", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.8, "streams": 4,
            "layers": layers, "max_positions": CONTEXT}


FAMILIES = {"derupel": derupel_config, "sarulix": sarulix_config, "fonuvik": fonuvik_config, "nasozen": nasozen_config}
# the design that stands beside a family's where it is not Qwen3: the framework's closest model
BESIDE = {"nasozen": "fonuvik"}


def qwen3_config(s: dict) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": VOCAB, "hidden_size": s["width"],
            "intermediate_size": s["ff"], "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"],
            "num_key_value_heads": max(1, s["heads"] // 2), "head_dim": s["hd"], "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "max_position_embeddings": CONTEXT, "tie_word_embeddings": False, "hidden_act": "silu"}


def _peaks(root: str) -> Dict[str, float]:
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d.get("hbm_gbs", 6650.0)), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _throughput(torch, model, batch: int, steps: int, warmup: int, seed: int) -> dict:
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    import numpy as np
    rng = np.random.default_rng(seed)
    V = model.spec.vocab_size
    ex = Executor(model, EngineLimits(max_num_seqs=batch, max_model_len=CONTEXT, max_step_tokens=PROMPT, page_size=16,
                                      num_pages=batch * CONTEXT // 16))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(warmup + 3):                          # prefill: one prompt a step, the last three timed
        ids = rng.integers(0, V, PROMPT).tolist()
        assert ex.admit("p") and ex.reserve("p", 0, PROMPT)
        torch.cuda.synchronize()
        start.record()
        ex.step([StepEntry("p", ids, 0, [PROMPT - 1])], sample=True, return_logits=False)
        end.record()
        torch.cuda.synchronize()
        ex.release("p")
        if i >= warmup:
            times.append(start.elapsed_time(end))
    prefill_ms = sorted(times)[len(times) // 2]
    reqs = list(range(batch))
    P = 512
    toks = []
    for r in reqs:
        assert ex.admit(r) and ex.reserve(r, 0, P + warmup + steps + 1)
        toks.append(ex.step([StepEntry(r, rng.integers(0, V, P).tolist(), 0, [P - 1])], sample=True, return_logits=False).token_ids[0])
    pos = P
    launches = 0
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches = ex.launch_count
            start.record()
        toks = ex.step([StepEntry(r, [t], pos, [0]) for r, t in zip(reqs, toks)], sample=True, return_logits=False).token_ids
        pos += 1
    end.record()
    torch.cuda.synchronize()
    decode_ms = start.elapsed_time(end) / steps
    out = {"prefill_tokens": PROMPT, "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PROMPT / prefill_ms * 1e3),
           "decode_batch": batch, "decode_ms_per_step": round(decode_ms, 4), "decode_tokens_per_s": round(batch / decode_ms * 1e3),
           "decode_launches_per_step": (ex.launch_count - launches) // steps, "graph_steps": ex.n_graph_steps}
    for r in reqs:
        ex.release(r)
    del ex
    return out


def _kernels(torch, model, batch: int, peaks: Dict[str, float], seed: int) -> Dict[str, List[dict]]:
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.profiler import DECODE, PREFILL, OpProfiler
    import numpy as np
    rng = np.random.default_rng(seed)
    V = model.spec.vocab_size
    ex = Executor(model, EngineLimits(max_num_seqs=batch, max_model_len=CONTEXT, max_step_tokens=PROMPT, page_size=16,
                                      num_pages=batch * CONTEXT // 16), eager=True)
    reqs = list(range(batch))

    def run():
        toks = []
        for r in reqs:
            assert ex.admit(r) and ex.reserve(r, 0, PROMPT + 8)
            ids = rng.integers(0, V, PROMPT if r == 0 else 512).tolist()
            toks.append((len(ids), ex.step([StepEntry(r, ids, 0, [len(ids) - 1])], sample=True, return_logits=False).token_ids[0]))
        for k in range(4):
            out = ex.step([StepEntry(r, [t], n + k, [0]) for r, (n, t) in zip(reqs, toks)], sample=True, return_logits=False).token_ids
            toks = [(n, t) for (n, _), t in zip(toks, out)]
        for r in reqs:
            ex.release(r)
    run()                                                # warm-up: loads every kernel, creates the workspaces
    prof = OpProfiler().enable()
    ex.profiler = prof
    try:
        run()
    finally:
        prof.disable()
        ex.profiler = None
    tables = {}
    for phase in (PREFILL, DECODE):
        rows = []
        for r in prof.rows(phase):
            rows.append({"op": r["op"], "calls": r["calls"], "avg_us": round(r["avg_us"], 2), "pct": round(r["pct"], 1),
                         "tflops": round(r["gflops"] / 1e3, 2), "gbs": round(r["gbps"], 1),
                         "of_bf16_peak": round(r["gflops"] / 1e3 / peaks["bf16_tflops"], 4),
                         "of_hbm": round(r["gbps"] / peaks["hbm_gbs"], 4)})
        tables[phase] = rows
    del ex
    return tables


def run(args, root: str, sampler=None) -> dict:
    import torch
    from llmgen_b200.engine.api import random_model
    peaks = _peaks(root)
    steps, warmup = max(8, min(args.steps, 64)), max(3, min(args.warmup, 8))
    wanted = [n for n in SIZES if not args.designs_size or n in args.designs_size.split(",")]
    out = {"designs": {}, "peaks": peaks, "gpu": torch.cuda.get_device_name(0), "dtype": "bf16", "data": "synthetic (random weights and ids)",
           "timing": "CUDA events; inputs larger than L2, nothing flushed"}
    w0 = sampler.mark() if sampler is not None else None
    for name in wanted:
        entry = {}
        family = getattr(args, "designs_family", "") or "derupel"
        beside = getattr(args, "designs_beside", "") or BESIDE.get(family, "qwen3")
        other = qwen3_config(SIZES[name]) if beside == "qwen3" else FAMILIES[beside](SIZES[name])
        for design, cfg in ((family, FAMILIES[family](SIZES[name])), (beside, other)):
            model = random_model(cfg, 2, "bfloat16", init_on_device=True)
            res = _throughput(torch, model, args.batch, steps, warmup, 3)
            res["weights_gb"] = round(model.weight_bytes() / 1e9, 3)
            if not args.skip_points:
                res["kernels"] = _kernels(torch, model, args.batch, peaks, 4)
            entry[design] = res
            del model
            torch.cuda.empty_cache()
        out["designs"][name] = entry
    if sampler is not None:
        out["clocks"] = sampler.stop([(w0, sampler.mark())])
    return out


def as_markdown(result: dict) -> str:
    lines = []
    for name, entry in result["designs"].items():
        lines.append(f"### {name}\n")
        lines.append("| design | weights GB | prefill ms (2,048 tokens) | prefill tokens/s | decode ms/step (batch 8) | decode tokens/s |")
        lines.append("|---|---|---|---|---|---|")
        for design, r in entry.items():
            lines.append(f"| {design} | {r['weights_gb']} | {r['prefill_ms']} | {r['prefill_tokens_per_s']} | {r['decode_ms_per_step']} | {r['decode_tokens_per_s']} |")
        for design, r in entry.items():
            for phase, rows in (r.get("kernels") or {}).items():
                lines.append(f"\n{design}, {phase}: kernel, calls, µs a call, share, TFLOP/s (of bf16 peak), GB/s (of copy bandwidth)\n")
                lines.append("| op | calls | avg µs | % | TFLOP/s | of peak | GB/s | of HBM |")
                lines.append("|---|---|---|---|---|---|---|---|")
                for k in rows:
                    lines.append(f"| {k['op']} | {k['calls']} | {k['avg_us']} | {k['pct']} | {k['tflops']} | {k['of_bf16_peak']} | {k['gbs']} | {k['of_hbm']} |")
        lines.append("")
    return "\n".join(lines)
