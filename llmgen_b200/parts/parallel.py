"""Several mixers side by side on the same input, their outputs added with a weight each."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateRequest
from .registry import build_mixer, mixer_class, register_mixer
from .spec import ParallelMixerSpec


def finish_pair(ctx, y, dtype):
    """A mixer's result as one array (or `Partials`): a `WeightedPair` is added up into a float32 buffer of the step's
    workspace; anything else passes through.  For consumers that have no kernel taking the pair."""
    if not isinstance(y, ops.WeightedPair):
        return y
    out = ctx.workspace.flat("pair_sum", ctx.workspace.default_rows * y.cols, torch.float32)[:y.rows * y.cols]
    return ops.scaled_sum(out.view(1, y.rows, y.cols), y, dtype)


class ParallelMixer(Mixer):
    """sum_i scales[i] * branch_i(x).  The branches are built from their own specs and know nothing of each other.

    Cache: the one branch that keeps paged keys and values (at most one may) receives the run item's pages; the
    branches that keep a per-request state share the item's state row, each its own stretch of it, in branch order.
    With two branches the result is handed on as an `ops.WeightedPair`, which the kernel that norms a sublayer's output
    adds up on the way (`norm_add`); more branches are added up pair by pair into a float32 buffer."""

    @staticmethod
    def weight_decls(spec: ParallelMixerSpec):
        return [d for b in spec.branches for d in mixer_class(b).weight_decls(b)]

    @staticmethod
    def kernel_modules(spec):
        return ("rowwise",) + tuple(m for b in spec.branches for m in mixer_class(b).kernel_modules(b))

    def __init__(self, spec: ParallelMixerSpec, weights, dtype, device):
        if len(spec.branches) < 2 or len(spec.branches) != len(spec.scales):
            raise ValueError("parallel mixer: two or more branches, one scale each")
        self.spec, self.dtype = spec, dtype
        self.branches = [build_mixer(b, weights, dtype, device) for b in spec.branches]
        self.scales = [float(s) for s in spec.scales]
        if sum(1 for b in self.branches if b.cache_request() is not None) > 1:
            raise ValueError("parallel mixer: at most one branch keeps paged keys and values")
        self.state_ranges = []
        at = 0
        for b in self.branches:
            req = b.state_request()
            if req is None:
                self.state_ranges.append(None)
                continue
            if req.dtype != torch.float32:
                raise ValueError("parallel mixer: the branches' states are float32 rows")
            n = 1
            for d in req.shape:
                n *= d
            self.state_ranges.append((at, at + n, tuple(req.shape)))
            at += n
        self.state_size = at
        self.replay_any_step = all(getattr(b, "replay_any_step", False) for b in self.branches)
        self.step_arrays_follow_shapes = all(getattr(b, "step_arrays_follow_shapes", False) or not hasattr(b, "prepare_step")
                                             for b in self.branches)
        self.capturable = all(getattr(b, "capturable", True) for b in self.branches)

    # -- what the engine asks
    def cache_request(self):
        for b in self.branches:
            req = b.cache_request()
            if req is not None:
                return req
        return None

    def state_request(self):
        return StateRequest((self.state_size,), torch.float32) if self.state_size else None

    def max_positions(self):
        limits = [b.max_positions() for b in self.branches if hasattr(b, "max_positions")]
        limits = [m for m in limits if m is not None]
        return min(limits) if limits else None

    def step_arrays_key(self):
        return ("parallel",) + tuple(b.step_arrays_key() if hasattr(b, "step_arrays_key") else id(b) for b in self.branches)

    def prepare_step(self, builder) -> None:
        for b in self.branches:
            if hasattr(b, "prepare_step"):
                b.prepare_step(builder)

    def workspace_bytes(self, tokens: int) -> int:
        asks = [getattr(b, "workspace_bytes", None) for b in self.branches]
        return sum(f(tokens) for f in asks if f is not None) + tokens * self.cols_hint() * 4

    def cols_hint(self) -> int:
        return int(getattr(self.spec.branches[0], "hidden_size", 0))

    def _branch_cache(self, i: int, cache: LayerCache) -> LayerCache:
        b = self.branches[i]
        keeps_pages = b.cache_request() is not None
        state = None
        if self.state_ranges[i] is not None and cache.state is not None:
            lo, hi, shape = self.state_ranges[i]
            state = cache.state[:, lo:hi]
            if len(shape) > 1:
                state = state.unflatten(1, shape) if state.is_contiguous() else state
        return LayerCache(k=cache.k if keeps_pages else None, v=cache.v if keeps_pages else None, group=cache.group,
                          page_size=cache.page_size, writes=cache.writes, state=state)

    def forward(self, ctx, x, cache: LayerCache):
        outs = [b.forward(ctx, x, self._branch_cache(i, cache)) for i, b in enumerate(self.branches)]
        pair = ops.WeightedPair(outs[0], self.scales[0], outs[1], self.scales[1])
        for y, s in zip(outs[2:], self.scales[2:]):
            pair = ops.WeightedPair(finish_pair(ctx, pair, self.dtype), 1.0, y, s)
        return pair


register_mixer("parallel", ParallelMixer)
