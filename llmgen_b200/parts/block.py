"""The arrangement of a layer's parts."""
from __future__ import annotations

import torch

from .base import LayerCache, Part
from .registry import (build_feed_forward, build_mixer, build_norm, feed_forward_class, mixer_class, norm_class,
                       register_block)
from ..kernels import ops
from .parallel import finish_pair
from .spec import INIT_EYE_PLUS_NORMAL, INIT_ONE_PLUS_NORMAL, VECTOR, MultiStreamBlockSpec, PostNormBlockSpec, PreNormBlockSpec, SandwichBlockSpec, WeightDecl


class PreNormBlock(Part):
    """x1 = x + mixer(norm(x)); x2 = x1 + ffn(norm(x1))  (src/models/qwen3.zig:224-236).

    The residual stream is float32 and lives in one buffer.  Each sum is folded into the norm
    that follows it: the block receives the previous block's output as `delta`, adds it in its
    first norm, adds the mixer's output in its second norm and returns the feed-forward's
    output as the next `delta` (an array or the float32 slices of a product cut along K, which the
    norm adds up: `kernels.ops.Partials`)."""

    @staticmethod
    def weight_decls(spec: PreNormBlockSpec):
        decls = norm_class(spec.mixer_norm).weight_decls(spec.mixer_norm) + mixer_class(spec.mixer).weight_decls(spec.mixer)
        if spec.ffn is not None:
            decls = decls + norm_class(spec.ffn_norm).weight_decls(spec.ffn_norm) + feed_forward_class(spec.ffn).weight_decls(spec.ffn)
        return decls

    @staticmethod
    def kernel_modules(spec: PreNormBlockSpec):
        mods = (tuple(norm_class(spec.mixer_norm).kernel_modules(spec.mixer_norm))
                + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer)))
        if spec.ffn is not None:
            mods += tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn))
        return mods

    def __init__(self, spec: PreNormBlockSpec, weights, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_norm(spec.mixer_norm, weights, dtype, device)
        self.mixer = build_mixer(spec.mixer, weights, dtype, device)
        self.ffn_norm = build_norm(spec.ffn_norm, weights, dtype, device) if spec.ffn is not None else None
        self.ffn = build_feed_forward(spec.ffn, weights, dtype, device) if spec.ffn is not None else None

    def workspace_bytes(self, tokens: int) -> int:
        """Bytes of activations a step of `tokens` rows keeps in the workspace for this layer: the normed
        input plus what the mixer and the feed-forward say they need (a part without `workspace_bytes`
        counts as nothing and must allocate before any graph is captured, like every part)."""
        elem = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * self.spec.mixer_norm.dim * elem
        parts = [getattr(p, "workspace_bytes", None) for p in (self.mixer, self.ffn) if p is not None]
        return own + max([f(tokens) for f in parts if f is not None] or [0])

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        T, H = resid.shape
        x = self.mixer_norm.add_norm(resid, delta, ctx.workspace.buffer("block_normed", T, H, self.dtype))
        mixed = finish_pair(ctx, self.mixer.forward(ctx, x, cache), self.dtype)
        if self.ffn is None:
            return mixed          # a layer without a feed-forward: the next norm adds the mixer's output
        x = self.ffn_norm.add_norm(resid, mixed, ctx.workspace.buffer("block_normed", T, H, self.dtype))
        return self.ffn.forward(ctx, x)


class PostNormBlock(Part):
    """x1 = x + norm(mixer(x)); x2 = x1 + norm(ffn(x1)): the norm sits on each sublayer's output, and the sublayers read the
    residual stream itself.

    The residual stream is the same float32 buffer as in every other block.  `norm_add` normalises a sublayer's output
    (an array or the float32 slices of a product cut along K), adds it to the residual and, in bfloat16, leaves a copy of
    the new residual rows in the storage dtype for the products of the sublayer that follows (the next block's mixer
    included: the copy is kept in a workspace buffer that blocks of this kind share).  The block finishes both sums
    itself and hands on nothing to add.  A block without a feed-forward stops after the first sum."""

    @staticmethod
    def weight_decls(spec: PostNormBlockSpec):
        decls = norm_class(spec.mixer_norm).weight_decls(spec.mixer_norm) + mixer_class(spec.mixer).weight_decls(spec.mixer)
        if spec.ffn is not None:
            decls += norm_class(spec.ffn_norm).weight_decls(spec.ffn_norm) + feed_forward_class(spec.ffn).weight_decls(spec.ffn)
        return decls

    @staticmethod
    def kernel_modules(spec: PostNormBlockSpec):
        mods = ("rowwise",) + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer))
        if spec.ffn is not None:
            mods += tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn))
        return mods

    def __init__(self, spec: PostNormBlockSpec, weights, dtype, device):
        for norm in (spec.mixer_norm, spec.ffn_norm if spec.ffn is not None else None):
            if norm is not None and (norm.kind != "rmsnorm" or norm.weight_offset != 0.0):
                raise ValueError("post-norm block: the norms on the sublayers' outputs are plain RMSNorms")
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_norm(spec.mixer_norm, weights, dtype, device)
        self.mixer = build_mixer(spec.mixer, weights, dtype, device)
        self.ffn_norm = build_norm(spec.ffn_norm, weights, dtype, device) if spec.ffn is not None else None
        self.ffn = build_feed_forward(spec.ffn, weights, dtype, device) if spec.ffn is not None else None

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * self.spec.mixer_norm.dim * elem
        parts = [getattr(p, "workspace_bytes", None) for p in (self.mixer, self.ffn) if p is not None]
        return own + max([f(tokens) for f in parts if f is not None] or [0])

    def _stream_copy(self, ctx, resid):
        """The residual rows as the products read them: the float32 buffer itself, or its copy in bfloat16."""
        if self.dtype == torch.float32:
            return resid, None
        T, H = resid.shape
        return None, ctx.workspace.buffer("stream_copy", T, H, self.dtype)

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        x, copy = self._stream_copy(ctx, resid)
        if delta is not None or getattr(ctx, "stream_copy_of", None) is not resid:
            # the block before was of another kind (or this is the first one): finish its sum, make the copy
            if delta is not None:
                resid.add_(delta.sum() if isinstance(delta, ops.Partials) else delta.float())
            if copy is not None:
                ops.cast_rows(copy, resid)
            ctx.stream_copy_of = resid
        x = resid if copy is None else copy
        mixed = self.mixer.forward(ctx, x, cache)
        ops.norm_add(resid, mixed, self.mixer_norm.weight, self.mixer_norm.eps, copy, self.dtype)
        if self.ffn is not None:
            out = self.ffn.forward(ctx, x)
            ops.norm_add(resid, out, self.ffn_norm.weight, self.ffn_norm.eps, copy, self.dtype)
        return None


class SandwichBlock(Part):
    """x1 = x + norm_b(mixer(norm_a(x))); x2 = x1 + norm_d(ffn(norm_c(x1))): every sublayer reads a normed stream and has
    its output normed before it joins the stream.

    The residual stream is the one float32 buffer of every other block.  One kernel a sublayer does what lies between
    two sublayers: `norm_add` normalises the sublayer's output (an array, float32 slices, or the weighted pair a parallel
    mixer returns), adds it to the residual and writes the NEXT sublayer's normed input in the same pass (the next
    block's first norm included, when the run list's next item is a block of this kind too: the model names it in
    `ctx.next_block`).  A block whose input nobody prepared norms it with `add_rmsnorm`, which also finishes a sum the
    block before left open."""

    @staticmethod
    def weight_decls(spec: SandwichBlockSpec):
        decls = (norm_class(spec.mixer_norm).weight_decls(spec.mixer_norm) + mixer_class(spec.mixer).weight_decls(spec.mixer)
                 + norm_class(spec.mixer_out_norm).weight_decls(spec.mixer_out_norm))
        if spec.ffn is not None:
            decls += (norm_class(spec.ffn_norm).weight_decls(spec.ffn_norm) + feed_forward_class(spec.ffn).weight_decls(spec.ffn)
                      + norm_class(spec.ffn_out_norm).weight_decls(spec.ffn_out_norm))
        return decls

    @staticmethod
    def kernel_modules(spec: SandwichBlockSpec):
        mods = ("rowwise", "elementwise") + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer))
        if spec.ffn is not None:
            mods += tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn))
        return mods

    def __init__(self, spec: SandwichBlockSpec, weights, dtype, device):
        norms = [spec.mixer_norm, spec.mixer_out_norm] + ([spec.ffn_norm, spec.ffn_out_norm] if spec.ffn is not None else [])
        for norm in norms:
            if norm is None or norm.kind != "rmsnorm" or norm.weight_offset != 0.0:
                raise ValueError("sandwich block: its norms are plain RMSNorms")
        self.spec, self.dtype = spec, dtype
        self.mixer_norm = build_norm(spec.mixer_norm, weights, dtype, device)
        self.mixer = build_mixer(spec.mixer, weights, dtype, device)
        self.mixer_out_norm = build_norm(spec.mixer_out_norm, weights, dtype, device)
        self.ffn_norm = build_norm(spec.ffn_norm, weights, dtype, device) if spec.ffn is not None else None
        self.ffn = build_feed_forward(spec.ffn, weights, dtype, device) if spec.ffn is not None else None
        self.ffn_out_norm = build_norm(spec.ffn_out_norm, weights, dtype, device) if spec.ffn is not None else None

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * self.spec.mixer_norm.dim * elem
        parts = [getattr(p, "workspace_bytes", None) for p in (self.mixer, self.ffn) if p is not None]
        return own + max([f(tokens) for f in parts if f is not None] or [0])

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        T, H = resid.shape
        normed = ctx.workspace.buffer("block_normed", T, H, self.dtype)
        if delta is not None or getattr(ctx, "normed_for", None) is not self:
            # nobody prepared this block's input: norm it here (and finish the sum a block of another kind left open)
            self.mixer_norm.add_norm(resid, finish_pair(ctx, delta, self.dtype) if delta is not None else None, normed)
        ctx.normed_for = None
        # the block that runs next, if it is of this kind, finds its normed input ready
        follower = getattr(ctx, "next_block", None)
        follow = follower.mixer_norm if isinstance(follower, SandwichBlock) else None
        mixed = self.mixer.forward(ctx, normed, cache)
        nxt = self.ffn_norm if self.ffn is not None else follow
        ops.norm_add(resid, mixed, self.mixer_out_norm.weight, self.mixer_out_norm.eps, normed if nxt is not None else None, self.dtype,
                     next_gain=nxt.weight if nxt is not None else None, next_eps=nxt.eps if nxt is not None else 0.0)
        if self.ffn is not None:
            out = self.ffn.forward(ctx, normed)
            nxt = follow
            ops.norm_add(resid, out, self.ffn_out_norm.weight, self.ffn_out_norm.eps, normed if nxt is not None else None, self.dtype,
                         next_gain=nxt.weight if nxt is not None else None, next_eps=nxt.eps if nxt is not None else 0.0)
        ctx.normed_for = follower if follow is not None else None
        return None


class MultiStreamBlock(Part):
    """A pre-norm layer over several residual streams per token (hyper-connections).

    The block's `resid` is the float32 array [tokens, streams * hidden] that the model keeps for architectures with
    `residual_streams`.  One kernel (`stream_step`) lies between two sublayers: it rewrites every stream from all the old ones
    and the sublayer's output (an array, float32 slices, or the weighted pair a parallel mixer returns), x_t <- sum_s mix[s, t] x_s +
    mult write[t] y, and in the same pass reads the streams for the sublayer that follows, norm(sum_t read[t] x_t) (the next block's
    mixer included, when the run list's next item is a block of this kind: the model names it in `ctx.next_block`).  The
    coefficients stay float32; `mult write` is folded at load.  A block whose input nobody prepared reads the streams itself.
    It finishes its sums and hands on nothing to add."""

    @staticmethod
    def weight_decls(spec: MultiStreamBlockSpec):
        S = spec.streams

        def coefficients(c):
            # the random-weights mode draws them around "every stream read, kept and written as it is"
            return [] if c is None else [WeightDecl(c.read, (S,), VECTOR, INIT_ONE_PLUS_NORMAL), WeightDecl(c.write, (S,), VECTOR, INIT_ONE_PLUS_NORMAL),
                                         WeightDecl(c.mix, (S, S), VECTOR, INIT_EYE_PLUS_NORMAL)]

        decls = norm_class(spec.mixer_norm).weight_decls(spec.mixer_norm) + mixer_class(spec.mixer).weight_decls(spec.mixer) \
            + coefficients(spec.mixer_streams)
        if spec.ffn is not None:
            decls += norm_class(spec.ffn_norm).weight_decls(spec.ffn_norm) + feed_forward_class(spec.ffn).weight_decls(spec.ffn) \
                + coefficients(spec.ffn_streams)
        return decls

    @staticmethod
    def kernel_modules(spec: MultiStreamBlockSpec):
        mods = ("rowwise", "elementwise") + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer))
        if spec.ffn is not None:
            mods += tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn))
        return mods

    def __init__(self, spec: MultiStreamBlockSpec, weights, dtype, device):
        S = spec.streams
        if not 1 <= S <= ops.MAX_STREAMS:
            raise ValueError(f"multi-stream block: {S} streams (1 to {ops.MAX_STREAMS})")
        for norm in (spec.mixer_norm, spec.ffn_norm if spec.ffn is not None else None):
            if norm is not None and (norm.kind != "rmsnorm" or norm.weight_offset != 0.0):
                raise ValueError("multi-stream block: its norms are plain RMSNorms")
        if S > 1 and (spec.mixer_streams is None or (spec.ffn is not None and spec.ffn_streams is None)):
            raise ValueError("multi-stream block: several streams need coefficients for every sublayer")
        self.spec, self.dtype, self.S = spec, dtype, S
        self.mixer_norm = build_norm(spec.mixer_norm, weights, dtype, device)
        self.mixer = build_mixer(spec.mixer, weights, dtype, device)
        self.ffn_norm = build_norm(spec.ffn_norm, weights, dtype, device) if spec.ffn is not None else None
        self.ffn = build_feed_forward(spec.ffn, weights, dtype, device) if spec.ffn is not None else None
        mult = float(spec.residual_mult)

        def coefficients(c):
            # (read, mult * write, mix); without tensors: one stream read as it is, kept as it is, y added times mult
            if c is None:
                one = torch.ones(1, dtype=torch.float32, device=device)
                return one, one * mult, one.clone()
            return (weights.device_tensor(c.read, dtype, device).contiguous(),
                    (weights.device_tensor(c.write, dtype, device).float() * mult).contiguous(),
                    weights.device_tensor(c.mix, dtype, device).contiguous())

        self.read1, self.write1, self.mix1 = coefficients(spec.mixer_streams)
        self.read2, self.write2, self.mix2 = coefficients(spec.ffn_streams) if spec.ffn is not None else (None, None, None)

    def workspace_bytes(self, tokens: int) -> int:
        elem = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * self.spec.mixer_norm.dim * (elem + 4 * self.S)
        parts = [getattr(p, "workspace_bytes", None) for p in (self.mixer, self.ffn) if p is not None]
        return own + max([f(tokens) for f in parts if f is not None] or [0])

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        T = resid.shape[0]
        H = self.spec.mixer_norm.dim
        if delta is not None or resid.shape[1] != self.S * H:
            raise ValueError("multi-stream block: it runs on the model's array of streams and takes no pending sum")
        streams = resid.view(T, self.S, H)
        normed = ctx.workspace.buffer("block_normed", T, H, self.dtype)
        if getattr(ctx, "normed_for", None) is not self:
            ops.stream_step(streams, None, None, None, self.read1, self.mixer_norm.weight, self.mixer_norm.eps, normed, self.dtype)
        ctx.normed_for = None
        follower = getattr(ctx, "next_block", None)
        follow = follower if isinstance(follower, MultiStreamBlock) and follower.S == self.S else None
        mixed = self.mixer.forward(ctx, normed, cache)
        if self.ffn is not None:
            ops.stream_step(streams, mixed, self.mix1, self.write1, self.read2, self.ffn_norm.weight, self.ffn_norm.eps, normed, self.dtype)
            mixed = self.ffn.forward(ctx, normed)
            mix, write = self.mix2, self.write2
        else:
            mix, write = self.mix1, self.write1
        if follow is not None:
            ops.stream_step(streams, mixed, mix, write, follow.read1, follow.mixer_norm.weight, follow.mixer_norm.eps, normed, self.dtype)
        else:
            ops.stream_step(streams, mixed, mix, write, None, None, 0.0, None, self.dtype)
        ctx.normed_for = follow
        return None


register_block("prenorm", PreNormBlock)
register_block("multi_stream", MultiStreamBlock)
register_block("sandwich", SandwichBlock)
register_block("postnorm", PostNormBlock)
