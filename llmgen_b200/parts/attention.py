"""Causal grouped-query attention over the paged cache, as a mixer."""
from __future__ import annotations

import torch

from ..cache.manager import FULL, WINDOW
from ..kernels import ops
from .base import KVRequest, LayerCache, Mixer, StateRequest
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import build_position, norm_class, register_mixer
from .spec import INIT_ONE_PLUS_NORMAL, VECTOR, AttentionSpec, RopeSpec, WeightDecl


def add_query_tiles(builder, bq: int, window: int = 0, heaviest_first: bool = False) -> str:
    """Adds to a step's arrays the (sequence, first query) of every tile of `bq` queries, under the name it returns
    (with `_seq` and `_q0` appended); mixers that cut their queries the same way share one pair of arrays.
    `heaviest_first`: in the order of the keys a tile has to read, most first; the blocks of a launch start in the
    order of the list, and a prompt's last tiles read the whole prompt while its first read one tile of keys."""
    name = f"attention_tiles_bq{bq}"
    if builder.has(name + "_seq"):
        return name
    tiles = []
    bound = getattr(builder, "token_bound", 0)
    for s, n in enumerate(builder.q_lens):
        if bound and n == 0:
            continue
        for start in range(0, max(n, 1), bq):
            keys = builder.starts[s] + min(start + bq, max(n, 1))
            tiles.append((min(keys, window + bq) if window else keys, s, start))
    if heaviest_first:
        tiles.sort(key=lambda t: -t[0])
    if bound:
        # a list of fixed length for the step's shape: no more tiles than this exist for `bound` tokens in
        # `n_seqs` sequences; the rest is padding (sequence -1), which the kernels skip
        most = bound // bq + builder.n_seqs
        tiles += [(0, -1, 0)] * (most - len(tiles))
    builder.add(name + "_seq", [t[1] for t in tiles])
    builder.add(name + "_q0", [t[2] for t in tiles])
    return name


class GQAAttention(Mixer):
    """q, k, v projections (packed into one [(nq + 2 nkv) hd, H] matrix at load) -> per-head
    RMSNorm of q and k, rotary encoding, cache write (one kernel) -> attention over the block
    table -> output projection.

    Attention kernels: in bfloat16 a step of single decoded tokens runs the bandwidth-shaped
    flash-decoding kernel (csrc/attention_decode.cu), any other step the tensor-core kernel
    (csrc/attention_tc.cu); float32, and sizes those two refuse, run the general CUDA-core kernel
    (csrc/attention.cu).

    Order and formulas: src/models/qwen3.zig:192-207 (q/k norm before RoPE, norm weights
    shared by all heads), src/module/attention.zig:85-92, src/backend/cpu/attention.zig:64-118.
    A run item with `writes=False` projects q only and reads the cache another item wrote.

    Variations (`AttentionSpec`): biases on the projections, values of another width than keys, a bound on the scores
    (softcap), a sink in the softmax's denominator, an output gate, rotation of pairs (2i, 2i + 1), heads of q and k divided
    by their root mean square after the rotation, and a mask in blocks of positions (its pages are a window group's).  The gate's matrix is packed behind q, k and v,
    the biases of q, k and v are added by the preparation kernel before the per-head norms, and bound, sink and gate
    are applied inside the attention kernels that take the steps of a layer that has any of them: in bfloat16 portions of
    prompts run on the tensor cores with float32 softmax weights (csrc/attention_mma.cu), single decoded tokens (their
    keys in parts), float32 and other sizes on the general kernel (csrc/attention.cu); the output projection's bias is
    added to its result (or to the first of its slices)."""

    # what `prepare_step` adds depends on the lengths of the step's portions only, not on their
    # positions or requests: the engine may keep it across decode steps of one batch size
    step_arrays_follow_shapes = True
    # its launches follow from a step's shape (token rows, sequences) alone, its lists of tiles have the length
    # that the shape bounds, and token rows that belong to no sequence pass through untouched: any step may be
    # replayed from the graph of its shape
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: AttentionSpec):
        qd, kd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        vd, od = spec.num_kv_heads * spec.value_dim, spec.num_heads * spec.value_dim
        decls = [WeightDecl(spec.q_proj, (qd, spec.hidden_size)), WeightDecl(spec.k_proj, (kd, spec.hidden_size)),
                 WeightDecl(spec.v_proj, (vd, spec.hidden_size)), WeightDecl(spec.o_proj, (spec.hidden_size, od))]
        for name, width in ((spec.q_bias, qd), (spec.k_bias, kd), (spec.v_bias, vd), (spec.o_bias, spec.hidden_size)):
            if name:
                decls.append(WeightDecl(name, (width,), VECTOR))
        if spec.gate_proj:
            decls.append(WeightDecl(spec.gate_proj, (spec.num_heads if spec.gate_per_head else od, spec.hidden_size)))
        for n in (spec.q_norm, spec.k_norm):
            if n is not None:
                decls += norm_class(n).weight_decls(n)
        if spec.conv is not None:
            decls += [WeightDecl(n, (w, spec.conv.taps), VECTOR) for n, w in zip(spec.conv_weights, (qd, kd, vd))]
        if spec.sink_scores:
            decls.append(WeightDecl(spec.sink_scores, (spec.num_heads,), VECTOR))
        return decls

    @staticmethod
    def kernel_modules(spec):
        if GQAAttention.varied(spec):
            return ("attn_prep", "attention", "attention_mma", "rowwise") + (("recurrent",) if spec.conv is not None else ()) + GEMM_MODULES
        return ("attn_prep", "attention", "attention_decode", "attention_tc") + GEMM_MODULES

    @staticmethod
    def varied(spec: AttentionSpec) -> bool:
        """True for a layer that only the general kernels take (see the class's last paragraph)."""
        return bool(spec.q_bias or spec.k_bias or spec.v_bias or spec.o_bias or spec.gate_proj or spec.sink or spec.softcap > 0
                    or spec.value_dim != spec.head_dim or spec.chunk or spec.unit_norm_eps is not None
                    or spec.conv is not None or spec.row_norms or spec.rotate_values or spec.sink_scores or spec.gate_per_head
                    or (spec.position is not None and getattr(spec.position, "pairing", "half") != "half"))

    def __init__(self, spec: AttentionSpec, weights, dtype, device):
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError(f"attention: {spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.head_dim % 2 != 0 or spec.head_dim > 512:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be even, at most 512")
        for n, heads in ((spec.q_norm, spec.num_heads), (spec.k_norm, spec.num_kv_heads)):
            if n is not None and spec.row_norms:
                if n.kind != "rmsnorm" or n.dim != heads * spec.head_dim or n.weight_offset != 0.0:
                    raise ValueError("attention: norms over a whole projection are plain RMSNorms of that width")
            elif n is not None and (n.kind not in ops.HEAD_NORMS or n.dim != spec.head_dim):
                raise ValueError(f"attention: per-head norms must run over head_dim and be one of {sorted(ops.HEAD_NORMS)}")
        self.spec = spec
        self.dtype = dtype
        self.nq, self.nkv, self.hd, self.vd = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        if self.vd > 512:
            raise ValueError(f"attention: the values' width {self.vd} must be at most 512")
        self.is_varied = self.varied(spec)
        # packed on the device: each matrix goes up through the loader's pinned stage as the file holds it
        names = [spec.q_proj, spec.k_proj, spec.v_proj] + ([spec.gate_proj] if spec.gate_proj else [])
        self.w_qkv = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in names], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.nq * self.hd]
        self.gate_off = (self.nq + self.nkv) * self.hd + self.nkv * self.vd if spec.gate_proj else -1
        # a run item that reads another item's cache projects q (and the gate) only
        self.w_q_gate = (torch.cat([self.w_q, self.w_qkv[self.gate_off:]], dim=0).contiguous() if spec.gate_proj else self.w_q)
        self.bias = None
        if spec.q_bias or spec.k_bias or spec.v_bias:
            widths = (self.nq * self.hd, self.nkv * self.hd, self.nkv * self.vd)
            self.bias = torch.cat([weights.device_tensor(n, dtype, device, keep=False) if n else
                                   torch.zeros(w, dtype=torch.float32, device=device)
                                   for n, w in zip((spec.q_bias, spec.k_bias, spec.v_bias), widths)]).contiguous()
        self.o_bias = weights.device_tensor(spec.o_bias, dtype, device) if spec.o_bias else None
        self.softcap, self.sink = float(spec.softcap), bool(spec.sink)
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.q_gain = weights.device_tensor(spec.q_norm.weight, dtype, device) if spec.q_norm else None
        self.k_gain = weights.device_tensor(spec.k_norm.weight, dtype, device) if spec.k_norm else None
        self.norm_eps = float((spec.q_norm or spec.k_norm).eps) if (spec.q_norm or spec.k_norm) else 0.0
        if spec.q_norm and spec.k_norm and spec.q_norm.eps != spec.k_norm.eps:
            raise ValueError("attention: q and k norms must share eps")
        self.q_off = float(spec.q_norm.weight_offset) if spec.q_norm else 0.0
        self.k_off = float(spec.k_norm.weight_offset) if spec.k_norm else 0.0
        self.position = build_position(spec.position, weights, dtype, device) if spec.position is not None else None
        # which values of a head the position encoding turns together, and the kind of the per-head norms: the
        # kernels are told and refuse what they do not implement
        self.pairing = getattr(self.position, "pairing", "half") if self.position is not None else "half"
        self.head_norm = (spec.q_norm or spec.k_norm).kind if (spec.q_norm or spec.k_norm) else "rmsnorm"
        if spec.unit_norm_eps is not None:
            # no gains, and after the rotation (the preparation kernel's general form)
            if spec.q_norm or spec.k_norm:
                raise ValueError("attention: per-head norms before the rotation and a unit norm after it exclude each other")
            self.head_norm, self.norm_eps = "unit_rms_after", float(spec.unit_norm_eps)
        # the variations that come with norms over whole projections: a short convolution after the projections (its last
        # inputs are state), values rotated by their position and outputs turned back, learned sink scores, a gate per head
        self.row_norms = bool(spec.row_norms)
        self.conv_w = None
        if spec.conv is not None:
            C = (self.nq + self.nkv) * self.hd + self.nkv * self.vd
            if spec.conv.channels != C or not 1 <= spec.conv.taps <= 8 or len(spec.conv_weights) != 3:
                raise ValueError("attention: one convolution of 1 to 8 taps over the channels of q, k and v")
            if not spec.row_norms:
                raise ValueError("attention: the convolution after the projections comes with norms over whole projections")
            self.conv_w = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in spec.conv_weights], dim=0).contiguous()
        self.value_position = None
        if spec.rotate_values:
            if spec.position is None or self.vd % 2 != 0 or not spec.row_norms:
                raise ValueError("attention: rotated values need a position encoding, an even width and norms over whole projections")
            if getattr(spec.position, "pairing", "half") != "half" or getattr(spec.position, "scaling", None) is not None:
                raise ValueError("attention: rotated values are turned in half-split pairs by plain frequencies")
            self.value_position = build_position(RopeSpec(rotary_dim=self.vd, theta=spec.position.theta,
                                                          max_positions=spec.position.max_positions), weights, dtype, device)
        if spec.row_norms and (spec.q_bias or spec.k_bias or spec.v_bias or spec.softcap > 0 or spec.chunk or spec.unit_norm_eps is not None
                               or self.pairing != "half"):
            raise ValueError("attention: norms over whole projections exclude biases, a bound, a mask in blocks and other pairings")
        if (spec.sink_scores or spec.gate_per_head) and not spec.row_norms:
            raise ValueError("attention: learned sink scores and a gate per head come with norms over whole projections")
        self.sink_scores = weights.device_tensor(spec.sink_scores, dtype, device).contiguous() if spec.sink_scores else None
        if self.sink_scores is not None and not spec.sink:
            raise ValueError("attention: sink scores without a sink")
        self.chunk = int(spec.chunk or 0)
        if self.chunk and spec.window:
            raise ValueError("attention: a window and a mask in blocks exclude each other")
        self.sm_count = ops.sm_count(device)
        self.window = int(spec.window or 0)
        self.bq = ops.attention_tile_queries(self.nq, self.nkv)
        self.tiles_name = f"attention_tiles_bq{self.bq}"
        self._tc_bq = {}       # page size -> queries per tile of the tensor-core kernel (0: not taken)
        self._mma_bq = None

    # -- what the engine asks
    def cache_request(self) -> KVRequest:
        # a mask in blocks of `chunk` positions never looks further back than chunk - 1 keys: its pages are a
        # window group's, given back as the blocks pass
        held = self.window or self.chunk
        return KVRequest(WINDOW if held else FULL, held, self.nkv, self.hd,
                         v_head_dim=self.vd if self.vd != self.hd else 0)

    def state_request(self):
        # the convolution's last taps - 1 inputs over the channels of q, k and v side by side, oldest first
        if self.conv_w is None or self.spec.conv.taps <= 1:
            return None
        return StateRequest(((self.spec.conv.taps - 1) * self.conv_w.shape[0],), torch.float32)

    def max_positions(self):
        return self.position.max_positions if self.position is not None else None

    def _tiles(self, builder, bq: int, heaviest_first: bool = False) -> None:
        add_query_tiles(builder, bq, self.window or self.chunk, heaviest_first)

    def tc_tile_queries(self, page_size: int) -> int:
        if self.dtype != torch.bfloat16 or self.is_varied:
            return 0
        if page_size not in self._tc_bq:
            self._tc_bq[page_size] = ops.attention_tc_tile_queries(self.nq, self.nkv, self.hd, page_size)
        return self._tc_bq[page_size]

    def mma_tile_queries(self) -> int:
        """Queries per tile of the tensor-core kernel that keeps float32 softmax weights (0: this layer's steps do not
        run on it): bfloat16 layers with variations, key and value widths it takes."""
        if self.dtype != torch.bfloat16 or not self.is_varied:
            return 0
        if self._mma_bq is None:
            self._mma_bq = ops.attention_mma_tile_queries(self.nq, self.nkv, self.hd, self.vd)
        return self._mma_bq

    def step_arrays_key(self):
        """Mixers with equal keys add the same arrays in `prepare_step`: the engine asks one of them."""
        return ("attention_tiles", self.bq, self.nq, self.nkv, self.hd, self.window, self.chunk, str(self.dtype), self.is_varied)

    def prepare_step(self, builder) -> None:
        """Tiles of queries, (sequence, first query of the tile) pairs, for the kernel this step will
        run: the tensor-core kernel's where it takes the step, else the CUDA-core kernel's."""
        page_size = getattr(builder, "page_size", 0)
        tc_bq = self.tc_tile_queries(page_size) if page_size and not builder.pure_decode else 0
        mma_bq = self.mma_tile_queries() if not builder.pure_decode else 0
        if tc_bq or mma_bq:
            self._tiles(builder, tc_bq or mma_bq, heaviest_first=True)
        else:
            self._tiles(builder, self.bq)

    def _split(self, ctx):
        """(num_parts, part_size) for flash-decoding; only pure-decode steps are split."""
        if not ctx.pure_decode:
            return 1, 0
        G = self.nq // self.nkv
        chunks = (G + 15) // 16
        blocks = max(1, ctx.n_seqs * self.nkv * chunks)
        longest = ctx.max_ctx_bound if ctx.fixed_shapes else ctx.max_ctx
        if self.window or self.chunk:
            longest = min(longest, self.window or self.chunk)
        by_sms = (2 * self.sm_count + blocks - 1) // blocks
        by_len = max(1, longest // 128)
        # under a window (as under a mask in blocks) the kernel cuts the keys a query can see, not the whole context
        return max(1, min(by_sms, by_len, 64)), 0

    def workspace_bytes(self, tokens: int) -> int:
        """Bytes of activations this part keeps in the step's workspace for `tokens` rows: the packed projection
        (and the float32 slices of two products cut along K), q, the attention's output and the output projection."""
        elem = 2 if self.dtype == torch.bfloat16 else 4
        packed = self.w_qkv.shape[0]
        return tokens * (packed + 2 * self.nq * max(self.hd, self.vd) + self.spec.hidden_size) * elem + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T = ctx.n_tokens
        ws = ctx.workspace
        group = ctx.groups[cache.group]
        nk = self.nkv if cache.writes else 0
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rot = self.position.rotary_dim if self.position is not None else 0
        if self.is_varied:
            return self._forward_varied(ctx, x, cache, group, nk, cos, sin, rot)
        decode = (self.dtype == torch.bfloat16 and ctx.pure_decode
                  and ops.attention_decode_usable(self.nq, self.nkv, self.hd, cache.page_size))
        fused = decode and ops.attention_decode_fuses_prep(self.hd, rot)
        w = self.w_qkv if cache.writes else self.w_q
        name = "attn_qkv" if cache.writes else "attn_q_only"
        if fused or T <= ops.SKINNY_BEST_ROWS or self.dtype != torch.bfloat16:
            packed = linear_sliced(ws, name, x, w, self.dtype)
        else:
            # the preparation kernel's fast path wants finished rows: with hundreds of them a product cut along K
            # would save less than adding its slices up there costs
            packed = linear(x, w, ws.buffer(name, T, w.shape[0], self.dtype))
        o = ws.buffer("attn_o", T, self.nq * self.hd, self.dtype)
        scale = float(self.spec.scale)
        if fused:
            # single decoded tokens: the attention kernel normalises, rotates and stores q, k and v itself
            self._decode(ctx, o, None, cache, group, scale,
                         prep=dict(packed=packed, nk=nk, rot=rot, positions=ctx.positions, slots=group.slots, cos=cos,
                                   sin=sin, q_gain=self.q_gain, k_gain=self.k_gain, eps=self.norm_eps,
                                   q_offset=self.q_off, k_offset=self.k_off, pairing=self.pairing,
                                   head_norm=self.head_norm))
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        q = ws.buffer("attn_q", T, self.nq * self.hd, self.dtype) if isinstance(packed, ops.Partials) else packed
        ops.attn_prep(packed, cache.k, cache.v, ctx.positions, group.slots, cos, sin, self.q_gain, self.k_gain,
                      self.nq, nk, self.hd, rot, cache.page_size, self.norm_eps, self.q_off, self.k_off, q_out=q,
                      pairing=self.pairing, head_norm=self.head_norm)
        packed = q
        if decode:
            self._decode(ctx, o, packed, cache, group, scale)
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        tc_bq = 0 if ctx.pure_decode else self.tc_tile_queries(cache.page_size)
        if tc_bq and ctx.has_array(f"attention_tiles_bq{tc_bq}_seq"):
            tile_seq = ctx.array(f"attention_tiles_bq{tc_bq}_seq")
            tile_q0 = ctx.array(f"attention_tiles_bq{tc_bq}_q0")
            ops.attention_tc(o, packed, packed.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks,
                             ctx.ctx_len, ctx.cu_q, tile_seq, tile_q0, tile_seq.numel(), T, self.nq, self.nkv,
                             self.hd, cache.page_size, self.window, scale)
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        tile_seq = ctx.array(self.tiles_name + "_seq")
        tile_q0 = ctx.array(self.tiles_name + "_q0")
        parts, part_size = self._split(ctx)
        scratch = None
        if parts > 1:
            scratch = ws.flat("attn_split", ops.attention_scratch_floats(T, self.nq, self.hd, parts), torch.float32)
        ops.paged_attention(o, packed, packed.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks,
                            ctx.ctx_len, ctx.cu_q, tile_seq, tile_q0, tile_seq.numel(), T, self.nq, self.nkv,
                            self.hd, cache.page_size, self.window, float(self.spec.scale), parts, part_size, scratch)
        return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)

    def _forward_varied(self, ctx, x, cache, group, nk, cos, sin, rot):
        """A layer with biases, another value width, a bound on the scores, a sink or a gate: the packed projection as
        an array (the gate's columns are read from it as they are), the general preparation and attention kernels."""
        T, ws = ctx.n_tokens, ctx.workspace
        if self.row_norms:
            return self._forward_row_norms(ctx, x, cache, group, cos, sin, rot)
        w = self.w_qkv if cache.writes else self.w_q_gate
        packed = linear(x, w, ws.buffer("attn_qkvg" if cache.writes else "attn_qg", T, w.shape[0], self.dtype))
        gate = None
        if self.gate_off >= 0:
            gate = packed[:, self.gate_off:] if cache.writes else packed[:, self.nq * self.hd:]
        bias = self.bias if (self.bias is None or cache.writes) else self.bias[: self.nq * self.hd]
        q = ws.buffer("attn_q", T, self.nq * self.hd, self.dtype)
        ops.attn_prep(packed, cache.k, cache.v, ctx.positions, group.slots, cos, sin, self.q_gain, self.k_gain,
                      self.nq, nk, self.hd, rot, cache.page_size, self.norm_eps, self.q_off, self.k_off, q_out=q,
                      pairing=self.pairing, head_norm=self.head_norm, bias=bias, vd=self.vd)
        o = ws.buffer("attn_o", T, self.nq * self.vd, self.dtype)
        mma_bq = 0 if ctx.pure_decode else self.mma_tile_queries()
        if mma_bq and ctx.has_array(f"attention_tiles_bq{mma_bq}_seq"):
            # portions of prompts in bfloat16: the products on the tensor cores, the weights float32 (three terms)
            tile_seq = ctx.array(f"attention_tiles_bq{mma_bq}_seq")
            ops.attention_mma(o, q, cache.k, cache.v, group.block_tables, group.max_blocks, ctx.ctx_len, ctx.cu_q, tile_seq,
                              ctx.array(f"attention_tiles_bq{mma_bq}_q0"), tile_seq.numel(), self.nq, self.nkv, self.hd, self.vd,
                              cache.page_size, self.window, float(self.spec.scale), softcap=self.softcap, sink=self.sink, gate=gate,
                              chunk=self.chunk)
            out = linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
            if self.o_bias is not None:
                ops.add_bias(out, self.o_bias)
            return out
        tile_seq = ctx.array(self.tiles_name + "_seq")
        tile_q0 = ctx.array(self.tiles_name + "_q0")
        # single decoded tokens: the keys in parts that are merged afterwards (the sink enters once, in the merge)
        parts, part_size = self._split(ctx)
        scratch = None
        if parts > 1:
            scratch = ws.flat("attn_split", ops.attention_scratch_floats(T, self.nq, self.vd, parts), torch.float32)
        ops.paged_attention(o, q, q.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks,
                            ctx.ctx_len, ctx.cu_q, tile_seq, tile_q0, tile_seq.numel(), T, self.nq, self.nkv,
                            self.hd, cache.page_size, self.window, float(self.spec.scale), parts, part_size, scratch,
                            vd=self.vd, softcap=self.softcap, sink=self.sink, gate=gate, chunk=self.chunk)
        out = linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        if self.o_bias is not None:
            ops.add_bias(out, self.o_bias)
        return out

    def _forward_row_norms(self, ctx, x, cache, group, cos, sin, rot):
        """A layer whose q and k are normed over their whole projections: the packed projection [q | k | v | gate], the short
        convolution over the channels of q, k, v (float32 out; its history from and to the request's state), one kernel for both
        norms, the rotation of q and k, the rotation of v and the cache write, and attention with the heads' sink scores, which
        turns each head's output back and applies the head's gate as it writes a row (value widths 64 and 128; one more kernel
        does that for other widths)."""
        T, ws = ctx.n_tokens, ctx.workspace
        if not cache.writes:
            raise ValueError("attention: a layer with norms over whole projections writes its own cache")
        nq, nk, hd, vd = self.nq, self.nkv, self.hd, self.vd
        C = (nq + nk) * hd + nk * vd
        if self.conv_w is not None:
            packed = linear(x, self.w_qkv, ws.buffer("attn_qkvg", T, self.w_qkv.shape[0], self.dtype))
            rows = ws.buffer("attn_conv", T, C, torch.float32)
            state = cache.state if cache.state is not None else ws.buffer("attn_no_state", 1, 1, torch.float32)
            ops.short_conv(rows, packed[:, :C], self.conv_w, state, ctx.cu_q, ctx.state_slots, ctx.n_seqs,
                           update_state=cache.state is not None)
            gate = packed[:, self.gate_off:] if self.gate_off >= 0 else None
        else:
            # the norms' kernel reads float32 rows: the projection leaves in float32
            rows = linear(x, self.w_qkv, ws.buffer("attn_qkvg32", T, self.w_qkv.shape[0], torch.float32))
            gate = None
            if self.gate_off >= 0:
                gate = ws.buffer("attn_gate", T, self.w_qkv.shape[0] - self.gate_off, self.dtype)
                ops.cast_rows(gate, rows[:, self.gate_off:].contiguous())
        vcos, vsin = self.value_position.tables() if self.value_position is not None else (None, None)
        q = ws.buffer("attn_q", T, nq * hd, self.dtype)
        ops.attn_prep_rows(rows, q, cache.k, cache.v, ctx.positions, group.slots, cos, sin, vcos, vsin, self.q_gain, self.k_gain,
                           nq, nk, hd, vd, rot, cache.page_size, self.norm_eps)
        o = ws.buffer("attn_o", T, nq * vd, self.dtype)
        per_head = bool(self.spec.gate_per_head and gate is not None)
        # value widths 64 and 128: the attention kernels turn a head's row back and apply the head's gate as they write it;
        # other widths leave that to one more kernel
        inside = vd in ops.ATTENTION_TURN_WIDTHS or (vcos is None and not per_head)
        turn = (vcos, vsin) if (inside and vcos is not None) else None
        kgate = gate if (inside or not per_head) else None
        mma_bq = 0 if ctx.pure_decode else self.mma_tile_queries()
        if mma_bq and ctx.has_array(f"attention_tiles_bq{mma_bq}_seq"):
            tile_seq = ctx.array(f"attention_tiles_bq{mma_bq}_seq")
            ops.attention_mma(o, q, cache.k, cache.v, group.block_tables, group.max_blocks, ctx.ctx_len, ctx.cu_q, tile_seq,
                              ctx.array(f"attention_tiles_bq{mma_bq}_q0"), tile_seq.numel(), nq, nk, hd, vd, cache.page_size, self.window,
                              float(self.spec.scale), sink=self.sink, gate=kgate, sink_values=self.sink_scores,
                              gate_per_head=per_head and kgate is not None, turn_back=turn)
        else:
            tile_seq = ctx.array(self.tiles_name + "_seq")
            tile_q0 = ctx.array(self.tiles_name + "_q0")
            parts, part_size = self._split(ctx)
            scratch = None
            if parts > 1:
                scratch = ws.flat("attn_split", ops.attention_scratch_floats(T, nq, vd, parts), torch.float32)
            ops.paged_attention(o, q, q.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks, ctx.ctx_len, ctx.cu_q,
                                tile_seq, tile_q0, tile_seq.numel(), T, nq, nk, hd, cache.page_size, self.window,
                                float(self.spec.scale), parts, part_size, scratch, vd=vd, sink=self.sink, gate=kgate,
                                sink_values=self.sink_scores, gate_per_head=per_head and kgate is not None, turn_back=turn,
                                positions=ctx.positions)
        if not inside:
            ops.unrotate_gate(o, gate if per_head else None, ctx.positions, vcos, vsin, nq, vd)
        out = linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        if self.o_bias is not None:
            ops.add_bias(out, self.o_bias)
        return out

    def _decode(self, ctx, o, q, cache, group, scale, prep=None) -> None:
        """Single decoded tokens: as many key parts as fill the SMs, at least 128 keys a part; the
        bound of the step's context class decides, not the lengths."""
        ws = ctx.workspace
        S = ctx.n_seqs
        G = self.nq // self.nkv
        chunks = (G + 7) // 8
        # the bound of the step's context class, for eager steps too: a step then cuts its keys the
        # same way whether it is replayed from a graph or launched directly, and gives the same bits
        bound = max(ctx.max_ctx_bound, ctx.max_ctx, 1)
        visible = min(bound, self.window) if self.window else bound
        blocks = max(1, S * self.nkv * chunks)
        # Key parts: at least 128 keys each, at most 64.  A block an SM where that still cuts every sequence's keys
        # into 4 parts or more (up to 4 sequences on 8 kv heads): two blocks an SM (the most that are resident) leave
        # the kernels after this one no room to start, and to ask for their weights, under it (a step of 4 sequences
        # of 640 keys: 0.898 ms with 8 parts, 0.798 with 4; of 1,500 keys: 0.994 with 9, 0.888 with 4).  Two blocks
        # an SM otherwise: with 8 sequences 2 parts are too few (0.935 against 0.907 ms with 4; at 1,500 keys 1.095
        # against 1.022).
        one_each = self.sm_count // blocks
        target = one_each if one_each >= 4 else (2 * self.sm_count) // blocks
        parts = max(1, min(target, visible // 128, 64))
        scratch = counters = None
        if parts > 1:
            scratch = ws.flat("attn_decode_split", ops.attention_decode_scratch_floats(S, self.nq, self.hd, parts),
                              torch.float32)
            counters = ws.flat("attn_decode_counters", ops.attention_decode_counters(max(ctx.max_seqs_bound, S), self.nq, self.nkv),
                               torch.int32, zero=True)
        ops.attention_decode(o, q, q.stride(0) if q is not None else 0, cache.k, cache.v, group.block_tables,
                             group.max_blocks, ctx.ctx_len, ctx.cu_q, S, self.nq, self.nkv, self.hd, cache.page_size,
                             self.window, scale, parts, bound, scratch, counters, **(prep or {}))


register_mixer("attention", GQAAttention)
