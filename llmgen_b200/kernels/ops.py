"""Python bindings of the CUDA kernels: thin functions from torch tensors to the C ABI.

torch is used as the allocator and for stream handles only; every function launches on
`torch.cuda.current_stream()`, allocates nothing and never synchronises, so a sequence of
calls can be captured into a CUDA graph.  There is no CPU path: a tensor that is not on a
CUDA device raises `KernelError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel arguments must live on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked of torch's C layer directly where it offers that: the
    `torch.cuda.current_stream()` object costs several microseconds, more than a launch."""
    if _raw_stream is not None and _raw_device is not None:
        return c_void_p(_raw_stream(_raw_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class _Counter:
    """How many kernels of this package were launched (a claim for benchmarks' records)."""
    launches = 0


def launches() -> int:
    return _Counter.launches


def _check(lib, rc: int, n_kernels: int = 1) -> None:
    if rc != 0:
        raise KernelError(lib.llmk_last_error().decode("utf-8", "replace"))
    _Counter.launches += n_kernels


def _row_stride(t: torch.Tensor) -> int:
    if t.dim() < 2:
        return t.shape[-1] if t.dim() == 1 else 1
    if t.stride(-1) != 1:
        raise KernelError("kernel operands must be contiguous in their last dimension")
    return t.stride(-2)


class Partials:
    """The result of a matrix product cut along K: float32 slices [splits, rows, cols] whose sum, in
    slice order, is the product.  The kernels that consume a product (`add_rmsnorm`, `attn_prep`,
    `attention_decode`, `silu_mul`) take a `Partials` in place of the finished array and do the sum themselves."""

    def __init__(self, tensor: torch.Tensor):
        if tensor.dim() != 3 or tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError("partial sums are a contiguous float32 [splits, rows, cols] array")
        self.tensor = tensor
        self.splits, self.rows, self.cols = tensor.shape

    @property
    def split_stride(self) -> int:
        return self.rows * self.cols

    def sum(self) -> torch.Tensor:
        """The finished product (float32), for callers that have no kernel taking slices."""
        return self.tensor.sum(dim=0)


# ---------------------------------------------------------------------------- elementwise
def embed_rows(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, bad_flag: Optional[torch.Tensor] = None,
               ids_from: Optional[torch.Tensor] = None, sampled: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[t] (float32 [n, H]) = table[ids[t]] * scale; ids int32 on the device.  With `ids_from` and
    `sampled` (int32, device) a row whose ids_from[t] >= 0 takes the id sampled[ids_from[t]]."""
    lib = build.load("elementwise")
    n, H = out.shape
    _check(lib, lib.llmk_embed_rows(_ptr(out), _ptr(table), _ptr(ids), _ptr(ids_from), _ptr(sampled), c_int(n), c_int(H),
                                    c_int(table.shape[0]), _ptr(bad_flag), c_int(dtype_code(table.dtype)), c_float(scale),
                                    _stream()))


def logit_cap(logits: torch.Tensor, cap: float, scale: float = 1.0) -> None:
    """logits (float32, contiguous) = scale * logits, then (cap > 0) cap * tanh(logits / cap), in place."""
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("logit_cap: logits must be contiguous float32")
    lib = build.load("elementwise")
    _check(lib, lib.llmk_logit_cap(_ptr(logits), c_longlong(logits.numel()), c_float(scale), c_float(cap), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, out: torch.Tensor,
                eps: float, weight_offset: float = 0.0, rows: Optional[torch.Tensor] = None,
                write_resid: bool = True) -> None:
    """resid (float32 [n, H]) += delta; out = rmsnorm(resid) * (weight + offset).  `delta` is an
    array of the output's dtype, a `Partials`, or None.

    With `rows` (int32 [m]) output row r is computed from source row rows[r] and the
    residual is left untouched."""
    lib = build.load("elementwise")
    H = resid.shape[-1]
    n_rows = out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("add_rmsnorm: residual and gain must be float32")
    splits, split_stride = 0, 0
    if isinstance(delta, Partials):
        if delta.cols != H or delta.rows != resid.shape[0]:
            raise KernelError("add_rmsnorm: partial sums do not have the residual's shape")
        splits, split_stride, delta = delta.splits, delta.split_stride, delta.tensor
    elif delta is not None and (delta.dtype != out.dtype or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must be contiguous and of the output's dtype")
    if rows is not None:
        write_resid = False
    _check(lib, lib.llmk_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), c_int(n_rows),
                                     c_int(H), c_float(eps), c_float(weight_offset), c_int(1 if write_resid else 0),
                                     c_int(splits), c_longlong(split_stride), c_int(dtype_code(out.dtype)), _stream()))


def silu_mul(out: torch.Tensor, gate_up, group: int = 0) -> None:
    """out[n, F] = silu(gate) * up, where gate_up[n, 2F] (an array or a `Partials`) alternates `group`
    gate columns and `group` up columns (group 0 or F: gate in columns [0, F), up in [F, 2F))."""
    lib = build.load("elementwise")
    n, F = out.shape
    splits, split_stride = 0, 0
    if isinstance(gate_up, Partials):
        splits, split_stride, ld = gate_up.splits, gate_up.split_stride, gate_up.cols
        gate_up = gate_up.tensor
    else:
        ld = _row_stride(gate_up)
    _check(lib, lib.llmk_silu_mul(_ptr(out), _ptr(gate_up), c_int(n), c_int(F), c_int(ld),
                                  c_int(group if group else F), c_int(splits), c_longlong(split_stride),
                                  c_int(dtype_code(out.dtype)), _stream()))


def widen(out: torch.Tensor, src: torch.Tensor) -> None:
    """out (float32) = src, element by element (both contiguous)."""
    lib = build.load("elementwise")
    _check(lib, lib.llmk_widen(_ptr(out), _ptr(src), c_longlong(src.numel()), c_int(dtype_code(src.dtype)), _stream()))


# ------------------------------------------------------------------------------ attn_prep
# Codes of the C ABI (csrc/common.cuh).  "half": pairs (i, i + rot / 2), the reference's pairing
# (src/backend/cpu/rope.zig:13-45); "interleaved": pairs (2i, 2i + 1).  The latent-attention kernels implement both; the
# grouped-query attention's preparation kernel implements both in its general form ("half" alone in the 16-byte forms
# and inside the decode kernel); what a kernel does not implement it refuses with a message, never rotates wrongly.
ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}
# "rmsnorm": gains, before the rotation; "unit_rms_after": no gains, over the rotated head
HEAD_NORMS = {"rmsnorm": 0, "unit_rms_after": 1}


def pairing_code(pairing: str) -> int:
    try:
        return ROTARY_PAIRINGS[pairing]
    except KeyError:
        raise KernelError(f"unknown rotary pairing {pairing!r} (known: {', '.join(ROTARY_PAIRINGS)})") from None


def head_norm_code(kind: str) -> int:
    try:
        return HEAD_NORMS[kind]
    except KeyError:
        raise KernelError(f"no kernel normalises heads with {kind!r} (known: {', '.join(HEAD_NORMS)})") from None


def attn_prep_set_by_token(on: bool) -> None:
    """Which 16-byte variant `attn_prep` runs on prompts: a warp on several heads of one token at a
    time (the default) or a row at a time (for comparisons and tests)."""
    build.load("attn_prep").llmk_attn_prep_set_by_token(c_int(1 if on else 0))


def attn_prep(qkv, kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
              positions: Optional[torch.Tensor], slots: Optional[torch.Tensor], cos: Optional[torch.Tensor],
              sin: Optional[torch.Tensor], q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
              nq: int, nk: int, hd: int, rot: int, page_size: int, eps: float,
              q_offset: float = 0.0, k_offset: float = 0.0, q_out: Optional[torch.Tensor] = None,
              pairing: str = "half", head_norm: str = "rmsnorm", bias: Optional[torch.Tensor] = None, vd: int = 0) -> None:
    """Per-head norm and rotary encoding of q and k, and the cache write of k, v.  `qkv` holds the
    packed rows [n, (nq + 2 nk) hd] as an array (q is then rewritten in place unless `q_out` is
    given) or as a `Partials` (q goes to `q_out`, which gives the storage dtype).  `pairing` says which
    values of a head the rotary encoding turns together and `head_norm` which norm runs over a head
    (see `ROTARY_PAIRINGS`, `HEAD_NORMS`); the kernel refuses the ones it does not implement.  `bias` (float32 over the
    packed columns) is added before the norms; `vd` is the width of a value head where it differs from `hd`."""
    lib = build.load("attn_prep")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != (nq + nk) * hd + nk * (vd or hd)):
        raise KernelError("attn_prep: the bias is one float32 per packed column")
    nkv_cache = kcache.shape[1] if kcache is not None else 0
    splits, split_stride = 0, 0
    if isinstance(qkv, Partials):
        if q_out is None:
            raise KernelError("attn_prep: partial sums need a place for q")
        n, stride, src = qkv.rows, qkv.cols, qkv.tensor
        splits, split_stride = qkv.splits, qkv.split_stride
        dtype = q_out.dtype
    else:
        n, stride, src = qkv.shape[0], _row_stride(qkv), qkv
        dtype = qkv.dtype
        if q_out is None:
            q_out = qkv
    if q_out.dtype != dtype:
        raise KernelError("attn_prep: q_out must have the storage dtype")
    _check(lib, lib.llmk_attn_prep(_ptr(src), c_longlong(stride), c_int(splits), c_longlong(split_stride),
                                   _ptr(q_out), c_longlong(_row_stride(q_out)), _ptr(kcache), _ptr(vcache),
                                   _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(q_gain), _ptr(k_gain),
                                   c_int(n), c_int(nq), c_int(nk), c_int(nkv_cache), c_int(hd), c_int(rot),
                                   c_int(page_size), c_float(eps), c_float(q_offset), c_float(k_offset),
                                   c_int(pairing_code(pairing)), c_int(head_norm_code(head_norm)),
                                   _ptr(bias), c_int(vd), c_int(dtype_code(dtype)), _stream()))


# ------------------------------------------------------------------------- matrix products
def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores (float32 multiply-add, fixed k order)."""
    lib = build.load("gemm_simt")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    if a.dtype != w.dtype:
        raise KernelError("gemm: a and w must share a dtype")
    _check(lib, lib.llmk_gemm_simt(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                   c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                   c_int(1 if accumulate else 0), c_int(dtype_code(a.dtype)),
                                   c_int(dtype_code(out.dtype)), _stream()))


GEMV_MAX_ROWS = 4


def gemv_bf16(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T for M <= 4 in bfloat16, float32 accumulation."""
    lib = build.load("gemv")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemv: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    _check(lib, lib.llmk_gemv_bf16(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                   c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                   c_int(1 if accumulate else 0), c_int(dtype_code(out.dtype)), _stream()))


def gemv_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 8 == 0
            and _row_stride(a) % 8 == 0 and _row_stride(w) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_tc_plans = {}


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the tiled product is best cut when its tiles are too few for the SMs (1: not cut)."""
    key = (M, N, K)
    v = _tc_plans.get(key)
    if v is None:
        v = int(build.load("gemm_tc").llmk_gemm_tc_splits(c_int(M), c_int(N), c_int(K)))
        _tc_plans[key] = v
    return v


def gemm_tc_sliced(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """The tiled tensor-core product cut along K: out is float32 [splits, M, N] and receives the sums
    of `splits` slices of K, for a consumer that adds them up (`Partials`)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_tc: operands a{list(a.shape)} {a.dtype} w{list(w.shape)} {w.dtype} do not fit")
    if out.dim() != 3 or out.shape[1] != M or out.shape[2] != N or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("gemm_tc: the slices go to a contiguous float32 [splits, M, N] array")
    _check(lib, lib.llmk_gemm_tc_sliced(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_longlong(_row_stride(a)),
                                        c_longlong(_row_stride(w)), c_longlong(N), c_int(out.shape[0]),
                                        _ptr(tc_error_flag(a.device)), c_int(1), _stream()))


def gemm_tc_set_pair_mode(mode: int) -> None:
    """How `gemm_tc` uses pairs of blocks on 256-row tiles (`tcgen05.mma.cta_group::2`): 0 never,
    1 where the product has the rows for it (the default), 2 / 3 always, with tiles 256 / 128 columns
    wide (for measurements and tests)."""
    build.load("gemm_tc").llmk_gemm_tc_set_pair_mode(c_int(mode))


def gemm_tc_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the tensor-core product takes these operands: bfloat16, rows starting on 16-byte
    boundaries (what its TMA loads need)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and _row_stride(a) % 8 == 0 and _row_stride(w) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_status = {}      # device (object or its string) -> (both flags, view of [0], view of [1])


def _status_of(device):
    entry = _status.get(device)
    if entry is None:
        entry = _status.get(str(device))
        if entry is None:
            flags = torch.zeros(2, dtype=torch.int32, device=device)
            entry = (flags, flags[0:1], flags[1:2])
            _status[str(device)] = entry
        _status[device] = entry              # the device object itself as a second key: no string per launch
    return entry


def status_flags(device) -> torch.Tensor:
    """Two device ints that kernels raise and the engine reads with a step's results: [0] a kernel's error
    (1: a bounded wait ran out; 2: a sequence longer than its attention launch was sized for), [1] a token
    id outside the vocabulary met by the embedding kernel."""
    return _status_of(device)[0]


def tc_error_flag(device) -> torch.Tensor:
    """Device int that a kernel raises when one of its bounded waits gave up or an input broke its bounds."""
    return _status_of(device)[1]


def bad_token_flag(device) -> torch.Tensor:
    """Device int that `embed_rows` raises when it meets an id outside the table."""
    return _status_of(device)[2]


def status_message(kernel_error: int, bad_token: int) -> Optional[str]:
    """What the two flags say, or None when both are clear."""
    if kernel_error == 2:
        return "a sequence was longer than the bound its attention launch was sized for (results of that step are invalid)"
    if kernel_error != 0:
        return "a kernel gave up waiting on a barrier (results of that step are invalid)"
    if bad_token != 0:
        return "a token id outside the vocabulary reached the embedding (its row was read as zeros)"
    return None


def check_tc_errors(device) -> None:
    """Raise if a kernel reported a wait that ran out or an input beyond its launch's bounds (synchronises)."""
    entry = _status.get(str(device))
    code = int(entry[1].item()) if entry is not None else 0
    if code != 0:
        entry[1].zero_()
        raise KernelError(status_message(code, 0))


_sm_counts: Dict[str, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (launch plans are made from it, not from a constant)."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    key = str(dev)
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _sm_counts[key]


GATED_ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gated: bool = False, pdl: bool = True,
            activation: str = "silu") -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tensor cores (tcgen05), bfloat16 operands, float32
    accumulation; `out` is bfloat16 or float32.  With `gated`, w interleaves gate and up rows in
    groups of 16 and out[M, N/2] = act(gate) * up, act = `activation` ("silu" or "gelu_tanh").  `pdl`: launched as a programmatic dependent of the
    kernel before it, like every other kernel here (its set-up then runs under that kernel's tail; a
    2,048-token prompt took 4.85 ms without and 4.45 ms with it)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if gated else N
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != n_out:
        raise KernelError(f"gemm_tc: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    _check(lib, lib.llmk_gemm_tc(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                 c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                 c_int(GATED_ACTIVATIONS[activation] if gated else 0), c_int(dtype_code(out.dtype)),
                                 _ptr(tc_error_flag(a.device)), c_int(1 if pdl else 0), _stream()))


ROWS8_MAX_ROWS = 8           # what the kernel takes
ROWS8_BEST_ROWS = 4          # up to here the engine uses it (decode steps of 1 / 2 / 4 / 8 sequences: +2.3 / +5.5 / +0.7 / -1.0 %)
ROWS8_GATED_BEST_ROWS = 1    # and its gated form (a step of one sequence 0.780 -> 0.767 ms; of 2 and 4: 0.773 -> 0.817, 0.898 -> 1.015)
_rows8_plans = {}


def gemm_rows8_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product for up to 8 rows that loads W straight from global memory into `mma.sync`
    (csrc/gemm_rows8.cu) takes these operands."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] > ROWS8_MAX_ROWS:
        return False
    lib = build.load("gemm_rows8")
    M, K = a.shape
    return bool(lib.llmk_gemm_rows8_usable(_ptr(a), _ptr(w), c_int(M), c_int(w.shape[0]), c_int(K), c_longlong(_row_stride(a)),
                                           c_longlong(_row_stride(w))))


def gemm_rows8_slices(N: int, K: int) -> int:
    """Into how many slices of K that product cuts [M, K] x [N, K]^T."""
    v = _rows8_plans.get((N, K))
    if v is None:
        v = int(build.load("gemm_rows8").llmk_gemm_rows8_slices(c_int(N), c_int(K)))
        _rows8_plans[(N, K)] = v
    return v


def gemm_rows8(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[slices, M, N] (float32, contiguous; slices = gemm_rows8_slices(N, K)) = the partial sums of a[M, K] @ w[N, K]^T
    over the slices of K, M <= 8."""
    lib = build.load("gemm_rows8")
    M, K = a.shape
    N = w.shape[0]
    if out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (gemm_rows8_slices(N, K), M, N) or w.shape[1] != K:
        raise KernelError(f"gemm_rows8: a{list(a.shape)} w{list(w.shape)} need contiguous float32 slices "
                          f"[{gemm_rows8_slices(N, K)}, {M}, {N}], got {list(out.shape)} {out.dtype}")
    _check(lib, lib.llmk_gemm_rows8(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_longlong(_row_stride(a)),
                                    c_longlong(_row_stride(w)), _stream()))


def gemm_rows8_gated_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the gated form of that product (w interleaving 16 gate and 16 up rows) takes these operands."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] > ROWS8_MAX_ROWS:
        return False
    lib = build.load("gemm_rows8")
    M, K = a.shape
    return bool(lib.llmk_gemm_rows8_gated_usable(_ptr(a), _ptr(w), c_int(M), c_int(w.shape[0]), c_int(K), c_longlong(_row_stride(a)),
                                                 c_longlong(_row_stride(w))))


def gemm_rows8_gated(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M, N/2] (bfloat16) = silu(gate) * up of a[M, K] @ w[N, K]^T, w interleaving gate and up rows in groups of 16, M <= 8."""
    lib = build.load("gemm_rows8")
    M, K = a.shape
    N = w.shape[0]
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N // 2) or w.shape[1] != K:
        raise KernelError(f"gemm_rows8_gated: a{list(a.shape)} w{list(w.shape)} need a bfloat16 result [{M}, {N // 2}], got {list(out.shape)} {out.dtype}")
    _check(lib, lib.llmk_gemm_rows8_gated(_ptr(out), c_longlong(_row_stride(out)), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                          c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), _stream()))


SKINNY_MAX_ROWS = 256        # what the kernel takes
SKINNY_BEST_ROWS = 32        # up to here it is the faster product (measured at 16, 32, 48 and 64 rows against the tiled product cut along K)
# most bytes of float32 slices one cut product leaves: about one 128 x 128 item per SM for the tiled product,
# 8 slices of 64 rows by the widest matrix for the few-rows one
SLICED_PRODUCT_BYTES = 16 << 20
SKINNY_DIRECT, SKINNY_PARTIAL, SKINNY_GATED = 0, 1, 2
SKINNY_CLUSTER_GATED = 5     # slices of K added up inside a cluster (2 or 4), then silu(gate) * up: out[M, N/2]
SKINNY_CLUSTER_MAX_ROWS = 64
_cluster_plans = {}
_skinny_plans = {}


def gemm_skinny_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the few-rows product cuts [M, K] x [N, K]^T (1: no cut)."""
    key = (M, N, K)
    v = _skinny_plans.get(key)
    if v is None:
        v = int(build.load("gemm_skinny").llmk_gemm_skinny_splits(c_int(M), c_int(N), c_int(K)))
        _skinny_plans[key] = v
    return v


def gemm_skinny_cluster_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the product is cut when a thread-block cluster adds them up
    (1: it is not cut)."""
    key = (M, N, K)
    v = _cluster_plans.get(key)
    if v is None:
        v = int(build.load("gemm_skinny").llmk_gemm_skinny_cluster_splits(c_int(M), c_int(N), c_int(K)))
        _cluster_plans[key] = v
    return v


def gemm_skinny(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, mode: int = SKINNY_DIRECT, splits: int = 1) -> None:
    """The weight-streaming tensor-core product for M <= 256 rows (csrc/gemm_skinny.cu).
    SKINNY_DIRECT: out[M, N]; SKINNY_GATED: out[M, N/2] = silu(gate) * up; SKINNY_PARTIAL: out is
    float32 [splits, M, N] and receives the partial sums of `splits` slices of K;
    SKINNY_CLUSTER_GATED: out[M, N/2] = silu(gate) * up from `splits` slices of K (2 or 4) added up
    inside a thread-block cluster (M <= 64)."""
    lib = build.load("gemm_skinny")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_skinny: operands a{list(a.shape)} {a.dtype} w{list(w.shape)} {w.dtype} do not fit")
    if mode == SKINNY_PARTIAL:
        if out.dim() != 3 or out.shape[1] != M or out.shape[2] != N or out.dtype != torch.float32 or not out.is_contiguous():
            raise KernelError("gemm_skinny: partial sums go to a contiguous float32 [splits, M, N] array")
        splits, ldc = out.shape[0], N
    else:
        n_out = N // 2 if mode in (SKINNY_GATED, SKINNY_CLUSTER_GATED) else N
        if out.shape[0] != M or out.shape[1] != n_out:
            raise KernelError(f"gemm_skinny: out{list(out.shape)} does not fit [{M}, {n_out}]")
        splits, ldc = (splits if mode == SKINNY_CLUSTER_GATED else 1), _row_stride(out)
    _check(lib, lib.llmk_gemm_skinny(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                     c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(ldc),
                                     c_int(splits), c_int(mode), c_int(dtype_code(out.dtype)),
                                     _ptr(tc_error_flag(a.device)), _stream()))


def gemm_skinny_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return a.shape[0] <= SKINNY_MAX_ROWS and gemm_tc_usable(a, w)


# ------------------------------------------------------------------------------ attention
def attention_tile_queries(nq: int, nkv: int) -> int:
    """Queries per tile of `paged_attention` for this group size."""
    lib = build.load("attention")
    return int(lib.llmk_attention_tile_queries(c_int(nq), c_int(nkv)))


def attention_scratch_floats(n_tokens: int, nq: int, hd: int, num_parts: int) -> int:
    return 0 if num_parts <= 1 else n_tokens * nq * num_parts * (hd + 2)


def _check_sinks(who: str, sink: bool, sink_values: Optional[torch.Tensor], nq: int) -> None:
    if sink_values is not None and (not sink or sink_values.dtype != torch.float32 or sink_values.numel() != nq
                                    or not sink_values.is_contiguous()):
        raise KernelError(f"{who}: the sinks' scores are one float32 per query head, with `sink` set")


ATTENTION_TURN_WIDTHS = (64, 128)    # value widths whose rows the attention kernels turn back themselves


def _check_turn(who: str, turn_back, positions, vd: int, gate, gate_per_head: bool, nq: int):
    if gate is not None and gate_per_head and gate.shape[1] != nq:
        raise KernelError(f"{who}: a gate per head is [tokens, heads]")
    if turn_back is None:
        return None, None
    cos, sin = turn_back
    if vd not in ATTENTION_TURN_WIDTHS or positions is None or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
            or cos.shape[1] != vd // 2 or tuple(sin.shape) != tuple(cos.shape) or not cos.is_contiguous() or not sin.is_contiguous():
        raise KernelError(f"{who}: rows are turned back for value widths {ATTENTION_TURN_WIDTHS}, by float32 tables [positions, vd / 2]")
    return cos, sin


def paged_attention(out: torch.Tensor, q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, n_tokens: int, nq: int, nkv: int,
                    hd: int, page_size: int, window: int, scale: float, num_parts: int = 1, part_size: int = 0,
                    scratch: Optional[torch.Tensor] = None, vd: int = 0, softcap: float = 0.0, sink: bool = False,
                    gate: Optional[torch.Tensor] = None, chunk: int = 0, sink_values: Optional[torch.Tensor] = None,
                    gate_per_head: bool = False, turn_back: Optional[tuple] = None, positions: Optional[torch.Tensor] = None) -> None:
    """out[t, nq*vd] = causal GQA of q[t] over the paged cache (see csrc/attention.cu).  `vd`: the values' width where
    it differs from `hd`; `softcap` > 0 bounds the scores by softcap * tanh(s / softcap); `sink` adds exp(0) to the
    softmax's denominator (exp(sink_values[head]) with `sink_values`, float32 [nq]); `gate` [tokens, nq*vd] (storage dtype): the result is multiplied by sigmoid(gate)
    (`gate_per_head`: [tokens, nq], one number per head); `turn_back` = (cos, sin) float32 [positions, vd / 2] with `positions` (the
    tokens' positions): each head's row is turned back in pairs (m, m + vd / 2) by minus its position before the gate (value widths
    `ATTENTION_TURN_WIDTHS`); `chunk` > 0:
    a query sees the keys at or before it inside its own block of that many positions, counted from the sequence's start."""
    lib = build.load("attention")
    if gate is not None and gate.dtype != q.dtype:
        raise KernelError("paged_attention: the gate has the storage dtype")
    _check_sinks("paged_attention", sink, sink_values, nq)
    tcos, tsin = _check_turn("paged_attention", turn_back, positions, vd or hd, gate, gate_per_head, nq)
    if num_parts > 1:
        need = attention_scratch_floats(n_tokens, nq, vd or hd, num_parts)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"paged_attention: split into {num_parts} parts needs {need} float32 of scratch")
    _check(lib, lib.llmk_paged_attention(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                         _ptr(kcache), _ptr(vcache), _ptr(block_tables), c_int(max_blocks),
                                         _ptr(ctx_len), _ptr(cu_q), _ptr(tile_seq), _ptr(tile_q0), c_int(n_tiles),
                                         c_int(n_tokens), c_int(nq), c_int(nkv), c_int(hd), c_int(page_size),
                                         c_int(window), c_float(scale), c_int(num_parts), c_int(part_size),
                                         _ptr(scratch), c_int(vd), c_float(softcap), c_int(1 if sink else 0), _ptr(sink_values),
                                         _ptr(gate), c_longlong(_row_stride(gate) if gate is not None else 0), c_int(chunk),
                                         c_int(1 if gate_per_head else 0), _ptr(tcos), _ptr(tsin), _ptr(positions),
                                         c_int(dtype_code(q.dtype)), _stream()),
           2 if num_parts > 1 else 1)


def attention_mma_tile_queries(nq: int, nkv: int, hd: int, vd: int) -> int:
    """Queries per tile of `attention_mma` (0: it does not take these sizes)."""
    return int(build.load("attention_mma").llmk_attention_mma_tile_queries(c_int(nq), c_int(nkv), c_int(hd), c_int(vd)))


def attention_mma(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                  max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor,
                  n_tiles: int, nq: int, nkv: int, hd: int, vd: int, page_size: int, window: int, scale: float,
                  softcap: float = 0.0, sink: bool = False, gate: Optional[torch.Tensor] = None, chunk: int = 0,
                  sink_values: Optional[torch.Tensor] = None, gate_per_head: bool = False, turn_back: Optional[tuple] = None) -> None:
    """Prompt portions in bfloat16 with 32-bit softmax weights on the tensor cores (csrc/attention_mma.cu): the same
    result as `paged_attention` with these options, tiles of `attention_mma_tile_queries` queries."""
    lib = build.load("attention_mma")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or (gate is not None and gate.dtype != torch.bfloat16):
        raise KernelError("attention_mma: bfloat16 only")
    _check_sinks("attention_mma", sink, sink_values, nq)
    tcos, tsin = _check_turn("attention_mma", turn_back, ctx_len, vd, gate, gate_per_head, nq)
    _check(lib, lib.llmk_attention_mma(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(_row_stride(q)), _ptr(kcache),
                                       _ptr(vcache), _ptr(block_tables), c_int(max_blocks), _ptr(ctx_len), _ptr(cu_q), _ptr(tile_seq),
                                       _ptr(tile_q0), c_int(n_tiles), c_int(nq), c_int(nkv), c_int(hd), c_int(vd), c_int(page_size),
                                       c_int(window), c_float(scale), c_float(softcap), c_int(1 if sink else 0), _ptr(sink_values),
                                       _ptr(gate), c_longlong(_row_stride(gate) if gate is not None else 0), c_int(chunk),
                                       c_int(1 if gate_per_head else 0), _ptr(tcos), _ptr(tsin), _stream()))


def attention_decode_set_cluster_merge(on: bool) -> None:
    """Whether `attention_decode` merges up to 8 key parts through the shared memory of a thread-block
    cluster (the default) or through global memory and a ticket (for measurements and tests)."""
    build.load("attention_decode").llmk_attention_decode_set_cluster_merge(c_int(1 if on else 0))


def attention_decode_usable(nq: int, nkv: int, hd: int, page_size: int) -> bool:
    return bool(build.load("attention_decode").llmk_attention_decode_usable(c_int(nq), c_int(nkv), c_int(hd), c_int(page_size)))


def attention_decode_scratch_floats(n_seqs: int, nq: int, hd: int, parts: int) -> int:
    return 0 if parts <= 1 else n_seqs * nq * parts * (hd + 2)


def attention_decode_counters(n_seqs: int, nq: int, nkv: int) -> int:
    lib = build.load("attention_decode")
    lib.llmk_attention_decode_counters.restype = c_longlong
    return int(lib.llmk_attention_decode_counters(c_int(n_seqs), c_int(nq), c_int(nkv)))


def attention_decode_fuses_prep(hd: int, rot: int) -> bool:
    return bool(build.load("attention_decode").llmk_attention_decode_fuses_prep(c_int(hd), c_int(rot)))


def attention_decode(out: torch.Tensor, q: Optional[torch.Tensor], q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                     n_seqs: int, nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                     parts: int, max_ctx: int, scratch: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                     packed=None, nk: int = 0, rot: int = 0, positions: Optional[torch.Tensor] = None,
                     slots: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                     sin: Optional[torch.Tensor] = None, q_gain: Optional[torch.Tensor] = None,
                     k_gain: Optional[torch.Tensor] = None, eps: float = 0.0, q_offset: float = 0.0,
                     k_offset: float = 0.0, pairing: str = "half", head_norm: str = "rmsnorm") -> None:
    """out[t] = attention of the single token of each sequence over the paged cache, bfloat16
    (csrc/attention_decode.cu).  `counters` (int32) must be zero before the first call.  With
    `packed` (the q/k/v projection rows as an array or a `Partials`) the kernel also normalises and
    rotates q and k and writes k and v to the cache, and `q` is not read.  `max_ctx` must bound every
    sequence's length: a longer one is skipped and raises the device error flag (`check_tc_errors`)."""
    lib = build.load("attention_decode")
    if kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or (q is not None and q.dtype != torch.bfloat16):
        raise KernelError("attention_decode: bfloat16 only")
    if parts > 1:
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < attention_decode_scratch_floats(n_seqs, nq, hd, parts):
            raise KernelError("attention_decode: scratch too small")
        if counters is None or counters.dtype != torch.int32 or counters.numel() < attention_decode_counters(n_seqs, nq, nkv):
            raise KernelError("attention_decode: counters too small")
    splits, split_stride, packed_stride, src = 0, 0, 0, None
    if isinstance(packed, Partials):
        src, splits, split_stride, packed_stride = packed.tensor, packed.splits, packed.split_stride, packed.cols
    elif packed is not None:
        if packed.dtype != torch.bfloat16:
            raise KernelError("attention_decode: packed rows must be bfloat16 or partial sums")
        src, packed_stride = packed, _row_stride(packed)
    _check(lib, lib.llmk_attention_decode(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                          _ptr(kcache), _ptr(vcache), _ptr(block_tables), c_int(max_blocks),
                                          _ptr(ctx_len), _ptr(cu_q), c_int(n_seqs), c_int(nq), c_int(nkv), c_int(hd),
                                          c_int(page_size), c_int(window), c_float(scale), c_int(parts), c_int(max_ctx),
                                          _ptr(scratch), _ptr(counters), _ptr(src), c_longlong(packed_stride),
                                          c_int(splits), c_longlong(split_stride), c_int(nk), c_int(rot),
                                          _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(q_gain), _ptr(k_gain),
                                          c_float(eps), c_float(q_offset), c_float(k_offset),
                                          c_int(pairing_code(pairing)), c_int(head_norm_code(head_norm)),
                                          _ptr(tc_error_flag(out.device)), _stream()))


def attention_tc_tile_queries(nq: int, nkv: int, hd: int, page_size: int) -> int:
    """Queries per tile of the tensor-core attention; 0 when it does not take these sizes."""
    return int(build.load("attention_tc").llmk_attention_tc_tile_queries(c_int(nq), c_int(nkv), c_int(hd), c_int(page_size)))


def attention_tc(out: torch.Tensor, q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, n_tokens: int, nq: int, nkv: int,
                 hd: int, page_size: int, window: int, scale: float, v_lbo: int = 0, v_sbo: int = 0) -> None:
    """out[t, nq*hd] = causal GQA of q[t] over the paged cache on the tensor cores, bfloat16
    (csrc/attention_tc.cu).  q is [n_tokens, >= nq*hd] with row stride q_stride."""
    lib = build.load("attention_tc")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_tc: bfloat16 only")
    _check(lib, lib.llmk_attention_tc(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                      c_int(n_tokens), _ptr(kcache), _ptr(vcache), c_longlong(kcache.shape[0]),
                                      _ptr(block_tables), c_int(max_blocks), _ptr(ctx_len), _ptr(cu_q),
                                      _ptr(tile_seq), _ptr(tile_q0), c_int(n_tiles), c_int(nq), c_int(nkv), c_int(hd),
                                      c_int(page_size), c_int(window), c_float(scale), _ptr(tc_error_flag(q.device)),
                                      ctypes.c_uint(v_lbo), ctypes.c_uint(v_sbo), _stream()))


# ------------------------------------------------------------------------------- sampling
SAMPLE_SPLIT = 32
_SAMPLE_ROW_BYTES = SAMPLE_SPLIT * 8 + 4        # a row's candidates and its ticket counter


def sample_scratch_bytes(max_rows: int) -> int:
    return max_rows * _SAMPLE_ROW_BYTES


def sample_scratch(max_rows: int, device) -> torch.Tensor:
    """Scratch for `sample` with up to `max_rows` rows: zeroed, because the ticket counters in it must start
    at zero (every launch leaves them at zero)."""
    return torch.zeros(sample_scratch_bytes(max_rows) // 4, dtype=torch.int32, device=device)


def sample(out_ids: torch.Tensor, logits: torch.Tensor, temps: torch.Tensor, seed: Optional[torch.Tensor],
           scratch: torch.Tensor, row_keys: Optional[torch.Tensor] = None) -> None:
    """out_ids[s] (int32) = argmax or Gumbel-max draw of logits[s] (float32 [n, V]); `scratch` from
    `sample_scratch`.  The random numbers of row s come from `seed` (one 64-bit value) and s, or, with
    `row_keys` (64 bits a row, as int64 or pairs of int32), from that row's key alone."""
    lib = build.load("sampling")
    n, V = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    rows = scratch.numel() * scratch.element_size() // _SAMPLE_ROW_BYTES
    if rows < n:
        raise KernelError("sample: scratch too small")
    if row_keys is not None and row_keys.numel() * row_keys.element_size() < 8 * n:
        raise KernelError("sample: one 64-bit key per row is required")
    _check(lib, lib.llmk_sample(_ptr(out_ids), _ptr(logits), c_longlong(_row_stride(logits)), _ptr(temps),
                                _ptr(seed), _ptr(row_keys), c_int(n), c_int(V), _ptr(scratch), c_int(rows), _stream()))


# ---------------------------------------------------------------------- rows of post-norm layers
ACTIVATIONS = {"relu2": 0, "clamped_glu": 1, "gelu_tanh_glu": 2, "tanh": 3, "silu_glu": 4, "gelu_tanh": 5}


def _delta_args(y, dtype: torch.dtype):
    """(pointer source, splits, split stride) of a product's result: an array of `dtype`, or float32 slices."""
    if isinstance(y, Partials):
        return y.tensor, y.splits, y.split_stride
    if y.dtype != dtype or not y.is_contiguous():
        raise KernelError("a product's result must be contiguous and of the storage dtype (or float32 slices)")
    return y, 0, 0


def norm_add(resid: torch.Tensor, y, weight: torch.Tensor, eps: float, copy: Optional[torch.Tensor], dtype: torch.dtype,
             next_gain: Optional[torch.Tensor] = None, next_eps: float = 0.0) -> None:
    """resid (float32 [n, H]) += rmsnorm(y) * weight; `copy` (storage dtype [n, H], or None) receives the new rows, or,
    with `next_gain`, rmsnorm(new rows) * next_gain: the input of a sublayer that norms what it reads.
    `y` is an array of the storage dtype, a `Partials`, or a `WeightedPair` of two such (a y1 + b y2)."""
    lib = build.load("rowwise")
    n, H = resid.shape
    if resid.dtype != torch.float32 or weight.dtype != torch.float32 or (next_gain is not None and next_gain.dtype != torch.float32):
        raise KernelError("norm_add: residual and gains must be float32")
    second, a, b = None, 1.0, 0.0
    if isinstance(y, WeightedPair):
        y, second, a, b = y.first, y.second, y.a, y.b
    src, splits, stride = _delta_args(y, dtype)
    src2, splits2, stride2 = _delta_args(second, dtype) if second is not None else (None, 0, 0)
    rows = y.rows if isinstance(y, Partials) else y.shape[0]
    if rows != n or (copy is not None and (copy.dtype != dtype or tuple(copy.shape) != (n, H) or not copy.is_contiguous())):
        raise KernelError("norm_add: shapes do not fit")
    if next_gain is not None and copy is None:
        raise KernelError("norm_add: the next norm's output needs a place")
    _check(lib, lib.llmk_norm_add2(_ptr(resid), _ptr(src), _ptr(weight), _ptr(copy), c_int(n), c_int(H), c_float(eps),
                                   c_int(splits), c_longlong(stride), _ptr(src2), c_int(splits2), c_longlong(stride2), c_float(a),
                                   c_float(b), _ptr(next_gain), c_float(next_eps), c_int(dtype_code(dtype)), _stream()))


class WeightedPair:
    """a * first + b * second, not yet added up: what a mixer made of two mixers side by side returns.  Each of the two
    is an array of the storage dtype or a `Partials`.  `norm_add` takes it as it is; `scaled_sum` adds it up for
    consumers that take one array."""

    def __init__(self, first, a: float, second, b: float):
        self.first, self.a, self.second, self.b = first, float(a), second, float(b)

    @property
    def rows(self) -> int:
        return self.first.rows if isinstance(self.first, Partials) else self.first.shape[0]

    @property
    def cols(self) -> int:
        return self.first.cols if isinstance(self.first, Partials) else self.first.shape[1]


def scaled_sum(out: torch.Tensor, pair: WeightedPair, dtype: torch.dtype) -> Partials:
    """out (float32 [1, n, H], contiguous) = a * first + b * second; returned as a one-slice `Partials`."""
    lib = build.load("rowwise")
    if out.dtype != torch.float32 or not out.is_contiguous() or out.dim() != 3 or out.shape[0] != 1 or out.shape[1] != pair.rows \
            or out.shape[2] != pair.cols:
        raise KernelError("scaled_sum: the sum goes to a contiguous float32 [1, rows, cols] array")
    src, splits, stride = _delta_args(pair.first, dtype)
    src2, splits2, stride2 = _delta_args(pair.second, dtype)
    _check(lib, lib.llmk_scaled_sum(_ptr(out), _ptr(src), c_int(splits), c_longlong(stride), _ptr(src2), c_int(splits2),
                                    c_longlong(stride2), c_float(pair.a), c_float(pair.b), c_longlong(pair.rows * pair.cols),
                                    c_int(dtype_code(dtype)), _stream()))
    return Partials(out)


def cast_rows(out: torch.Tensor, src: torch.Tensor) -> None:
    """out (storage dtype, contiguous) = src (float32, contiguous), element by element."""
    lib = build.load("rowwise")
    if src.dtype != torch.float32 or not src.is_contiguous() or not out.is_contiguous() or out.numel() != src.numel():
        raise KernelError("cast_rows: contiguous float32 in, as many values out")
    _check(lib, lib.llmk_cast_rows(_ptr(out), _ptr(src), c_longlong(src.numel()), c_int(dtype_code(out.dtype)), _stream()))


def act_rows(out: torch.Tensor, x, activation: str, alpha: float = 1.0, limit: float = 0.0, group: int = 0) -> None:
    """out[n, F] = relu(x)^2 ("relu2", x [n, F]) or the clamped gated unit of x [n, 2F] ("clamped_glu": gate in
    the first F columns, up in the last): g' = min(g, limit), u' = clamp(u, -limit, limit),
    out = g' sigmoid(alpha g') (u' + 1); or gelu_tanh(gate) * up / silu(gate) * up of x [n, 2F] ("gelu_tanh_glu", "silu_glu",
    where `group` > 0 says that gate and up columns alternate in groups of that many); or tanh(x) / the tanh form of gelu
    ("tanh", "gelu_tanh", x [n, F]).
    `x` is an array or a `Partials`."""
    lib = build.load("rowwise")
    try:
        mode = ACTIVATIONS[activation]
    except KeyError:
        raise KernelError(f"unknown activation {activation!r} (known: {', '.join(ACTIVATIONS)})") from None
    n, F = out.shape
    if isinstance(x, Partials):
        src, splits, stride, ld = x.tensor, x.splits, x.split_stride, x.cols
    else:
        src, splits, stride, ld = x, 0, 0, _row_stride(x)
        if x.dtype != out.dtype:
            raise KernelError("act_rows: input and output share the storage dtype")
    _check(lib, lib.llmk_act_rows(_ptr(out), _ptr(src), c_int(n), c_int(F), c_longlong(ld), c_int(mode), c_float(alpha), c_float(limit),
                                  c_int(splits), c_longlong(stride), c_int(group), c_int(dtype_code(out.dtype)), _stream()))


GATE_FORMS = {"sigmoid": 0, "silu": 1, "plain": 2}


def gated_rmsnorm(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                  gate_form: str = "sigmoid", heads: int = 1, gains_per_head: bool = False) -> None:
    """out[n, H] (storage dtype) = rmsnorm(o) * weight * f(gate), f the sigmoid, silu, or the gate as it is (`gate_form`);
    o float32 [n, H] contiguous, gate of the storage dtype with any row stride.  Without `weight`: o * f(gate).
    `heads` > 1: every row of out and o is one head of a token (row = token * heads + head) and the gate is
    [n / heads, heads * H] with any row stride; `weight` is then [H], shared by the heads, or, with `gains_per_head`,
    [heads, H]."""
    lib = build.load("rowwise")
    n, H = out.shape
    if o.dtype != torch.float32 or not o.is_contiguous() or gate.dtype != out.dtype or n % heads != 0:
        raise KernelError("gated_rmsnorm: o must be contiguous float32 and the gate of the storage dtype")
    w_rows = heads if gains_per_head else 1
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != w_rows * H or not weight.is_contiguous()):
        raise KernelError("gated_rmsnorm: the gains are float32 [H] or [heads, H]")
    if tuple(gate.shape) != (n // heads, heads * H):
        raise KernelError("gated_rmsnorm: the gate is [tokens, heads * H]")
    _check(lib, lib.llmk_gated_rmsnorm(_ptr(out), _ptr(o), _ptr(gate), _ptr(weight), c_int(n), c_int(H), c_longlong(_row_stride(gate)),
                                       c_float(eps), c_int(GATE_FORMS[gate_form]), c_int(w_rows), c_int(heads),
                                       c_int(dtype_code(out.dtype)), _stream()))


def add_bias(y, bias: torch.Tensor) -> None:
    """y[r, :] += bias (float32 [H]); y is an array [n, H] (bfloat16 or float32, rows any stride apart) or a `Partials`,
    whose first slice takes the bias."""
    lib = build.load("rowwise")
    t = y.tensor[0] if isinstance(y, Partials) else y
    if bias.dtype != torch.float32 or bias.numel() != t.shape[-1]:
        raise KernelError("add_bias: one float32 per column")
    _check(lib, lib.llmk_add_bias(_ptr(t), _ptr(bias), c_int(t.shape[0]), c_int(t.shape[1]), c_longlong(_row_stride(t)),
                                  c_int(dtype_code(t.dtype)), _stream()))


def concat_stream(out: torch.Tensor, resid: torch.Tensor, delta, x0: torch.Tensor) -> None:
    """out[n, 2H] (storage dtype) = [resid + delta | x0]; resid and x0 float32 [n, H]; `delta` None, an array of the
    storage dtype or a `Partials`."""
    lib = build.load("rowwise")
    n, H = resid.shape
    if resid.dtype != torch.float32 or x0.dtype != torch.float32 or tuple(out.shape) != (n, 2 * H) or not out.is_contiguous():
        raise KernelError("concat_stream: float32 [n, H] twice in, [n, 2H] out")
    src, splits, stride = (None, 0, 0) if delta is None else _delta_args(delta, out.dtype)
    _check(lib, lib.llmk_concat_stream(_ptr(out), _ptr(resid), _ptr(src), _ptr(x0), c_int(n), c_int(H), c_int(splits),
                                       c_longlong(stride), c_int(dtype_code(out.dtype)), _stream()))


# ------------------------------------------------------------------------- several residual streams
MAX_STREAMS = 16


def stream_step(streams: torch.Tensor, y, mix: Optional[torch.Tensor], out_coef: Optional[torch.Tensor], next_in: Optional[torch.Tensor],
                next_gain: Optional[torch.Tensor], eps: float, normed: Optional[torch.Tensor], dtype: torch.dtype) -> None:
    """One step of a layer that keeps S residual streams per token, `streams` float32 [n, S, H] (csrc/rowwise.cu).  With `y` (a
    sublayer's output: an array of the storage dtype, a `Partials`, or a `WeightedPair` of two such): every stream is rewritten
    from all the old ones, x_t <- sum_s mix[s, t] x_s + out_coef[t] y.  With `next_in`: normed [n, H] (storage dtype) =
    rmsnorm(sum_t next_in[t] x_t) * next_gain over the new streams.  Either half may be left out."""
    lib = build.load("rowwise")
    if streams.dtype != torch.float32 or streams.dim() != 3 or not streams.is_contiguous():
        raise KernelError("stream_step: the streams are a contiguous float32 [n, S, H] array")
    n, S, H = streams.shape
    if S > MAX_STREAMS:
        raise KernelError(f"stream_step: at most {MAX_STREAMS} streams")
    second, a, b = None, 1.0, 0.0
    src, splits, stride, src2, splits2, stride2 = None, 0, 0, None, 0, 0
    if y is not None:
        if isinstance(y, WeightedPair):
            y, second, a, b = y.first, y.second, y.a, y.b
        src, splits, stride = _delta_args(y, dtype)
        if second is not None:
            src2, splits2, stride2 = _delta_args(second, dtype)
        rows = y.rows if isinstance(y, Partials) else y.shape[0]
        cols = y.cols if isinstance(y, Partials) else y.shape[1]
        if rows != n or cols != H or mix is None or out_coef is None or mix.numel() != S * S or out_coef.numel() != S:
            raise KernelError("stream_step: the sublayer's output is [n, H] and comes with mix [S, S] and out [S]")
    for c in (mix, out_coef, next_in, next_gain):
        if c is not None and (c.dtype != torch.float32 or not c.is_contiguous()):
            raise KernelError("stream_step: coefficients and gains are contiguous float32")
    if next_in is not None and (next_in.numel() != S or next_gain is None or next_gain.numel() != H or normed is None
                                or normed.dtype != dtype or tuple(normed.shape) != (n, H) or not normed.is_contiguous()):
        raise KernelError("stream_step: the next sublayer's input needs in [S], gains [H] and a place [n, H]")
    _check(lib, lib.llmk_stream_step(_ptr(streams), _ptr(src), c_int(splits), c_longlong(stride), _ptr(src2), c_int(splits2),
                                     c_longlong(stride2), c_float(a), c_float(b), _ptr(mix), _ptr(out_coef), _ptr(next_in),
                                     _ptr(next_gain), c_float(eps), _ptr(normed), c_int(n), c_int(S), c_int(H),
                                     c_int(dtype_code(dtype)), _stream()))


def stream_spread(streams: torch.Tensor, row: torch.Tensor, collapse: bool = False) -> None:
    """streams (float32 [n, S, H]) <- every stream a copy of row (float32 [n, H]); `collapse`: row <- the sum of the streams."""
    lib = build.load("rowwise")
    if streams.dtype != torch.float32 or row.dtype != torch.float32 or streams.dim() != 3 or not streams.is_contiguous() \
            or not row.is_contiguous() or tuple(row.shape) != (streams.shape[0], streams.shape[2]):
        raise KernelError("stream_spread: float32 [n, S, H] and [n, H], contiguous")
    n, S, H = streams.shape
    _check(lib, lib.llmk_stream_spread(_ptr(streams), _ptr(row), c_int(n), c_int(S), c_int(H), c_int(1 if collapse else 0), _stream()))


# ------------------------------------------------------------ norms over whole projections, rotated values
def attn_prep_rows(x: torch.Tensor, q_out: torch.Tensor, kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                   positions: torch.Tensor, slots: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                   vcos: Optional[torch.Tensor], vsin: Optional[torch.Tensor], q_gain: Optional[torch.Tensor],
                   k_gain: Optional[torch.Tensor], nq: int, nk: int, hd: int, vd: int, rot: int, page_size: int, eps: float) -> None:
    """x float32 [n, >= nq hd + nk hd + nk vd] = [q | k | v] of each token: q and k divided by the root mean square of their whole
    row and multiplied by gains of that size (`q_gain` [nq hd], `k_gain` [nk hd]), the first `rot` values of every head turned
    in half-split pairs; v turned over all of its width by `vcos` / `vsin` [positions, vd / 2] (None: as it is).  q goes to
    `q_out` (storage dtype), k and v to the paged cache (csrc/attn_prep.cu)."""
    lib = build.load("attn_prep")
    n = x.shape[0]
    if x.dtype != torch.float32 or x.shape[1] < nq * hd + nk * (hd + vd) or q_out.shape[0] != n or q_out.shape[1] < nq * hd:
        raise KernelError("attn_prep_rows: float32 rows [q | k | v] in, q of the storage dtype out")
    for g, w in ((q_gain, nq * hd), (k_gain, nk * hd)):
        if g is not None and (g.dtype != torch.float32 or g.numel() != w or not g.is_contiguous()):
            raise KernelError("attn_prep_rows: gains are float32 over a whole projection")
    if kcache is not None and kcache.dtype != q_out.dtype:
        raise KernelError("attn_prep_rows: the cache has the storage dtype")
    nkv_cache = kcache.shape[1] if kcache is not None else 0
    _check(lib, lib.llmk_attn_prep_rows(_ptr(x), c_longlong(_row_stride(x)), _ptr(q_out), c_longlong(_row_stride(q_out)), _ptr(kcache),
                                        _ptr(vcache), _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(vcos), _ptr(vsin),
                                        _ptr(q_gain), _ptr(k_gain), c_int(n), c_int(nq), c_int(nk), c_int(nkv_cache), c_int(hd), c_int(vd),
                                        c_int(rot), c_int(page_size), c_float(eps), c_int(dtype_code(q_out.dtype)), _stream()))


def unrotate_gate(o: torch.Tensor, gate: Optional[torch.Tensor], positions: torch.Tensor, vcos: Optional[torch.Tensor],
                  vsin: Optional[torch.Tensor], nq: int, vd: int) -> None:
    """o [n, nq vd] in place: every head turned back by minus its position's angles (pairs (m, m + vd / 2), tables
    [positions, vd / 2]; None: not turned), then multiplied by sigmoid(gate[t, head]), `gate` [n, nq] of o's dtype with any row
    stride (None: no gate)."""
    lib = build.load("attn_prep")
    if o.shape[1] != nq * vd or (gate is not None and (gate.dtype != o.dtype or gate.shape[0] != o.shape[0] or gate.shape[1] != nq)):
        raise KernelError("unrotate_gate: o is [n, nq vd], the gate [n, nq] of the same dtype")
    _check(lib, lib.llmk_unrotate_gate(_ptr(o), c_longlong(_row_stride(o)), _ptr(gate), c_longlong(_row_stride(gate) if gate is not None else 0),
                                       _ptr(positions), _ptr(vcos), _ptr(vsin), c_int(o.shape[0]), c_int(nq), c_int(vd),
                                       c_int(dtype_code(o.dtype)), _stream()))


# ------------------------------------------------------------ gates on the current token, matrix memories
def min_gru(out: torch.Tensor, zxg: torch.Tensor, bias_z: Optional[torch.Tensor], bias_x: Optional[torch.Tensor], state: torch.Tensor,
            cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int) -> None:
    """out[t, c] (storage dtype) = S_t silu(g_t), S_t = (1 - z) S_(t-1) + z cand, z = sigmoid(zxg[t, c] + bias_z), u = zxg[t, C + c] +
    bias_x, cand = u + 1/2 where u >= 0 else sigmoid(u), g = zxg[t, 2C + c]; zxg float32 [n, 3C]; state float32 [slots, >= C]
    (csrc/memory_scan.cu)."""
    lib = build.load("memory_scan")
    n, C = out.shape
    if zxg.dtype != torch.float32 or tuple(zxg.shape) != (n, 3 * C) or state.dtype != torch.float32 or state.shape[1] < C \
            or not out.is_contiguous():
        raise KernelError("min_gru: float32 [n, 3C] in, [n, C] out, float32 state rows of at least C")
    _check(lib, lib.llmk_min_gru(_ptr(out), _ptr(zxg), c_longlong(_row_stride(zxg)), _ptr(bias_z), _ptr(bias_x), _ptr(state),
                                 c_longlong(_row_stride(state)), _ptr(cu_q), _ptr(state_slots), c_int(n_seqs), c_int(n), c_int(C),
                                 c_int(dtype_code(out.dtype)), _stream()))


def mlstm_gates(gates: torch.Tensor, q: torch.Tensor, k: torch.Tensor, gi: torch.Tensor, gf: torch.Tensor, bias_i: Optional[torch.Tensor],
                bias_f: Optional[torch.Tensor], m_state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int,
                heads: int, dim: int, cap: float, q_scale: float) -> None:
    """gates float32 [n, heads, 4] <- (i, f, (q . k) q_scale, m_(t-1)) of a matrix memory with a running maximum:
    i = cap tanh((gi + bias_i) / cap), f = logsigmoid(cap tanh((gf + bias_f) / cap)), m_t = max(f + m_(t-1), i) (from which
    `memory_scan` makes keep = exp(f + m_(t-1) - m_t), take = exp(i - m_t) and exp(-m_t)); m is carried in `m_state` (float32
    [slots, >= heads]).  q, k [n, heads dim] and gi, gf
    [n, heads] of the storage dtype with any row stride.  Two launches (csrc/memory_scan.cu)."""
    lib = build.load("memory_scan")
    n = q.shape[0]
    if gates.dtype != torch.float32 or not gates.is_contiguous() or gates.numel() < n * heads * 4 or m_state.dtype != torch.float32:
        raise KernelError("mlstm_gates: gates and the maxima are float32")
    _check(lib, lib.llmk_mlstm_gates(_ptr(gates), _ptr(q), c_longlong(_row_stride(q)), _ptr(k), c_longlong(_row_stride(k)), _ptr(gi),
                                     c_longlong(_row_stride(gi)), _ptr(gf), c_longlong(_row_stride(gf)), _ptr(bias_i), _ptr(bias_f),
                                     _ptr(m_state), c_longlong(_row_stride(m_state)), _ptr(cu_q), _ptr(state_slots), c_int(n_seqs),
                                     c_int(n), c_int(heads), c_int(dim), c_float(cap), c_float(q_scale), c_int(dtype_code(q.dtype)),
                                     _stream()), 2)


def delta_rule_prep(aux: torch.Tensor, dots: torch.Tensor, r: torch.Tensor, k: torch.Tensor, a: torch.Tensor, decay: torch.Tensor,
                    a_bias: Optional[torch.Tensor], w_bias: Optional[torch.Tensor], cu_q: torch.Tensor, n_seqs: int, heads: int, dim: int,
                    decay_scale: float, unit_eps: float) -> None:
    """The generalized delta rule's vectors per token and head: aux float32 [n, 3 heads dim] = [w | b | u] with w = exp(-decay_scale
    sigmoid(decay + w_bias)), u = k / sqrt(sum k^2 + unit_eps), b = sigmoid(a + a_bias) u; dots float32 [n, heads, 2] = (b . r, k . r).
    r, k, a of the storage dtype with any row stride; decay float32."""
    lib = build.load("memory_scan")
    n = r.shape[0]
    if aux.dtype != torch.float32 or dots.dtype != torch.float32 or decay.dtype != torch.float32 or not aux.is_contiguous() \
            or not dots.is_contiguous() or aux.numel() < n * 3 * heads * dim or dots.numel() < n * heads * 2:
        raise KernelError("delta_rule_prep: aux, dots and the decay's input are float32")
    _check(lib, lib.llmk_delta_rule_prep(_ptr(aux), _ptr(dots), _ptr(r), c_longlong(_row_stride(r)), _ptr(k), c_longlong(_row_stride(k)),
                                         _ptr(a), c_longlong(_row_stride(a)), _ptr(decay), c_longlong(_row_stride(decay)), _ptr(a_bias),
                                         _ptr(w_bias), _ptr(cu_q), c_int(n_seqs), c_int(n), c_int(heads), c_int(dim),
                                         c_float(decay_scale), c_float(unit_eps), c_int(dtype_code(r.dtype)), _stream()))


MEMORY_FORMS = {"delta": 0, "mlstm": 1}


def memory_scan(out: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, aux: Optional[torch.Tensor], dots: torch.Tensor,
                state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, heads: int, dim: int, vdim: int,
                form: str, r_scale: float = 1.0, den_eps: float = 0.0) -> None:
    """A matrix memory S [dim, vdim] per head walked over each sequence's new tokens (csrc/memory_scan.cu); out float32
    [n, heads vdim].  "delta": S_t = diag(w) S - b (u^T S) + k v^T, o = S_t^T r, with `aux` and `dots` from `delta_rule_prep`.
    "mlstm": S_t = keep S + take k v^T, n_t = keep n + take k, o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps), q = r r_scale,
    with `dots` from `mlstm_gates`.  state float32 [slots, >= heads dim vdim (+ heads dim for n)]."""
    lib = build.load("memory_scan")
    need = heads * dim * vdim + (heads * dim if form == "mlstm" else 0)
    if out.dtype != torch.float32 or not out.is_contiguous() or state.dtype != torch.float32 or state.shape[1] < need \
            or dots.dtype != torch.float32 or r.dtype != k.dtype or r.dtype != v.dtype:
        raise KernelError("memory_scan: out, dots and state are float32; r, k, v share the storage dtype")
    _check(lib, lib.llmk_memory_scan(_ptr(out), _ptr(r), c_longlong(_row_stride(r)), _ptr(k), c_longlong(_row_stride(k)), _ptr(v),
                                     c_longlong(_row_stride(v)), _ptr(aux), _ptr(dots), _ptr(state), c_longlong(_row_stride(state)),
                                     _ptr(cu_q), _ptr(state_slots), c_int(n_seqs), c_int(heads), c_int(dim), c_int(vdim),
                                     c_int(MEMORY_FORMS[form]), c_float(r_scale), c_float(den_eps), c_int(dtype_code(r.dtype)), _stream()))


# ------------------------------------------------------------------------------ recurrent mixers
CONV_ACTIVATIONS = {"none": 0, "silu": 1}
SHORT_CONV_FEW_TOKENS = 64     # steps of up to this many token rows: the convolution and its state's update in one launch


def short_conv(out: torch.Tensor, x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
               state_slots: torch.Tensor, n_seqs: int, in_bias: Optional[torch.Tensor] = None,
               conv_bias: Optional[torch.Tensor] = None, activation: str = "none", update_state: bool = True) -> None:
    """out[t, c] (float32) = act(sum_i taps[c, i] in(t - (K-1) + i, c) + conv_bias[c]) over each sequence of the step, in
    = x + in_bias; a sequence's first tokens read the last K - 1 inputs of the step before from `state` [slots, >= (K-1) C]
    (a view whose rows are the slots), which is then brought up to date (csrc/recurrent.cu)."""
    lib = build.load("recurrent")
    n, C = out.shape
    K = taps.shape[1]
    if out.dtype != torch.float32 or taps.dtype != torch.float32 or state.dtype != torch.float32 or tuple(taps.shape) != (C, K):
        raise KernelError("short_conv: out, taps [channels, K] and state are float32")
    if x.shape[0] != n or x.shape[1] != C or state.shape[1] < (K - 1) * C:
        raise KernelError("short_conv: shapes do not fit")
    _check(lib, lib.llmk_short_conv(_ptr(out), c_longlong(_row_stride(out)), _ptr(x), c_longlong(_row_stride(x)), _ptr(in_bias),
                                    _ptr(taps), _ptr(conv_bias), _ptr(state), c_longlong(_row_stride(state)), _ptr(cu_q),
                                    _ptr(state_slots), c_int(n_seqs), c_int(n), c_int(C), c_int(K),
                                    c_int(CONV_ACTIVATIONS[activation]), c_int(1 if update_state else 0),
                                    c_int(dtype_code(x.dtype)), _stream()),
           2 if update_state and K > 1 and n > SHORT_CONV_FEW_TOKENS else 1)


def rglru_scratch_rows(n_tokens: int, n_seqs: int, dtype: torch.dtype) -> int:
    """Rows of the float32 scratch [rows, C] that `rglru` needs for a step of this shape."""
    lib = build.load("recurrent")
    lib.llmk_rglru_scratch_rows.restype = c_longlong
    return int(lib.llmk_rglru_scratch_rows(c_int(n_tokens), c_int(n_seqs), c_int(dtype_code(dtype))))


def rglru(out: torch.Tensor, scratch: torch.Tensor, u: torch.Tensor, w_a: torch.Tensor, w_i: torch.Tensor,
          b_a: Optional[torch.Tensor], b_i: Optional[torch.Tensor], lam: torch.Tensor, y: torch.Tensor,
          y_bias: Optional[torch.Tensor], state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int,
          blocks: int, decay_scale: float) -> None:
    """The real-gated linear recurrent unit over each sequence's new tokens (csrc/recurrent.cu): gates from u (float32
    [n, C], the convolution's output) by the block-diagonal matrices w_a, w_i [blocks, C/blocks, C/blocks], then
    S = a S + sqrt(1 - a^2) i u from `state` [slots, >= C] and out[n, C] (storage dtype) = S * gelu_tanh(y + y_bias).
    `scratch`: contiguous float32, `rglru_scratch_rows` rows of C (long steps of the bfloat16 engine scan in segments)."""
    lib = build.load("recurrent")
    n, C = u.shape
    need = rglru_scratch_rows(n, n_seqs, out.dtype) * C
    if u.dtype != torch.float32 or not u.is_contiguous() or scratch.dtype != torch.float32 or scratch.numel() < need \
            or not scratch.is_contiguous():
        raise KernelError(f"rglru: u and the scratch ({need} values) are contiguous float32")
    if w_a.dtype != out.dtype or w_i.dtype != out.dtype or y.dtype != out.dtype or not w_a.is_contiguous() or not w_i.is_contiguous():
        raise KernelError("rglru: gate matrices, y and out share the storage dtype")
    if tuple(w_a.shape) != (blocks, C // blocks, C // blocks) or w_i.shape != w_a.shape or state.shape[1] < C:
        raise KernelError("rglru: shapes do not fit")
    flat = scratch.view(-1)
    _check(lib, lib.llmk_rglru(_ptr(out), c_longlong(_row_stride(out)), _ptr(flat), c_void_p(flat.data_ptr() + 4 * n * C), _ptr(u),
                               _ptr(w_a), _ptr(w_i), _ptr(b_a), _ptr(b_i), _ptr(lam), _ptr(y), c_longlong(_row_stride(y)),
                               _ptr(y_bias), _ptr(state), c_longlong(_row_stride(state)), _ptr(cu_q), _ptr(state_slots),
                               c_int(n_seqs), c_int(n), c_int(C), c_int(blocks), c_float(decay_scale),
                               c_int(dtype_code(out.dtype)), _stream()), 4 if need > 2 * n * C else 2)


def delta_scan(out: torch.Tensor, qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int,
               heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float, q_scale: float, beta_buf: torch.Tensor) -> None:
    """The gated delta rule with a decay per key channel over each sequence's new tokens (csrc/recurrent.cu).  qkv float32
    [n, 2 kv_heads dim + heads vdim] (after convolution and silu); beta [n, heads] (storage dtype, any row stride, before
    its sigmoid); decay float32 [n, heads dim] (before dt_bias and softplus); state [slots, >= heads dim vdim] float32;
    out float32 [n, heads vdim].  `qkv` and `decay` are REWRITTEN (q and k as unit vectors, 1 - g); `beta_buf`: float32
    scratch [n, heads + kv_heads]."""
    lib = build.load("recurrent")
    n = out.shape[0]
    if out.dtype != torch.float32 or qkv.dtype != torch.float32 or decay.dtype != torch.float32 or state.dtype != torch.float32 \
            or beta_buf.dtype != torch.float32:
        raise KernelError("delta_scan: out, qkv, decay, state and the scratch are float32")
    if not out.is_contiguous() or not decay.is_contiguous() or out.shape[1] != heads * vdim or decay.shape[1] != heads * dim \
            or qkv.shape[1] != 2 * kv_heads * dim + heads * vdim or state.shape[1] < heads * dim * vdim or beta_buf.numel() < n * (heads + kv_heads) \
            or not beta_buf.is_contiguous():
        raise KernelError("delta_scan: shapes do not fit")
    _check(lib, lib.llmk_delta_scan(_ptr(out), _ptr(qkv), c_longlong(_row_stride(qkv)), _ptr(beta), c_longlong(_row_stride(beta)),
                                    _ptr(decay), _ptr(beta_buf), _ptr(dt_bias), _ptr(a_log), _ptr(state), c_longlong(_row_stride(state)),
                                    _ptr(cu_q), _ptr(state_slots), c_int(n_seqs), c_int(n), c_int(heads), c_int(kv_heads), c_int(dim),
                                    c_int(vdim), c_float(unit_eps), c_float(q_scale), c_int(dtype_code(beta.dtype)), _stream()), 2)


DECAY_FORMS = {"sigmoid_pow": 0, "exp_exp": 1}


def token_shift_mix(out: torch.Tensor, x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
                    state_slots: torch.Tensor, n_seqs: int) -> None:
    """out[i, t] = x[t] + (x[t - 1] - x[t]) * mu[i] for every blend i (csrc/recurrent.cu): out [n_mix, n, W] of the storage
    dtype, x [n, W], mu float32 [n_mix, W].  A sequence's first token of the step reads its state row (float32 [slots, >= W],
    zeros for a fresh request) as the token before it, and the sequence's last row is left there."""
    lib = build.load("recurrent")
    n_mix, n, W = out.shape
    if x.dtype != out.dtype or tuple(x.shape) != (n, W) or not out.is_contiguous() or mu.dtype != torch.float32 or tuple(mu.shape) != (n_mix, W) \
            or not mu.is_contiguous() or state.dtype != torch.float32 or state.shape[1] < W:
        raise KernelError("token_shift_mix: shapes or dtypes do not fit")
    _check(lib, lib.llmk_token_shift_mix(_ptr(out), c_longlong(n * W), _ptr(x), c_longlong(_row_stride(x)), _ptr(mu), _ptr(state),
                                         c_longlong(_row_stride(state)), _ptr(cu_q), _ptr(state_slots), c_int(n_seqs), c_int(n), c_int(W),
                                         c_int(n_mix), c_int(dtype_code(x.dtype)), _stream()))


def decay_scan_segment_floats(heads: int, dim: int, vdim: int) -> int:
    """float32 values of the scratch that lets `decay_scan` walk long sequences in segments: 64 segments' states and
    decay products (eight sequences of eight segments, or fewer of more)."""
    return 64 * heads * (dim * vdim + dim)


def decay_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, bias: Optional[torch.Tensor],
               bonus: Optional[torch.Tensor], state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, heads: int,
               dim: int, vdim: int, form: str, tau: float, q_scale: float, read_first: bool, qkv_buf: torch.Tensor, dots: torch.Tensor,
               segments: Optional[torch.Tensor] = None) -> None:
    """Linear attention with a decay per head and key channel over each sequence's new tokens (csrc/recurrent.cu).
    q, k [n, heads dim], v [n, heads vdim] of the storage dtype (any row stride); decay float32 [n, heads dim], the decays'
    pre-activations z, REWRITTEN; with b = `bias` (float32 [heads dim]) the decay is sigmoid(z + b)^(1/tau) ("sigmoid_pow")
    or exp(-exp(z + b)) ("exp_exp").  state float32 [slots, >= heads dim vdim]; out float32 [n, heads vdim].
    `read_first`: o = (S + diag(bonus) k v^T)^T q before S <- diag(a) S + k v^T; else o = S^T q after it.  q is multiplied
    by `q_scale`.  `qkv_buf` float32 scratch [n, 2 heads dim + heads vdim], `dots` float32 scratch [n, 2 heads].
    `segments` (float32, `decay_scan_segment_floats` values): with it, steps of some hundred token rows of a few sequences
    walk each sequence in segments side by side (two launches) instead of token by token from its first to its last."""
    lib = build.load("recurrent")
    n = out.shape[0]
    if any(t.dtype != torch.float32 for t in (out, decay, state, qkv_buf, dots)) or q.dtype != k.dtype or q.dtype != v.dtype:
        raise KernelError("decay_scan: out, decay, state and the scratch are float32; q, k, v share the storage dtype")
    if not out.is_contiguous() or not decay.is_contiguous() or out.shape[1] != heads * vdim or decay.shape[1] != heads * dim \
            or q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim or state.shape[1] < heads * dim * vdim \
            or qkv_buf.numel() < n * (2 * heads * dim + heads * vdim) or dots.numel() < 2 * n * heads or not qkv_buf.is_contiguous() \
            or not dots.is_contiguous():
        raise KernelError("decay_scan: shapes do not fit")
    for name, t in (("bias", bias), ("bonus", bonus)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads * dim or not t.is_contiguous()):
            raise KernelError(f"decay_scan: {name} is float32 [heads, dim]")
    if segments is not None and (segments.dtype != torch.float32 or not segments.is_contiguous()):
        raise KernelError("decay_scan: the segments' scratch is a contiguous float32 array")
    launched = c_int(0)
    _check(lib, lib.llmk_decay_scan(_ptr(out), _ptr(q), c_longlong(_row_stride(q)), _ptr(k), c_longlong(_row_stride(k)), _ptr(v),
                                    c_longlong(_row_stride(v)), _ptr(decay), _ptr(bias), _ptr(bonus), _ptr(qkv_buf), _ptr(dots), _ptr(state),
                                    c_longlong(_row_stride(state)), _ptr(cu_q), _ptr(state_slots), c_int(n_seqs), c_int(n), c_int(heads),
                                    c_int(dim), c_int(vdim), c_int(DECAY_FORMS[form]), c_float(tau), c_float(q_scale),
                                    c_int(1 if read_first else 0), _ptr(segments), c_longlong(segments.numel() if segments is not None else 0),
                                    ctypes.byref(launched), c_int(dtype_code(q.dtype)), _stream()), 0)
    _Counter.launches += launched.value


# ------------------------------------------------------------------------------ linear attention
def linear_attention_scratch_floats(n_tokens: int, n_seqs: int, heads: int, dim: int, vdim: int) -> int:
    """float32 values of scratch `linear_attention` needs for a step of this shape (0: none)."""
    lib = build.load("linear_attention")
    lib.llmk_linear_attention_scratch_floats.restype = c_longlong
    return int(lib.llmk_linear_attention_scratch_floats(c_int(n_tokens), c_int(n_seqs), c_int(heads), c_int(dim), c_int(vdim)))


def linear_attention(out: torch.Tensor, packed: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor,
                     decay: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, heads: int, dim: int,
                     vdim: int, silu: bool = True, scratch: Optional[torch.Tensor] = None) -> None:
    """The decayed outer-product recurrence over each sequence's new tokens (csrc/linear_attention.cu).  `packed`
    [tokens, >= ...] holds q, k (heads x dim) and v (heads x vdim) at the column offsets given; `state` float32
    [slots, heads, dim, vdim] is read and written at each sequence's slot; out float32 [tokens, heads * vdim]."""
    lib = build.load("linear_attention")
    if out.dtype != torch.float32 or state.dtype != torch.float32 or decay.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("linear_attention: out, state and decay are float32")
    if tuple(state.shape[1:]) != (heads, dim, vdim) or not state.is_contiguous():
        raise KernelError(f"linear_attention: state must be [slots, {heads}, {dim}, {vdim}], got {list(state.shape)}")
    es = packed.element_size()
    base = packed.data_ptr()
    n_tokens = out.shape[0]
    need = linear_attention_scratch_floats(n_tokens, n_seqs, heads, dim, vdim)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"linear_attention: a step of {n_tokens} tokens needs {need} float32 of scratch")
    _check(lib, lib.llmk_linear_attention(_ptr(out), c_void_p(base + q_off * es), c_void_p(base + k_off * es), c_void_p(base + v_off * es),
                                          c_longlong(_row_stride(packed)), _ptr(state), _ptr(decay), _ptr(cu_q), _ptr(state_slots),
                                          c_int(n_seqs), c_int(heads), c_int(dim), c_int(vdim), c_int(1 if silu else 0),
                                          c_int(n_tokens), _ptr(scratch if need else None), c_int(dtype_code(packed.dtype)), _stream()),
           3 if need else 1)


# ------------------------------------------------------------------------------ latent attention
def latent_prep(packed: torch.Tensor, dq_off: int, dkv_off: int, q_rank: int, rank: int, rot: int, q_gain: Optional[torch.Tensor],
                kv_gain: torch.Tensor, eps: float, cq_out: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                positions: torch.Tensor, slots: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                pairing: str) -> None:
    """Per token of `packed` [n, ...]: cq_out[n, q_rank] = rmsnorm(packed[:, dq_off:+q_rank]) * q_gain, and the cached
    vector [rmsnorm(c) * kv_gain | rotate(kr)] written at `slots` (csrc/latent_attention.cu)."""
    lib = build.load("latent_attention")
    n = packed.shape[0]
    _check(lib, lib.llmk_latent_prep(_ptr(packed), c_longlong(_row_stride(packed)), c_int(dq_off), c_int(dkv_off), c_int(q_rank),
                                     c_int(rank), c_int(rot), _ptr(q_gain), _ptr(kv_gain), c_float(eps), _ptr(cq_out), _ptr(cache),
                                     _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), c_int(pairing_code(pairing)), c_int(n),
                                     c_int(dtype_code(packed.dtype)), _stream()))


def latent_absorb(qa: torch.Tensor, q: torch.Tensor, wuk: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], heads: int, dim: int, rot: int, rank: int, pairing: str) -> None:
    """qa float32 [n, heads, rank + rot] = [Wuk_h^T q_unrotated | rotate(q_rotated)] of q [n, heads * (dim + rot)]."""
    lib = build.load("latent_attention")
    n = q.shape[0]
    if qa.dtype != torch.float32 or not qa.is_contiguous() or qa.numel() != n * heads * (rank + rot) or wuk.dtype != q.dtype:
        raise KernelError("latent_absorb: shapes or dtypes do not fit")
    _check(lib, lib.llmk_latent_absorb(_ptr(qa), _ptr(q), c_longlong(_row_stride(q)), _ptr(wuk), _ptr(positions), _ptr(cos), _ptr(sin),
                                       c_int(n), c_int(heads), c_int(dim), c_int(rot), c_int(rank), c_int(pairing_code(pairing)),
                                       c_int(dtype_code(q.dtype)), _stream()))


def latent_rotate(qa: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], heads: int,
                  rank: int, rot: int, pairing: str) -> None:
    """Turns the rotated part of every head of qa (float32 [n, heads * (rank + rot)], contiguous) in place."""
    lib = build.load("latent_attention")
    n = qa.shape[0]
    if qa.dtype != torch.float32 or not qa.is_contiguous() or qa.numel() != n * heads * (rank + rot):
        raise KernelError("latent_rotate: qa is contiguous float32 [n, heads * (rank + rot)]")
    _check(lib, lib.llmk_latent_rotate(_ptr(qa), _ptr(positions), _ptr(cos), _ptr(sin), c_int(n), c_int(heads), c_int(rank), c_int(rot),
                                       c_int(pairing_code(pairing)), _stream()))


def latent_attention_set_mma(on: bool) -> None:
    """Whether `latent_attention` takes bfloat16 caches whose sizes fit to the tensor cores (the default) or runs its
    float32 kernel for them too (for measurements and tests)."""
    build.load("latent_attention").llmk_latent_attention_set_mma(c_int(1 if on else 0))


def latent_attention_tile_queries(heads: int) -> int:
    return int(build.load("latent_attention").llmk_latent_attention_tile_queries(c_int(heads)))


def latent_attention_scratch_floats(n_tokens: int, heads: int, rank: int, parts: int) -> int:
    return 0 if parts <= 1 else n_tokens * heads * parts * (rank + 2)


def latent_attention_on_tensor_cores(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """Whether `latent_attention` takes a cache of this dtype and these sizes to the tensor cores."""
    return bool(build.load("latent_attention").llmk_latent_attention_on_tensor_cores(c_int(rank), c_int(rot), c_int(dtype_code(dtype))))


def latent_attention(out: Optional[torch.Tensor], qa: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, max_blocks: int,
                     ctx_len: torch.Tensor, cu_q: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tokens: int,
                     heads: int, rank: int, rot: int, page_size: int, scale: float, parts: int = 1,
                     scratch: Optional[torch.Tensor] = None, out_head_major: Optional[torch.Tensor] = None) -> None:
    """out float32 [n, heads, rank] = causal softmax attention of qa over the cached vectors (one shared kv head whose
    values are the first `rank` entries of the cached vector).  With `out_head_major` (bfloat16 [heads, t_pad, rank]; the
    tensor-core form only) the result goes there instead, rounded, for the grouped product that follows."""
    lib = build.load("latent_attention")
    t_pad = 0
    if out_head_major is not None:
        if out_head_major.dtype != torch.bfloat16 or out_head_major.dim() != 3 or out_head_major.shape[0] != heads \
                or out_head_major.shape[2] != rank or not out_head_major.is_contiguous():
            raise KernelError("latent_attention: the head-major result is contiguous bfloat16 [heads, t_pad, rank]")
        t_pad = out_head_major.shape[1]
    elif out is None or out.dtype != torch.float32:
        raise KernelError("latent_attention: outputs are float32")
    if qa.dtype != torch.float32:
        raise KernelError("latent_attention: queries are float32")
    if parts > 1 and (scratch is None or scratch.numel() < latent_attention_scratch_floats(n_tokens, heads, rank, parts)):
        raise KernelError("latent_attention: scratch too small")
    _check(lib, lib.llmk_latent_attention(_ptr(out), _ptr(qa), _ptr(cache), _ptr(block_tables), c_int(max_blocks), _ptr(ctx_len),
                                          _ptr(cu_q), _ptr(tile_seq), _ptr(tile_q0), c_int(tile_seq.numel()), c_int(n_tokens),
                                          c_int(heads), c_int(rank), c_int(rot), c_int(page_size), c_float(scale), c_int(parts),
                                          _ptr(scratch), _ptr(out_head_major), c_int(t_pad), c_int(dtype_code(cache.dtype)), _stream()),
           2 if parts > 1 else 1)


def latent_gate(out: torch.Tensor, o: torch.Tensor, gate: Optional[torch.Tensor], heads: int, vdim: int, t_pad: int) -> None:
    """out[n, heads * vdim] (storage dtype) = o (float32 [heads, t_pad, vdim], head-major) * sigmoid(gate)."""
    lib = build.load("latent_attention")
    n = out.shape[0]
    if o.dtype != torch.float32 or not o.is_contiguous() or o.numel() < heads * t_pad * vdim or (gate is not None and gate.dtype != out.dtype):
        raise KernelError("latent_gate: shapes or dtypes do not fit")
    _check(lib, lib.llmk_latent_gate(_ptr(out), _ptr(o), _ptr(gate), c_longlong(_row_stride(gate) if gate is not None else 0), c_int(n),
                                     c_int(heads), c_int(vdim), c_int(t_pad), c_int(dtype_code(out.dtype)), _stream()))


def latent_expand(out: torch.Tensor, oa: torch.Tensor, wuv: torch.Tensor, gate: Optional[torch.Tensor], heads: int, rank: int,
                  vdim: int) -> None:
    """out[n, heads * vdim] (storage dtype) = (Wuv_h oa[n, h]) * sigmoid(gate)."""
    lib = build.load("latent_attention")
    n = out.shape[0]
    if oa.dtype != torch.float32 or wuv.dtype != out.dtype or (gate is not None and gate.dtype != out.dtype):
        raise KernelError("latent_expand: dtypes do not fit")
    _check(lib, lib.llmk_latent_expand(_ptr(out), _ptr(oa), _ptr(wuv), _ptr(gate), c_longlong(_row_stride(gate) if gate is not None else 0),
                                       c_int(n), c_int(heads), c_int(rank), c_int(vdim), c_int(dtype_code(out.dtype)), _stream()))


# -------------------------------------------------------------------------- routed feed-forward
# "softmax_top": the logits choose, the weights are the softmax over the chosen logits alone
ROUTER_SCORINGS = {"sigmoid": 0, "softmax": 1, "softmax_top": 2}


MOE_GROUPED_TILE = 128      # rows per tile of the grouped tensor-core product


def moe_max_tiles(n_slots: int, experts: int, tile: int = 0) -> int:
    """The most tiles of `tile` rows (0: the 16 of `moe_experts`) that `n_slots` rows grouped by expert can need."""
    return int(build.load("moe").llmk_moe_max_tiles(c_int(n_slots), c_int(experts), c_int(tile)))


def moe_route(h: torch.Tensor, router: torch.Tensor, slot_expert: torch.Tensor, slot_weight: torch.Tensor, top: int,
              scoring: str = "sigmoid", renormalize: bool = False, bias: Optional[torch.Tensor] = None) -> None:
    """Per row of h [n, K]: scores of router (float32 [E, K]) h (+ `bias`, float32 [E]), the `top` largest choose; slot
    n * top + c receives (expert, score)."""
    lib = build.load("moe")
    n, K = h.shape
    E = router.shape[0]
    if router.dtype != torch.float32 or slot_expert.dtype != torch.int32 or slot_weight.dtype != torch.float32 \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != E)):
        raise KernelError("moe_route: router, bias and weights float32, experts int32")
    _check(lib, lib.llmk_moe_route(_ptr(h), c_longlong(_row_stride(h)), _ptr(router), _ptr(bias), _ptr(slot_expert), _ptr(slot_weight), c_int(n),
                                   c_int(K), c_int(E), c_int(top), c_int(ROUTER_SCORINGS[scoring]), c_int(1 if renormalize else 0),
                                   c_int(dtype_code(h.dtype)), _stream()))


def moe_plan(slot_expert: torch.Tensor, n_slots: int, experts: int, order: torch.Tensor, pos_of_slot: torch.Tensor,
             tile_expert: torch.Tensor, tile_start: torch.Tensor, tile_rows: torch.Tensor, tile: int = 0, padded: bool = False) -> None:
    """Groups the slots by expert into tiles of `tile` rows (0: 16).  `padded`: every expert's rows start on a tile, `order`
    has moe_max_tiles(...) * tile entries (-1 where a tile has no row) and tile i is rows [i * tile, (i + 1) * tile)."""
    lib = build.load("moe")
    need = moe_max_tiles(n_slots, experts, tile) * tile if padded else n_slots
    if order.numel() < need or tile_expert.numel() < moe_max_tiles(n_slots, experts, tile):
        raise KernelError("moe_plan: arrays too small")
    _check(lib, lib.llmk_moe_plan(_ptr(slot_expert), c_int(n_slots), c_int(experts), c_int(tile), c_int(1 if padded else 0), _ptr(order),
                                  _ptr(pos_of_slot), _ptr(tile_expert), _ptr(tile_start), _ptr(tile_rows), _stream()))


def moe_gather(out: torch.Tensor, h: torch.Tensor, order: torch.Tensor, slot_weight: torch.Tensor, top: int, scale_rows: bool) -> None:
    """out[pos] = h[order[pos] // top] (times the slot's weight if `scale_rows`), zeros where order[pos] < 0."""
    lib = build.load("moe")
    n, K = out.shape
    if out.dtype != h.dtype or not out.is_contiguous() or order.numel() < n:
        raise KernelError("moe_gather: shapes or dtypes do not fit")
    _check(lib, lib.llmk_moe_gather(_ptr(out), _ptr(h), c_longlong(_row_stride(h)), _ptr(order), _ptr(slot_weight), c_int(n), c_int(top),
                                    c_int(K), c_int(1 if scale_rows else 0), c_int(dtype_code(out.dtype)), _stream()))


def gemm_tc_grouped(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, real_rows: int = 0) -> None:
    """out[m] = a[m] @ w[g]^T where g = tile_group[m // 128] (int32 on the device; -1: the tile is skipped): a [M, K] with
    M a multiple of 128, w [groups, N, K] contiguous, both bfloat16; out [M, N] bfloat16 or float32 (csrc/gemm_tc.cu).
    `real_rows`: how many rows hold data (for the profiler's count of the work; the kernel does not read it)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    G, N, Kw = w.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or Kw != K or not w.is_contiguous() or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc_grouped: a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    if tile_group.dtype != torch.int32 or tile_group.numel() < M // MOE_GROUPED_TILE:
        raise KernelError("gemm_tc_grouped: one int32 group per tile of 128 rows")
    _check(lib, lib.llmk_gemm_tc_grouped(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_longlong(_row_stride(a)),
                                         c_longlong(K), c_longlong(_row_stride(out)), c_int(G), _ptr(tile_group),
                                         c_int(dtype_code(out.dtype)), _ptr(tc_error_flag(a.device)), c_int(1), _stream()))


def moe_experts(out: torch.Tensor, x: torch.Tensor, w0: torch.Tensor, w1: Optional[torch.Tensor], order: torch.Tensor,
                slot_weight: torch.Tensor, tile_expert: torch.Tensor, tile_start: torch.Tensor, tile_rows: torch.Tensor,
                n_slots: int, top: int, first: bool, weight_on_input: bool, alpha: float = 1.0, limit: float = 0.0,
                plain: bool = False) -> None:
    """first: out float32 [slots, ff] = gated activation of the rows' products with w0 = gate, w1 = up [E, ff, K]
    (`plain`: silu(gate) * up instead of the clamped unit);
    else out float32 [slots, K] = rows of x (float32 [slots, ff]) times w0 = down [E, K, ff]."""
    lib = build.load("moe")
    E, N, K = w0.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape[1] != N:
        raise KernelError("moe_experts: out is contiguous float32 [slots, columns]")
    _check(lib, lib.llmk_moe_experts(_ptr(out), _ptr(x), c_longlong(_row_stride(x)), _ptr(w0), _ptr(w1), _ptr(order), _ptr(slot_weight),
                                     _ptr(tile_expert), _ptr(tile_start), _ptr(tile_rows), c_int(n_slots), c_int(E), c_int(top),
                                     c_int(K), c_int(N), c_int(1 if first else 0), c_int(1 if weight_on_input else 0), c_float(alpha),
                                     c_float(limit), c_int(1 if plain else 0), c_int(dtype_code(w0.dtype)), _stream()))


def moe_combine(out: torch.Tensor, rows: torch.Tensor, pos_of_slot: torch.Tensor, shared_out: Optional[torch.Tensor], top: int,
                slot_weight: Optional[torch.Tensor] = None) -> None:
    """out float32 [n, H] = shared_out (storage dtype, or None) + the token's `top` rows of `rows` (float32 [slots, H]), each
    times its slot's weight where `slot_weight` (float32 [n * top]) is given."""
    lib = build.load("moe")
    n, H = out.shape
    dt = shared_out.dtype if shared_out is not None else torch.float32
    _check(lib, lib.llmk_moe_combine(_ptr(out), _ptr(rows), _ptr(pos_of_slot), _ptr(shared_out), _ptr(slot_weight), c_int(n), c_int(top), c_int(H),
                                     c_int(dtype_code(dt)), _stream()))
