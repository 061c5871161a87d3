"""Python launchers of the hand-written CUDA kernels (ctypes over the libraries csrc/build.py makes).

Tensors are torch tensors used as plain device memory: every launcher checks device, dtype and
layout, passes raw pointers and the current CUDA stream, and turns a non-zero status into a
`KernelError`.  Nothing here computes: if a library cannot be built or loaded the call raises;
there is no CPU or library-op fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_uint64, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import build

DT_F32, DT_BF16 = 0, 1
_STATUS = {-1: "unsupported dtype", -2: "unsupported shape", -3: "misaligned pointer or stride",
           -4: "size beyond the kernel's limit", -5: "device-side wait ran out"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """Kernel launches made through this module since import (launch counting for measurements)."""
    return _launches


def count_launches(n: int) -> None:
    """Account for launches made on this module's behalf elsewhere (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")
    raise KernelError(f"{what}: CUDA error {status} (cudaError_t)")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return DT_F32
    if dt == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)     # the short way to the stream's handle
_device_index: Optional[int] = None


def _stream() -> c_void_p:
    """The current stream of the current device (under a graph capture: the capturing stream).  Asked for at
    every launch, so by the shortest route torch offers."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (no CPU path exists)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_sigs_done = set()
_profile: Optional[list] = None          # (function name, start event, end event) per launch while profiling


def profile_start() -> None:
    """From now on every launch made through this module is bracketed by two CUDA events (for launch-by-launch
    runs; launches replayed inside a CUDA graph are not seen)."""
    global _profile
    _profile = []


def profile_report():
    """Stop profiling; [(function, calls, seconds on the device)] sorted by time, the reference's per-kind
    totals (stratum/native/stratum_arch_llama.inc.c:2081-2091) with kernels in place of weight types."""
    global _profile
    rows, _profile = _profile or [], None
    torch.cuda.synchronize()
    totals = {}
    for name, e0, e1 in rows:
        calls, secs = totals.get(name, (0, 0.0))
        totals[name] = (calls + 1, secs + e0.elapsed_time(e1) * 1e-3)
    return sorted(((n, c, t) for n, (c, t) in totals.items()), key=lambda r: -r[2])


class _Timed:
    """A launcher whose calls are bracketed by events while profiling is on."""
    __slots__ = ("f", "name")

    def __init__(self, f, name):
        self.f, self.name = f, name

    def __call__(self, *args):
        if _profile is None:
            return self.f(*args)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        status = self.f(*args)
        e1.record()
        _profile.append((self.name, e0, e1))
        return status


_timed = {}


def _fn(libname: str, fname: str, argtypes):
    key = (libname, fname)
    t = _timed.get(key)
    if t is None:
        lib = build.load(libname)
        f = getattr(lib, fname)
        f.argtypes = argtypes
        f.restype = c_int
        t = _timed[key] = _Timed(f, fname.replace("stratum_", "", 1))
    return t if _profile is not None else t.f


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] as float32.  table [V,H] float32|bfloat16, ids int32 [T], out float32 [T,H]."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    f = _fn("elementwise", "stratum_embed_gather",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), ids.numel(), table.shape[1],
             table.shape[0], _stream()), "embed_gather")


class _EmbedPairs(ctypes.Structure):
    """Mirror of struct EmbedPairs in csrc/elementwise.cu."""
    _fields_ = [("table", c_void_p), ("pairs", c_void_p), ("ids", c_void_p), ("token_pos", c_void_p),
                ("token_seq", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p), ("last", c_void_p),
                ("out", c_void_p), ("out2", c_void_p),
                ("n_tokens", c_int), ("hidden", c_int), ("vocab", c_int), ("buckets", c_int),
                ("mul_prev", c_int), ("mul_cur", c_int), ("write_state", c_int), ("reserved", c_int),
                ("scale", c_float), ("reserved2", c_float)]


def embed_pairs(table: torch.Tensor, pairs: Optional[torch.Tensor], ids: torch.Tensor, token_pos: torch.Tensor,
                token_seq: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor, last: Optional[torch.Tensor],
                out: torch.Tensor, out2: Optional[torch.Tensor], scale: float, mul_prev: int, mul_cur: int,
                write_state: bool = True) -> None:
    """out[t] = table[ids[t]] * scale + pairs[(prev * mul_prev + ids[t] * mul_cur) mod buckets], float32; prev is the
    token in front of t in its sequence (from the step, or from `last`, int32 [slots, 1], which then takes the
    sequence's last token of this step); a sequence's first token reads the last row of pairs [buckets + 1, hidden].
    out2 (or None) receives the same rows.  pairs None: out[t] = table[ids[t]] * scale, and `last` is not touched."""
    _need(table, "table"); _need(ids, "ids", torch.int32)
    _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
    _need(seq_start, "seq_start", torch.int32); _need(seq_slot, "seq_slot", torch.int32)
    _need(out, "out", torch.float32)
    if out.shape != (ids.numel(), table.shape[1]):
        raise KernelError("embed_pairs: shapes disagree")
    p = _EmbedPairs()
    p.table, p.ids, p.token_pos = table.data_ptr(), ids.data_ptr(), token_pos.data_ptr()
    p.token_seq, p.seq_start, p.seq_slot = token_seq.data_ptr(), seq_start.data_ptr(), seq_slot.data_ptr()
    p.out = out.data_ptr()
    if pairs is not None:
        _need(pairs, "pairs", table.dtype); _need(last, "last", torch.int32)
        if pairs.shape[1] != table.shape[1] or pairs.shape[0] < 2:
            raise KernelError("embed_pairs: shapes disagree")
        p.pairs, p.last, p.buckets = pairs.data_ptr(), last.data_ptr(), pairs.shape[0] - 1
    if out2 is not None:
        _need(out2, "out2", torch.float32)
        if out2.shape != out.shape:
            raise KernelError("embed_pairs: out2 and out disagree")
        p.out2 = out2.data_ptr()
    p.n_tokens, p.hidden, p.vocab = ids.numel(), table.shape[1], table.shape[0]
    p.mul_prev, p.mul_cur, p.write_state, p.scale = int(mul_prev), int(mul_cur), int(bool(write_state)), float(scale)
    f = _fn("elementwise", "stratum_embed_pairs", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(table.dtype), _stream()), "embed_pairs")


def add_rows(x: torch.Tensor, a: Optional[torch.Tensor], row: torch.Tensor) -> None:
    """x[t] += a[t] (where given) + row: x, a float32 [tokens, hidden], row float32 [hidden]."""
    _need(x, "x", torch.float32); _need(row, "row", torch.float32)
    if a is not None:
        _need(a, "a", torch.float32)
        if a.shape != x.shape:
            raise KernelError("add_rows: a and x disagree")
    if row.numel() != x.shape[1]:
        raise KernelError("add_rows: row and x disagree")
    f = _fn("elementwise", "stratum_add_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(a), _ptr(row), x.shape[0], x.shape[1], _stream()), "add_rows")


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * gain.  x float32 [*,H], gain float32 [H]."""
    _need(x, "x", torch.float32); _need(gain, "gain", torch.float32); _need(out, "out")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("rmsnorm: rows and out disagree")
    elif x.shape[0] != n_rows:
        raise KernelError("rmsnorm: x and out disagree")
    f = _fn("elementwise", "stratum_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), _ptr(gain), _ptr(rows), _ptr(out), dtype_code(out.dtype), n_rows, x.shape[-1],
             c_float(eps), _stream()), "rmsnorm")


def rmsnorm_pair(x: torch.Tensor, gain_a: torch.Tensor, gain_b: torch.Tensor, eps: float, out_a: torch.Tensor,
                 out_b: torch.Tensor) -> None:
    """out_a[r] = rmsnorm(x[r]) * gain_a and out_b[r] = rmsnorm(x[r]) * gain_b from one pass over x (float32 [rows, H];
    the outputs of one dtype)."""
    _need(x, "x", torch.float32); _need(gain_a, "gain_a", torch.float32); _need(gain_b, "gain_b", torch.float32)
    _need(out_a, "out_a"); _need(out_b, "out_b", out_a.dtype)
    if out_a.shape != x.shape or out_b.shape != x.shape or gain_a.numel() != x.shape[1] or gain_b.numel() != x.shape[1]:
        raise KernelError("rmsnorm_pair: shapes disagree")
    f = _fn("elementwise", "stratum_rmsnorm_pair",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), _ptr(gain_a), _ptr(gain_b), _ptr(out_a), _ptr(out_b), dtype_code(out_a.dtype), x.shape[0],
             x.shape[1], c_float(eps), _stream()), "rmsnorm_pair")


def rmsnorm_heads(x: torch.Tensor, first_col: int, n_heads: int, head_dim: int, gain: torch.Tensor,
                  eps: float) -> None:
    """In place, in every row of x [T, width]: each of the n_heads stretches of head_dim values from column
    first_col on becomes rmsnorm(stretch) * gain.  gain float32 [head_dim]."""
    _need(x, "x", contiguous=False); _need(gain, "gain", torch.float32)
    if x.dim() != 2 or x.stride(1) != 1 or first_col < 0 or first_col + n_heads * head_dim > x.shape[1]:
        raise KernelError("rmsnorm_heads: the heads do not lie inside the rows of x")
    if gain.numel() != head_dim:
        raise KernelError("rmsnorm_heads: gain and head_dim disagree")
    f = _fn("elementwise", "stratum_rmsnorm_heads",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p])
    _check(f(_ptr(x), dtype_code(x.dtype), x.shape[0], x.stride(0), first_col, n_heads, head_dim, _ptr(gain),
             c_float(eps), _stream()), "rmsnorm_heads")


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = tanh(alpha * x[rows[r]] or x[r]) * w + b.  x float32 [*,H]; alpha float32 (one number, on the
    device); w, b float32 [H]."""
    _need(x, "x", torch.float32); _need(alpha, "alpha", torch.float32); _need(w, "w", torch.float32)
    _need(b, "b", torch.float32); _need(out, "out")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("dynamic_tanh: rows and out disagree")
    elif x.shape[0] != n_rows:
        raise KernelError("dynamic_tanh: x and out disagree")
    if alpha.numel() != 1 or w.numel() != x.shape[-1] or b.numel() != x.shape[-1]:
        raise KernelError("dynamic_tanh: alpha is one number, w and b have the row's length")
    f = _fn("elementwise", "stratum_dynamic_tanh",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(alpha), _ptr(w), _ptr(b), _ptr(rows), _ptr(out), dtype_code(out.dtype), n_rows,
             x.shape[-1], _stream()), "dynamic_tanh")


GELU_ERF, GELU_TANH = 0, 1


def gelu(x: torch.Tensor, kind: int = GELU_ERF) -> None:
    """In place over the rows of x [rows, width]: the exact GELU (kind GELU_ERF) or its tanh form (GELU_TANH)."""
    _need(x, "x", contiguous=False)
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gelu: rows must be contiguous")
    f = _fn("elementwise", "stratum_gelu", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), dtype_code(x.dtype), x.shape[0], x.shape[1], x.stride(0), kind, _stream()), "gelu")


def swiglu(gu: torch.Tensor, out: torch.Tensor, act: int = 0) -> None:
    """out[r][j] = silu(gu[r][2j]) * gu[r][2j+1]; with act (ACT_*), that activation takes silu's place."""
    _need(gu, "gu"); _need(out, "out", gu.dtype)
    f = _fn("elementwise", "stratum_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gu), _ptr(out), dtype_code(gu.dtype), out.shape[0], out.shape[1], int(act), _stream()), "swiglu")


def rope_store(qkv: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
               block_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], interleaved: bool,
               mscale: float, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
               n_q: int, n_kv: int, head_dim: int, page_tokens: int, write_cache: bool) -> None:
    """Rotate q (in place) and k, and store k and v into the paged cache."""
    _need(qkv, "qkv"); _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
    n_pairs = 0 if inv_freq is None else inv_freq.numel()
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
    if write_cache:
        _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
        _need(block_table, "block_table", torch.int32)
    if qkv.shape[-1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width is not (n_q + 2 n_kv) * head_dim")
    f = _fn("elementwise", "stratum_rope_store",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), dtype_code(qkv.dtype), _ptr(token_pos), _ptr(token_seq), _ptr(block_table),
             0 if block_table is None else block_table.stride(0), _ptr(inv_freq), n_pairs, int(interleaved),
             c_float(mscale), _ptr(k_cache), _ptr(v_cache), qkv.shape[0], n_q, n_kv, head_dim, page_tokens,
             int(write_cache), _stream()), "rope_store")


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor, mscale: float, out: torch.Tensor) -> None:
    """out[t][k] = mscale * (cos, sin)((float)pos[t] * inv_freq[k]): float32 [tokens, pairs, 2], once per step, for
    the matrix-product epilogues that rotate queries and keys."""
    _need(token_pos, "token_pos", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(out, "out", torch.float32)
    if tuple(out.shape) != (token_pos.numel(), inv_freq.numel(), 2):
        raise KernelError("rope_table: out must be [tokens, pairs, 2]")
    f = _fn("elementwise", "stratum_rope_table", [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(token_pos), _ptr(inv_freq), c_float(mscale), _ptr(out), token_pos.numel(), inv_freq.numel(),
             _stream()), "rope_table")


def fill_normal(out: torch.Tensor, seed: int, std: float) -> None:
    """Fill with std * N(0,1) from a counter-based generator keyed by (seed, element index)."""
    _need(out, "out")
    f = _fn("elementwise", "stratum_fill_normal", [c_void_p, c_int, c_size_t, c_uint64, c_float, c_void_p])
    _check(f(_ptr(out), dtype_code(out.dtype), out.numel(), c_uint64(seed & (2**64 - 1)), c_float(std),
             _stream()), "fill_normal")


# ------------------------------------------------------------------ linear (any shape, CUDA cores)
EPI_STORE, EPI_ADD_F32, EPI_STORE_F32, EPI_SWIGLU = 0, 1, 2, 3
EPI_ADD_F32_EMIT, EPI_QKV_ROPE = 4, 5          # gemm_tc only: see GemmExtra


# what a product with EPI_STORE may apply to what it stores; with EPI_SWIGLU: the gate's activation (0 = silu)
ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH, ACT_RELU_SQ = 0, 1, 2, 3


def linear_simple(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  epilogue: int, act: int = ACT_NONE) -> None:
    """out (=|+=) x @ w.T + bias.  x [M,K] and w [N,K] of one dtype; bias float32; see EPI_*.  act (EPI_STORE
    only): the activation applied to what is stored, see ACT_*."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("linear: rows must be contiguous")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"linear: epilogue {epilogue} writes {want}, out is {out.dtype}")
    f = _fn("linear_simple", "stratum_linear_simple",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), dtype_code(x.dtype), epilogue, M, N, K, x.stride(0),
             out.stride(0), act, _stream()), "linear_simple")


def linear_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_step: int, o_step: int) -> None:
    """One product per head on the CUDA cores: out[:, j*o_step : j*o_step+N] = x[:, j*x_step : j*x_step+K] @ w[j].T.
    x [M, >= (heads-1)*x_step+K] and w [heads, N, K] of one dtype, out of the same dtype."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", x.dtype, contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1 or w.dim() != 3:
        raise KernelError("linear_heads: rows must be contiguous and w [heads, N, K]")
    heads, N, Kd = w.shape
    f = _fn("linear_simple", "stratum_linear_heads",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(out), dtype_code(x.dtype), EPI_STORE, heads, x.shape[0], N, Kd, x.stride(0),
             out.stride(0), x_step, o_step, _stream()), "linear_heads")


def head_gemm_ok(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_step: int, o_step: int) -> bool:
    """Whether the tensor-core form of linear_heads takes this call."""
    return (x.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0 and x_step % 8 == 0
            and x.stride(0) % 8 == 0 and o_step % 2 == 0 and out.stride(0) % 2 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0)


def head_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_step: int, o_step: int) -> None:
    """linear_heads in bfloat16 on tensor cores: every head's product in one launch (see head_gemm_ok)."""
    _need(x, "x", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1 or w.dim() != 3:
        raise KernelError("head_gemm: rows must be contiguous and w [heads, N, K]")
    heads, N, Kd = w.shape
    f = _fn("head_gemm", "stratum_head_gemm",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(out), heads, x.shape[0], N, Kd, x.stride(0), out.stride(0), x_step, o_step,
             _stream()), "head_gemm")


def _linear_shapes(x, w, bias, out, epilogue, what):
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", contiguous=False)
    if x.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError(f"{what}: rows must be contiguous")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    M, Kd = x.shape
    N = w.shape[0]
    width = N // 2 if epilogue == EPI_SWIGLU else N
    if w.shape[1] != Kd or out.shape[0] != M or out.shape[1] != width:
        raise KernelError(f"{what}: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    want = x.dtype if epilogue in (EPI_STORE, EPI_SWIGLU) else torch.float32
    if out.dtype != want:
        raise KernelError(f"{what}: epilogue {epilogue} writes {want}, out is {out.dtype}")
    return M, N, Kd


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                epilogue: int, act: int = ACT_NONE) -> None:
    """bfloat16, at most 32 rows of x: the weight-streaming tensor-core kernel (see EPI_*; act as linear_simple's)."""
    M, N, Kd = _linear_shapes(x, w, bias, out, epilogue, "gemm_skinny")
    _need(x, "x", torch.bfloat16, contiguous=False)
    f = _fn("gemm_skinny", "stratum_gemm_skinny",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), epilogue, M, N, Kd, x.stride(0), out.stride(0), act,
             _stream()), "gemm_skinny")


_scratch_epoch = 0


def scratch_epoch() -> int:
    """Grows whenever a scratch buffer that kernels are given is replaced by a larger one (the old one is freed).
    A captured CUDA graph recorded the old address: whoever replays graphs compares this number with the one
    at capture and captures again when it has moved."""
    return _scratch_epoch


def scratch_regrown() -> None:
    global _scratch_epoch
    _scratch_epoch += 1


_status_word: Optional[torch.Tensor] = None


def status_word() -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits write to when a wait runs out."""
    global _status_word
    if _status_word is None:
        _status_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status_word


def check_status() -> None:
    """Synchronise and raise if a kernel gave up a wait (the word is cleared for the next run)."""
    if _status_word is None:
        return
    code = int(_status_word.item())
    if code != 0:
        _status_word.zero_()
        where = {101: "the TMA producer waiting for a free stage", 102: "the MMA warp waiting for a free accumulator",
                 103: "the MMA warp waiting for a loaded stage", 104: "the epilogue waiting for an accumulator"}
        raise KernelError(f"a device-side wait ran out in {where.get(code, f'code {code}')}; results are invalid")


_gemm_scratch = None


def _gemm_tc_scratch(device):
    """float32 scratch for the partial tiles of tiles that several CTAs share."""
    global _gemm_scratch
    if _gemm_scratch is None or _gemm_scratch.device != device:
        lib = build.load("gemm_tc")
        lib.stratum_gemm_tc_scratch_floats.restype = ctypes.c_longlong
        _gemm_scratch = torch.empty(int(lib.stratum_gemm_tc_scratch_floats()), dtype=torch.float32, device=device)
        scratch_regrown()
    return _gemm_scratch


class _EpiExtra(ctypes.Structure):
    """Mirror of struct EpiExtra in csrc/gemm_tc.cu (pointers first, then 4-byte fields)."""
    _fields_ = [("norm_ss", c_void_p), ("emit_x", c_void_p), ("emit_gain", c_void_p), ("emit_ss", c_void_p),
                ("rope_cs", c_void_p), ("token_pos", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("norm_parts", c_int), ("norm_ld", c_int), ("norm_size", c_float), ("norm_eps", c_float),
                ("emit_ldx", c_int), ("emit_ld", c_int),
                ("rope_pairs", c_int), ("bt_stride", c_int), ("n_q", c_int), ("n_kv", c_int), ("head_dim", c_int),
                ("page_tokens", c_int), ("write_cache", c_int), ("act", c_int)]


class GemmExtra:
    """What a gemm_tc call does beyond its basic epilogue (all optional):

    scaled rows   norm_ss float32 [parts, rows] partial sums of squares of the rows a norm handed over as
                  r * gain: the product's rows are multiplied by 1 / sqrt(sum / norm_size + norm_eps);
    EPI_ADD_F32_EMIT   emit_x bfloat16 [rows, N] receives bf16(new residual * emit_gain), emit_ss float32
                  [parts, rows] the sums of squares of the new residual values per tile of columns (how many
                  parts were written: `last_parts()` after the call);
    EPI_QKV_ROPE  the columns are query, key and value heads (pairs of rotated dimensions neighbours): queries
                  are rotated and stored to `out`, keys rotated and written, values written, into the paged cache;
    activation    EPI_STORE applies ACT_* to what it stores.
    """

    def __init__(self):
        self.c = _EpiExtra()
        self.keep = []                      # tensors whose memory the struct points into

    def activation(self, act: int) -> "GemmExtra":
        self.c.act = int(act)
        return self

    def scaled_rows(self, norm_ss: torch.Tensor, parts: int, size: int, eps: float) -> "GemmExtra":
        _need(norm_ss, "norm_ss", torch.float32)
        if norm_ss.dim() != 2 or norm_ss.shape[0] < parts:
            raise KernelError("gemm_tc: norm_ss must be [parts or more, rows]")
        self.c.norm_ss, self.c.norm_parts, self.c.norm_ld = norm_ss.data_ptr(), parts, norm_ss.stride(0)
        self.c.norm_size, self.c.norm_eps = float(size), float(eps)
        self.keep.append(norm_ss)
        return self

    def emit(self, emit_x: torch.Tensor, gain: torch.Tensor, emit_ss: torch.Tensor) -> "GemmExtra":
        _need(emit_x, "emit_x", torch.bfloat16); _need(gain, "gain", torch.float32)
        _need(emit_ss, "emit_ss", torch.float32)
        self.c.emit_x, self.c.emit_gain, self.c.emit_ss = emit_x.data_ptr(), gain.data_ptr(), emit_ss.data_ptr()
        self.c.emit_ldx, self.c.emit_ld = emit_x.stride(0), emit_ss.stride(0)
        self.keep += [emit_x, gain, emit_ss]
        return self

    def qkv_rope(self, rope_cs: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
                 block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                 v_cache: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, page_tokens: int,
                 write_cache: bool) -> "GemmExtra":
        _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
        if rope_cs is not None:
            _need(rope_cs, "rope_cs", torch.float32)
            if rope_cs.dim() != 3 or rope_cs.shape[0] != token_pos.numel() or rope_cs.shape[2] != 2:
                raise KernelError("gemm_tc: rope_cs must be [rows, pairs, 2]")
            self.c.rope_cs, self.c.rope_pairs = rope_cs.data_ptr(), rope_cs.shape[1]
        if write_cache:
            _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
            _need(block_table, "block_table", torch.int32, contiguous=False)
            self.c.k_cache, self.c.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
            self.c.block_table, self.c.bt_stride = block_table.data_ptr(), block_table.stride(0)
        self.c.token_pos, self.c.token_seq = token_pos.data_ptr(), token_seq.data_ptr()
        self.c.n_q, self.c.n_kv, self.c.head_dim, self.c.page_tokens = n_q, n_kv, head_dim, page_tokens
        self.c.write_cache = int(bool(write_cache))
        self.keep += [rope_cs, token_pos, token_seq, block_table, k_cache, v_cache]
        return self


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epilogue: int, extra: Optional[GemmExtra] = None) -> int:
    """bfloat16 matrix product on the 5th-generation tensor cores (TMA + tcgen05/TMEM); see EPI_* and GemmExtra.
    The form (k shared inside clusters, stream-K, tiles, tiles on pairs of CTAs) is chosen from the shapes in
    gemm_tc.cu.  Returns the number of parts written per row with EPI_ADD_F32_EMIT (else 0)."""
    basic = {EPI_ADD_F32_EMIT: EPI_ADD_F32, EPI_QKV_ROPE: EPI_STORE}.get(epilogue, epilogue)
    M, N, Kd = _linear_shapes(x, w, bias, out, basic, "gemm_tc")
    _need(x, "x", torch.bfloat16, contiguous=False)
    if epilogue in (EPI_ADD_F32_EMIT, EPI_QKV_ROPE) and extra is None:
        raise KernelError("gemm_tc: this epilogue needs a GemmExtra")
    part = _gemm_tc_scratch(x.device)
    lib = build.load("gemm_tc")
    f = _fn("gemm_tc", "stratum_gemm_tc_ex",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), epilogue, M, N, Kd, x.stride(0), out.stride(0),
             _ptr(status_word()), _ptr(part), None if extra is None else ctypes.addressof(extra.c), _stream()),
           "gemm_tc")
    count_launches(lib.stratum_gemm_tc_last_launches() - 1)      # a second pass, if there was one
    return int(lib.stratum_gemm_tc_last_parts()) if epilogue == EPI_ADD_F32_EMIT else 0


def gemm_tc_last_form() -> Tuple[str, int]:
    """The form the last gemm_tc call took, for tests:
    ("tiles" | "pairs" | "pairs-shared" | "stream-k" | "cluster-k", cluster size)."""
    code = int(build.load("gemm_tc").stratum_gemm_tc_last_form())
    return {1: "tiles", 2: "pairs", 3: "stream-k", 4: "cluster-k", 5: "pairs-shared"}.get(code % 16, "none"), code // 16


# ------------------------------------------------------------------ attention (any sizes, CUDA cores)
def attention_simple(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                     token_seq: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_tokens: int, window: int, scale: float) -> None:
    """Causal GQA attention of every token of the step over its sequence's cached keys."""
    _need(qkv, "qkv"); _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
    _need(out, "out", qkv.dtype); _need(block_table, "block_table", torch.int32)
    f = _fn("attention_simple", "stratum_attention_simple",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), dtype_code(qkv.dtype), _ptr(token_pos),
             _ptr(token_seq), _ptr(block_table), block_table.stride(0), _ptr(out), out.stride(0), qkv.shape[0],
             n_q, n_kv, head_dim, page_tokens, window, c_float(scale), _stream()), "attention_simple")


class _MixerPrep(ctypes.Structure):
    """Mirror of struct MixerPrep in csrc/mixer_prep.cu."""
    _fields_ = [("x", c_void_p), ("token_pos", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("inv_freq", c_void_p), ("k_norm_gain", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("q_out", c_void_p), ("k_out", c_void_p), ("ld", c_int), ("bt_stride", c_int), ("n_tokens", c_int), ("rot_pairs", c_int),
                ("n_q", c_int), ("q_dim", c_int), ("q_col", c_int), ("q_rot_off", c_int),
                ("n_k", c_int), ("k_dim", c_int), ("k_col", c_int), ("k_rot_off", c_int), ("k_norm_n", c_int),
                ("n_v", c_int), ("v_dim", c_int), ("v_col", c_int),
                ("page_tokens", c_int), ("write_cache", c_int), ("eps", c_float),
                ("q_out_ld", c_int), ("q_out_step", c_int), ("q_out_off", c_int), ("k_out_ld", c_int),
                ("interleaved", c_int)]


def mixer_prep(x: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor, block_table: Optional[torch.Tensor],
               k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_tokens: int, write_cache: bool,
               *, queries=(0, 0, 0), keys=(0, 0, 0), values=(0, 0, 0), inv_freq: Optional[torch.Tensor] = None,
               q_rot_off: int = 0, k_rot_off: int = 0, k_norm_gain: Optional[torch.Tensor] = None,
               eps: float = 0.0, q_out: Optional[torch.Tensor] = None, q_out_step: int = 0,
               q_out_off: int = 0, k_out: Optional[torch.Tensor] = None, interleaved: bool = False) -> None:
    """Between a fused projection and attention.  x [tokens, ld] holds runs of equal heads: queries, keys, values,
    each given as (heads, head size, first column).  Queries: dimensions [q_rot_off, q_rot_off + 2R) rotated in
    place (R = len(inv_freq), pairs (i, i + R), or the neighbours (2i, 2i + 1) when `interleaved`); with q_out [tokens, *] the dimensions from q_rot_off on go, the
    first 2R rotated, to q_out[:, j * q_out_step + q_out_off ...] for head j instead.  Keys: the first len(k_norm_gain) dimensions divided by their
    root mean square (eps inside the root) times the gain, dimensions [k_rot_off, k_rot_off + 2R) rotated, then
    appended to k_cache, and with k_out [tokens, *] also written to its row t (zeros for tokens of no sequence).
    Values: appended to v_cache.  Tokens of no sequence are left alone otherwise."""
    _need(x, "x", contiguous=False); _need(token_pos, "token_pos", torch.int32)
    _need(token_seq, "token_seq", torch.int32)
    p = _MixerPrep()
    p.x, p.token_pos, p.token_seq = x.data_ptr(), token_pos.data_ptr(), token_seq.data_ptr()
    p.ld, p.n_tokens = x.stride(0), x.shape[0]
    p.n_q, p.q_dim, p.q_col = queries
    p.n_k, p.k_dim, p.k_col = keys
    p.n_v, p.v_dim, p.v_col = values
    p.q_rot_off, p.k_rot_off = q_rot_off, k_rot_off
    p.interleaved = int(bool(interleaved))
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        p.inv_freq, p.rot_pairs = inv_freq.data_ptr(), inv_freq.numel()
    if k_norm_gain is not None:
        _need(k_norm_gain, "k_norm_gain", torch.float32)
        p.k_norm_gain, p.k_norm_n = k_norm_gain.data_ptr(), k_norm_gain.numel()
    p.eps, p.page_tokens, p.write_cache = float(eps), page_tokens, int(bool(write_cache))
    if q_out is not None:
        _need(q_out, "q_out", x.dtype, contiguous=False)
        p.q_out, p.q_out_ld, p.q_out_step, p.q_out_off = q_out.data_ptr(), q_out.stride(0), q_out_step, q_out_off
    if k_out is not None:
        _need(k_out, "k_out", x.dtype, contiguous=False)
        if not write_cache:
            raise KernelError("mixer_prep: k_out goes with the cache write")
        p.k_out, p.k_out_ld = k_out.data_ptr(), k_out.stride(0)
    if write_cache:
        _need(block_table, "block_table", torch.int32, contiguous=False)
        p.block_table, p.bt_stride = block_table.data_ptr(), block_table.stride(0)
        if p.n_k:
            _need(k_cache, "k_cache", x.dtype)
            p.k_cache = k_cache.data_ptr()
        if p.n_v:
            _need(v_cache, "v_cache", x.dtype)
            p.v_cache = v_cache.data_ptr()
    f = _fn("mixer_prep", "stratum_mixer_prep", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(x.dtype), _stream()), "mixer_prep")


def gate_heads(a: torch.Tensor, g: torch.Tensor, n_heads: int, block: int) -> None:
    """In place: a[t, j * block + i] *= sigmoid(g[t, j]) for j < n_heads, i < block; a and g of one dtype, rows of
    any stride."""
    _need(a, "a", contiguous=False); _need(g, "g", a.dtype, contiguous=False)
    if a.shape[0] != g.shape[0] or a.shape[1] < n_heads * block or g.shape[1] < n_heads or a.stride(1) != 1 \
            or g.stride(1) != 1:
        raise KernelError("gate_heads: shapes disagree")
    f = _fn("mixer_prep", "stratum_gate_heads",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), a.stride(0), _ptr(g), g.stride(0), a.shape[0], n_heads, block, dtype_code(a.dtype), _stream()),
           "gate_heads")


class _GeneralAttention(ctypes.Structure):
    """Mirror of struct GeneralAttention in csrc/attention_general.h."""
    _fields_ = [("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("out", c_void_p),
                ("token_pos", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("qb_seq", c_void_p), ("qb_tok0", c_void_p), ("qb_ntok", c_void_p),
                ("part_o", c_void_p), ("part_ml", c_void_p), ("seq_start", c_void_p), ("sink", c_void_p),
                ("ldq", c_int), ("ldo", c_int), ("bt_stride", c_int), ("n_tokens", c_int),
                ("n_heads", c_int), ("group", c_int), ("maps", c_int),
                ("qk_dim", c_int), ("v_dim", c_int), ("n_k_heads", c_int), ("n_v_heads", c_int), ("v_in_k", c_int),
                ("page_tokens", c_int), ("window", c_int), ("combine", c_int), ("gate_col", c_int),
                ("temp_every", c_int), ("n_qblocks", c_int), ("tokens_per_block", c_int), ("n_splits", c_int),
                ("chunk", c_int), ("reserved", c_int),
                ("dense", c_int), ("ldk", c_int), ("ldv", c_int), ("keep_first", c_int),
                ("scale", c_float), ("softcap", c_float), ("temp_coef", c_float), ("lam", c_float),
                ("out_scale", c_float), ("eps", c_float)]


class AttentionShape:
    """The constants of a general attention (see csrc/attention_general.cu): heads, query heads per key/value
    head (`group`), score maps per head, key and value sizes, whether the values are the first v_dim values of
    the key rows, scale, softcap (0: none), window (0: every key; keep_first: with a window, the positions below it stay
    visible), the query factor
    1 + temp_coef ln(floor((p + 1) / temp_every) + 1), and for two maps the combination
    (a_0 - lam a_1) / rms * out_scale with its eps and the column of the output gate (-1: none)."""

    def __init__(self, n_heads: int, group: int, maps: int, qk_dim: int, v_dim: int, v_in_k: bool, scale: float,
                 softcap: float = 0.0, window: int = 0, temp_coef: float = 0.0, temp_every: int = 1,
                 lam: float = 0.0, out_scale: float = 1.0, eps: float = 0.0, gate_col: int = -1,
                 sink: Optional[torch.Tensor] = None, keep_first: int = 0):
        self.keep_first = int(keep_first) if window > 0 else 0
        self.n_heads, self.group, self.maps, self.qk_dim, self.v_dim = n_heads, group, maps, qk_dim, v_dim
        self.v_in_k, self.scale, self.softcap, self.window = bool(v_in_k), scale, softcap, window
        self.temp_coef, self.temp_every, self.lam, self.out_scale = temp_coef, temp_every, lam, out_scale
        self.eps, self.gate_col = eps, gate_col
        if sink is not None:
            _need(sink, "sink", torch.float32)
            if sink.numel() != n_heads:
                raise KernelError("attention: one sink per head")
        self.sink = sink

    def fill(self, p: "_GeneralAttention") -> None:
        p.n_heads, p.group, p.maps, p.qk_dim, p.v_dim = self.n_heads, self.group, self.maps, self.qk_dim, self.v_dim
        p.n_k_heads = (self.n_heads // self.group) * self.maps
        p.n_v_heads = 0 if self.v_in_k else self.n_heads // self.group
        p.v_in_k, p.window, p.combine, p.gate_col = int(self.v_in_k), self.window, int(self.maps == 2), self.gate_col
        p.temp_every, p.scale, p.softcap, p.temp_coef = self.temp_every, self.scale, self.softcap, self.temp_coef
        p.lam, p.out_scale, p.eps, p.keep_first = self.lam, self.out_scale, self.eps, self.keep_first
        p.sink = None if self.sink is None else self.sink.data_ptr()


def _general_params(shape: AttentionShape, q, k_cache, v_cache, token_pos, token_seq, block_table, out,
                    page_tokens: int, seq_start: Optional[torch.Tensor] = None) -> "_GeneralAttention":
    _need(q, "q", contiguous=False); _need(k_cache, "k_cache", q.dtype); _need(out, "out", q.dtype, contiguous=False)
    _need(token_pos, "token_pos", torch.int32); _need(token_seq, "token_seq", torch.int32)
    if seq_start is not None:                 # keys and values as plain matrices, rows by sequence and position
        _need(seq_start, "seq_start", torch.int32); _need(v_cache, "v_cache", q.dtype)
        if k_cache.dim() != 2 or v_cache.dim() != 2 or shape.v_in_k:
            raise KernelError("attention_general: dense keys and values are two matrices [rows, heads * size]")
        p = _GeneralAttention()
        shape.fill(p)
        p.q, p.k_cache, p.v_cache, p.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
        p.token_pos, p.token_seq, p.seq_start = token_pos.data_ptr(), token_seq.data_ptr(), seq_start.data_ptr()
        p.dense, p.ldk, p.ldv = 1, k_cache.stride(0), v_cache.stride(0)
        p.ldq, p.ldo, p.n_tokens, p.page_tokens = q.stride(0), out.stride(0), q.shape[0], page_tokens
        return p
    _need(block_table, "block_table", torch.int32, contiguous=False)
    if q.stride(-1) != 1 or out.stride(-1) != 1:
        raise KernelError("attention_general: rows must be contiguous")
    p = _GeneralAttention()
    shape.fill(p)
    p.q, p.k_cache, p.out = q.data_ptr(), k_cache.data_ptr(), out.data_ptr()
    if not shape.v_in_k:
        _need(v_cache, "v_cache", q.dtype)
        p.v_cache = v_cache.data_ptr()
    p.token_pos, p.token_seq, p.block_table = token_pos.data_ptr(), token_seq.data_ptr(), block_table.data_ptr()
    p.ldq, p.ldo, p.bt_stride, p.n_tokens, p.page_tokens = q.stride(0), out.stride(0), block_table.stride(0), \
        q.shape[0], page_tokens
    return p


def attention_general(shape: AttentionShape, q: torch.Tensor, k_cache: torch.Tensor, v_cache: Optional[torch.Tensor],
                      token_pos: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor,
                      page_tokens: int) -> None:
    """Causal attention of every token of the step over its sequence's cached keys for the shapes AttentionShape
    describes, on the CUDA cores in float32 (q, the cache and out in one dtype)."""
    p = _general_params(shape, q, k_cache, v_cache, token_pos, token_seq, block_table, out, page_tokens)
    f = _fn("attention_general", "stratum_attention_general", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(q.dtype), _stream()), "attention_general")


def attention_general_mma_ok(shape: AttentionShape, q: torch.Tensor, out: torch.Tensor, page_tokens: int) -> bool:
    """Whether the tensor-core form of the general attention takes this call (else: attention_general)."""
    return (q.dtype == torch.bfloat16 and shape.qk_dim % 8 == 0 and shape.v_dim % 8 == 0 and shape.v_dim <= 512
            and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0 and page_tokens == 64)


def attention_general_mma_row_groups(v_dim: int) -> int:
    """Groups of 16 query rows a CTA of the tensor-core general attention takes in prompt steps."""
    return int(build.load("attention_general_mma").stratum_attention_general_mma_row_groups(int(v_dim)))


def attention_general_mma(shape: AttentionShape, q: torch.Tensor, k_cache: torch.Tensor,
                          v_cache: Optional[torch.Tensor], token_pos: torch.Tensor, token_seq: torch.Tensor,
                          block_table: torch.Tensor, out: torch.Tensor, page_tokens: int, qblocks,
                          tokens_per_block: int, n_splits: int, chunk: int, part_o: Optional[torch.Tensor],
                          part_ml: Optional[torch.Tensor], row_groups: int = 1,
                          seq_start: Optional[torch.Tensor] = None) -> None:
    """The general attention in bfloat16 on tensor cores.  qblocks: None (one token per sequence, block i is row i)
    or (seq, first row, tokens) int32 tensors with tokens <= row_groups * tokens_per_block, where
    tokens_per_block = 16 // min(group, 16) tokens make one group of 16 rows and row_groups is 1 or
    attention_general_mma_row_groups(v_dim) (a CTA then takes that many groups through every tile of keys).  The keys
    of a sequence are cut into n_splits ranges of `chunk` keys (a multiple of 64).  With more than one range or
    more than one map the items' results go through scratch: part_o float32 [tokens*heads*maps*n_splits*v_dim],
    part_ml float32 [tokens*heads*maps*n_splits*2].  seq_start (int32, the first row of every sequence of the step):
    k_cache and v_cache are then plain matrices [rows, heads * size] that hold sequence s's keys and values by
    position from row seq_start[s] on, with 64 readable rows beyond the last sequence's; no block table."""
    p = _general_params(shape, q, k_cache, v_cache, token_pos, token_seq, block_table, out, page_tokens, seq_start)
    if qblocks is None:
        p.n_qblocks = q.shape[0]
    else:
        qs, qt, qn = qblocks
        p.qb_seq, p.qb_tok0, p.qb_ntok, p.n_qblocks = qs.data_ptr(), qt.data_ptr(), qn.data_ptr(), qs.numel()
    p.tokens_per_block, p.n_splits, p.chunk, p.reserved = tokens_per_block, n_splits, chunk, row_groups
    through_scratch = n_splits > 1 or shape.maps > 1
    if through_scratch:
        need = q.shape[0] * shape.n_heads * shape.maps * n_splits
        _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < need * shape.v_dim or part_ml.numel() < need * 2:
            raise KernelError("attention_general_mma: scratch too small")
        p.part_o, p.part_ml = part_o.data_ptr(), part_ml.data_ptr()
    f = _fn("attention_general_mma", "stratum_attention_general_mma", [c_void_p, c_void_p])
    _check(f(ctypes.addressof(p), _stream()), "attention_general_mma")
    if through_scratch:
        count_launches(1)          # the finishing kernel


# ------------------------------------------------------------------ norms behind a sublayer
def norm_into_residual(y: torch.Tensor, gain: torch.Tensor, eps: float, x: torch.Tensor, accumulate: bool = True,
                       copy: Optional[torch.Tensor] = None) -> None:
    """x[r] (+)= y[r] / sqrt(mean(y[r]^2) + eps) * gain, all float32 [rows, H]; y may be x when nothing is
    accumulated.  copy (bfloat16 [rows, H]): the new rows of x, rounded, for the products that read them."""
    _need(y, "y", torch.float32); _need(x, "x", torch.float32); _need(gain, "gain", torch.float32)
    if y.shape != x.shape or gain.numel() != x.shape[-1]:
        raise KernelError("norm_into_residual: y, x and gain disagree")
    if copy is not None:
        _need(copy, "copy", torch.bfloat16)
        if copy.shape != x.shape:
            raise KernelError("norm_into_residual: copy and x disagree")
    f = _fn("sublayer_norm", "stratum_norm_into_residual",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(gain), _ptr(x), _ptr(copy), x.shape[0], x.shape[1], c_float(eps), int(bool(accumulate)),
             _stream()), "norm_into_residual")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = bfloat16(x); both contiguous and of one shape."""
    _need(x, "x", torch.float32); _need(out, "out", torch.bfloat16)
    if x.shape != out.shape:
        raise KernelError("cast_rows: x and out disagree")
    f = _fn("sublayer_norm", "stratum_cast_rows", [c_void_p, c_void_p, ctypes.c_longlong, c_void_p])
    _check(f(_ptr(x), _ptr(out), x.numel(), _stream()), "cast_rows")


# ------------------------------------------------------------------ layer norm (weight, no bias)
def layernorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = (v - mean v) / sqrt(var v + eps) * gain with v = x[rows[r]] or x[r].  x float32 [*, H], gain float32
    [H], out [rows, H] float32 or bfloat16."""
    _need(x, "x", torch.float32); _need(gain, "gain", torch.float32); _need(out, "out")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() != n_rows:
            raise KernelError("layernorm: rows and out disagree")
    elif x.shape[0] != n_rows:
        raise KernelError("layernorm: x and out disagree")
    if gain.numel() != x.shape[-1] or out.shape[-1] != x.shape[-1]:
        raise KernelError("layernorm: gain, x and out disagree")
    f = _fn("layer_norm", "stratum_layernorm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), _ptr(gain), _ptr(rows), _ptr(out), dtype_code(out.dtype), n_rows, x.shape[-1], c_float(eps),
             _stream()), "layernorm")


def layernorm_into_residual(y: torch.Tensor, gain: torch.Tensor, eps: float, x: torch.Tensor,
                            accumulate: bool = True, next_gain: Optional[torch.Tensor] = None,
                            next_eps: float = 0.0, next_out: Optional[torch.Tensor] = None) -> None:
    """x[r] (+)= layer norm of y[r] times gain, float32 [rows, H] both; with next_out [rows, H] (float32 or
    bfloat16) also next_out[r] = layer norm of the new x[r] times next_gain: the norm in front of the next sublayer."""
    _need(y, "y", torch.float32); _need(x, "x", torch.float32); _need(gain, "gain", torch.float32)
    if y.shape != x.shape or gain.numel() != x.shape[-1]:
        raise KernelError("layernorm_into_residual: y, x and gain disagree")
    code = 0
    if next_out is not None:
        _need(next_out, "next_out"); _need(next_gain, "next_gain", torch.float32)
        if next_out.shape != x.shape or next_gain.numel() != x.shape[-1]:
            raise KernelError("layernorm_into_residual: next_out, next_gain and x disagree")
        code = dtype_code(next_out.dtype)
    f = _fn("layer_norm", "stratum_layernorm_into_residual",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(gain), _ptr(x), _ptr(next_gain if next_out is not None else None), _ptr(next_out), code,
             x.shape[0], x.shape[1], c_float(eps), c_float(next_eps), int(bool(accumulate)), _stream()),
           "layernorm_into_residual")


def pack_columns(x: torch.Tensor, out: torch.Tensor, col0: int) -> None:
    """out[:, col0 : col0 + W] = x, rounded to out's dtype.  x float32 [rows, W] contiguous; out [rows, >= col0 + W]."""
    _need(x, "x", torch.float32); _need(out, "out", contiguous=False)
    if out.shape[0] != x.shape[0] or out.stride(1) != 1 or col0 < 0 or col0 + x.shape[1] > out.shape[1]:
        raise KernelError("pack_columns: shapes disagree")
    f = _fn("layer_norm", "stratum_pack_columns", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(out), dtype_code(out.dtype), x.shape[0], x.shape[1], out.stride(0), col0, _stream()),
           "pack_columns")


class _QKNormRope(ctypes.Structure):
    """Mirror of struct QKNormRope in csrc/qk_norm_rope.cu."""
    _fields_ = [("proj", c_void_p), ("token_pos", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("q_gain", c_void_p), ("k_gain", c_void_p), ("inv_freq", c_void_p), ("q_out", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("ld", c_int), ("ldq", c_int), ("bt_stride", c_int), ("n_tokens", c_int),
                ("n_heads", c_int), ("n_kv", c_int), ("dim", c_int), ("rot_pairs", c_int),
                ("page_tokens", c_int), ("write_cache", c_int), ("eps", c_float), ("magnitude", c_float),
                ("v_dim", c_int), ("per_head", c_int), ("half", c_int), ("reserved", c_int)]


def qk_norm_rope(proj: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                 q_gain: torch.Tensor, k_gain: torch.Tensor, inv_freq: Optional[torch.Tensor], eps: float,
                 q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv: int,
                 dim: int, page_tokens: int, write_cache: bool, v_dim: int = 0, per_head: bool = False,
                 half: bool = False, magnitude: float = 1.0) -> None:
    """proj float32 [tokens, >= (n_heads + n_kv) * dim + n_kv * v_dim] holds queries, keys and (v_dim > 0) values as
    projected.  v_dim = 0: the key columns go, as they are, to v_cache; else the value columns do (v_cache [pages,
    n_kv, page_tokens, v_dim]).  Queries and keys are divided by a root mean square (eps inside the root) and
    multiplied by a gain: of their whole stretch with a gain per column, or (per_head) of each head with one gain of
    `dim` values for all heads; the first 2 * len(inv_freq) dimensions of every head are rotated by position *
    inv_freq[i], pairs (2i, 2i + 1) or (half) (i, i + len(inv_freq)), cos and sin times `magnitude`; queries go to
    q_out [tokens, >= n_heads * dim], keys to k_cache [pages, n_kv, page_tokens, dim] (of q_out's dtype)."""
    _need(proj, "proj", torch.float32, contiguous=False); _need(token_pos, "token_pos", torch.int32)
    _need(token_seq, "token_seq", torch.int32); _need(q_gain, "q_gain", torch.float32)
    _need(k_gain, "k_gain", torch.float32); _need(q_out, "q_out", contiguous=False)
    if per_head:
        if q_gain.numel() != dim or k_gain.numel() != dim:
            raise KernelError("qk_norm_rope: one gain per dimension of a head")
    elif q_gain.numel() != n_heads * dim or k_gain.numel() != n_kv * dim:
        raise KernelError("qk_norm_rope: one gain per projected column")
    p = _QKNormRope()
    p.proj, p.token_pos, p.token_seq = proj.data_ptr(), token_pos.data_ptr(), token_seq.data_ptr()
    p.q_gain, p.k_gain, p.q_out = q_gain.data_ptr(), k_gain.data_ptr(), q_out.data_ptr()
    if inv_freq is not None and inv_freq.numel():
        _need(inv_freq, "inv_freq", torch.float32)
        p.inv_freq, p.rot_pairs = inv_freq.data_ptr(), inv_freq.numel()
    p.ld, p.ldq, p.n_tokens = proj.stride(0), q_out.stride(0), proj.shape[0]
    p.n_heads, p.n_kv, p.dim, p.page_tokens, p.eps = n_heads, n_kv, dim, page_tokens, float(eps)
    p.v_dim, p.per_head, p.half, p.magnitude = int(v_dim), int(bool(per_head)), int(bool(half)), float(magnitude)
    p.write_cache = int(bool(write_cache))
    if write_cache:
        _need(block_table, "block_table", torch.int32, contiguous=False)
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype)
        if k_cache.shape[-1] != dim or v_cache.shape[-1] != (v_dim or dim):
            raise KernelError("qk_norm_rope: the caches' rows and the head sizes disagree")
        p.block_table, p.bt_stride = block_table.data_ptr(), block_table.stride(0)
        p.k_cache, p.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    f = _fn("qk_norm_rope", "stratum_qk_norm_rope", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(q_out.dtype), _stream()), "qk_norm_rope")


# ------------------------------------------------------------------ the gated delta rule
class _DeltaRule(ctypes.Structure):
    """Mirror of struct DeltaRule in csrc/delta_rule.cu."""
    _fields_ = [("proj", c_void_p), ("conv_w", c_void_p), ("a_log", c_void_p), ("dt_bias", c_void_p),
                ("gain", c_void_p), ("act", c_void_p), ("o_raw", c_void_p), ("out", c_void_p), ("state", c_void_p),
                ("token_pos", c_void_p), ("token_seq", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p),
                ("ld", c_int), ("lda", c_int), ("ldo", c_int), ("n_tokens", c_int), ("n_seqs", c_int),
                ("n_heads", c_int), ("n_kv", c_int), ("dim", c_int), ("vdim", c_int), ("taps", c_int),
                ("state_stride", c_int), ("write_state", c_int), ("eps", c_float), ("reserved", c_float)]


def delta_rule(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               gain: torch.Tensor, act: torch.Tensor, o_raw: torch.Tensor, out: torch.Tensor, state: torch.Tensor,
               token_pos: torch.Tensor, token_seq: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor,
               n_heads: int, n_kv: int, dim: int, vdim: int, eps: float, write_state: bool) -> None:
    """One step of the gated delta rule for every sequence of the step (see csrc/delta_rule.cu).  proj float32
    [tokens, >= C + 2 n_heads + n_heads vdim] with C = 2 n_kv dim + n_heads vdim conv channels; conv_w float32
    [C, taps]; act [tokens, >= C + 2 n_heads + n_kv] and o_raw [tokens, n_heads vdim] float32 scratch; out [tokens, >=
    n_heads vdim] in the compute dtype; state float32 [slots, n_heads dim vdim + (taps - 1) C]."""
    for name, t in (("proj", proj), ("act", act)):
        _need(t, name, torch.float32, contiguous=False)
    for name, t in (("conv_w", conv_w), ("a_log", a_log), ("dt_bias", dt_bias), ("gain", gain), ("o_raw", o_raw),
                    ("state", state)):
        _need(t, name, torch.float32)
    for name, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_start", seq_start),
                    ("seq_slot", seq_slot)):
        _need(t, name, torch.int32)
    _need(out, "out", contiguous=False)
    C = 2 * n_kv * dim + n_heads * vdim
    if conv_w.shape[0] != C or gain.numel() != vdim or a_log.numel() != n_heads or dt_bias.numel() != n_heads:
        raise KernelError("delta_rule: weights and sizes disagree")
    if o_raw.numel() < proj.shape[0] * n_heads * vdim or out.shape[0] != proj.shape[0]:
        raise KernelError("delta_rule: buffers and tokens disagree")
    p = _DeltaRule()
    p.proj, p.conv_w, p.a_log, p.dt_bias, p.gain = (proj.data_ptr(), conv_w.data_ptr(), a_log.data_ptr(),
                                                    dt_bias.data_ptr(), gain.data_ptr())
    p.act, p.o_raw, p.out, p.state = act.data_ptr(), o_raw.data_ptr(), out.data_ptr(), state.data_ptr()
    p.token_pos, p.token_seq, p.seq_start, p.seq_slot = (token_pos.data_ptr(), token_seq.data_ptr(),
                                                         seq_start.data_ptr(), seq_slot.data_ptr())
    p.ld, p.lda, p.ldo, p.n_tokens, p.n_seqs = proj.stride(0), act.stride(0), out.stride(0), proj.shape[0], seq_slot.numel()
    p.n_heads, p.n_kv, p.dim, p.vdim, p.taps = n_heads, n_kv, dim, vdim, conv_w.shape[1]
    p.state_stride, p.write_state, p.eps = state.stride(0), int(bool(write_state)), float(eps)
    f = _fn("delta_rule", "stratum_delta_rule", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(out.dtype), _stream()), "delta_rule")
    count_launches(2)


# ------------------------------------------------------------------ the selective state-space mixer
class _SsmScan(ctypes.Structure):
    """Mirror of struct SsmScan in csrc/ssm_scan.cu."""
    _fields_ = [("proj", c_void_p), ("conv_w", c_void_p), ("conv_b", c_void_p), ("a_log", c_void_p),
                ("dt_bias", c_void_p), ("d_skip", c_void_p), ("gain", c_void_p), ("act", c_void_p),
                ("y_raw", c_void_p), ("out", c_void_p), ("state", c_void_p),
                ("token_pos", c_void_p), ("token_seq", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p),
                ("ld", c_int), ("lda", c_int), ("ldo", c_int), ("n_tokens", c_int), ("n_seqs", c_int),
                ("n_heads", c_int), ("vdim", c_int), ("n_state", c_int), ("n_groups", c_int), ("taps", c_int),
                ("norm_groups", c_int), ("state_stride", c_int), ("write_state", c_int), ("eps", c_float)]


def ssm_scan(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, a_log: torch.Tensor,
             dt_bias: torch.Tensor, d_skip: torch.Tensor, gain: torch.Tensor, act: torch.Tensor, y_raw: torch.Tensor,
             out: torch.Tensor, state: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
             seq_start: torch.Tensor, seq_slot: torch.Tensor, n_heads: int, vdim: int, n_state: int, n_groups: int,
             norm_groups: int, eps: float, write_state: bool) -> None:
    """One step of the selective state-space mixer for every sequence of the step (see csrc/ssm_scan.cu).  With inner
    = n_heads vdim and C = inner + 2 n_groups n_state: proj float32 [tokens, >= inner + C + n_heads] ([z | x | B | C |
    dt]); conv_w float32 [C, taps], conv_b [C]; a_log, dt_bias, d_skip [n_heads]; gain [inner]; act [tokens, >= C + 2
    n_heads] and y_raw [tokens, inner] float32 scratch; out [tokens, >= inner] in the compute dtype; state float32
    [slots, inner n_state + (taps - 1) C]."""
    for name, t in (("proj", proj), ("act", act)):
        _need(t, name, torch.float32, contiguous=False)
    for name, t in (("conv_w", conv_w), ("conv_b", conv_b), ("a_log", a_log), ("dt_bias", dt_bias),
                    ("d_skip", d_skip), ("gain", gain), ("y_raw", y_raw), ("state", state)):
        _need(t, name, torch.float32)
    for name, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_start", seq_start),
                    ("seq_slot", seq_slot)):
        _need(t, name, torch.int32)
    _need(out, "out", contiguous=False)
    inner = n_heads * vdim
    C = inner + 2 * n_groups * n_state
    if conv_w.shape[0] != C or conv_b.numel() != C or gain.numel() != inner or a_log.numel() != n_heads \
            or dt_bias.numel() != n_heads or d_skip.numel() != n_heads:
        raise KernelError("ssm_scan: weights and sizes disagree")
    if y_raw.numel() < proj.shape[0] * inner or out.shape[0] != proj.shape[0]:
        raise KernelError("ssm_scan: buffers and tokens disagree")
    p = _SsmScan()
    p.proj, p.conv_w, p.conv_b, p.a_log = proj.data_ptr(), conv_w.data_ptr(), conv_b.data_ptr(), a_log.data_ptr()
    p.dt_bias, p.d_skip, p.gain = dt_bias.data_ptr(), d_skip.data_ptr(), gain.data_ptr()
    p.act, p.y_raw, p.out, p.state = act.data_ptr(), y_raw.data_ptr(), out.data_ptr(), state.data_ptr()
    p.token_pos, p.token_seq, p.seq_start, p.seq_slot = (token_pos.data_ptr(), token_seq.data_ptr(),
                                                         seq_start.data_ptr(), seq_slot.data_ptr())
    p.ld, p.lda, p.ldo, p.n_tokens, p.n_seqs = proj.stride(0), act.stride(0), out.stride(0), proj.shape[0], seq_slot.numel()
    p.n_heads, p.vdim, p.n_state, p.n_groups, p.taps = n_heads, vdim, n_state, n_groups, conv_w.shape[1]
    p.norm_groups, p.state_stride, p.write_state, p.eps = norm_groups, state.stride(0), int(bool(write_state)), float(eps)
    f = _fn("ssm_scan", "stratum_ssm_scan", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(out.dtype), _stream()), "ssm_scan")
    count_launches(2)


# ------------------------------------------------------------------ gated linear attention
class _Gla(ctypes.Structure):
    """Mirror of struct Gla in csrc/gla.cu."""
    _fields_ = [("proj", c_void_p), ("inner", c_void_p), ("reserved_p", c_void_p), ("gain", c_void_p),
                ("alpha", c_void_p), ("o_raw", c_void_p), ("out", c_void_p), ("state", c_void_p),
                ("token_seq", c_void_p), ("seq_start", c_void_p), ("seq_slot", c_void_p),
                ("ld", c_int), ("ldo", c_int), ("n_tokens", c_int), ("n_seqs", c_int),
                ("n_heads", c_int), ("dim", c_int), ("vdim", c_int), ("rank", c_int),
                ("state_stride", c_int), ("write_state", c_int), ("ld_inner", c_int), ("reserved_i", c_int),
                ("eps", c_float), ("inv_tau", c_float), ("q_scale", c_float), ("reserved", c_float)]


class GlaStep:
    """One step of gated linear attention over a fused projection (see csrc/gla.cu): proj float32 [tokens, >= 2 heads
    dim + 2 heads vdim + rank] holds q | k | v | g | the decay's inner projection.  In order: `cast(inner)` leaves the
    inner projection in a matrix of the compute dtype [tokens, >= rank]; the caller's matrix product turns it into z
    float32 [tokens, heads * dim]; `decay(z)` makes the decays of z in place; `recur(...)` runs the recurrence over
    every sequence's state (float32 [slots, >= heads * vdim * dim], S^T) and leaves the read-outs in o_raw float32
    [tokens, heads * vdim]; `finish(...)` norms and gates them into out (compute dtype [tokens, >= heads * vdim])."""

    def __init__(self, proj: torch.Tensor, n_heads: int, dim: int, vdim: int, rank: int, tau: float, q_scale: float,
                 eps: float):
        _need(proj, "proj", torch.float32, contiguous=False)
        p = self.p = _Gla()
        p.proj, p.ld, p.n_tokens = proj.data_ptr(), proj.stride(0), proj.shape[0]
        p.n_heads, p.dim, p.vdim, p.rank = n_heads, dim, vdim, rank
        p.state_stride = n_heads * dim * vdim           # until recur() is told the real one
        p.ldo = n_heads * vdim
        p.eps, p.inv_tau, p.q_scale = float(eps), 1.0 / float(tau), float(q_scale)
        p.n_seqs = 1
        self.T, self.keep = proj.shape[0], [proj]

    def cast(self, inner: torch.Tensor) -> None:
        _need(inner, "inner", contiguous=False)
        if inner.shape[0] != self.T or inner.shape[1] < self.p.rank or inner.stride(1) != 1:
            raise KernelError("gla: the inner projection's matrix and the step disagree")
        self.p.inner, self.p.ld_inner = inner.data_ptr(), inner.stride(0)
        f = _fn("gla", "stratum_gla_cast", [c_void_p, c_int, c_void_p])
        _check(f(ctypes.addressof(self.p), dtype_code(inner.dtype), _stream()), "gla_cast")

    def _run(self, which: int, dtype: torch.dtype, what: str) -> None:
        f = _fn("gla", "stratum_gla", [c_void_p, c_int, c_int, c_void_p])
        _check(f(ctypes.addressof(self.p), which, dtype_code(dtype), _stream()), what)

    def decay(self, z: torch.Tensor) -> None:
        _need(z, "z", torch.float32)
        if z.shape != (self.T, self.p.n_heads * self.p.dim):
            raise KernelError("gla: z and the step disagree")
        self.p.alpha = z.data_ptr()
        self.keep.append(z)
        self._run(0, torch.float32, "gla_decay")

    def recur(self, o_raw: torch.Tensor, state: torch.Tensor, token_seq: torch.Tensor, seq_start: torch.Tensor,
              seq_slot: torch.Tensor, write_state: bool = True) -> None:
        _need(o_raw, "o_raw", torch.float32); _need(state, "state", torch.float32)
        _need(token_seq, "token_seq", torch.int32); _need(seq_start, "seq_start", torch.int32)
        _need(seq_slot, "seq_slot", torch.int32)
        p = self.p
        if o_raw.shape != (self.T, p.n_heads * p.vdim) or state.dim() != 2 or not p.alpha:
            raise KernelError("gla: shapes disagree, or the decays were not made")
        p.o_raw, p.state, p.state_stride = o_raw.data_ptr(), state.data_ptr(), state.stride(0)
        p.token_seq, p.seq_start, p.seq_slot = token_seq.data_ptr(), seq_start.data_ptr(), seq_slot.data_ptr()
        p.n_seqs, p.write_state = seq_slot.numel(), int(bool(write_state))
        self._run(1, torch.float32, "gla_recur")

    def finish(self, gain: torch.Tensor, out: torch.Tensor) -> None:
        _need(gain, "gain", torch.float32); _need(out, "out", contiguous=False)
        p = self.p
        if gain.numel() != p.vdim or out.shape[0] != self.T or out.shape[1] < p.n_heads * p.vdim or not p.o_raw:
            raise KernelError("gla: shapes disagree, or the recurrence has not run")
        p.gain, p.out, p.ldo = gain.data_ptr(), out.data_ptr(), out.stride(0)
        self._run(2, out.dtype, "gla_finish")


# ------------------------------------------------------------------ routed experts
class _MoeRoute(ctypes.Structure):
    """Mirror of struct MoeRoute in csrc/moe_router.cu."""
    _fields_ = [("x", c_void_p), ("w_router", c_void_p), ("correction", c_void_p), ("dense", c_void_p),
                ("chosen", c_void_p), ("weights", c_void_p),
                ("ldx", c_int), ("ldd", c_int), ("n_tokens", c_int), ("width", c_int),
                ("n_experts", c_int), ("top", c_int), ("n_groups", c_int), ("keep", c_int),
                ("scale", c_float), ("reserved", c_float), ("w_gate", c_void_p), ("score", c_int), ("renorm", c_int),
                ("bias", c_void_p)]


def moe_route(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], dense: torch.Tensor,
              chosen: torch.Tensor, weights: torch.Tensor, top: int, n_groups: int, keep: int, scale: float,
              softmax: bool = False, renorm: bool = True, w_gate: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None) -> None:
    """Routing with a choice correction and groups (see csrc/moe_router.cu): scores by sigmoid, or by softmax over all
    experts; the chosen scores divided by their sum (renorm) or left as they are.  x [tokens, width] float32 or
    bfloat16; w_router float32 [experts, width]; correction float32 [experts] or None; dense float32 [tokens, >=
    experts] (weights, zeros for experts not chosen); chosen int32 and weights float32 [tokens, top].  w_gate
    float32 [width]: dense[:, experts] receives sigmoid(x . w_gate), the gate of a shared expert.  bias float32
    [experts]: added to the router's products before they are scored."""
    _need(x, "x", contiguous=False); _need(w_router, "w_router", torch.float32)
    _need(dense, "dense", torch.float32, contiguous=False)
    _need(chosen, "chosen", torch.int32); _need(weights, "weights", torch.float32)
    E = w_router.shape[0]
    if correction is not None:
        _need(correction, "correction", torch.float32)
    if w_router.shape[1] != x.shape[1] or (correction is not None and correction.numel() != E) \
            or chosen.shape != (x.shape[0], top) or weights.shape != (x.shape[0], top) or dense.shape[0] != x.shape[0]:
        raise KernelError("moe_route: shapes disagree")
    p = _MoeRoute()
    p.x, p.w_router, p.correction = x.data_ptr(), w_router.data_ptr(), (0 if correction is None else correction.data_ptr())
    p.score, p.renorm = int(bool(softmax)), int(bool(renorm))
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != E:
            raise KernelError("moe_route: one bias per expert")
        p.bias = bias.data_ptr()
    if w_gate is not None:
        _need(w_gate, "w_gate", torch.float32)
        if w_gate.numel() != x.shape[1] or dense.shape[1] < E + 1:
            raise KernelError("moe_route: the shared gate needs one row of weights and one more column of dense")
        p.w_gate = w_gate.data_ptr()
    p.dense, p.chosen, p.weights = dense.data_ptr(), chosen.data_ptr(), weights.data_ptr()
    p.ldx, p.ldd, p.n_tokens, p.width = x.stride(0), dense.stride(0), x.shape[0], x.shape[1]
    p.n_experts, p.top, p.n_groups, p.keep, p.scale = E, top, n_groups, keep, float(scale)
    f = _fn("moe_router", "stratum_moe_route", [c_void_p, c_int, c_void_p])
    _check(f(ctypes.addressof(p), dtype_code(x.dtype), _stream()), "moe_route")


def scale_column_blocks(a: torch.Tensor, w: torch.Tensor, block: int, n_blocks: int) -> None:
    """In place: a[t, e * block + j] *= w[t, e] for e < n_blocks, j < block; columns beyond stay.  w float32."""
    _need(a, "a", contiguous=False); _need(w, "w", torch.float32, contiguous=False)
    if a.shape[0] != w.shape[0] or a.shape[1] < block * n_blocks or w.shape[1] < n_blocks:
        raise KernelError("scale_column_blocks: shapes disagree")
    f = _fn("moe_router", "stratum_scale_column_blocks",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), dtype_code(a.dtype), a.stride(0), _ptr(w), w.stride(0), a.shape[0], block, n_blocks,
             _stream()), "scale_column_blocks")


def moe_group(chosen: torch.Tensor, n_experts: int):
    """The (token, choice) pairs of chosen [tokens, top] in the order of their experts, within an expert in the order
    of the tokens: (counts int32 [experts], order int32 [pairs]: the pair at every place, where int32 [pairs]: the
    place of every pair), all on the device."""
    _need(chosen, "chosen", torch.int32)
    n = chosen.numel()
    counts = torch.empty(n_experts, dtype=torch.int32, device=chosen.device)
    order = torch.empty(n, dtype=torch.int32, device=chosen.device)
    where = torch.empty(n, dtype=torch.int32, device=chosen.device)
    f = _fn("moe_router", "stratum_moe_group", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(chosen), n, n_experts, _ptr(counts), _ptr(order), _ptr(where), _stream()), "moe_group")
    count_launches(1)
    return counts, order, where


def gather_rows(x: torch.Tensor, order: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[r] = x[order[r] // top]; out contiguous [len(order), width] of x's dtype."""
    _need(x, "x", contiguous=False); _need(order, "order", torch.int32); _need(out, "out", x.dtype)
    if out.shape != (order.numel(), x.shape[1]):
        raise KernelError("gather_rows: shapes disagree")
    f = _fn("moe_router", "stratum_gather_rows",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(order), top, _ptr(out), out.shape[0], x.shape[1],
             _stream()), "gather_rows")


def moe_combine(outs: torch.Tensor, where: torch.Tensor, weights: torch.Tensor, y: torch.Tensor,
                accumulate: bool) -> None:
    """y[t] (+)= sum_k weights[t, k] * outs[where[t * top + k]]; outs float32 [pairs, width], y float32 [tokens, width]."""
    _need(outs, "outs", torch.float32); _need(where, "where", torch.int32); _need(weights, "weights", torch.float32)
    _need(y, "y", torch.float32)
    T, top = weights.shape
    if where.numel() != T * top or outs.shape != (T * top, y.shape[1]) or y.shape[0] != T:
        raise KernelError("moe_combine: shapes disagree")
    f = _fn("moe_router", "stratum_moe_combine",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(outs), _ptr(where), _ptr(weights), _ptr(y), T, top, y.shape[1], int(bool(accumulate)), _stream()),
           "moe_combine")


def attention_mma(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                  token_seq: torch.Tensor, block_table: torch.Tensor, qblocks, tokens_per_block: int,
                  out: torch.Tensor, part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], n_q: int,
                  n_kv: int, head_dim: int, page_tokens: int, window: int, scale: float, n_splits: int,
                  chunk: int) -> None:
    """bfloat16 tensor-core attention over the paged cache.  qblocks: None (one token per sequence, block i is
    sequence i) or (seq, first row, tokens) int32 tensors of equal length.  n_splits > 1 needs scratch:
    part_o float32 [tokens*n_q*n_splits*head_dim], part_ml float32 [tokens*n_q*n_splits*2]."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    n_tokens = qkv.shape[0]
    if qblocks is None:
        qs = qt = qn = None
        n_qb = n_tokens
    else:
        qs, qt, qn = qblocks
        n_qb = qs.numel()
    if n_splits > 1:
        need = n_tokens * n_q * n_splits
        _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
            raise KernelError("attention_mma: scratch too small for the splits")
    f = _fn("attention_mma", "stratum_attention_mma",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), n_qb, tokens_per_block,
             _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), n_tokens, n_q, n_kv, head_dim, page_tokens,
             window, c_float(scale), n_splits, chunk, _stream()), "attention_mma")
    if n_splits > 1:
        count_launches(1)          # the merge kernel


def attention_tile(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                   token_seq: torch.Tensor, block_table: torch.Tensor, qblocks, tokens_per_warp: int,
                   out: torch.Tensor, n_q: int, n_kv: int, head_dim: int, page_tokens: int, window: int,
                   scale: float) -> None:
    """bfloat16 tensor-core attention for prompts: query tiles of 4 * tokens_per_warp tokens share their key
    tiles through shared memory.  qblocks: (seq, first row, tokens) int32 tensors, tokens <= 4 * tokens_per_warp."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    qs, qt, qn = qblocks
    f = _fn("attention_mma", "stratum_attention_tile",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), qs.numel(), tokens_per_warp,
             _ptr(out), out.stride(0), qkv.shape[0], n_q, n_kv, head_dim, page_tokens, window, c_float(scale),
             _stream()), "attention_tile")


def attention_tc(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                 block_table: torch.Tensor, qblocks, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                 page_tokens: int, window: int, scale: float, halves: int = 1) -> None:
    """bfloat16 attention for prompts on tcgen05/TMEM: query tiles of halves * 128 / (n_q / n_kv) tokens (qblocks
    as for attention_tile).  halves 2: a CTA owns 256 query rows whose two halves share every key and value tile.
    head_dim 64 or 128, group size dividing 128, pages of 64 tokens."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    qs, qt, qn = qblocks
    f = _fn("attention_tc", "stratum_attention_tc",
            [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
             c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(token_pos),
             _ptr(block_table), block_table.stride(0), _ptr(qs), _ptr(qt), _ptr(qn), qs.numel(), _ptr(out),
             out.stride(0), qkv.shape[0], n_q, n_kv, head_dim, page_tokens, window, c_float(scale), halves,
             _ptr(status_word()), _stream()), "attention_tc")


_stream_scratch = None


def attention_stream(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_pos: torch.Tensor,
                     token_seq: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_tokens: int, window: int, scale: float, late_trigger: bool = True,
                     whole_pages: bool = False) -> None:
    """bfloat16 attention for decode steps (one new token per sequence, row i of qkv): the pages of all
    sequences are spread evenly over the SMs and streamed by TMA.  head_dim 64 or 128, at most 8 query heads per
    kv head, pages of 64 tokens, at most 1024 sequences.  late_trigger: a CTA that has asked for its last page lets
    the kernels after this one start (they then wait on the SMs for this one to end).  whole_pages (head_dim 64):
    eight warps take whole pages in turn, instead of four warps a quarter of every page."""
    global _stream_scratch
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32, contiguous=False)
    gs = n_q // max(n_kv, 1)
    if _stream_scratch is None or _stream_scratch[0] < gs * (head_dim + 2) or _stream_scratch[1].device != qkv.device:
        lib = build.load("attention_stream")
        lib.stratum_attention_stream_scratch_floats.restype = ctypes.c_longlong
        floats = int(lib.stratum_attention_stream_scratch_floats(max(gs, 8), max(head_dim, 128)))
        _stream_scratch = (max(gs, 8) * (max(head_dim, 128) + 2),
                           torch.empty(floats, dtype=torch.float32, device=qkv.device))
        scratch_regrown()
    f = _fn("attention_stream", "stratum_attention_stream",
            [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(token_pos),
             _ptr(token_seq), _ptr(block_table), block_table.stride(0), _ptr(out), out.stride(0), qkv.shape[0],
             n_q, n_kv, head_dim, page_tokens, window, c_float(scale), int(bool(late_trigger)),
             int(bool(whole_pages)), _ptr(_stream_scratch[1]),
             _ptr(status_word()),
             _stream()), "attention_stream")
    count_launches(1)


# ------------------------------------------------------------------ sampling
ARGMAX_SPLITS = 32
_argmax_scratch = None


def _argmax_scratch_for(rows: int, device):
    """(best values, best ids, counters) for the many-blocks-per-row argmax; the counters start at zero and
    every launch leaves them at zero."""
    global _argmax_scratch
    if _argmax_scratch is None or _argmax_scratch[2].numel() < rows:
        n = max(rows, 64)
        _argmax_scratch = (torch.empty(n * ARGMAX_SPLITS, dtype=torch.float32, device=device),
                           torch.empty(n * ARGMAX_SPLITS, dtype=torch.int32, device=device),
                           torch.zeros(n, dtype=torch.int32, device=device))
        scratch_regrown()
    return _argmax_scratch


def argmax(logits: torch.Tensor, ids: torch.Tensor, values: Optional[torch.Tensor] = None) -> None:
    """ids[r] = index of the largest logit of row r, the lowest index among equals."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(ids, "ids", torch.int32)
    if values is not None:
        _need(values, "values", torch.float32)
    pv, pi, cnt = _argmax_scratch_for(logits.shape[0], logits.device)
    f = _fn("sampling", "stratum_argmax",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(ids), _ptr(values),
             _ptr(pv), _ptr(pi), _ptr(cnt), _stream()), "argmax")


def feed_ids(ids: torch.Tensor, feed: torch.Tensor, prev: torch.Tensor) -> None:
    """ids[i] = prev[feed[i]] where feed[i] >= 0 (int32 tensors on the device): picked ids fed back without the host."""
    _need(ids, "ids", torch.int32); _need(feed, "feed", torch.int32); _need(prev, "prev", torch.int32)
    if feed.numel() != ids.numel():
        raise KernelError("feed_ids: ids and feed disagree")
    f = _fn("sampling", "stratum_feed_ids", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(feed), _ptr(prev), ids.numel(), _stream()), "feed_ids")


SAMPLE_SPLITS, SAMPLE_KEEP = 32, 64
_sample_scratch = None


def _sample_scratch_for(rows: int, device):
    """What the many-blocks-per-row sampling kernel leaves between its two stages (per row: the stretches' best
    logits, ids, sums and last kept keys, their lists of candidates, a counter that starts at zero and is left
    at zero, a mark for the one-block kernel)."""
    global _sample_scratch
    if _sample_scratch is None or _sample_scratch[6].numel() < rows:
        n = max(rows, 64)
        f32, i32 = torch.float32, torch.int32
        _sample_scratch = (torch.empty(n * SAMPLE_SPLITS, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS, dtype=i32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * 8, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS, dtype=i32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * SAMPLE_KEEP, dtype=f32, device=device),
                           torch.empty(n * SAMPLE_SPLITS * SAMPLE_KEEP, dtype=i32, device=device),
                           torch.zeros(n, dtype=i32, device=device),
                           torch.zeros(n, dtype=i32, device=device))
        scratch_regrown()
    return _sample_scratch


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, ids: torch.Tensor, values: Optional[torch.Tensor] = None,
           one_block_per_row: bool = False) -> None:
    """Per row: temperature <= 0 greedy, else a draw by `uniform` from exp((l - max) / T), optionally among the
    top_k largest (0: off, at most 512) cut after the prefix that reaches top_p (1: off).  Rows of 8,192 logits
    or more are cut over 32 blocks each (one_block_per_row: the single-block kernel, for comparison)."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(ids, "ids", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32); _need(uniform, "uniform", torch.float32)
    scratch = (None,) * 8 if one_block_per_row else _sample_scratch_for(logits.shape[0], logits.device)
    f = _fn("sampling", "stratum_sample",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(uniform), _ptr(ids), _ptr(values), *[_ptr(t) for t in scratch], _stream()), "sample")
    if not one_block_per_row and 8192 <= logits.shape[1] <= 262144:
        count_launches(1)                      # the one-block kernel behind, for marked rows
