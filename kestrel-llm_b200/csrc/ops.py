"""Python face of the sm_100a kernel library: one function per exported entry point.

Tensors are torch CUDA tensors used as typed device memory; every function checks dtypes,
shapes and contiguity, then launches on torch's current stream.  There is no CPU fallback and
no other implementation behind these names: if the library cannot be built or loaded, the
first call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build
from . import cdecl as _cdecl

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def library() -> ctypes.CDLL:
    """The loaded kernel library, built on first use."""
    global _lib
    if _lib is None:
        path = _build.build_cuda()
        try:
            # the kernel library calls the host runtime (cache manager), which is found beside it
            ctypes.CDLL(_build.build_host(verbose=False), mode=ctypes.RTLD_GLOBAL)
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _declare(lib)
        _lib = lib
        if os.environ.get("KESTREL_PDL", "1") == "0":      # for A/B measurements only
            set_pdl(False)
    return _lib


def library_path() -> str:
    library()
    return _build.build_cuda(verbose=False)


_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare(lib) -> None:
    """Argument and result types of every exported function, from the package's C header."""
    _cdecl.declare(lib, ("kestrel_", "kprog_", "krunner_"))


launches = 0     # kernels launched through this module since import (graph replays are counted by their runner)


def _check(rc: int) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise KernelError(library().kestrel_last_error().decode("utf-8", "replace"))


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current device's current stream as a raw handle.  Asked for at every launch, so it
    takes torch's two C calls where they exist (a step of a few tokens is bound by the host)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype) and (dims is None or t.dim() == dims):
        return
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got shape {tuple(t.shape)}")


def _code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name}: dtype {t.dtype} is neither float32 nor bfloat16")
    return _DT[t.dtype]


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for all kernels of the library (default on)."""
    fn = library().kestrel_set_pdl
    fn(1 if on else 0)


def device_arch() -> int:
    return library().kestrel_device_arch()


class Partials:
    """A projection's output before its consumer: ``data`` float32 [S, T, N] whose slices sum to
    the result, plus an optional float32 bias [N] still to be added."""

    __slots__ = ("data", "bias")

    def __init__(self, data: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if data.dim() == 2:
            data = data.unsqueeze(0)
        _need(data, "partials", torch.float32, 3)
        self.data = data
        self.bias = bias

    @property
    def slices(self) -> int:
        return self.data.shape[0]

    @property
    def tokens(self) -> int:
        return self.data.shape[1]

    @property
    def width(self) -> int:
        return self.data.shape[2]

    @property
    def slice_stride(self) -> int:
        return self.data.stride(0)

    def reduce(self, dtype: torch.dtype) -> torch.Tensor:
        """The summed result [T, N] in ``dtype``, for consumers without a fused form."""
        out = torch.empty((self.tokens, self.width), dtype=dtype, device=self.data.device)
        _check(library().kestrel_reduce_partials(self.data.data_ptr(), self.slices, self.slice_stride,
                                                 _p(self.bias), out.data_ptr(), _code(out, "reduce"),
                                                 self.tokens, self.width, _stream()))
        return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] widened to float32, times ``scale``."""
    _need(table, "embed.table", dims=2)
    _need(ids, "embed.ids", torch.int32, 1)
    _need(out, "embed.out", torch.float32, 2)
    T, d = out.shape
    if ids.shape[0] != T or table.shape[1] != d:
        raise KernelError(f"embed: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
    if scale != 1.0:
        _check(library().kestrel_embed_scaled(table.data_ptr(), _code(table, "embed.table"), ids.data_ptr(), out.data_ptr(), T, d, float(scale),
                                              _stream()))
        return
    _check(library().kestrel_embed(table.data_ptr(), _code(table, "embed.table"), ids.data_ptr(),
                                   out.data_ptr(), T, d, _stream()))


def norm_set_warp_rows(rows: int = 0, with_slices: bool = False) -> None:
    """From how many rows on a norm that only reads the stream takes the kernel with a warp a row
    (0: the default, 1024), and whether a norm that adds slices takes it too (by default it does
    not: the block-a-row kernel is faster there).  For tests of both kernels."""
    library().kestrel_set_norm_warp_rows(int(rows), 1 if with_slices else 0)


def add_rmsnorm(residual: torch.Tensor, delta: Optional[Partials], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """x = residual[t] + delta[t]; residual[t] = x if write_back; out[r] = rmsnorm(x) * weight,
    where t = rows[r] if rows is given, else r."""
    _need(residual, "add_rmsnorm.residual", torch.float32, 2)
    _need(weight, "add_rmsnorm.weight", torch.float32, 1)
    _need(out, "add_rmsnorm.out", dims=2)
    T, d = residual.shape
    R = out.shape[0]
    if weight.shape[0] != d or out.shape[1] != d:
        raise KernelError("add_rmsnorm: widths differ")
    if rows is not None:
        _need(rows, "add_rmsnorm.rows", torch.int32, 1)
        if rows.shape[0] != R:
            raise KernelError("add_rmsnorm: rows and out differ in length")
        write_back = False
    elif R != T:
        raise KernelError("add_rmsnorm: out and residual differ in rows")
    if delta is not None and (delta.tokens != T or delta.width != d):
        raise KernelError(f"add_rmsnorm: delta [{delta.tokens},{delta.width}] against residual [{T},{d}]")
    _check(library().kestrel_add_rmsnorm(
        residual.data_ptr(), _p(delta.data) if delta else None, delta.slices if delta else 0,
        delta.slice_stride if delta else 0, _p(delta.bias) if delta else None, _p(rows),
        weight.data_ptr(), float(eps), out.data_ptr(), _code(out, "add_rmsnorm.out"), R, d,
        1 if (write_back and delta is not None) else 0, _stream()))


def swiglu(gate_up: Partials, out: torch.Tensor) -> None:
    """out[t, i] = silu(g[t, i]) * u[t, i] with g, u the two halves of gate_up's width."""
    _need(out, "swiglu.out", dims=2)
    T, ff = out.shape
    if gate_up.tokens != T or gate_up.width != 2 * ff or gate_up.bias is not None:
        raise KernelError("swiglu: shapes differ, or a bias is pending")
    _check(library().kestrel_swiglu(gate_up.data.data_ptr(), gate_up.slices, gate_up.slice_stride,
                                    out.data_ptr(), _code(out, "swiglu.out"), T, ff, _stream()))


def attn_prepare(qkv: Partials, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                 norm_eps: float, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                 page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor,
                 nq: int, nkv: int, hd: int, write_kv: bool = True, rot_mode: int = 0, rot_scale: float = 1.0) -> None:
    """Bias, per-head RMSNorm, rotation; q to q_out, K and V into their cache pages.  ``rot_mode``
    0 pairs dimension j with j + rotary_dim / 2 (rotate-half), 1 pairs 2j with 2j + 1
    (interleaved); ``rot_scale`` multiplies cos and sin."""
    _need(q_out, "attn_prepare.q_out", dims=2)
    _need(positions, "attn_prepare.positions", torch.int32, 1)
    _need(seq_of_token, "attn_prepare.seq_of_token", torch.int32, 1)
    _need(block_table, "attn_prepare.block_table", torch.int32, 2)
    _need(k_cache, "attn_prepare.k_cache", q_out.dtype)
    _need(v_cache, "attn_prepare.v_cache", q_out.dtype)
    T = q_out.shape[0]
    if qkv.tokens != T or qkv.width != (nq + 2 * nkv) * hd or q_out.shape[1] != nq * hd:
        raise KernelError("attn_prepare: shapes differ")
    if rotary_dim and inv_freq is None:
        raise KernelError("attn_prepare: rotation asked for without frequencies")
    _check(library().kestrel_attn_prepare(
        qkv.data.data_ptr(), qkv.slices, qkv.slice_stride, _p(qkv.bias), _p(q_norm_w), _p(k_norm_w),
        float(norm_eps), _p(inv_freq), int(rotary_dim), int(rot_mode), float(rot_scale), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), k_cache.data_ptr(),
        v_cache.data_ptr(), q_out.data_ptr(), _code(q_out, "attn_prepare.q_out"), T, nq, nkv, hd,
        1 if write_kv else 0, _stream()))


def qkv_prepare_fused(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor],
                      k_norm_w: Optional[torch.Tensor], norm_eps: float, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor, nq: int, nkv: int, hd: int,
                      write_kv: bool = True, rot_mode: int = 0, rot_scale: float = 1.0) -> bool:
    """The q, k, v product of x [T, K] with w [(nq + 2 nkv) hd, K] and all of ``attn_prepare`` in
    one tcgen05 kernel.  False, and nothing launched, where that kernel does not take the case
    (float32, few tokens, a head size or rotation other than 128 / rotate-half over the whole
    head): the caller then runs the product and ``attn_prepare``."""
    if x.dtype != torch.bfloat16 or inv_freq is None or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    _need(x, "qkv_prepare.x", torch.bfloat16, 2)
    _need(w, "qkv_prepare.w", torch.bfloat16, 2)
    _need(q_out, "qkv_prepare.q_out", torch.bfloat16, 2)
    _need(positions, "qkv_prepare.positions", torch.int32, 1)
    _need(seq_of_token, "qkv_prepare.seq_of_token", torch.int32, 1)
    _need(block_table, "qkv_prepare.block_table", torch.int32, 2)
    _need(k_cache, "qkv_prepare.k_cache", torch.bfloat16)
    _need(v_cache, "qkv_prepare.v_cache", torch.bfloat16)
    T, K = x.shape
    if w.shape != ((nq + 2 * nkv) * hd, K) or q_out.shape != (T, nq * hd) or not q_out.is_contiguous():
        raise KernelError("qkv_prepare: shapes differ")
    rc = library().kestrel_gemm_tc_qkv_prepare(
        x.data_ptr(), w.data_ptr(), T, K, x.stride(0), w.stride(0), _p(bias), _p(q_norm_w), _p(k_norm_w), float(norm_eps),
        _p(inv_freq), int(rotary_dim), int(rot_mode), float(rot_scale), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), k_cache.data_ptr(), v_cache.data_ptr(),
        q_out.data_ptr(), nq, nkv, hd, 1 if write_kv else 0, _stream())
    if rc == 1:
        return False
    _check(rc)
    return True


def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, n] = sum_k x[t, k] w[n, k] on the CUDA cores, float32 accumulation in ascending k."""
    _need(x, "gemm.x", dims=2)
    _need(w, "gemm.w", x.dtype, 2)
    _need(out, "gemm.out", torch.float32, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(library().kestrel_gemm_plain(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(x, "gemm.x"),
                                        T, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()))


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                    page_size: int, out: torch.Tensor, nq: int, nkv: int, hd: int, window: int,
                    scale: float) -> None:
    _need(q, "attention.q", dims=2)
    _need(out, "attention.out", q.dtype, 2)
    _need(k_cache, "attention.k_cache", q.dtype)
    _need(v_cache, "attention.v_cache", q.dtype)
    _need(block_table, "attention.block_table", torch.int32, 2)
    T = q.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape:
        raise KernelError("attention: shapes differ")
    _check(library().kestrel_attention_plain(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
        seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(page_size),
        out.data_ptr(), _code(q, "attention.q"), T, nq, nkv, hd, int(window), float(scale), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r]."""
    _need(logits, "argmax.logits", torch.float32, 2)
    _need(out, "argmax.out", torch.int32, 1)
    R, V = logits.shape
    lib = library()
    chunks = lib.kestrel_argmax_chunks(V)
    cand_v = cand_i = None
    if chunks > 1:              # a large vocabulary is scanned by many blocks; their candidates go to scratch
        cand_v = torch.empty((R, chunks), dtype=torch.float32, device=logits.device)
        cand_i = torch.empty((R, chunks), dtype=torch.int32, device=logits.device)
    _check(lib.kestrel_argmax(logits.data_ptr(), logits.stride(0), R, V, out.data_ptr(), _p(cand_v), _p(cand_i),
                              _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row; per-row options; rows with temperature <= 0 take the first maximum."""
    _need(logits, "sample.logits", torch.float32, 2)
    R, V = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (uniform, "uniform", torch.float32), (out, "out", torch.int32)):
        _need(t, f"sample.{name}", dt, 1)
        if t.shape[0] != R:
            raise KernelError(f"sample.{name}: {t.shape[0]} entries for {R} rows")
    _check(library().kestrel_sample(logits.data_ptr(), logits.stride(0), R, V, temperature.data_ptr(),
                                    top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                                    uniform.data_ptr(), out.data_ptr(), _stream()))


def repetition_penalty(logits: torch.Tensor, history: torch.Tensor, counts: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for each of the first counts[r] tokens of history[r] (int32 [R, width], a request's
    last generated tokens), logits[r, token] becomes l / penalty[r] if l >= 0, else l * penalty[r] -
    once per occurrence; rows with penalty <= 1 are left alone."""
    _need(logits, "repetition_penalty.logits", torch.float32, 2)
    _need(history, "repetition_penalty.history", torch.int32, 2)
    _need(counts, "repetition_penalty.counts", torch.int32, 1)
    _need(penalty, "repetition_penalty.penalty", torch.float32, 1)
    R, V = logits.shape
    if history.shape[0] != R or counts.shape[0] != R or penalty.shape[0] != R:
        raise KernelError("repetition_penalty: one row of history, one count and one penalty per row of logits")
    fn = library().kestrel_repetition_penalty
    _check(fn(logits.data_ptr(), logits.stride(0), R, V, history.data_ptr(), history.shape[1], counts.data_ptr(),
              penalty.data_ptr(), _stream()))


def sample_set_cluster(on: bool = True) -> None:
    """Whether `sample` may take the kernel that keeps a row in the shared memory of a cluster
    (the default); off: always the one-block kernel over global memory.  For tests of the latter."""
    fn = library().kestrel_sample_set_cluster
    fn(1 if on else 0)


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, K and both row strides
    multiples of 8 elements, bases 16-byte aligned (the TMA rules)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    return bool(library().kestrel_gemm_tc_supported(x.data_ptr(), w.data_ptr(), x.shape[0], w.shape[0], x.shape[1],
                                                    x.stride(0), w.stride(0)))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
            splits: Optional[int] = None, weights_static: bool = False) -> torch.Tensor:
    """y = x w^T on the tensor cores (tcgen05, TMA, TMEM) as float32 slices [S, T, N].
    ``weights_static``: w was complete before the kernel that precedes this call in the stream
    began (a model's weights, never something the step itself computes); few-token products then
    fetch their first weight tiles while that kernel still runs."""
    _need(x, "gemm_tc.x", torch.bfloat16, 2)
    _need(w, "gemm_tc.w", torch.bfloat16, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)}")
    lib = library()
    if out is not None:
        if out.dim() == 2:
            out = out.unsqueeze(0)
        _need(out, "gemm_tc.out", torch.float32, 3)
        if out.shape[1:] != (T, N):
            raise KernelError(f"gemm_tc: out {tuple(out.shape)} for T={T}, N={N}")
        S = out.shape[0]
    else:
        S = splits if splits is not None else lib.kestrel_gemm_tc_splits(T, N, K)
        out = torch.empty((S, T, N), dtype=torch.float32, device=x.device)
    _check(lib.kestrel_gemm_tc_w(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, x.stride(0), w.stride(0),
                                 out.stride(1), S, out.stride(0), 1 if weights_static else 0, _stream()))
    return out


def gemm_tc_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, weights_static: bool = False) -> None:
    """out = silu(x Wg^T) * (x Wu^T) in one tcgen05 kernel with two accumulators."""
    _need(x, "gemm_tc_swiglu.x", torch.bfloat16, 2)
    _need(w_gate_up, "gemm_tc_swiglu.w", torch.bfloat16, 2)
    _need(out, "gemm_tc_swiglu.out", torch.bfloat16, 2)
    T, K = x.shape
    ff = out.shape[1]
    if w_gate_up.shape != (2 * ff, K) or out.shape[0] != T:
        raise KernelError("gemm_tc_swiglu: shapes differ")
    _check(library().kestrel_gemm_tc_swiglu_w(x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), T, ff, K,
                                              x.stride(0), w_gate_up.stride(0), out.stride(0),
                                              1 if weights_static else 0, _stream()))


def gemm_tc_set_tuning(overhead_kb: int = -1, ctas_per_sm: int = 0) -> None:
    """Tuning of the split heuristic of few-token products (see gemm_tcgen05.cu)."""
    fn = library().kestrel_gemm_tc_set_tuning
    fn(int(overhead_kb), int(ctas_per_sm))


def gemm_tc_set_wide(on: bool = True, more_than_tokens: int = -1) -> None:
    """Whether products of more than ``more_than_tokens`` (32) and at most 128 tokens take two
    weight tiles a CTA (the default).  For tests and measurements of the one-tile kernel."""
    fn = library().kestrel_gemm_tc_set_wide
    fn(1 if on else 0, int(more_than_tokens))


def gemm_tc_set_pair_tuning(min_tokens: int = -1, overhead_kb: int = -1) -> None:
    """Tuning of many-token products on CTA pairs: products of more than ``min_tokens`` tokens
    take them; a K slice is priced at ``overhead_kb`` k-blocks beyond its own (see gemm_tcgen05.cu)."""
    fn = library().kestrel_gemm_tc_set_pair_tuning
    fn(int(min_tokens), int(overhead_kb))


def gemm_tc_set_many_token_path(pairs: bool = True, persistent: bool = True, swiglu_tile: int = 256,
                                swiglu_swapped: Optional[bool] = None) -> None:
    """Which kernel a many-token product (more than 128 tokens) takes: CTA pairs (the default),
    else one persistent CTA per SM (what runs where pairs cannot be scheduled; ``swiglu_tile``
    128 or 256 tokens for its SwiGLU form), else one tile per CTA.  ``swiglu_swapped``: the
    SwiGLU product on pairs takes the tokens as the M operand always (True), never (False), or
    where its finer tiles save a round of tiles (None, the default).  For tests of every path."""
    lib = library()
    for name, v in (("kestrel_gemm_tc_set_pairs", 1 if pairs else 0), ("kestrel_gemm_tc_set_persistent", 1 if persistent else 0),
                    ("kestrel_gemm_tc_set_swiglu_tile", int(swiglu_tile)), ("kestrel_gemm_tc_set_swiglu_swapped", 1 if swiglu_swapped is None else (2 if swiglu_swapped else 0))):
        fn = getattr(lib, name)
        fn(v)


def gemm_tc_set_qkv_fused(on: Optional[bool] = None) -> None:
    """Whether a q, k, v product of many tokens does ``attn_prepare``'s work in its epilogue: where
    the product would not be cut along K (None, the default), wherever the kernel takes the
    sizes (True), never (False).  For tests of both paths."""
    library().kestrel_gemm_tc_set_qkv_fused(1 if on is None else (2 if on else 0))


def gemm_tc_error() -> int:
    """Error word of the tcgen05 kernels' bounded waits (0 = none); synchronises the device."""
    return library().kestrel_gemm_tc_error()


def linear(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
           weights_static: bool = False) -> torch.Tensor:
    """y = x w^T as float32 slices [S, T, N] (S = 1 unless a split-K kernel ran).
    ``weights_static`` as in `gemm_tc`.

    float32 operands always take the CUDA-core product; bfloat16 operands take the tcgen05
    product when its tiling rules hold (see `gemm_tc_supported`) and the CUDA-core one
    otherwise."""
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2:
        # one question to the library: do the operands fit, and into how many K slices
        plan = library().kestrel_gemm_tc_plan(x.data_ptr(), w.data_ptr(), T, N, x.shape[1], x.stride(0), w.stride(0))
        if plan > 0:
            return gemm_tc(x, w, out, splits=plan if out is None else None, weights_static=weights_static)
    if out is None:
        out = torch.empty((1, T, N), dtype=torch.float32, device=x.device)
    elif out.dim() == 2:
        out = out.unsqueeze(0)
    gemm_plain(x, w, out[0])
    return out


def linear_add_into(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual += x w^T inside the product's epilogue, where the product can do that (bfloat16,
    many tokens, one pass over K); False if it cannot - nothing has run then and the caller takes
    the product as slices."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    _need(x, "linear_add_into.x", torch.bfloat16, 2)
    _need(w, "linear_add_into.w", torch.bfloat16, 2)
    _need(residual, "linear_add_into.residual", torch.float32, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or residual.shape != (T, N):
        raise KernelError(f"linear_add_into: x {tuple(x.shape)}, w {tuple(w.shape)}, residual {tuple(residual.shape)}")
    rc = library().kestrel_gemm_tc_add(x.data_ptr(), w.data_ptr(), residual.data_ptr(), T, N, K, x.stride(0), w.stride(0),
                                       residual.stride(0), _stream())
    if rc == 1:
        return False
    _check(rc)
    return True


def linear_act(x: torch.Tensor, w: torch.Tensor, act: str, weights_static: bool = False) -> torch.Tensor:
    """act(x w^T) in x's dtype, ``act`` one of `COLUMN_ACTS`.  bfloat16 with many tokens: the activation is the
    product's epilogue and the float32 product never reaches memory; otherwise the product comes as slices and
    `partial_columns_act` sums and activates them.  Both ways give the same bits where the product is one slice."""
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and linear_act_fused:
        out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        rc = library().kestrel_gemm_tc_act(x.data_ptr(), w.data_ptr(), out.data_ptr(), COLUMN_ACTS[act], T, N, x.shape[1], x.stride(0),
                                           w.stride(0), out.stride(0), _stream())
        if rc != 1:
            _check(rc)
            return out
    return partial_columns_act(Partials(linear(x, w, weights_static=weights_static)), 0, N, x.dtype, act)


linear_act_fused = True          # tests switch the epilogue form off to hold both forms against each other


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, ff: int, weights_static: bool = False) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in x's dtype, Wg and Wu being the two halves of w_gate_up's rows.
    ``weights_static`` as in `gemm_tc`."""
    out = torch.empty((x.shape[0], ff), dtype=x.dtype, device=x.device)
    if gemm_tc_supported(x, w_gate_up):
        # the activation is the product's epilogue: the K range is not split, whatever the number of
        # tokens, and the gate/up product never reaches memory
        gemm_tc_swiglu(x, w_gate_up, out, weights_static=weights_static)
    else:
        swiglu(Partials(linear(x, w_gate_up, weights_static=weights_static)), out)
    return out


def attention_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                  tile_seq: torch.Tensor, tile_row0: torch.Tensor, rows_per_tile: int, cu_seqlens: torch.Tensor,
                  kv_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int,
                  window: int, scale: float, slices: int = 1, slice_len: int = 1 << 30,
                  max_kv_dev: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention (mma.sync) of the tiles listed in tile_seq / tile_row0; rows of
    other requests in ``out`` are left alone.  With ``slices`` > 1 the key range is cut into
    slices of ``slice_len`` keys (a multiple of 64) that are merged in ascending order;
    ``slices * slice_len`` must reach the longest request, keys beyond it are not seen."""
    _need(q, "attention_mma.q", torch.bfloat16, 2)
    _need(out, "attention_mma.out", torch.bfloat16, 2)
    _need(k_cache, "attention_mma.k_cache", torch.bfloat16)
    _need(v_cache, "attention_mma.v_cache", torch.bfloat16)
    _need(block_table, "attention_mma.block_table", torch.int32, 2)
    _need(tile_seq, "attention_mma.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_mma.tile_row0", torch.int32, 1)
    T = q.shape[0]
    tiles = tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_mma: shapes differ")
    part_o = part_ml = None
    if slices > 1:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), 1 << 30)
    _check(library().kestrel_attention_mma(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, rows_per_tile, cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), T, nq, nkv, hd, int(window), int(slices),
        slice_len, _p(max_kv_dev), float(scale), _stream()))
    if slices > 1:
        global launches
        launches += 1          # the merge kernel


def attention_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                 tile_seq: torch.Tensor, tile_row0: torch.Tensor, cu_seqlens: torch.Tensor, kv_lens: torch.Tensor,
                 block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int, window: int, scale: float,
                 slices: int = 1, slice_len: int = 1 << 30, max_kv_dev: Optional[torch.Tensor] = None,
                 rows_per_tile: int = 128, score: Optional["ScoreOptions"] = None) -> None:
    """tcgen05 attention of the listed tiles, head size 128 (with a layer's `ScoreOptions`; sigmoid weights in one slice): tiles of ``rows_per_tile`` rows, up
    to 256 (prompt portions; 16 for decode tokens); the key range may be cut into
    ``slices`` slices of ``slice_len`` keys (a multiple of 128) that are merged in ascending
    order; ``slices * slice_len`` must reach the longest request.  The cache tensors are
    [pages, kv heads, page size, 128], contiguous, with a page size the kernel's page-wise TMA
    boxes fit (``attention_tc_supported``)."""
    _need(q, "attention_tc.q", torch.bfloat16, 2)
    _need(out, "attention_tc.out", torch.bfloat16, 2)
    _need(k_cache, "attention_tc.k_cache", torch.bfloat16)
    _need(v_cache, "attention_tc.v_cache", torch.bfloat16)
    _need(block_table, "attention_tc.block_table", torch.int32, 2)
    _need(tile_seq, "attention_tc.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_tc.tile_row0", torch.int32, 1)
    T, tiles = q.shape[0], tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_tc: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention_tc: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    part_o = part_ml = None
    if slices > 1:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), (1 << 30) // 128 * 128)
    _check(library().kestrel_attention_tc_biased(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, int(rows_per_tile), cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], block_table.stride(0), int(page_size), int(k_cache.shape[0]), T, nq, nkv, hd,
        int(window), int(slices), slice_len, _p(max_kv_dev), float(scale), *(score or ScoreOptions()).args(nq), *(score or ScoreOptions()).rel_args(nq),
        _stream()))
    if slices > 1:
        global launches
        launches += 1          # the merge kernel


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     tile_seq: torch.Tensor, tile_row0: torch.Tensor, cu_seqlens: torch.Tensor, kv_lens: torch.Tensor,
                     block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int, window: int, scale: float,
                     slices: int = 1, slice_len: int = 1 << 30, max_kv_dev: Optional[torch.Tensor] = None) -> None:
    """Attention of decode tokens (tiles of at most 16 rows) with a TMA loader warp in front of
    four mma.sync warps, head size 64 or 128; the key range is cut into ``slices`` slices of
    ``slice_len`` keys (a multiple of 64) that are merged in ascending order (up to 4 inside the
    kernel, by the CTAs of a cluster; more through scratch and a second kernel), and
    ``slices * slice_len`` must reach the longest request.  The cache tensors are
    [pages, kv heads, page size, head size], contiguous (``attention_decode_supported``).  Keys
    and values of positions before a request's first token of this step must have been written
    by earlier steps, not by the kernel in front of this one: they are fetched before it ends."""
    _need(q, "attention_decode.q", torch.bfloat16, 2)
    _need(out, "attention_decode.out", torch.bfloat16, 2)
    _need(k_cache, "attention_decode.k_cache", torch.bfloat16)
    _need(v_cache, "attention_decode.v_cache", torch.bfloat16)
    _need(block_table, "attention_decode.block_table", torch.int32, 2)
    _need(tile_seq, "attention_decode.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_decode.tile_row0", torch.int32, 1)
    T, tiles = q.shape[0], tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_decode: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention_decode: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    part_o = part_ml = None
    scratch = slices > library().kestrel_attention_decode_cluster_slices()    # fewer are merged inside the kernel
    if scratch:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), (1 << 30) // 128 * 128)
    _check(library().kestrel_attention_decode(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], block_table.stride(0), int(page_size), int(k_cache.shape[0]), T,
        nq, nkv, hd, int(window), int(slices), slice_len, _p(max_kv_dev), float(scale), _stream()))
    if scratch:
        global launches
        launches += 1          # the merge kernel


def attention_decode_supported(hd: int, page_size: int) -> bool:
    """Whether the decode attention kernel takes this head size and page size."""
    return bool(library().kestrel_attention_decode_supported(int(hd), int(page_size)))


def attention_decode_error() -> int:
    """Error word of the decode attention kernel's bounded waits (0 = none); synchronises the device."""
    return library().kestrel_attention_decode_error()


def attention_tc_supported(hd: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel takes this head size and page size."""
    return bool(library().kestrel_attention_tc_supported(int(hd), int(page_size)))


def raise_on_kernel_error() -> None:
    """Reads the error words of the kernels with bounded waits (matrix product, the two attention
    kernels) and raises if one of them gave up a wait: its output is not to be trusted.
    Synchronises the device; callers use it where they synchronise anyway."""
    lib = library()
    bad = [(name, code) for name, code in (("gemm_tcgen05", lib.kestrel_gemm_tc_error()),
                                           ("attention_tc", lib.kestrel_attention_tc_error()),
                                           ("attention_decode", lib.kestrel_attention_decode_error()),
                                           ("moe_tcgen05", lib.kestrel_moe_tc_error())) if code]
    if bad:
        raise KernelError("a bounded wait ran out in " + ", ".join(f"{n} (wait {c})" for n, c in bad) +
                          ": the step's results are invalid")


def wait_probe():
    """Runs one block that waits, with the kernels' bounded wait, on a barrier nobody completes.
    Returns (gave_up, milliseconds): the wait must give up within seconds and leave the
    device usable."""
    ms = ctypes.c_float(0.0)
    rc = library().kestrel_wait_probe(ctypes.addressof(ms))
    if rc < 0:
        raise KernelError(library().kestrel_last_error().decode("utf-8", "replace"))
    return rc == 1, float(ms.value)


def attention_tc_error() -> int:
    """Error word of the tcgen05 attention kernel's bounded waits (0 = none); synchronises the device."""
    return library().kestrel_attention_tc_error()


def attention_set_small_portions(per_cent: int = -1) -> None:
    """Short prompt portions (at most 512 rows of (token, head) per kv head) go to the attention
    kernel for decode tokens while their keys stay under limits by row count; ``per_cent`` scales
    those limits (0: never, negative: the default).  For tests of both routes."""
    library().kestrel_attention_set_small_portions(int(per_cent))


class AttentionPlanner:
    """What the attention kernels keep between the layers of a step: the tile lists of the
    step's requests on the device (made once per step from the step's host description) and
    scratch for key-range slices.  One planner serves all attention layers of a model; its
    launches must stay on one stream."""

    def __init__(self, max_tokens: int = 4096, max_seqs: int = 256):
        self._lib = library()
        self._h = self._lib.kestrel_attn_planner_create(int(max_tokens), int(max_seqs))
        if not self._h:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.kestrel_attn_planner_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def attention(planner: Optional[AttentionPlanner], q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch,
              group: int, page_size: int, out: torch.Tensor, nq: int, nkv: int, hd: int, window: int, scale: float) -> None:
    """Causal attention of this step's queries over their requests' cache pages.  ``batch``
    is the step's description: its packed int32 buffer on the host (``host``) and on the device
    (``device_buffer``), the buffer's ``layout``, a ``serial`` that changes with every step, and
    ``captured`` (the launch is being recorded for replay).  Which kernel takes which requests,
    the tiling of their rows and the cutting of key ranges into slices are decided natively
    (csrc/kernels/attention_dispatch.cu); float32 always takes the plain kernel."""
    _need(q, "attention.q", dims=2)
    _need(out, "attention.out", q.dtype, 2)
    _need(k_cache, "attention.k_cache", q.dtype, 4)
    _need(v_cache, "attention.v_cache", q.dtype, 4)
    if q.shape[1] != nq * hd or out.shape != q.shape:
        raise KernelError("attention: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    if q.shape[0] != batch.num_tokens:
        raise KernelError(f"attention: {q.shape[0]} query rows for a step of {batch.num_tokens} tokens")
    lib = library()
    global launches
    rc = lib.kestrel_attention(planner.handle if planner is not None else None, int(batch.serial), batch.host.ctypes.data,
                               batch.device_buffer.data_ptr(), batch.layout.ctypes.data, int(group), 1 if batch.captured else 0,
                               q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _code(q, "attention.q"),
                               int(k_cache.shape[0]), int(page_size), nq, nkv, hd, int(window), float(scale), _stream())
    if rc != 0:
        raise KernelError(lib.kestrel_last_error().decode("utf-8", "replace"))
    launches += lib.kestrel_attn_planner_last_launches(planner.handle) if planner is not None else 1


# ---- kernels around the residual stream for arrangements other than the pre-norm block ---------

def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> None:
    """x[t, 2i] += sin(pos[t] * freq[i]), x[t, 2i + 1] += cos(pos[t] * freq[i]), angles in float32."""
    _need(x, "add_sinusoid.x", torch.float32, 2)
    _need(positions, "add_sinusoid.positions", torch.int32, 1)
    _need(freq, "add_sinusoid.freq", torch.float32, 1)
    T, d = x.shape
    if positions.shape[0] != T or freq.shape[0] < (d + 1) // 2:
        raise KernelError("add_sinusoid: shapes differ")
    _check(library().kestrel_add_sinusoid(x.data_ptr(), positions.data_ptr(), freq.data_ptr(), T, d, _stream()))


def add_two(residual: torch.Tensor, a: Partials, b: Optional[Partials], cast: Optional[torch.Tensor], c: Optional[Partials] = None) -> None:
    """residual += a + b (the sums of their slices, a's first), + c where a third product is given;
    ``cast``, if given, receives the new residual stream in its own dtype."""
    _need(residual, "add_two.residual", torch.float32, 2)
    T, d = residual.shape
    if b is None and c is not None:
        b, c = c, None
    for p in (a, b, c):
        if p is not None and (p.tokens != T or p.width != d or p.bias is not None):
            raise KernelError("add_two: a product does not fit the residual stream, or carries a bias")
    if cast is not None:
        _need(cast, "add_two.cast", dims=2)
        if cast.shape != residual.shape:
            raise KernelError("add_two: cast and residual differ in shape")
    if c is not None:
        _check(library().kestrel_add_three(residual.data_ptr(), a.data.data_ptr(), a.slices, a.slice_stride, b.data.data_ptr(), b.slices,
                                           b.slice_stride, c.data.data_ptr(), c.slices, c.slice_stride, _p(cast),
                                           _code(cast, "add_two.cast") if cast is not None else F32, T, d, _stream()))
        return
    _check(library().kestrel_add_two(residual.data_ptr(), a.data.data_ptr(), a.slices, a.slice_stride,
                                     _p(b.data) if b is not None else None, b.slices if b is not None else 0,
                                     b.slice_stride if b is not None else 0, _p(cast),
                                     _code(cast, "add_two.cast") if cast is not None else F32, T, d, _stream()))


def gelu_table_mul(g: Partials, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = gelu_tanh(g[t, i]) * table[ids[t], col0 + i] for the out.shape[1] columns of g."""
    _need(table, "gelu_table_mul.table", out.dtype, 2)
    _need(out, "gelu_table_mul.out", dims=2)
    _need(ids, "gelu_table_mul.ids", torch.int32, 1)
    T, n = out.shape
    if g.tokens != T or g.width < n or ids.shape[0] != T or col0 < 0 or col0 + n > table.shape[1] or g.bias is not None:
        raise KernelError("gelu_table_mul: shapes differ")
    _check(library().kestrel_gelu_table_mul(g.data.data_ptr(), g.slices, g.slice_stride, g.width, table.data_ptr(), table.stride(0),
                                            int(col0), ids.data_ptr(), out.data_ptr(), _code(out, "gelu_table_mul.out"), T, n, _stream()))


def add_normed(residual: torch.Tensor, p: Partials, weight: torch.Tensor, eps: float) -> None:
    """residual += y / sqrt(mean(y^2) + eps) * weight with y the sum of p's slices."""
    _need(residual, "add_normed.residual", torch.float32, 2)
    _need(weight, "add_normed.weight", torch.float32, 1)
    T, d = residual.shape
    if p.tokens != T or p.width != d or weight.shape[0] != d or p.bias is not None:
        raise KernelError("add_normed: shapes differ")
    _check(library().kestrel_add_normed(residual.data_ptr(), p.data.data_ptr(), p.slices, p.slice_stride, weight.data_ptr(), float(eps),
                                        T, d, _stream()))


def partial_columns(p: Partials, col0: int, n: int, dtype: torch.dtype) -> torch.Tensor:
    """Columns [col0, col0 + n) of a product, summed over its slices, in ``dtype``."""
    out = torch.empty((p.tokens, n), dtype=dtype, device=p.data.device)
    if p.bias is not None:
        raise KernelError("partial_columns: a bias is pending")
    _check(library().kestrel_partial_columns(p.data.data_ptr(), p.slices, p.slice_stride, p.width, int(col0), out.data_ptr(),
                                             _code(out, "partial_columns.out"), p.tokens, int(n), _stream()))
    return out


COLUMN_ACTS = {None: 0, "none": 0, "relu2": 1, "tanh": 2, "silu": 3, "gelu": 4, "gelu_tanh": 5}


def partial_columns_act(p: Partials, col0: int, n: int, dtype: torch.dtype, act: Optional[str]) -> torch.Tensor:
    """act(columns [col0, col0 + n) of a product, summed over its slices, plus its bias) in ``dtype``;
    ``act`` None, "relu2" (the square of relu), "tanh", "silu", "gelu" (the exact one, with erf) or "gelu_tanh"."""
    if act not in COLUMN_ACTS:
        raise KernelError(f"partial_columns_act: activation {act!r} is none of {', '.join(str(k) for k in COLUMN_ACTS)}")
    out = torch.empty((p.tokens, n), dtype=dtype, device=p.data.device)
    if p.bias is not None and p.bias.shape[0] != p.width:
        raise KernelError("partial_columns_act: the bias does not fit the product's columns")
    _check(library().kestrel_partial_columns_act(p.data.data_ptr(), p.slices, p.slice_stride, p.width, int(col0), _p(p.bias), COLUMN_ACTS[act],
                                                 out.data_ptr(), _code(out, "partial_columns_act.out"), p.tokens, int(n), _stream()))
    return out


def combine_normed(a: Partials, wa: torch.Tensor, b: Partials, wb: torch.Tensor, eps: float, mix: float) -> Partials:
    """mix * (rmsnorm(a) * wa + rmsnorm(b) * wb) over the rows of two products, as a product of one slice."""
    _need(wa, "combine_normed.wa", torch.float32, 1)
    _need(wb, "combine_normed.wb", torch.float32, 1)
    T, d = a.tokens, a.width
    if b.tokens != T or b.width != d or wa.shape[0] != d or wb.shape[0] != d or a.bias is not None or b.bias is not None:
        raise KernelError("combine_normed: shapes differ, or a bias is pending")
    out = torch.empty((1, T, d), dtype=torch.float32, device=a.data.device)
    _check(library().kestrel_combine_normed(a.data.data_ptr(), a.slices, a.slice_stride, wa.data_ptr(), b.data.data_ptr(), b.slices, b.slice_stride,
                                            wb.data_ptr(), float(eps), float(mix), out.data_ptr(), T, d, _stream()))
    return Partials(out)


def add_gated_normed(residual: torch.Tensor, y: Partials, gate: Optional[Partials], weight: torch.Tensor, eps: float,
                     next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0, next_out: Optional[torch.Tensor] = None) -> None:
    """residual += rmsnorm(y * sigmoid(gate)) * weight, y and gate the sums of their slices plus their
    biases (no gate: y alone); with ``next_weight`` also next_out = rmsnorm(residual) * next_weight."""
    _need(residual, "add_gated_normed.residual", torch.float32, 2)
    _need(weight, "add_gated_normed.weight", torch.float32, 1)
    T, d = residual.shape
    for p in (y, gate):
        if p is not None and (p.tokens != T or p.width != d or (p.bias is not None and p.bias.shape[0] != d)):
            raise KernelError("add_gated_normed: a product does not fit the residual stream")
    if (next_weight is None) != (next_out is None):
        raise KernelError("add_gated_normed: the next norm needs its weight and its output")
    if next_out is not None:
        _need(next_out, "add_gated_normed.next_out", dims=2)
        _need(next_weight, "add_gated_normed.next_weight", torch.float32, 1)
        if next_out.shape != residual.shape or next_weight.shape[0] != d:
            raise KernelError("add_gated_normed: the next norm's shapes differ")
    if weight.shape[0] != d:
        raise KernelError("add_gated_normed: the weight does not fit the row")
    _check(library().kestrel_add_gated_normed(
        residual.data_ptr(), y.data.data_ptr(), y.slices, y.slice_stride, _p(y.bias), _p(gate.data) if gate is not None else None,
        gate.slices if gate is not None else 0, gate.slice_stride if gate is not None else 0, _p(gate.bias) if gate is not None else None,
        weight.data_ptr(), float(eps), _p(next_weight), float(next_eps), _p(next_out),
        _code(next_out, "add_gated_normed.next_out") if next_out is not None else F32, T, d, _stream()))


def embed_add(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor) -> None:
    """x[t] += table[ids[t]] widened to float32."""
    _need(table, "embed_add.table", dims=2)
    _need(ids, "embed_add.ids", torch.int32, 1)
    _need(x, "embed_add.x", torch.float32, 2)
    if ids.shape[0] != x.shape[0] or table.shape[1] != x.shape[1]:
        raise KernelError("embed_add: shapes differ")
    _check(library().kestrel_embed_add(table.data_ptr(), _code(table, "embed_add.table"), ids.data_ptr(), x.data_ptr(), x.shape[0], x.shape[1],
                                       _stream()))


def gate_columns_mul(x: torch.Tensor, g: Partials, col0: int) -> None:
    """x[t, i] *= sigmoid(columns [col0, col0 + x.shape[1]) of a product, summed over its slices, plus its bias), in place:
    a gate per element of a mixer's output."""
    _need(x, "gate_columns_mul.x", dims=2)
    T, n = x.shape
    if g.tokens != T or col0 < 0 or col0 + n > g.width or (g.bias is not None and g.bias.shape[0] != g.width):
        raise KernelError("gate_columns_mul: shapes differ")
    _check(library().kestrel_gate_columns_mul(x.data_ptr(), _code(x, "gate_columns_mul.x"), g.data.data_ptr(), g.slices, g.slice_stride, g.width,
                                              int(col0), _p(g.bias), T, n, _stream()))


def add_row(x: torch.Tensor, row: torch.Tensor) -> None:
    """x[t] += row for every token: float32 [T, d] and float32 [d]."""
    _need(x, "add_row.x", torch.float32, 2)
    _need(row, "add_row.row", torch.float32, 1)
    if row.shape[0] != x.shape[1]:
        raise KernelError("add_row: the row does not fit the stream")
    _check(library().kestrel_add_row(x.data_ptr(), row.data_ptr(), x.shape[0], x.shape[1], _stream()))


def logit_scale_cap(logits: torch.Tensor, scale: float, cap: float) -> None:
    """In place: logits * scale, then cap * tanh(. / cap) where cap > 0."""
    _need(logits, "logit_scale_cap.logits", torch.float32, 2)
    _check(library().kestrel_logit_scale_cap(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], float(scale), float(cap),
                                             _stream()))


# ---- attention without rotation, values of their own size, kept first tokens, an output gate -----

QK_NORM_MODES = {None: 0, False: 0, "none": 0, True: 1, "head": 1, "projection": 2}


def attn_prepare_ex(qkv: Partials, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], qk_norm, norm_eps: float,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor, gate_out: Optional[torch.Tensor],
                    nq: int, nkv: int, hd: int, vd: int, has_kv: bool, v_norm: bool = False, rotation=None, q_temp=None) -> None:
    """Columns [q | k | v | gate] of a fused product, plus the product's bias where it carries one:
    q and k divided by their root mean square - ``qk_norm`` "head" (or True): per head, times a
    weight [hd] where given; "projection": over all of q's columns at once and all of k's, times
    weights [nq hd] and [nkv hd]; None: left as they are - and v per head if ``v_norm``; q to
    ``q_out``, k and v into the cache pages (absent if ``has_kv`` is False), sigmoid of the gate
    columns to ``gate_out`` float32 [T, nq].  With ``rotation`` (a `Rotation` of parts/base.py: frequencies,
    rotated size, pairing, scale) q and k are turned by position after their norm.  ``q_temp`` = (coef, every): q
    times 1 + coef ln(floor((position + 1) / every) + 1), a temperature that grows with the position."""
    _need(q_out, "attn_prepare_ex.q_out", dims=2)
    _need(block_table, "attn_prepare_ex.block_table", torch.int32, 2)
    _need(k_cache, "attn_prepare_ex.k_cache", q_out.dtype, 4)
    _need(v_cache, "attn_prepare_ex.v_cache", q_out.dtype, 4)
    T = q_out.shape[0]
    if qkv.tokens != T or q_out.shape[1] != nq * hd:
        raise KernelError("attn_prepare_ex: shapes differ")
    if qk_norm not in QK_NORM_MODES:
        raise KernelError(f"attn_prepare_ex: qk_norm {qk_norm!r} is none of None, 'head', 'projection'")
    mode = QK_NORM_MODES[qk_norm]
    if qkv.bias is not None:
        _need(qkv.bias, "attn_prepare_ex.bias", torch.float32, 1)
        if qkv.bias.shape[0] != qkv.width:
            raise KernelError("attn_prepare_ex: the bias does not fit the product's columns")
    if mode == 2:
        for w, n, name in ((q_norm_w, nq * hd, "q"), (k_norm_w, nkv * hd, "k")):
            if (w is None and (name == "q" or has_kv)) or (w is not None and (w.dtype != torch.float32 or w.numel() != n)):
                raise KernelError(f"attn_prepare_ex: the norm over the whole {name} projection needs a float32 weight of {n} entries")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or tuple(v_cache.shape[1:]) != (nkv, page_size, vd):
        raise KernelError("attn_prepare_ex: the cache planes do not fit the heads")
    if gate_out is not None:
        _need(gate_out, "attn_prepare_ex.gate_out", torch.float32, 2)
    inv_freq = rot = rot_mode = None
    if rotation is not None:
        inv_freq, rot, rot_mode = rotation.inv_freq, int(rotation.dim), rotation.mode
        _need(inv_freq, "attn_prepare_ex.inv_freq", torch.float32, 1)
        if rot <= 0 or rot % 2 or rot > hd or inv_freq.shape[0] < rot // 2:
            raise KernelError(f"attn_prepare_ex: {rot} rotated dimensions of a head of {hd} with {inv_freq.shape[0]} frequencies")
    if mode == 1:
        for w, name in ((q_norm_w, "q"), (k_norm_w, "k")):
            if w is not None and (w.dtype != torch.float32 or w.numel() != hd):
                raise KernelError(f"attn_prepare_ex: the norm per head takes a float32 weight of {hd} entries for {name}")
    t_coef, t_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if q_temp and t_every <= 0:
        raise KernelError("attn_prepare_ex: a query temperature needs a positive number of positions a step")
    _check(library().kestrel_attn_prepare_tempered(
        qkv.data.data_ptr(), qkv.slices, qkv.slice_stride, qkv.width, _p(qkv.bias), _p(q_norm_w), _p(k_norm_w), mode, 1 if v_norm else 0,
        float(norm_eps), _p(inv_freq), rot or 0, rot_mode or 0, float(rotation.scale) if rotation is not None else 1.0, t_coef, t_every, positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(page_size),
        k_cache.data_ptr(), v_cache.data_ptr(), q_out.data_ptr(), _p(gate_out), _code(q_out, "attn_prepare_ex.q_out"), T, nq, nkv, hd, vd,
        1 if has_kv else 0, _stream()))


WEIGHTINGS = {"softmax": 0, "softmax_sink": 1, "sigmoid": 2}


class ScoreOptions:
    """What a layer does to its scores s = q . k * scale and how it weighs keys, all in float32:
    ``softcap`` > 0: s <- softcap tanh(s / softcap); ``r1``, ``r2`` (float32 [heads], both or
    neither): s <- s - r1[h] ln(1 + r2[h] (i - j)) for the key j behind the query i; ``weighting``
    "softmax", "softmax_sink" (one more term in the denominator, without a value: exp(sink[h]) with
    ``sink`` float32 [heads], exp(0) without it) or "sigmoid" (every visible key weighs
    sigmoid(s + head_bias[h]), nothing is normalised).  ``rel`` (float32 [buckets, heads]) with ``rel_bucket``
    (int32 [far + 1], the bucket of every distance up to ``far``; longer distances share far's): s <- s +
    rel[bucket(i - j), h], a learned number per head and bucket of distances."""

    __slots__ = ("softcap", "r1", "r2", "head_bias", "weighting", "sink", "rel", "rel_bucket")

    def __init__(self, softcap: float = 0.0, r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None,
                 head_bias: Optional[torch.Tensor] = None, weighting: str = "softmax", sink: Optional[torch.Tensor] = None,
                 rel: Optional[torch.Tensor] = None, rel_bucket: Optional[torch.Tensor] = None):
        if (rel is None) != (rel_bucket is None):
            raise KernelError("a table of distance terms needs the buckets of the distances, and the other way round")
        self.rel, self.rel_bucket = rel, rel_bucket
        if weighting not in WEIGHTINGS:
            raise KernelError(f"weighting '{weighting}' is none of {', '.join(WEIGHTINGS)}")
        if (r1 is None) != (r2 is None):
            raise KernelError("the distance term needs both of its per-head numbers")
        if softcap < 0:
            raise KernelError("a score cap is positive, or 0 for none")
        if sink is not None and weighting != "softmax_sink":
            raise KernelError("numbers for the denominator's extra term belong to the weighting 'softmax_sink'")
        self.softcap, self.r1, self.r2, self.head_bias, self.weighting, self.sink = float(softcap), r1, r2, head_bias, weighting, sink

    def args(self, nq: int):
        for t, name in ((self.r1, "r1"), (self.r2, "r2"), (self.head_bias, "head_bias"), (self.sink, "sink")):
            if t is not None:
                _need(t, f"score.{name}", torch.float32, 1)
                if t.shape[0] != nq:
                    raise KernelError(f"score.{name}: {t.shape[0]} entries for {nq} heads")
        return self.softcap, _p(self.r1), _p(self.r2), _p(self.head_bias), WEIGHTINGS[self.weighting], _p(self.sink)

    def rel_args(self, nq: int):
        """(table, buckets, longest distance with a bucket of its own) for the kernels that take the distance table."""
        if self.rel is None:
            return None, None, 0
        _need(self.rel, "score.rel", torch.float32, 2)
        _need(self.rel_bucket, "score.rel_bucket", torch.int32, 1)
        if self.rel.shape[1] != nq or self.rel_bucket.shape[0] < 1:
            raise KernelError(f"score.rel: {tuple(self.rel.shape)} for {nq} heads")
        return self.rel.data_ptr(), self.rel_bucket.data_ptr(), self.rel_bucket.shape[0] - 1


_NO_SCORE = ScoreOptions()


def attention_plain_ex(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                       seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, out: torch.Tensor, nq: int, nkv: int,
                       hd: int, vd: int, window: int, keep_first: int, gate: Optional[torch.Tensor], scale: float,
                       score: Optional[ScoreOptions] = None, v_ld: int = 0) -> None:
    """`attention_plain` with values of size ``vd`` (the first ``vd`` numbers of V rows of ``v_ld``, where that is given), the first ``keep_first`` keys of a request
    visible beyond the window, each head's output multiplied by ``gate`` [T, nq], and the layer's
    `ScoreOptions`."""
    _need(q, "attention.q", dims=2)
    _need(out, "attention.out", q.dtype, 2)
    _need(k_cache, "attention.k_cache", q.dtype, 4)
    _need(v_cache, "attention.v_cache", q.dtype, 4)
    _need(block_table, "attention.block_table", torch.int32, 2)
    T = q.shape[0]
    if q.shape[1] != nq * hd or out.shape != (T, nq * vd):
        raise KernelError("attention: shapes differ")
    if gate is not None:
        _need(gate, "attention.gate", torch.float32, 2)
    _check(library().kestrel_attention_plain_biased(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), int(page_size), out.data_ptr(), _code(q, "attention.q"), T, nq, nkv, hd, vd, int(window), int(keep_first),
        _p(gate), float(scale), *(score or _NO_SCORE).args(nq), *(score or _NO_SCORE).rel_args(nq), int(v_ld), _stream()))


def attention_window_supported(hd: int, vd: int, nq: int, nkv: int) -> bool:
    """Whether the tensor-core kernel of `attention_window` takes these sizes."""
    return bool(library().kestrel_attention_window_supported(int(hd), int(vd), int(nq), int(nkv)))


def attention_window(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch, block_table: torch.Tensor, page_size: int,
                     out: torch.Tensor, nq: int, nkv: int, hd: int, vd: int, window: int, keep_first: int, gate: Optional[torch.Tensor],
                     scale: float, score: Optional[ScoreOptions] = None, v_ld: int = 0) -> None:
    """`attention_plain_ex` for bfloat16 on the tensor cores, over this step's requests as ``batch``
    describes them (cumulative lengths, lengths after the step, the most tokens of one request and the
    longest context).  A step of single tokens cuts its key rounds into shares, a CTA each, and a
    second kernel merges them (`attention_window_set_splits`)."""
    _need(q, "attention_window.q", torch.bfloat16, 2)
    _need(out, "attention_window.out", torch.bfloat16, 2)
    _need(k_cache, "attention_window.k_cache", torch.bfloat16, 4)
    _need(v_cache, "attention_window.v_cache", torch.bfloat16, 4)
    _need(block_table, "attention_window.block_table", torch.int32, 2)
    T = q.shape[0]
    if q.shape[1] != nq * hd or out.shape != (T, nq * vd) or T != batch.num_tokens:
        raise KernelError("attention_window: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or tuple(v_cache.shape[1:]) != (nkv, page_size, v_ld or vd):
        raise KernelError("attention_window: the cache planes do not fit the heads")
    if gate is not None:
        _need(gate, "attention_window.gate", torch.float32, 2)
    lib = library()
    # a step of single tokens: the key range shared out over CTAs; the longest context is the host's (a recorded step's: its class's)
    ksplit = lib.kestrel_attention_window_splits(int(batch.num_seqs), int(batch.max_count), nq, nkv, hd, vd, int(window), int(batch.max_kv_len)) \
        if _window_splits else 1
    scratch = None
    if ksplit > 1:
        scratch = torch.empty(lib.kestrel_attention_window_scratch_floats(int(batch.num_seqs), int(batch.max_count), nq, nkv, hd, vd, ksplit), dtype=torch.float32, device=q.device)
    _check(lib.kestrel_attention_window_biased(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(gate), batch.cu_seqlens.data_ptr(), batch.kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), int(batch.num_seqs), int(batch.max_count), nq, nkv, hd, vd, int(window),
        int(keep_first), float(scale), *(score or _NO_SCORE).args(nq), *(score or _NO_SCORE).rel_args(nq), int(v_ld), ksplit, _p(scratch), _stream()))
    if ksplit > 1:
        global launches
        launches += 1          # the merge kernel


_window_splits = True


def attention_window_set_splits(on: bool = True) -> None:
    """Whether `attention_window` shares the keys of single-token steps out over several CTAs (the default).  For tests of both."""
    global _window_splits
    _window_splits = bool(on)


def row_tiles(batch, rows_per_token: int, rows_per_tile: int = 256):
    """The step's rows - (token, head of a key head's group) pairs, ``rows_per_token`` a token - cut into tiles per
    request: (request of each tile, its first row) as int32 tensors on the device, made once a step from the
    host's copy of the requests' token counts and kept on ``batch``."""
    kept = batch.__dict__.setdefault("_row_tiles", {})
    key = (rows_per_token, rows_per_tile)
    if key not in kept:
        seq, row0 = [], []
        for i, n in enumerate(batch.counts):
            for r in range(0, n * rows_per_token, rows_per_tile):
                seq.append(i)
                row0.append(r)
        t = torch.tensor([seq, row0], dtype=torch.int32).to(batch.device_buffer.device, non_blocking=True)
        kept[key] = (t[0], t[1])
    return kept[key]


# ---- attention over cached latents -----------------------------------------------------------

def latent_prepare(fused: Partials, q_norm_w: torch.Tensor, kv_norm_w: torch.Tensor, norm_eps: float, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, latent_cache: torch.Tensor, q_out: torch.Tensor,
                   gate_out: Optional[torch.Tensor], kv_out: Optional[torch.Tensor] = None, rot_cols: int = 0, rotation=None) -> None:
    """Columns [query latent | key/value latent | shared key part | gate] of a fused product: both latents RMS-normed
    with their weights; the query latent to ``q_out`` [T, q_rank], the key/value latent into the
    token's slot of ``latent_cache`` [pages, 1, page size, kv_rank], sigmoid of the gate columns to
    ``gate_out`` float32 [T, heads]; ``kv_out`` [T, kv_rank], if given, receives the step's key/value
    latents as rows too.  With ``rot_cols`` the cache rows are [latent | ``rot_cols`` more]: a key part that all heads
    share, not normed, turned by position as ``rotation`` (a `Rotation` of parts/base.py) says."""
    _need(q_out, "latent_prepare.q_out", dims=2)
    _need(latent_cache, "latent_prepare.latent_cache", q_out.dtype, 4)
    _need(q_norm_w, "latent_prepare.q_norm_w", torch.float32, 1)
    _need(kv_norm_w, "latent_prepare.kv_norm_w", torch.float32, 1)
    _need(block_table, "latent_prepare.block_table", torch.int32, 2)
    T, q_rank = q_out.shape
    kv_rank = latent_cache.shape[3] - int(rot_cols)
    n_gate = 0
    inv_freq, rot, rot_mode, rot_scale = None, 0, 0, 1.0
    if rotation is not None:
        inv_freq, rot, rot_mode, rot_scale = rotation.inv_freq, int(rotation.dim), rotation.mode, float(rotation.scale)
        _need(inv_freq, "latent_prepare.inv_freq", torch.float32, 1)
        if rot > rot_cols or rot % 2 or inv_freq.shape[0] < rot // 2:
            raise KernelError(f"latent_prepare: {rot} rotated dimensions of a key part of {rot_cols}")
    if kv_rank <= 0 or rot_cols < 0:
        raise KernelError("latent_prepare: the cache rows are shorter than the shared key part")
    if gate_out is not None:
        _need(gate_out, "latent_prepare.gate_out", torch.float32, 2)
        n_gate = gate_out.shape[1]
    if kv_out is not None:
        _need(kv_out, "latent_prepare.kv_out", q_out.dtype, 2)
        if kv_out.shape != (T, kv_rank):
            raise KernelError("latent_prepare: kv_out has the wrong shape")
    if fused.tokens != T or fused.bias is not None or latent_cache.shape[1] != 1 or latent_cache.shape[2] != page_size or \
            q_norm_w.shape[0] != q_rank or kv_norm_w.shape[0] != kv_rank or (gate_out is not None and gate_out.shape[0] != T):
        raise KernelError("latent_prepare: shapes differ, or a bias is pending")
    _check(library().kestrel_latent_prepare_rotated(
        fused.data.data_ptr(), fused.slices, fused.slice_stride, fused.width, q_norm_w.data_ptr(), kv_norm_w.data_ptr(), float(norm_eps),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(page_size), latent_cache.data_ptr(),
        q_out.data_ptr(), _p(gate_out), _p(kv_out), _code(q_out, "latent_prepare.q_out"), T, q_rank, kv_rank, n_gate, int(rot_cols), _p(inv_freq),
        rot, rot_mode, rot_scale, _stream()))


def latent_rotate_queries(q: torch.Tensor, heads: int, d: int, rot_cols: int, q_lat: torch.Tensor, col0: int, positions: torch.Tensor,
                          rotation) -> None:
    """Columns [d, d + rot_cols) of every head of q [T, heads * (d + rot_cols)], turned by position as ``rotation`` says (None:
    copied), into columns [col0, col0 + rot_cols) of every head of q_lat [T, heads * (col0 + rot_cols)]."""
    _need(q, "latent_rotate_queries.q", dims=2)
    _need(q_lat, "latent_rotate_queries.q_lat", q.dtype, 2)
    T = q.shape[0]
    if q.shape[1] != heads * (d + rot_cols) or q_lat.shape != (T, heads * (col0 + rot_cols)):
        raise KernelError("latent_rotate_queries: shapes differ")
    inv_freq, rot, rot_mode, rot_scale = None, 0, 0, 1.0
    if rotation is not None:
        inv_freq, rot, rot_mode, rot_scale = rotation.inv_freq, int(rotation.dim), rotation.mode, float(rotation.scale)
    _check(library().kestrel_latent_rotate_queries(q.data_ptr(), q.stride(0), d + rot_cols, d, q_lat.data_ptr(), q_lat.stride(0), col0 + rot_cols, col0,
                                                   positions.data_ptr(), _code(q, "latent_rotate_queries.q"), T, heads, rot_cols, _p(inv_freq), rot,
                                                   rot_mode, rot_scale, _stream()))


def head_scale(x: torch.Tensor, gate: torch.Tensor, heads: int) -> None:
    """x[t, h, :] *= gate[t, h] in place: x [T, heads * d], gate float32 [T, heads]."""
    _need(x, "head_scale.x", dims=2)
    _need(gate, "head_scale.gate", torch.float32, 2)
    T = x.shape[0]
    if gate.shape != (T, heads) or x.shape[1] % heads:
        raise KernelError("head_scale: shapes differ")
    _check(library().kestrel_head_scale(x.data_ptr(), gate.data_ptr(), _code(x, "head_scale.x"), T, heads, x.shape[1] // heads, _stream()))


def head_gemm(x: torch.Tensor, w: torch.Tensor, heads: int, w_kn: bool, out: Optional[torch.Tensor] = None,
              x_head_stride: Optional[int] = None, out_head_stride: Optional[int] = None, out_f32: bool = False) -> torch.Tensor:
    """Every head's columns of x [T, heads * K] times that head's own matrix, a slice of ``w``:
    ``w_kn`` False: w [heads * N, K], out_h = x_h w_h^T; True: w [heads * K, N], out_h = x_h w_h (the
    transposed use of an expansion).  Returns [T, heads * N] in x's dtype (float32 if ``out_f32``); float32 sums.
    ``x_head_stride`` / ``out_head_stride``: a head's K input columns start every so many columns of x, its N
    output columns every so many columns of ``out`` (heads whose columns lie among others)."""
    _need(x, "head_gemm.x", dims=2)
    _need(w, "head_gemm.w", x.dtype, 2)
    T = x.shape[0]
    hsx = x.shape[1] // heads if x_head_stride is None else int(x_head_stride)
    if (x_head_stride is None and x.shape[1] % heads) or w.shape[0] % heads:
        raise KernelError("head_gemm: the columns of x or the rows of w do not divide by the heads")
    K = w.shape[0] // heads if w_kn else w.shape[1]
    N = w.shape[1] if w_kn else w.shape[0] // heads
    hso = N if out_head_stride is None else int(out_head_stride)
    if K > hsx or N > hso or x.shape[1] < (heads - 1) * hsx + K:
        raise KernelError(f"head_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, {heads} heads")
    out_dtype = torch.float32 if out_f32 else x.dtype
    if out is None:
        out = torch.empty((T, heads * hso), dtype=out_dtype, device=x.device)
    _need(out, "head_gemm.out", out_dtype, 2)
    if out.shape[0] != T or out.shape[1] < (heads - 1) * hso + N:
        raise KernelError("head_gemm: out has the wrong shape")
    _check(library().kestrel_head_gemm_strided(x.data_ptr(), x.stride(0), hsx, w.data_ptr(), w.stride(0), 1 if w_kn else 0, out.data_ptr(),
                                               out.stride(0), hso, 1 if out_f32 else 0, _code(x, "head_gemm.x"), T, heads, N, K, _stream()))
    return out


def head_gemm_set_plain(on: bool = True) -> None:
    """Whether bfloat16 head-wise products take the CUDA-core kernel instead of the tensor-core one
    (off by default).  For tests of both."""
    library().kestrel_head_gemm_set_plain(1 if on else 0)


# ---- gated delta rule ------------------------------------------------------------------------

def delta_conv_silu(x: Partials, conv_w: torch.Tensor, state: torch.Tensor, tail_off: int, batch, out: torch.Tensor) -> None:
    """out[t, c] = silu(causal convolution over time of x's first C columns), C = conv_w.shape[0];
    inputs before the step come from, and the last taps - 1 inputs go to, each request's state slot
    (``state`` float32 [slots, size], the tail [taps - 1, C] at ``tail_off``)."""
    _need(conv_w, "delta_conv.w", torch.float32, 2)
    _need(state, "delta_conv.state", torch.float32, 2)
    _need(out, "delta_conv.out", torch.float32, 2)
    C, taps = conv_w.shape
    T = out.shape[0]
    if x.tokens != T or x.width < C or out.shape[1] != C or x.bias is not None:
        raise KernelError("delta_conv_silu: shapes differ")
    _check(library().kestrel_delta_conv_silu(x.data.data_ptr(), x.slices, x.slice_stride, x.width, conv_w.data_ptr(), taps, state.data_ptr(),
                                             state.stride(0), int(tail_off), batch.seq_of_token.data_ptr(), batch.cu_seqlens.data_ptr(),
                                             batch.slots.data_ptr(), out.data_ptr(), T, batch.num_seqs, C, _stream()))
    global launches
    launches += 1 if taps > 1 else 0


def delta_gates(act: torch.Tensor, x: Partials, col_beta: int, a: Partials, A_log: torch.Tensor, dt_bias: torch.Tensor,
                qn: torch.Tensor, kn: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, H: int, G: int, d: int) -> None:
    """Unit query and key vectors (queries scaled by d^-1/2), beta = sigmoid, decay = exp(-exp(A_log) softplus(a + dt_bias))."""
    for t, n in ((act, "act"), (qn, "qn"), (kn, "kn"), (decay, "decay"), (beta, "beta")):
        _need(t, f"delta_gates.{n}", torch.float32, 2)
    T = act.shape[0]
    if a.tokens != T or a.width != H * d or qn.shape != (T, G * d) or decay.shape != (T, H * d) or beta.shape != (T, H):
        raise KernelError("delta_gates: shapes differ")
    _check(library().kestrel_delta_gates(act.data_ptr(), act.shape[1], x.data.data_ptr(), x.slices, x.slice_stride, x.width, int(col_beta),
                                         a.data.data_ptr(), a.slices, a.slice_stride, A_log.data_ptr(), dt_bias.data_ptr(), qn.data_ptr(),
                                         kn.data_ptr(), decay.data_ptr(), beta.data_ptr(), T, H, G, d, _stream()))


def delta_scan(qn: torch.Tensor, kn: torch.Tensor, decay: torch.Tensor, act: torch.Tensor, col_v: int, beta: torch.Tensor,
               state: torch.Tensor, batch, out: torch.Tensor, H: int, G: int, d: int, dv: int) -> None:
    """The recurrence S <- a S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over this step's
    tokens of every request, from and to the requests' state slots."""
    _need(out, "delta_scan.out", torch.float32, 2)
    _need(state, "delta_scan.state", torch.float32, 2)
    _check(library().kestrel_delta_scan(qn.data_ptr(), kn.data_ptr(), decay.data_ptr(), act.data_ptr(), act.shape[1], int(col_v), beta.data_ptr(),
                                        state.data_ptr(), state.stride(0), batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), out.data_ptr(),
                                        batch.num_seqs, H, G, d, dv, _stream()))


def delta_out(o: torch.Tensor, weight: torch.Tensor, eps: float, gate: Partials, out: torch.Tensor, H: int, dv: int) -> None:
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate) per head, in out's dtype."""
    _need(o, "delta_out.o", torch.float32, 2)
    _need(weight, "delta_out.weight", torch.float32, 1)
    _need(out, "delta_out.out", dims=2)
    T = o.shape[0]
    if o.shape[1] != H * dv or out.shape != o.shape or gate.tokens != T or gate.width != H * dv or weight.shape[0] != dv:
        raise KernelError("delta_out: shapes differ")
    _check(library().kestrel_delta_out(o.data_ptr(), weight.data_ptr(), float(eps), gate.data.data_ptr(), gate.slices, gate.slice_stride,
                                       out.data_ptr(), _code(out, "delta_out.out"), T, H, dv, _stream()))


# ---- linear recurrences with a matrix of state per head ---------------------------------------

def forget_gates(fused: Partials, col_q: int, col_f: int, col_v: int, f_bias: Optional[torch.Tensor], lower: Optional[torch.Tensor],
                 n: int, nv: int):
    """(r, w, k, v) float32 for `recurrence_scan` from a fused product's columns: r = silu(q),
    w = lower + (1 - lower) * sigmoid(f + f_bias), k = 1 - w, v as it is."""
    T, dev = fused.tokens, fused.data.device
    if fused.bias is not None:
        raise KernelError("forget_gates: a bias is pending on the fused product")
    r, w, k = (torch.empty((T, n), dtype=torch.float32, device=dev) for _ in range(3))
    v = torch.empty((T, nv), dtype=torch.float32, device=dev)
    _check(library().kestrel_forget_gates(fused.data.data_ptr(), fused.slices, fused.slice_stride, fused.width, int(col_q), int(col_f), int(col_v),
                                          _p(f_bias), _p(lower), r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), T, int(n), int(nv), _stream()))
    return r, w, k, v


def removal_gates(fused: Partials, col_r: int, col_k: int, col_v: int, col_a: int, a_bias: Optional[torch.Tensor], wz: Partials,
                  w_bias: Optional[torch.Tensor], decay_rate: float, H: int, d: int):
    """(r, w, k, v, a, b) float32 for `recurrence_scan` from a fused product's columns and the decay's
    second product ``wz``: u = k / sqrt(sum k^2 + 1e-6) per head, w = exp(-decay_rate * sigmoid(wz + w_bias)),
    a = -(sigmoid(rate + a_bias) * u), b = u."""
    T, dev, n = fused.tokens, fused.data.device, H * d
    if fused.bias is not None or wz.bias is not None or wz.tokens != T or wz.width != n:
        raise KernelError("removal_gates: shapes differ, or a bias is pending")
    r, w, k, v, a, b = (torch.empty((T, n), dtype=torch.float32, device=dev) for _ in range(6))
    _check(library().kestrel_removal_gates(fused.data.data_ptr(), fused.slices, fused.slice_stride, fused.width, int(col_r), int(col_k), int(col_v),
                                           int(col_a), _p(a_bias), wz.data.data_ptr(), wz.slices, wz.slice_stride, _p(w_bias), float(decay_rate),
                                           r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), a.data_ptr(), b.data_ptr(), T, H, d, _stream()))
    return r, w, k, v, a, b


def recurrence_scan(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor],
                    state: torch.Tensor, state_off: int, batch, H: int, d: int, dv: int) -> torch.Tensor:
    """S <- diag(w) S + a (b^T S) + k v^T, o = S^T r per head over this step's tokens of every request,
    from and to the requests' state slots (S [H, d, dv] at ``state_off`` floats into a slot); returns
    o float32 [T, H dv].  ``a`` and ``b`` None: no correction term."""
    _need(state, "recurrence_scan.state", torch.float32, 2)
    T = r.shape[0]
    for t, name, n in ((r, "r", H * d), (w, "w", H * d), (k, "k", H * d), (v, "v", H * dv), (a, "a", H * d), (b, "b", H * d)):
        if t is not None:
            _need(t, f"recurrence_scan.{name}", torch.float32, 2)
            if t.shape != (T, n):
                raise KernelError(f"recurrence_scan.{name}: shape {tuple(t.shape)}, expected ({T}, {n})")
    if state_off < 0 or state_off + H * d * dv > state.shape[1]:
        raise KernelError("recurrence_scan: the state does not fit the slot")
    out = torch.empty((T, H * dv), dtype=torch.float32, device=r.device)
    _check(library().kestrel_recurrence_scan(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), _p(a), _p(b), state.data_ptr(), state.stride(0),
                                             int(state_off), batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), out.data_ptr(), batch.num_seqs,
                                             H, d, dv, _stream()))
    return out


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, gate: Optional[Partials], gate_col0: int, out: torch.Tensor,
                   H: int, dv: int) -> None:
    """out = o / sqrt(mean(o^2) + eps) per head, times ``weight`` ([dv]: shared by the heads; [H dv]: one per
    head), times sigmoid of the columns [gate_col0, gate_col0 + H dv) of ``gate`` where given."""
    _need(o, "head_norm_gate.o", torch.float32, 2)
    _need(weight, "head_norm_gate.weight", torch.float32, 1)
    _need(out, "head_norm_gate.out", dims=2)
    T = o.shape[0]
    if o.shape[1] != H * dv or out.shape != o.shape or weight.shape[0] not in (dv, H * dv):
        raise KernelError("head_norm_gate: shapes differ")
    if gate is not None and (gate.tokens != T or gate.bias is not None or gate_col0 + H * dv > gate.width):
        raise KernelError("head_norm_gate: the gate's product does not fit, or carries a bias")
    w_stride = dv if (weight.shape[0] == H * dv and H > 1) else 0
    _check(library().kestrel_head_norm_gate(o.data_ptr(), weight.data_ptr(), w_stride, float(eps), _p(gate.data) if gate is not None else None,
                                            gate.slices if gate is not None else 0, gate.slice_stride if gate is not None else 0,
                                            gate.width if gate is not None else 0, int(gate_col0), out.data_ptr(), _code(out, "head_norm_gate.out"),
                                            T, H, dv, _stream()))


# ---- routed feed-forward -----------------------------------------------------------------------

MOE_TILE_ROWS = 64


MOE_TC_MIN_PAIRS = 1024     # from this many (token, choice) pairs on, the grouped products take the tcgen05 kernels
_moe_tc = True


def moe_set_tcgen05(on: bool = True) -> None:
    """Whether the grouped products of many pairs take the tcgen05 kernels (the default) or the
    mma.sync ones at every size.  For tests of both."""
    global _moe_tc
    _moe_tc = bool(on)


def moe_set_plain(on: bool = True) -> None:
    """Whether the bfloat16 grouped products of `moe_experts` take the CUDA-core kernel instead of
    the tensor-core one (off by default).  For tests of both."""
    library().kestrel_moe_set_plain(1 if on else 0)


def moe_route(z: Partials, bias: Optional[torch.Tensor], top: int):
    """(expert ids int32 [T, top], weights float32 [T, top]): the ``top`` largest router logits of
    each token and the softmax over them."""
    T, E = z.tokens, z.width
    ids = torch.empty((T, top), dtype=torch.int32, device=z.data.device)
    w = torch.empty((T, top), dtype=torch.float32, device=z.data.device)
    _check(library().kestrel_moe_route(z.data.data_ptr(), z.slices, z.slice_stride, _p(bias), ids.data_ptr(), w.data_ptr(), T, E, top,
                                       _stream()))
    return ids, w


def moe_route_sigmoid(z: Partials, correction: Optional[torch.Tensor], top: int, groups: int = 1, keep: int = 1, scale: float = 1.0):
    """(expert ids int32 [T, top], weights float32 [T, top]) of a router with sigmoid scores: experts are chosen by
    score + ``correction`` among the ``keep`` best of ``groups`` equal groups of neighbours (a group's score: the sum of its two
    largest choice scores), and weighted by their scores over the chosen scores' sum, times ``scale``."""
    T, E = z.tokens, z.width
    if z.bias is not None:
        raise KernelError("moe_route_sigmoid: a bias is pending")
    if correction is not None:
        _need(correction, "moe_route_sigmoid.correction", torch.float32, 1)
        if correction.shape[0] != E:
            raise KernelError("moe_route_sigmoid: a correction per expert")
    ids = torch.empty((T, top), dtype=torch.int32, device=z.data.device)
    w = torch.empty((T, top), dtype=torch.float32, device=z.data.device)
    _check(library().kestrel_moe_route_sigmoid(z.data.data_ptr(), z.slices, z.slice_stride, _p(correction), int(groups), int(keep), float(scale),
                                               ids.data_ptr(), w.data_ptr(), T, E, top, _stream()))
    return ids, w


UP_ACTS = {"gelu": 1, "gelu_tanh": 2, "silu": 3, "relu2": 4}


def moe_experts_ungated(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                        act: str) -> torch.Tensor:
    """The chosen experts' outputs W_down[e] act(W_up[e] x), weighted and summed per token: float32 [T, width].
    w_up [E, ff, width], w_down [E, width, ff]; ``act`` one of `UP_ACTS`.  The pairs' input rows are gathered in the
    order of their experts, then two grouped products run (tcgen05 from `MOE_TC_MIN_PAIRS` pairs on)."""
    _need(x, "moe.x", dims=2)
    _need(w_up, "moe.w_up", x.dtype, 3)
    _need(w_down, "moe.w_down", x.dtype, 3)
    if act not in UP_ACTS:
        raise KernelError(f"moe_experts_ungated: activation {act!r} is none of {', '.join(UP_ACTS)}")
    T, K = x.shape
    E, ff, _ = w_up.shape
    top, N = ids.shape[1], w_down.shape[1]
    if w_up.shape[2] != K or w_down.shape != (E, N, ff) or ids.shape[0] != T:
        raise KernelError("moe_experts_ungated: shapes differ")
    lib, dev, P, code = library(), x.device, T * top, _code(x, "moe.x")
    xs = torch.empty((P, K), dtype=x.dtype, device=dev)
    a = torch.empty((P, ff), dtype=x.dtype, device=dev)
    y = torch.empty((P, N), dtype=torch.float32, device=dev)
    out = torch.empty((T, N), dtype=torch.float32, device=dev)
    tc = bool(_moe_tc and x.dtype == torch.bfloat16 and P >= MOE_TC_MIN_PAIRS and
              lib.kestrel_moe_tc_supported(xs.data_ptr(), a.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), ff, K))
    rows = lib.kestrel_moe_tc_tile_rows() if tc else MOE_TILE_ROWS
    max_tiles = lib.kestrel_moe_max_tiles(P, E, rows)
    meta = torch.empty((E + 1) + 2 * P + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
    offsets, row_pair, pair_row = meta[:E + 1], meta[E + 1:E + 1 + P], meta[E + 1 + P:E + 1 + 2 * P]
    o = E + 1 + 2 * P
    tile_expert, tile_row0, n_tiles = meta[o:o + max_tiles], meta[o + max_tiles:o + 2 * max_tiles], meta[o + 2 * max_tiles:]
    _check(lib.kestrel_moe_group(ids.data_ptr(), P, E, rows, offsets.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(),
                                 tile_expert.data_ptr(), tile_row0.data_ptr(), n_tiles.data_ptr(), _stream()))
    _check(lib.kestrel_moe_gather_rows_any(x.data_ptr(), x.stride(0), row_pair.data_ptr(), top, xs.data_ptr(), code, P, K, _stream()))
    if tc:
        _check(lib.kestrel_moe_up_act_tc(xs.data_ptr(), w_up.data_ptr(), offsets.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(),
                                         n_tiles.data_ptr(), max_tiles, UP_ACTS[act], a.data_ptr(), P, E, ff, K, _stream()))
        _check(lib.kestrel_moe_down_tc(a.data_ptr(), w_down.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), tile_expert.data_ptr(),
                                       tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, weights.data_ptr(), y.data_ptr(), P, E, N, ff, _stream()))
    else:
        _check(lib.kestrel_moe_up_act(xs.data_ptr(), w_up.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), tile_expert.data_ptr(),
                                      tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, UP_ACTS[act], a.data_ptr(), code, ff, K, _stream()))
        _check(lib.kestrel_moe_down(a.data_ptr(), w_down.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), tile_expert.data_ptr(),
                                    tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, weights.data_ptr(), y.data_ptr(), code, N, ff, _stream()))
    _check(lib.kestrel_moe_combine(y.data_ptr(), pair_row.data_ptr(), top, out.data_ptr(), T, N, _stream()))
    return out


# ---- a diagonal recurrence with gates from its own input -------------------------------------------
def rglru_branches(fused: Partials, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], state: torch.Tensor, tail_off: int, batch,
                   y_out: torch.Tensor, u_out: torch.Tensor, u_st: torch.Tensor) -> None:
    """Columns [y | x] of a fused product (plus its bias): y_out = gelu_tanh(y), u_out = causal convolution over time of x per
    channel (``conv_w`` [C, taps], last column the current token's; ``conv_b`` [C]) as float32, ``u_st`` the same in the storage
    type; inputs before the step come from, and the last taps - 1 inputs go to, each request's state slot at ``tail_off``."""
    _need(conv_w, "rglru.conv_w", torch.float32, 2)
    _need(state, "rglru.state", torch.float32, 2)
    _need(y_out, "rglru.y_out", torch.float32, 2)
    _need(u_out, "rglru.u_out", torch.float32, 2)
    _need(u_st, "rglru.u_st", dims=2)
    C, taps = conv_w.shape
    T = y_out.shape[0]
    if fused.tokens != T or fused.width < 2 * C or y_out.shape != (T, C) or u_out.shape != (T, C) or u_st.shape != (T, C) or \
            (fused.bias is not None and fused.bias.shape[0] != fused.width) or (conv_b is not None and conv_b.shape[0] != C):
        raise KernelError("rglru_branches: shapes differ")
    _check(library().kestrel_rglru_branches(fused.data.data_ptr(), fused.slices, fused.slice_stride, fused.width, _p(fused.bias), conv_w.data_ptr(),
                                            _p(conv_b), taps, state.data_ptr(), state.stride(0), int(tail_off), batch.seq_of_token.data_ptr(),
                                            batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), y_out.data_ptr(), u_out.data_ptr(), u_st.data_ptr(),
                                            _code(u_st, "rglru.u_st"), T, batch.num_seqs, C, _stream()))
    global launches
    launches += 1 if taps > 1 else 0


RGLRU_CHUNKED_FROM = 128     # a step whose longest portion has this many tokens runs the recurrence in chunks
rglru_chunked = True         # tests switch the chunked form off to hold both against each other


def rglru_scan(y: torch.Tensor, u: torch.Tensor, gr: torch.Tensor, gi: torch.Tensor, r_bias: Optional[torch.Tensor],
               i_bias: Optional[torch.Tensor], lam: torch.Tensor, rate: float, state: torch.Tensor, batch, out: torch.Tensor) -> None:
    """Per channel: r = sigmoid(gr + r_bias), i = sigmoid(gi + i_bias), a = exp(-rate r softplus(lam)),
    S <- a S + sqrt(1 - a^2) i u, out = S y; S float32 at the start of each request's state slot.  Steps that bring a
    request `RGLRU_CHUNKED_FROM` tokens or more run the recurrence in chunks (two kernels; same result within rounding)."""
    T, C = y.shape
    for t, name in ((y, "y"), (u, "u"), (gr, "gr"), (gi, "gi")):
        _need(t, f"rglru_scan.{name}", torch.float32, 2)
        if t.shape != (T, C):
            raise KernelError("rglru_scan: shapes differ")
    _need(lam, "rglru_scan.lam", torch.float32, 1)
    _need(out, "rglru_scan.out", dims=2)
    if out.shape != (T, C) or lam.shape[0] != C:
        raise KernelError("rglru_scan: shapes differ")
    if not batch.captured and batch.max_count >= RGLRU_CHUNKED_FROM and rglru_chunked:
        # many tokens of a request: the recurrence in chunks, as many as keep the chip busy, of 32 tokens at least
        chunk = max(32, (-(-int(batch.max_count) // 64) + 7) // 8 * 8)
        chunks = -(-int(batch.max_count) // chunk)
        scratch = torch.empty((batch.num_seqs * chunks * 2 * C,), dtype=torch.float32, device=y.device)
        _check(library().kestrel_rglru_scan_chunked(y.data_ptr(), u.data_ptr(), gr.data_ptr(), gi.data_ptr(), _p(r_bias), _p(i_bias), lam.data_ptr(),
                                                    float(rate), state.data_ptr(), state.stride(0), batch.cu_seqlens.data_ptr(),
                                                    batch.slots.data_ptr(), out.data_ptr(), _code(out, "rglru_scan.out"), batch.num_seqs,
                                                    int(batch.max_count), chunk, scratch.data_ptr(), C, _stream()))
        global launches
        launches += 1
        return
    _check(library().kestrel_rglru_scan(y.data_ptr(), u.data_ptr(), gr.data_ptr(), gi.data_ptr(), _p(r_bias), _p(i_bias), lam.data_ptr(), float(rate),
                                        state.data_ptr(), state.stride(0), batch.cu_seqlens.data_ptr(), batch.slots.data_ptr(), out.data_ptr(),
                                        _code(out, "rglru_scan.out"), batch.num_seqs, C, _stream()))


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                limit: float) -> torch.Tensor:
    """The chosen experts' outputs, weighted and summed per token: float32 [T, width].
    w_gate_up [E, 2 ff, width] (gate rows, then up rows), w_down [E, width, ff]."""
    _need(x, "moe.x", dims=2)
    _need(w_gate_up, "moe.w_gate_up", x.dtype, 3)
    _need(w_down, "moe.w_down", x.dtype, 3)
    T, K = x.shape
    E, ff2, _ = w_gate_up.shape
    ff, top = ff2 // 2, ids.shape[1]
    N = w_down.shape[1]
    if w_gate_up.shape[2] != K or w_down.shape != (E, N, ff) or ids.shape[0] != T:
        raise KernelError("moe_experts: shapes differ")
    lib, dev, P = library(), x.device, T * top
    act = torch.empty((P, ff), dtype=x.dtype, device=dev)
    y = torch.empty((P, N), dtype=torch.float32, device=dev)
    out = torch.empty((T, N), dtype=torch.float32, device=dev)
    if _moe_tc and x.dtype == torch.bfloat16 and P >= MOE_TC_MIN_PAIRS and x.stride(0) % 8 == 0:
        xs = torch.empty((P, K), dtype=x.dtype, device=dev)
        if lib.kestrel_moe_tc_supported(xs.data_ptr(), act.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), ff, K):
            rows = lib.kestrel_moe_tc_tile_rows()
            max_tiles = lib.kestrel_moe_max_tiles(P, E, rows)
            meta = torch.empty((E + 1) + 2 * P + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
            offsets, row_pair, pair_row = meta[:E + 1], meta[E + 1:E + 1 + P], meta[E + 1 + P:E + 1 + 2 * P]
            o = E + 1 + 2 * P
            tile_expert, tile_row0, n_tiles = meta[o:o + max_tiles], meta[o + max_tiles:o + 2 * max_tiles], meta[o + 2 * max_tiles:]
            _check(lib.kestrel_moe_group(ids.data_ptr(), P, E, rows, offsets.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(),
                                         tile_expert.data_ptr(), tile_row0.data_ptr(), n_tiles.data_ptr(), _stream()))
            _check(lib.kestrel_moe_gather_rows(x.data_ptr(), x.stride(0), row_pair.data_ptr(), top, xs.data_ptr(), P, K, _stream()))
            _check(lib.kestrel_moe_gate_up_tc(xs.data_ptr(), w_gate_up.data_ptr(), offsets.data_ptr(), tile_expert.data_ptr(), tile_row0.data_ptr(),
                                              n_tiles.data_ptr(), max_tiles, float(limit), act.data_ptr(), P, E, ff, K, _stream()))
            _check(lib.kestrel_moe_down_tc(act.data_ptr(), w_down.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), tile_expert.data_ptr(),
                                           tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, weights.data_ptr(), y.data_ptr(), P, E, N, ff, _stream()))
            _check(lib.kestrel_moe_combine(y.data_ptr(), pair_row.data_ptr(), top, out.data_ptr(), T, N, _stream()))
            return out
    max_tiles = lib.kestrel_moe_max_tiles(P, E, MOE_TILE_ROWS)
    meta = torch.empty((E + 1) + 2 * P + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
    offsets, row_pair, pair_row = meta[:E + 1], meta[E + 1:E + 1 + P], meta[E + 1 + P:E + 1 + 2 * P]
    o = E + 1 + 2 * P
    tile_expert, tile_row0, n_tiles = meta[o:o + max_tiles], meta[o + max_tiles:o + 2 * max_tiles], meta[o + 2 * max_tiles:]
    _check(lib.kestrel_moe_group(ids.data_ptr(), P, E, MOE_TILE_ROWS, offsets.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(),
                                 tile_expert.data_ptr(), tile_row0.data_ptr(), n_tiles.data_ptr(), _stream()))
    _check(lib.kestrel_moe_gate_up(x.data_ptr(), x.stride(0), w_gate_up.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(),
                                   tile_expert.data_ptr(), tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, top, float(limit),
                                   act.data_ptr(), _code(x, "moe.x"), ff, K, _stream()))
    _check(lib.kestrel_moe_down(act.data_ptr(), w_down.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), tile_expert.data_ptr(),
                                tile_row0.data_ptr(), n_tiles.data_ptr(), max_tiles, weights.data_ptr(), y.data_ptr(), _code(x, "moe.x"), N, ff,
                                _stream()))
    _check(lib.kestrel_moe_combine(y.data_ptr(), pair_row.data_ptr(), top, out.data_ptr(), T, N, _stream()))
    return out


# ---- the step program and its runner ---------------------------------------------------------
PHASES = {name[4:].lower(): value for name, value in _cdecl.constants().items() if name.startswith("KPH_") and name != "KPH_COUNT"}
PHASE_COUNT = _cdecl.constants()["KPH_COUNT"]


class StepProgram:
    """A model's step as a list of kernel-level operations (csrc/kernels/step_program.cu).  Parts
    write their operations into it once, in the order in which they run (`emit` methods); the
    methods below return registers - small integers that name activations - or raise."""

    def __init__(self, dtype: torch.dtype):
        self._lib = library()
        self.dtype = dtype
        self._h = self._lib.kprog_create(_DT[dtype])
        if not self._h:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        self._keep = []          # tensors the program points into

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.kprog_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _reg(self, rc: int) -> int:
        if rc < 0:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        return rc

    def _ptr(self, t: Optional[torch.Tensor], name: str, dtype=None):
        if t is None:
            return None
        _need(t, name, dtype)
        self._keep.append(t)
        return t.data_ptr()

    def begin_call(self) -> None:
        self._reg(self._lib.kprog_begin_call(self._h))

    def embed(self, table: torch.Tensor) -> int:
        _need(table, "program.embed.table", dims=2)
        return self._reg(self._lib.kprog_embed(self._h, self._ptr(table, "table"), _code(table, "table"), table.shape[1]))

    def add_rmsnorm(self, residual: int, delta: Optional[int], weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                    logit_rows: bool = False, phase: str = "norm") -> int:
        return self._reg(self._lib.kprog_add_rmsnorm(self._h, residual, -1 if delta is None else delta,
                                                     self._ptr(weight, "norm weight", torch.float32), float(eps), weight.shape[0],
                                                     _DT[out_dtype], 1 if logit_rows else 0, PHASES[phase]))

    def linear(self, x: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, add_to: Optional[int] = None,
               phase: str = "other") -> int:
        _need(weight, "program.linear.weight", self.dtype, 2)
        return self._reg(self._lib.kprog_linear(self._h, x, self._ptr(weight, "weight"), weight.stride(0), weight.shape[0],
                                                weight.shape[1], self._ptr(bias, "bias", torch.float32),
                                                -1 if add_to is None else add_to, PHASES[phase]))

    def gate_up_swiglu(self, x: int, weight: torch.Tensor, ff: int, phase: str = "gate_up") -> int:
        _need(weight, "program.gate_up.weight", self.dtype, 2)
        if weight.shape[0] != 2 * ff:
            raise KernelError("program.gate_up_swiglu: the weight has not 2 x ff rows")
        return self._reg(self._lib.kprog_gate_up_swiglu(self._h, x, self._ptr(weight, "weight"), weight.stride(0), ff,
                                                        weight.shape[1], PHASES[phase]))

    def attn_prepare(self, qkv: int, q_norm_w, k_norm_w, norm_eps: float, inv_freq, rotary_dim: int, rot_mode: int,
                     rot_scale: float, group: int, page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, nq: int,
                     nkv: int, hd: int, write_kv: bool, phase: str = "rope") -> int:
        return self._reg(self._lib.kprog_attn_prepare(
            self._h, qkv, self._ptr(q_norm_w, "q_norm", torch.float32), self._ptr(k_norm_w, "k_norm", torch.float32),
            float(norm_eps), self._ptr(inv_freq, "inv_freq", torch.float32), int(rotary_dim), int(rot_mode), float(rot_scale),
            int(group), int(page_size), self._ptr(k_cache, "k_cache", self.dtype), self._ptr(v_cache, "v_cache", self.dtype),
            nq, nkv, hd, 1 if write_kv else 0, PHASES[phase]))

    def attention(self, q: int, planner: Optional[AttentionPlanner], group: int, page_size: int, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, nq: int, nkv: int, hd: int, window: int, scale: float, phase: str = "attn") -> int:
        if planner is not None:
            self._keep.append(planner)
        return self._reg(self._lib.kprog_attention(
            self._h, q, planner.handle if planner is not None else None, int(group), int(page_size), int(k_cache.shape[0]),
            self._ptr(k_cache, "k_cache", self.dtype), self._ptr(v_cache, "v_cache", self.dtype), nq, nkv, hd, int(window),
            float(scale), PHASES[phase]))

    def logits(self, x: int, weight: torch.Tensor, phase: str = "lm_head") -> None:
        _need(weight, "program.logits.weight", self.dtype, 2)
        self._reg(self._lib.kprog_logits(self._h, x, self._ptr(weight, "weight"), weight.stride(0), weight.shape[0],
                                         weight.shape[1], PHASES[phase]))

    @property
    def num_ops(self) -> int:
        return self._lib.kprog_num_ops(self._h)


def kernel_errors() -> int:
    """Bits of the kernels whose bounded waits ran out since the last call (0 = none); synchronises."""
    return library().kestrel_kernel_errors()
