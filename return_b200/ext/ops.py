"""Python face of the CUDA kernels: thin, checked wrappers over the ``extern "C"`` launchers.

Every function here launches hand-written sm_100a kernels on torch's current CUDA stream.
There is no CPU path and no library stand-in: a tensor that is not on a CUDA device, or a
missing extension, raises.  The only library product on the engine's path is the bfloat16
matrix product (cuBLAS through ``torch.mm``), where the reference's engine also calls a
library (rollout/monkey_patch/qwen3.py:21-22,29-31,56).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

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
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")
    return t.data_ptr()              # an int: ctypes makes the pointer from it (argtypes are set)


try:                                                  # the raw handle, without building a Stream object
    _raw_stream, _device_index = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:                                # a torch without these: the public way, slower
    _raw_stream = None


def _stream():
    """The current stream of the current device (each launch asks: a graph capture changes it)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_device_index()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


# kernels of this package launched by this process (a captured graph counts once, at capture)
launch_count = 0


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launch_count
    launch_count += kernels
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")


# How kernels of a step overlap through programmatic dependent launch (csrc/common.cuh): every kernel waits for
# its predecessor before it touches what that wrote, and lets its successor start when its main loop is done.
PDL_MODE = 2

_core = None

_CORE_SOURCES = ["elementwise.cu", "gemm_f32.cu", "gemm_skinny.cu", "rope_cache.cu", "attention_simt.cu", "sampling.cu",
                 "attention_prep.cu"]


def core() -> ctypes.CDLL:
    """The library of kernels that need no specialisation."""
    global _core
    if _core is None:
        lib = build.load("return_core", _CORE_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I, F = c_void_p, c_int, c_float
        lib.rb_embedding.argtypes = [P, I, P, P, I, I, I, F, I, P]
        L = ctypes.c_longlong
        lib.rb_activation.argtypes = [P, L, I, P, L, I, I, P, I, I, I, P]
        lib.rb_hyper_read_norm.argtypes = [P, P, P, P, I, F, F, P, I, I, I, I, P]
        lib.rb_hyper_write.argtypes = [P, P, I, P, P, P, P, I, F, F, P, I, I, I, I, P]
        lib.rb_add_rmsnorm.argtypes = [P, P, P, P, I, F, F, P, I, I, I, P]
        lib.rb_rmsnorm_rows.argtypes = [P, P, I, F, F, P, I, I, I, P]
        lib.rb_rmsnorm_rows_ld.argtypes = [P, I, P, I, F, F, P, I, I, I, I, P]
        lib.rb_rmsnorm_rows_ld.restype = c_int
        lib.rb_swiglu.argtypes = [P, P, I, I, I, I, P]
        lib.rb_gemm_f32.argtypes = [P, P, P, I, I, I, I, I, I, P]
        lib.rb_gemm_skinny.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P]
        lib.rb_gemm_skinny.restype = c_int
        lib.rb_gemm_skinny_act.argtypes = [P, P, P, I, I, P, I, I, I, I, I, I, I, P]
        lib.rb_gemm_skinny_act.restype = c_int
        lib.rb_gemm_skinny_fused.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, I, I, F, P, P, I, F, P, I, P]
        lib.rb_gemm_skinny_fused.restype = c_int
        lib.rb_gemm_skinny_ctas.argtypes = [I]
        lib.rb_gemm_skinny_ctas.restype = c_int
        lib.rb_qk_norm_rope_write.argtypes = [P, I, P, P, I, F, F, P, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, P]
        lib.rb_attention_simt.argtypes = [P, I, P, P, P, P, P, I, I, P, I, I, I, I, I, F, I, P]
        lib.rb_attention_simt_mod.argtypes = [P, I, P, P, P, P, P, I, I, P, I, I, I, I, I, F, I, I, F, P, P, P]
        lib.rb_attn_prep.argtypes = [P, I, I, I, I, P, P, P, I, P, P, I, F, P, P, I, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, I, P]
        lib.rb_attn_gate.argtypes = [P, P, I, I, I, I, I, I, I, I, P]
        lib.rb_embedding_pair.argtypes = [P, P, I, P, P, P, P, P, P, P, I, I, I, F, I, L, L, P]
        lib.rb_last_token.argtypes = [P, P, P, P, I, P]
        lib.rb_sample.argtypes = [P, I, I, I, P, P, P, P, P, P, I, P]
        lib.rb_argmax.argtypes = [P, I, I, I, P, P]
        lib.rb_postnorm_add_norm.argtypes = [P, P, P, I, F, F, P, I, F, F, P, I, I, I, P]
        lib.rb_softcap.argtypes = [P, F, ctypes.c_longlong, P]
        for name in ("rb_embedding", "rb_add_rmsnorm", "rb_rmsnorm_rows", "rb_swiglu", "rb_gemm_f32",
                     "rb_qk_norm_rope_write", "rb_attention_simt", "rb_sample", "rb_argmax", "rb_postnorm_add_norm",
                     "rb_softcap", "rb_activation", "rb_hyper_read_norm", "rb_hyper_write", "rb_attention_simt_mod",
                     "rb_attn_prep", "rb_attn_gate", "rb_embedding_pair", "rb_last_token"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


# head sizes compiled ahead of time by build_all(); any other multiple of 16 compiles on first use
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)


def build_all():
    """Compiles every library of the package (nvcc cross-compiles, no GPU needed); returns the paths."""
    paths = [build.library_path("return_core", _CORE_SOURCES, {"RB_PDL_MODE": PDL_MODE})]
    paths.append(build.library_path("return_tc5", _TC5_SOURCES, _tc5_defines()))
    paths.append(build.library_path("return_recurrent", _RECURRENT_SOURCES, {"RB_PDL_MODE": PDL_MODE}))
    paths.append(build.library_path("return_latent", _LATENT_SOURCES, {"RB_PDL_MODE": PDL_MODE}))
    paths.append(build.library_path("return_moe", _MOE_SOURCES, {"RB_PDL_MODE": PDL_MODE}))
    paths.append(build.library_path("return_moe_tc5", _MOE_TC5_SOURCES, {"RB_PDL_MODE": PDL_MODE}))
    for d in TC5_ATTENTION_HEAD_DIMS:
        paths.append(build.library_path(f"return_attn_tc5_d{d}", ["attention_tc5.cu"], _attn_tc5_defines(d)))
    for d in PREBUILT_HEAD_DIMS:
        paths.append(build.library_path(f"return_attn_d{d}", ["attention_mma.cu"], _attn_defines(d)))
    return paths


# ------------------------------------------------------------------------------- elementwise

def embedding(table: torch.Tensor, tokens: torch.Tensor, stream_out: torch.Tensor, scale: float = 1.0) -> None:
    """stream_out[t] = scale * float32(table[tokens[t]]); tokens int32 [T], stream_out float32 [T, H], or [T, S, H] for a
    model that keeps S residual streams (all S start as the embedded token)."""
    T, H = stream_out.shape[0], stream_out.shape[-1]
    copies = stream_out.shape[1] if stream_out.dim() == 3 else 1
    assert tokens.dtype == torch.int32 and stream_out.dtype == torch.float32
    assert table.shape[1] == H and table.is_contiguous() and stream_out.is_contiguous()
    _check(core().rb_embedding(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(stream_out),
                               T, H, table.shape[0], float(scale), copies, _stream()), "embedding")


def embedding_pair(table, pairs, batch, last_token, stream_out, scale: float, buckets: int, mul_prev: int, mul_cur: int) -> None:
    """stream_out[t] = scale * table[token] + pairs[row]: row = (previous token * mul_prev + token * mul_cur) mod buckets,
    or row ``buckets`` for a sequence's first token.  The token before a segment's first one is ``last_token`` (int32, one
    per state slot) of the segment's request; ``last_token_update`` renews it after the step."""
    T, H = stream_out.shape
    assert tuple(table.shape[1:]) == (H,) and tuple(pairs.shape) == (buckets + 1, H) and pairs.dtype == table.dtype
    assert table.is_contiguous() and pairs.is_contiguous() and stream_out.is_contiguous() and stream_out.dtype == torch.float32
    assert last_token.dtype == torch.int32 and batch.tokens.dtype == torch.int32
    _check(core().rb_embedding_pair(_ptr(table), _ptr(pairs), dtype_code(table.dtype), _ptr(batch.tokens), _ptr(batch.pos),
                                    _ptr(batch.tok_seg), _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(last_token),
                                    _ptr(stream_out), T, H, table.shape[0], scale, buckets, mul_prev, mul_cur, _stream()),
           "embedding_pair")


def last_token_update(batch, last_token) -> None:
    """last_token[slot of a segment's request] = the segment's last token, for every segment of the step."""
    assert last_token.dtype == torch.int32
    _check(core().rb_last_token(_ptr(batch.tokens), _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(last_token),
                                batch.num_segments, _stream()), "last_token")


ACTIVATIONS = {"relu2": 0, "tanh": 1, "gelu_tanh": 2, "silu": 3, "neg_exp_exp": 4}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str, bias: Optional[torch.Tensor] = None) -> None:
    """out = f(x) over 2-d views with unit stride along a row (in place when out is x): ``relu2`` max(x, 0)^2, ``tanh``,
    ``gelu_tanh``, ``silu``, ``neg_exp_exp`` exp(-exp(x + bias)) with a bias per column.  float32 arithmetic."""
    assert x.dim() == 2 and out.shape == x.shape and x.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert kind == "neg_exp_exp" and bias.numel() == x.shape[1] and bias.is_contiguous()
    _check(core().rb_activation(_ptr(x), x.stride(0), dtype_code(x.dtype), _ptr(out), out.stride(0), dtype_code(out.dtype),
                                ACTIVATIONS[kind], _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                x.shape[0], x.shape[1], _stream()), "activation")


HYPER_MAX_STREAMS = 8


def hyper_read_norm(streams: torch.Tensor, read: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                    rows: Optional[torch.Tensor] = None, offset: float = 0.0) -> None:
    """out = rmsnorm(sum_s read[s] * streams[:, s]) * (offset + weight).  streams float32 [T, S, H]; read float32 [S] or
    None for the plain sum of the streams; ``rows`` (int32) picks the token rows (out then has one row per entry)."""
    T, S, H = streams.shape
    n = T if rows is None else rows.numel()
    assert streams.dtype == torch.float32 and streams.is_contiguous() and out.is_contiguous() and out.shape == (n, H)
    assert weight.numel() == H and (read is None or (read.dtype == torch.float32 and read.numel() == S))
    assert rows is None or rows.dtype == torch.int32
    _check(core().rb_hyper_read_norm(_ptr(streams), _ptr(read), _ptr(rows), _ptr(weight), dtype_code(weight.dtype), eps, offset,
                                     _ptr(out), dtype_code(out.dtype), n, S, H, _stream()), "hyper_read_norm")


def hyper_write(streams: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, write: torch.Tensor, nxt=None,
                out: Optional[torch.Tensor] = None) -> None:
    """streams[:, t] <- sum_s mix[s, t] * streams[:, s] + write[t] * y for all t at once, in place (streams float32
    [T, S, H]; mix float32 [S, S] indexed [from, to]; write float32 [S]; y [T, H] float32 or the activation type).  With
    ``nxt`` = (read or None, weight, eps, offset) and ``out``, the read of the sublayer that runs next is done on the
    new streams in the same kernel: out = rmsnorm(sum_t read[t] * streams[:, t]) * (offset + weight)."""
    T, S, H = streams.shape
    assert streams.dtype == torch.float32 and streams.is_contiguous() and y.shape == (T, H) and y.is_contiguous()
    assert mix.dtype == write.dtype == torch.float32 and mix.shape == (S, S) and mix.is_contiguous() and write.numel() == S
    read, weight, eps, offset = nxt if nxt is not None else (None, None, 0.0, 0.0)
    if out is not None:
        assert weight is not None and weight.numel() == H and out.shape == (T, H) and out.is_contiguous()
        assert read is None or (read.dtype == torch.float32 and read.numel() == S)
        act = dtype_code(out.dtype)
    else:
        act = dtype_code(y.dtype)
    assert act == F32 or y.dtype in (torch.float32, torch.bfloat16)
    if act == F32:
        assert y.dtype == torch.float32
    _check(core().rb_hyper_write(_ptr(streams), _ptr(y), 1 if y.dtype == torch.float32 else 0, _ptr(mix), _ptr(write),
                                 _ptr(read), _ptr(weight), dtype_code(weight.dtype) if weight is not None else F32, eps,
                                 offset, _ptr(out), act, T, S, H, _stream()), "hyper_write")


def add_rmsnorm(stream: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, offset: float = 0.0) -> None:
    """stream += delta (written back unless ``rows``); out = rmsnorm(stream) * (offset + weight).

    ``rows`` (int32) picks the rows to normalise; out then has one row per entry of ``rows``.
    """
    H = stream.shape[1]
    n = out.shape[0]
    assert stream.dtype == torch.float32 and stream.is_contiguous() and out.is_contiguous()
    assert out.shape[1] == H and weight.numel() == H
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape == stream.shape and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert n == stream.shape[0]
    _check(core().rb_add_rmsnorm(_ptr(stream), _ptr(delta), _ptr(rows), _ptr(weight), dtype_code(weight.dtype),
                                 eps, offset, _ptr(out), dtype_code(out.dtype), n, H, _stream()), "add_rmsnorm")


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, offset: float = 0.0) -> None:
    """out = rmsnorm over the last dim of contiguous x [..., N]."""
    N = x.shape[-1]
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == x.dtype and weight.numel() == N
    _check(core().rb_rmsnorm_rows(_ptr(x), _ptr(weight), dtype_code(weight.dtype), eps, offset, _ptr(out),
                                  dtype_code(x.dtype), x.numel() // N, N, _stream()), "rmsnorm_rows")


def rmsnorm_columns(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, offset: float = 0.0) -> None:
    """out = rmsnorm over the last dim of x [T, N], where x and out may be runs of columns of wider buffers (any row
    stride, unit stride along a row)."""
    T, N = x.shape
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == x.shape and out.dtype == x.dtype and weight.numel() == N
    _check(core().rb_rmsnorm_rows_ld(_ptr(x), x.stride(0), _ptr(weight), dtype_code(weight.dtype), eps, offset, _ptr(out),
                                     out.stride(0), dtype_code(x.dtype), T, N, _stream()), "rmsnorm_columns")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
    """out = silu(gate) * up.  ``interleave`` 0: gate_up[t] = [gate | up]; 8: blocks of 8 gate then 8 up."""
    T, I2 = gate_up.shape
    assert out.shape == (T, I2 // 2) and gate_up.is_contiguous() and out.is_contiguous()
    assert out.dtype == gate_up.dtype and interleave in (0, 8)
    _check(core().rb_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I2 // 2, interleave, _stream()), "swiglu")


def postnorm_add_norm(stream: torch.Tensor, delta: torch.Tensor, post, nxt=None, out: Optional[torch.Tensor] = None) -> None:
    """stream (float32) += rmsnorm(delta) * (offset + w) with ``post`` = (w, eps, offset); with ``nxt`` = (w, eps, offset)
    and ``out``, also out = rmsnorm(stream) * (offset + w): the joint between two sublayers of a layer that norms a
    sublayer's output as well as its input."""
    T, H = stream.shape
    assert stream.dtype == torch.float32 and stream.is_contiguous() and delta.shape == stream.shape and delta.is_contiguous()
    wp, eps_p, off_p = post
    assert wp.numel() == H
    wn, eps_n, off_n = nxt if nxt is not None else (None, 0.0, 0.0)
    if out is not None:
        assert wn is not None and wn.numel() == H and out.shape == stream.shape and out.is_contiguous() and out.dtype == delta.dtype
    _check(core().rb_postnorm_add_norm(_ptr(stream), _ptr(delta), _ptr(wp), dtype_code(wp.dtype), eps_p, off_p, _ptr(wn),
                                       dtype_code(wn.dtype) if wn is not None else F32, eps_n, off_n, _ptr(out),
                                       dtype_code(delta.dtype), T, H, _stream()), "postnorm_add_norm")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap), in place; float32."""
    assert x.dtype == torch.float32 and x.is_contiguous() and cap > 0
    _check(core().rb_softcap(_ptr(x), float(cap), x.numel(), _stream()), "softcap")


# ------------------------------------------------------------------------------- matrix products

def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == out.dtype == torch.float32
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().rb_gemm_f32(_ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                              _stream()), "gemm_f32")


SKINNY_KERNEL_MAX_ROWS = 32     # what the kernel takes
SKINNY_MAX_ROWS = 8             # what the engine gives it: beyond 8 rows the library is faster (38 us against 58 at
                                # 16 rows and 106 at 32, for N = 24576, K = 4096)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False, act: Optional[str] = None,
                bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 32 in bfloat16: the weight-streaming kernel of decode steps
    (the engine uses it up to 8 rows).
    ``gated``: w holds gate and up rows interleaved in blocks of 8; out[M, N/2] = silu(gate) * up.
    ``act``: one of ``ACTIVATIONS`` applied to the float32 sums before they are stored (``bias``: its bias per column)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N) and M <= SKINNY_KERNEL_MAX_ROWS
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if act is not None:
        assert not gated and (bias is None or (act == "neg_exp_exp" and bias.numel() == N and bias.is_contiguous()))
        _check(core().rb_gemm_skinny_act(_ptr(x), _ptr(w), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                         ACTIVATIONS[act], _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                         M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()), "gemm_skinny_act")
        return
    _check(core().rb_gemm_skinny(_ptr(x), _ptr(w), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                 1 if gated else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()),
           "gemm_skinny")


class RowSums:
    """Where a product in its residual form leaves each CTA's share of sum(v^2) per token, for the norm that follows:
    the product that takes the normed rows multiplies its result by rstd = 1 / sqrt(sum / dim + eps) instead of
    anyone norming them.  ``parts``: float32 [8, width]; ``count``: the shares that were written; ``dim``: the length
    of the normed row."""
    WIDTH = 512

    def __init__(self, parts: torch.Tensor, dim: int, count: int = 0):
        self.parts, self.dim, self.count = parts, dim, count


def gemm_skinny_fused(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], gated: bool = False, scale=None,
                      residual=None) -> None:
    """The weight-streaming product for up to 8 rows with the norm and the residual add around it folded in.

    ``scale`` = (RowSums, eps): the accumulators are multiplied by each token's rstd, the factor that the norm
    before this product would have applied (its input rows are v * (offset + weight), not normed).
    ``residual`` = (stream, next_norm, sums): v = stream + acc goes to ``stream`` (float32 [M, N]); with
    ``next_norm`` = (weight, offset), ``out`` [M, N] gets v * (offset + weight) for the next product; ``sums``
    (a RowSums, or None) gets the shares of sum(v^2)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and M <= 8 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1
    lib = core()
    ssq_in, ssq_in_count, norm_dim, eps = None, 0, 0, 0.0
    if scale is not None:
        sums_in, eps = scale
        assert sums_in.count > 0 and sums_in.parts.dtype == torch.float32 and sums_in.parts.is_contiguous()
        ssq_in, ssq_in_count, norm_dim = sums_in.parts, sums_in.count, sums_in.dim
    stream = norm_w = ssq_out = None
    norm_w_dtype, offset = F32, 0.0
    if residual is not None:
        stream, next_norm, sums_out = residual
        assert not gated and stream.dtype == torch.float32 and stream.is_contiguous() and stream.shape == (M, N)
        if next_norm is not None:
            norm_w, offset = next_norm
            assert out is not None and norm_w.numel() == N
            norm_w_dtype = dtype_code(norm_w.dtype)
        if sums_out is not None:
            assert sums_out.parts.dtype == torch.float32 and sums_out.parts.is_contiguous() and sums_out.dim == N
            sums_out.count = lib.rb_gemm_skinny_ctas(N)
            assert sums_out.count <= sums_out.parts.shape[1]
            ssq_out = sums_out.parts
    if out is not None:
        assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    ld_sums = (ssq_in if ssq_in is not None else ssq_out).shape[1] if (ssq_in is not None or ssq_out is not None) else 0
    if ssq_in is not None and ssq_out is not None:
        assert ssq_in.shape[1] == ssq_out.shape[1]
    _check(lib.rb_gemm_skinny_fused(_ptr(x), _ptr(w), _ptr(out), 1 if residual is not None else 0, 1 if gated else 0,
                                    M, N, K, x.stride(0), w.stride(0), out.stride(0) if out is not None else 0,
                                    _ptr(ssq_in), ssq_in_count, norm_dim, eps, _ptr(stream), _ptr(norm_w), norm_w_dtype,
                                    offset, _ptr(ssq_out), ld_sums, _stream()), "gemm_skinny_fused")


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product (few rows, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# From this many rows on, the gated product of a feed-forward runs as 256 x 256 tiles by pairs of CTAs with the gating
# in the epilogue: measured against cuBLAS + the SwiGLU kernel at [rows, 4096] x [24576, 4096]: 83 / 81 us at 512 rows,
# 111 / 112 at 768, 276 / 302 at 2,048, 508 / 623 at 4,096.
PAIR_MIN_ROWS = 768


def pair_ok(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 kernels (TMA-fed) take this product: bfloat16, rows of whole 16-byte pieces."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and w.shape[0] % 16 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gated_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, interleave: int, ctx=None) -> None:
    """out[T, I] = silu(x @ gate^T) * (x @ up^T) for the fused weight ``w`` [2I, K] of a gated
    feed-forward.  With the interleaved layout the product's epilogue does the gating where an own kernel
    is the fastest: for few rows (weight streaming) and for many (tcgen05, pairs of CTAs); otherwise a product
    into a [T, 2I] buffer (from ``ctx``, a parts.base.LayerContext, if given) is followed by the SwiGLU kernel."""
    if interleave == 8 and skinny_ok(x, w):
        gemm_skinny(x, w, out, gated=True)
        return
    if interleave == 8 and x.shape[0] >= PAIR_MIN_ROWS and pair_ok(x, w, out):
        gemm_tc5(x, w, out, gated=True, pair=True)
        return
    if ctx is not None:
        gu = ctx.buffer("gated_linear.gate_up", (x.shape[0], w.shape[0]), x.dtype, x.device)
    else:
        gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
    linear(x, w, gu)
    swiglu(gu, out, interleave)


_tc5 = None
_TC5_SOURCES = ["gemm_tc5.cu", "gemm_stream.cu"]


def _tc5_defines():
    return {"RB_PDL_MODE": PDL_MODE}


def tc5_lib() -> ctypes.CDLL:
    """The tcgen05 / TMA matrix-product library."""
    global _tc5
    if _tc5 is None:
        lib = build.load("return_tc5", _TC5_SOURCES, _tc5_defines())
        P, I = c_void_p, c_int
        lib.rb_gemm_stream.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_gemm_stream.restype = c_int
        lib.rb_gemm_stream_plan.argtypes = [I, I, I, I, P]
        lib.rb_gemm_stream_plan.restype = None
        lib.rb_tc5_gemm.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_pair.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_pair.restype = c_int
        lib.rb_tc5_gemm_simple.argtypes = [P, P, P, I, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm_bmn.argtypes = [P, P, P, I, I, I, I, I, I, I, P, P]
        lib.rb_tc5_gemm.restype = lib.rb_tc5_gemm_simple.restype = lib.rb_tc5_gemm_bmn.restype = c_int
        _tc5 = lib
    return _tc5


_tc5_status = {}


def tc5_status(device) -> torch.Tensor:
    """One int per device that a tcgen05 kernel raises when one of its bounded waits gave up."""
    t = _tc5_status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _tc5_status[device] = t
    return t


_tc5_launched = set()          # devices on which a kernel with bounded waits ran since the status word was last read


def check_status(device) -> None:
    """Reads the status word of the tcgen05 kernels if one of them ran on ``device`` since the last check, and
    raises ``KernelError`` if a bounded wait gave up (the kernel's output is then not to be trusted).  It
    synchronises, so callers use it where they wait for the step anyway (after sampling, after a replayed step)."""
    device = torch.device(device)
    if device not in _tc5_launched:
        return
    _tc5_launched.discard(device)
    t = _tc5_status.get(device)
    if t is None:
        return
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelError(f"a kernel on {device} gave up a bounded wait (an mbarrier, or the other CTAs of its grid) or "
                          f"found its shared memory misaligned (status {code}); the step's output is not valid")


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False, simple_bn: int = 0,
             pair: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed).  ``gated``: SwiGLU epilogue over
    woven gate/up rows of w, out [M, N/2].  ``simple_bn``: run the one-stage twin with that tile width.
    ``pair``: 256 x 256 tiles by pairs of CTAs (two-SM MMAs)."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    status = tc5_status(x.device)
    f32 = 1 if out.dtype == torch.float32 else 0
    if simple_bn:
        rc = tc5_lib().rb_tc5_gemm_simple(_ptr(x), _ptr(w), _ptr(out), f32, simple_bn, M, N, K, x.stride(0),
                                          w.stride(0), out.stride(0), _ptr(status), _stream())
    else:
        fn = tc5_lib().rb_tc5_gemm_pair if pair else tc5_lib().rb_tc5_gemm
        rc = fn(_ptr(x), _ptr(w), _ptr(out), f32, 1 if gated else 0, M, N, K, x.stride(0),
                w.stride(0), out.stride(0), _ptr(status), _stream())
    _tc5_launched.add(x.device)
    _check(rc, "gemm_tc5")


STREAM_MAX_ROWS = 128


def stream_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 weight-streaming kernel takes this product."""
    return (x.dtype == torch.bfloat16 and x.shape[0] <= STREAM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 128 in bfloat16: weights streamed by TMA through tcgen05 with the
    operand roles exchanged (weight rows on the 128 tensor-memory lanes, tokens as columns), the rows dealt out
    evenly to one CTA per SM.  ``gated``: w holds gate and up rows woven in blocks of 8; out[M, N/2] = silu(gate) * up."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert w.shape[1] == K and out.shape == (M, N // 2 if gated else N) and M <= STREAM_MAX_ROWS
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(tc5_lib().rb_gemm_stream(_ptr(x), _ptr(w), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                    1 if gated else 0, M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                    _ptr(tc5_status(x.device)), _stream()), "gemm_stream")


def gemm_stream_plan(M: int, N: int, K: int, gated: bool = False):
    """(rows of the largest range, chunks per CTA, rows of the tallest chunk, parts of K side by side on the lanes)
    on the current device."""
    buf = (c_int * 4)()
    tc5_lib().rb_gemm_stream_plan(M, N, K, 1 if gated else 0, buf)
    return tuple(buf)


def gemm_tc5_bmn(x: torch.Tensor, b: torch.Tensor, out: torch.Tensor, bn: int = 128) -> None:
    """out[M, N] (float32) = x[M, K] @ b[K, N], b row-major: the tcgen05 twin with an MN-major B operand."""
    M, K = x.shape
    N = b.shape[1]
    assert x.dtype == b.dtype == torch.bfloat16 and out.dtype == torch.float32 and b.shape[0] == K
    _check(tc5_lib().rb_tc5_gemm_bmn(_ptr(x), _ptr(b), _ptr(out), bn, M, N, K, x.stride(0), b.stride(0), out.stride(0),
                                     _ptr(tc5_status(x.device)), _stream()), "gemm_tc5_bmn")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: Optional[str] = None,
           bias: Optional[torch.Tensor] = None) -> None:
    """out = x @ w^T.  float32: the engine's own FFMA kernel.  bfloat16 with up to 8 rows: the
    engine's weight-streaming kernel.  bfloat16 with more rows: cuBLAS with float32 accumulation.
    The output is bfloat16 or float32 (``out``'s dtype).  ``act``: out = f(x @ w^T) for one of ``ACTIVATIONS``
    (``bias``: its bias per column): in the weight-streaming kernel's epilogue, else a launch of its own in place."""
    if x.dtype == torch.float32:
        gemm_f32(x, w, out)
        if act is not None:
            activation(out, out, act, bias)
        return
    if not x.is_cuda:
        raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if skinny_ok(x, w):
        gemm_skinny(x, w, out, act=act, bias=bias)
        return
    if out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        torch.mm(x, w.t(), out=out)
    if act is not None:
        activation(out, out, act, bias)


# ------------------------------------------------------------------------------- attention

def qk_norm_rope_write(qkv, q_weight, k_weight, eps, cos, sin, rot_dim, pos, tok_seg, block_table,
                       page_size, k_pool, v_pool, num_heads, num_kv_heads, head_dim, write_kv=True,
                       offset=0.0) -> None:
    """In place on qkv [T, (Hq+2Hkv)*D]: q heads normed and rotated; k heads normed, rotated and
    written to ``k_pool``; v heads written to ``v_pool``.  Pools: [pages, Hkv, P, D]."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    assert pos.dtype == tok_seg.dtype == block_table.dtype == torch.int32
    assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
    if rot_dim:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32
        assert cos.shape[1] * 2 == rot_dim and cos.is_contiguous() and sin.is_contiguous()
        assert rot_dim <= head_dim
    else:
        cos = sin = pos            # never read: a rotary width of zero rotates nothing
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    if q_weight is not None:
        assert k_weight is not None and k_weight.dtype == q_weight.dtype
    _check(core().rb_qk_norm_rope_write(
        _ptr(qkv), qkv.stride(0), _ptr(q_weight), _ptr(k_weight), wd, eps, offset, _ptr(cos), _ptr(sin),
        rot_dim, _ptr(pos), _ptr(tok_seg), _ptr(block_table), block_table.stride(0), page_size,
        _ptr(k_pool), _ptr(v_pool), dtype_code(qkv.dtype), T, num_heads, num_kv_heads, head_dim,
        1 if write_kv else 0, _stream()), "qk_norm_rope_write")


def attention_simt(qkv, k_pool, v_pool, pos, tok_seg, block_table, page_size, out, num_heads,
                   num_kv_heads, head_dim, scale, window=0) -> None:
    """Paged causal attention, one warp per (token, head); out [T, Hq*D]."""
    T = qkv.shape[0]
    assert out.is_contiguous() and out.dtype == qkv.dtype and k_pool.dtype == qkv.dtype
    _check(core().rb_attention_simt(
        _ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(pos), _ptr(tok_seg), _ptr(block_table),
        block_table.stride(0), page_size, _ptr(out), dtype_code(qkv.dtype), T, num_heads, num_kv_heads,
        head_dim, scale, int(window or 0), _stream()), "attention_simt")


_attn_libs = {}


def _attn_defines(head_dim: int):
    return {"HEAD_DIM": head_dim, "RB_PDL_MODE": PDL_MODE}


def attention_lib(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels, compiled for this head size on first use."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise KernelError(f"head_dim={head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        lib = build.load(f"return_attn_d{head_dim}", ["attention_mma.cu"], _attn_defines(head_dim))
        P, I, F = c_void_p, c_int, c_float
        lib.rb_attn_prefill.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, P, P]
        lib.rb_attn_decode.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, P, I, I, F, I, I, P, P]
        lib.rb_attn_decode_fused.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, P, I, I, F, I, I, P, P, I, F, F, P, P, I, I, P]
        lib.rb_attn_decode_fused.restype = c_int
        lib.rb_attn_prefill_mod.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, P, I, F, P, P]
        lib.rb_attn_decode_mod.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, P, I, I, F, I, I, P, I, F, P, P]
        lib.rb_attn_prefill_mod.restype = lib.rb_attn_decode_mod.restype = c_int
        lib.rb_attn_decode_scratch_floats.argtypes = [I, I, I]
        lib.rb_attn_decode_scratch_floats.restype = ctypes.c_longlong
        lib.rb_attn_prefill.restype = lib.rb_attn_decode.restype = lib.rb_attn_head_dim.restype = c_int
        if lib.rb_attn_head_dim() != head_dim:
            raise KernelError("attention library was compiled for another head size")
        _attn_libs[head_dim] = lib
    return lib


_attn_tc5_libs = {}
TC5_ATTENTION_HEAD_DIMS = (64, 128)
TC5_TILE_ROWS = 256            # query rows of one CTA of the tcgen05 prefill attention kernel
MMA_TILE_ROWS = 64             # query rows of one CTA of the mma.sync prefill attention kernel
TILES_TC5, TILES_MMA = "attention.rows256", "attention.rows64"     # the names of their tables in a step's batch

_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device (asked of the driver once).  Where no device is
    visible (the dispatch rules are also tested on the host) the count of a B200 stands in."""
    global _num_sms
    if _num_sms is None:
        _num_sms = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                    if torch.cuda.is_available() else 148)
    return _num_sms


def _attn_tc5_defines(head_dim: int):
    return {"HEAD_DIM": head_dim}


def attention_tc5_lib(head_dim: int) -> ctypes.CDLL:
    """The tcgen05 prefill attention kernel, compiled for this head size (64 or 128) on first use."""
    lib = _attn_tc5_libs.get(head_dim)
    if lib is None:
        if head_dim not in TC5_ATTENTION_HEAD_DIMS:
            raise KernelError(f"head_dim={head_dim}: the tcgen05 attention kernel takes {TC5_ATTENTION_HEAD_DIMS}")
        lib = build.load(f"return_attn_tc5_d{head_dim}", ["attention_tc5.cu"], _attn_tc5_defines(head_dim))
        P, I, F = c_void_p, c_int, c_float
        lib.rb_attn_prefill_tc5.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, I, P, I, P, P, P]
        lib.rb_attn_prefill_tc5_mod.argtypes = [P, I, P, P, P, I, P, P, P, I, I, P, I, I, F, I, I, P, I, P, P, I, F, P, P]
        lib.rb_attn_prefill_tc5_mod.restype = c_int
        lib.rb_attn_tc5_split_floats.argtypes = [I, I, I]
        lib.rb_attn_tc5_split_floats.restype = ctypes.c_longlong
        lib.rb_attn_prefill_tc5.restype = c_int
        _attn_tc5_libs[head_dim] = lib
    return lib


def _sink_ptr(sink, num_heads):
    if sink is None:
        return None
    assert sink.dtype == torch.float32 and sink.numel() == num_heads and sink.is_contiguous()
    return _ptr(sink)


def attention_prefill_tc5(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, block_table, page_size, out, num_heads,
                          num_kv_heads, head_dim, scale, window=0, num_splits=1, held=None, sink=None,
                          chunk=0, softcap=0.0, slopes=None) -> None:
    """tcgen05 attention for the listed (segment, first row) blocks of up to TC5_TILE_ROWS query rows
    (the blocks with the longest contexts should come first: they take longest).  ``num_splits`` > 1 splits
    every block's keys over that many CTAs and merges them in a second launch; ``held``: the step's map of
    work buffers, so that the layers share the buffer of the partial results.  ``chunk``, ``softcap``, ``slopes``: the
    score options of ``paged_attention``."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.is_contiguous()
    lib = attention_tc5_lib(head_dim)
    T = qkv.shape[0]
    _tc5_launched.add(qkv.device)
    scratch = None
    if num_splits > 1:
        key = ("attention.prefill_split_scratch", num_splits, T, num_heads, head_dim)
        scratch = held.get(key) if held is not None else None
        if scratch is None:
            scratch = torch.empty(lib.rb_attn_tc5_split_floats(num_splits, T, num_heads), dtype=torch.float32, device=qkv.device)
            if held is not None:
                held[key] = scratch
    _check(lib.rb_attn_prefill_tc5_mod(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(tiles),
                                       tiles.shape[0], _ptr(cu_q), _ptr(seg_pos0), _ptr(block_table),
                                       block_table.stride(0), page_size, _ptr(out), num_heads, num_kv_heads, scale,
                                       int(window or 0), num_splits, _ptr(scratch), T, _ptr(tc5_status(qkv.device)),
                                       _sink_ptr(sink, num_heads), int(chunk or 0), float(softcap or 0.0),
                                       _sink_ptr(slopes, num_heads), _stream()), "attention_prefill_tc5", 2 if num_splits > 1 else 1)


PREFILL_SPLIT_MIN_KEYS = 512       # a CTA of a split block keeps at least this many keys


def prefill_splits(n_ctas: int, longest_context: int) -> int:
    """How many ways the keys of the prompt blocks are split: a CTA owns an SM, so blocks x heads below
    the SM count leave SMs idle (a short portion of a long prompt); the keys are then shared out until the
    CTAs fill the GPU once, as long as every share keeps PREFILL_SPLIT_MIN_KEYS keys."""
    return max(1, min(num_sms() // max(1, n_ctas), longest_context // PREFILL_SPLIT_MIN_KEYS, 64))


def _prefill_split_count(batch, num_heads, window) -> int:
    held = getattr(batch, "scratch", None)
    key = ("attention.prefill_splits", num_heads, window)
    if held is not None and key in held:
        return held[key]
    host = batch.host
    tiles = host.tiles[TILES_TC5]
    longest = int(host.seg_kv_len[tiles[:, 0]].max())
    if window:
        longest = min(longest, int(window) + TC5_TILE_ROWS)
    n = prefill_splits(tiles.shape[0] * num_heads, longest)
    if held is not None:
        held[key] = n
    return n


def decode_splits(n_ctas_base: int, max_kv_len: int, ctas_per_sm: int = 2) -> int:
    """How many ways the keys of a decoded token are split.  Two CTAs share an SM (head sizes up to
    128), so the time of the launch goes with (waves of CTAs) x (keys per CTA); the split count that
    makes this smallest wins, with at least 128 keys per CTA and the smaller count on a tie."""
    tiles = max(1, (max_kv_len + 15) // 16)
    slots = num_sms() * ctas_per_sm
    best, best_cost = 1, None
    for s in range(1, 65):
        if s > 1 and (max_kv_len + s - 1) // s < 128:
            break
        waves = (n_ctas_base * s + slots - 1) // slots
        cost = waves * ((tiles + s - 1) // s + 16)         # + the fixed work of a CTA, about 16 tiles' worth (3 us)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attention_prefill_mma(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, block_table, page_size, out, num_heads,
                          num_kv_heads, head_dim, scale, window=0, sink=None, chunk=0, softcap=0.0, slopes=None) -> None:
    """Tensor-core attention for the listed (segment, first row) tiles of up to 64 query rows.  ``chunk``, ``softcap``,
    ``slopes``: the score options of ``paged_attention``."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.is_contiguous()
    lib = attention_lib(head_dim)
    _check(lib.rb_attn_prefill_mod(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(tiles), tiles.shape[0],
                                   _ptr(cu_q), _ptr(seg_pos0), _ptr(block_table), block_table.stride(0), page_size,
                                   _ptr(out), num_heads, num_kv_heads, scale, int(window or 0), _sink_ptr(sink, num_heads),
                                   int(chunk or 0), float(softcap or 0.0), _sink_ptr(slopes, num_heads), _stream()),
           "attention_prefill")


def _split_scratch(lib, n, num_heads, num_splits, device, held=None):
    """The buffer in which the splits of the keys leave their partial results (none for one split).
    ``held``: the step's map of work buffers; every layer of the step then shares one."""
    key = ("attention.split_scratch", n, num_heads, num_splits)
    if held is not None and key in held:
        return held[key]
    floats = lib.rb_attn_decode_scratch_floats(n, num_heads, num_splits)
    scratch = torch.empty(floats, dtype=torch.float32, device=device) if floats else None
    if held is not None:
        held[key] = scratch
    return scratch


def attention_decode_mma(qkv, k_pool, v_pool, decode_segs, cu_q, seg_kv_len, block_table, page_size, out,
                         num_heads, num_kv_heads, head_dim, scale, window=0, num_splits=1, held=None, sink=None,
                         chunk=0, softcap=0.0, slopes=None) -> None:
    """Tensor-core attention for segments of one token, the keys split ``num_splits`` ways.  ``chunk``, ``softcap``,
    ``slopes``: the score options of ``paged_attention``."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    lib = attention_lib(head_dim)
    n = decode_segs.shape[0]
    scratch = _split_scratch(lib, n, num_heads, num_splits, qkv.device, held)
    _check(lib.rb_attn_decode_mod(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(decode_segs), n,
                                  _ptr(cu_q), _ptr(seg_kv_len), _ptr(block_table), block_table.stride(0), page_size,
                                  _ptr(scratch), _ptr(out), num_heads, num_kv_heads, scale, int(window or 0),
                                  num_splits, _sink_ptr(sink, num_heads), int(chunk or 0), float(softcap or 0.0),
                                  _sink_ptr(slopes, num_heads), _stream()), "attention_decode", 2 if num_splits > 1 else 1)


def _decode_split_count(batch, num_heads, num_kv_heads, window) -> int:
    """The split count of this step's decoded tokens, worked out once per step and kind of layer."""
    held = getattr(batch, "scratch", None)
    if held is None:
        return _decode_split_count_now(batch, num_heads, num_kv_heads, window)
    key = ("attention.splits", num_heads, num_kv_heads, window)
    n = held.get(key)
    if n is None:
        n = held[key] = _decode_split_count_now(batch, num_heads, num_kv_heads, window)
    return n


def _decode_split_count_now(batch, num_heads, num_kv_heads, window) -> int:
    host = batch.host
    n_dec = host.decode_segs.shape[0]
    group = num_heads // num_kv_heads
    base = n_dec * num_kv_heads * ((group + 15) // 16)
    longest = int(host.seg_kv_len[host.decode_segs].max())
    if window:
        longest = min(longest, int(window))
    fixed = getattr(batch, "variant", {}).get(decode_splits_key(num_heads, num_kv_heads, window))
    return fixed or decode_splits(base, longest)


def decode_splits_key(num_heads, num_kv_heads, window):
    """Under this key a captured step holds the split count of its decoded tokens (``batch.variant``)."""
    return ("attention.decode_splits", num_heads, num_kv_heads, window or 0)


def decode_splits_for(n_tokens: int, longest: int, num_heads: int, num_kv_heads: int, window=None) -> int:
    """The split count of a step of ``n_tokens`` single tokens whose contexts reach ``longest`` keys."""
    group = num_heads // num_kv_heads
    if window:
        longest = min(longest, int(window))
    return decode_splits(n_tokens * num_kv_heads * ((group + 15) // 16), longest)


def decode_only(batch, dtype, num_heads, num_kv_heads, window=None) -> bool:
    """Whether the step holds single decoded tokens only, runs on the tensor-core path, and is small enough
    that the decode attention kernel should norm, rotate and cache those tokens itself: the saved launch
    pays while the kernel's CTAs fit on the GPU at once; with more, the work added to every CTA costs
    more than the small kernel it replaces (measured: +1 % at 8 requests, -2 % at 64)."""
    host = batch.host
    if not (dtype == torch.bfloat16 and host.num_multi == 0
            and host.decode_segs.shape[0] == host.num_tokens and host.num_tokens > 0):
        return False
    group = num_heads // num_kv_heads
    ctas = host.num_tokens * num_kv_heads * ((group + 15) // 16) * _decode_split_count(batch, num_heads, num_kv_heads, window)
    return ctas <= 2 * num_sms()


def attention_decode_fused(qkv, q_weight, k_weight, eps, offset, cos, sin, rot_dim, k_pool, v_pool, batch,
                           block_table, page_size, out, num_heads, num_kv_heads, head_dim, scale, window=None,
                           write_kv=True) -> None:
    """A step of single tokens: per-head q/k norm, rotation, cache write and split-KV attention in one kernel
    (plus the merge of the splits).  ``qkv`` holds the raw projections and is left as it is."""
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    lib = attention_lib(head_dim)
    n = batch.decode_segs.shape[0]
    splits = _decode_split_count(batch, num_heads, num_kv_heads, window)
    scratch = _split_scratch(lib, n, num_heads, splits, qkv.device, getattr(batch, "scratch", None))
    if rot_dim:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] * 2 == rot_dim
        assert cos.is_contiguous() and sin.is_contiguous()
    else:
        cos = sin = batch.cu_q          # never read: a rotary width of zero rotates nothing
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    _check(lib.rb_attn_decode_fused(_ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(batch.decode_segs), n,
                                    _ptr(batch.cu_q), _ptr(batch.seg_kv_len), _ptr(block_table), block_table.stride(0),
                                    page_size, _ptr(scratch), _ptr(out), num_heads, num_kv_heads, scale,
                                    int(window or 0), splits, _ptr(q_weight), _ptr(k_weight), wd, eps, offset,
                                    _ptr(cos), _ptr(sin), rot_dim, 1 if write_kv else 0, _stream()),
           "attention_decode_fused", 2 if splits > 1 else 1)


def paged_attention(qkv, k_pool, v_pool, batch, block_table, page_size, out, num_heads, num_kv_heads,
                    head_dim, scale, window=None, sink=None, chunk=None, softcap=None, slopes=None) -> None:
    """Attention of every token of the step over its request's cached keys (its own included).

    float32: the CUDA-core kernel, whose result does not depend on how the work was cut.
    bfloat16: the tensor-core kernels, one for prompt portions and one (split over the keys) for
    single decoded tokens.

    Options of the score: ``window`` (the last n keys) or ``chunk`` (the keys of the query's own block of n positions,
    blocks counted from position 0), never both; ``sink`` (float32 [heads]: exp(sink) joins the softmax's denominator);
    ``softcap`` (a scaled score s becomes cap * tanh(s / cap)); ``slopes`` (float32 [heads]: slopes[h] * (i - j) is taken
    off the score of key j for query i)."""
    if window and chunk:
        raise KernelError("a window and a chunk exclude each other")
    if qkv.dtype == torch.float32:
        T = qkv.shape[0]
        assert out.is_contiguous() and out.dtype == qkv.dtype and k_pool.dtype == qkv.dtype
        _check(core().rb_attention_simt_mod(
            _ptr(qkv), qkv.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(batch.pos), _ptr(batch.tok_seg), _ptr(block_table),
            block_table.stride(0), page_size, _ptr(out), dtype_code(qkv.dtype), T, num_heads, num_kv_heads, head_dim, scale,
            int(window or 0), int(chunk or 0), float(softcap or 0.0), _sink_ptr(slopes, num_heads),
            _sink_ptr(sink, num_heads), _stream()), "attention_simt")
        return
    host = batch.host
    bound = window or chunk                       # either bounds the keys a query can see
    if host.num_multi:
        if head_dim in TC5_ATTENTION_HEAD_DIMS:
            attention_prefill_tc5(qkv, k_pool, v_pool, batch.tiles[TILES_TC5], batch.cu_q, batch.seg_pos0, block_table,
                                  page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0,
                                  _prefill_split_count(batch, num_heads, bound), getattr(batch, "scratch", None), sink,
                                  chunk, softcap, slopes)
        else:
            attention_prefill_mma(qkv, k_pool, v_pool, batch.tiles[TILES_MMA], batch.cu_q, batch.seg_pos0, block_table,
                                  page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0, sink,
                                  chunk, softcap, slopes)
    n_dec = host.decode_segs.shape[0]
    if n_dec:
        attention_decode_mma(qkv, k_pool, v_pool, batch.decode_segs, batch.cu_q, batch.seg_kv_len, block_table,
                             page_size, out, num_heads, num_kv_heads, head_dim, scale, window or 0,
                             _decode_split_count(batch, num_heads, num_kv_heads, bound), getattr(batch, "scratch", None), sink,
                             chunk, softcap, slopes)


def attention_prepare(proj, q_off: int, k_off: int, v_off: int, biases, norms, eps: float, tables, batch, kv, q_out,
                      num_heads: int, num_kv_heads: int, dim: int, vdim: int, head_dim: int, write_kv: bool = True) -> None:
    """From a step's projection rows to what the paged attention kernels read, for an attention that prepares a row as a
    whole (csrc/attention_prep.cu).  ``proj`` [T, >= ...]: q heads of ``dim`` from column ``q_off``, k heads from ``k_off``,
    v heads of ``vdim`` from ``v_off`` (``v_off`` < 0: the values are the key projection as it is).  ``biases``: None or
    (q, k, v) added first; ``norms``: None or (q weight, k weight) of an RMS norm over the whole q and the whole k
    projection; ``tables``: None or (cos, sin, rot) rotating elements (2i, 2i + 1), i < rot / 2, of every q and k head.
    q goes to ``q_out`` [T, heads * head_dim], keys and values into the pages of ``kv`` (heads padded to ``head_dim``)."""
    T = proj.shape[0]
    assert proj.stride(1) == 1 and q_out.is_contiguous() and q_out.dtype == proj.dtype
    assert tuple(q_out.shape) == (T, num_heads * head_dim) and kv.k.dtype == proj.dtype
    qb, kb, vb = biases if biases is not None else (None, None, None)
    qn, kn = norms if norms is not None else (None, None)
    cos, sin, rot = tables if tables is not None else (batch.pos, batch.pos, 0)      # never read with a width of zero
    if rot:
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] * 2 == rot and cos.is_contiguous() and sin.is_contiguous()
    _check(core().rb_attn_prep(
        _ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(qb), _ptr(kb), _ptr(vb),
        dtype_code(qb.dtype) if qb is not None else F32, _ptr(qn), _ptr(kn), dtype_code(qn.dtype) if qn is not None else F32,
        eps, _ptr(cos), _ptr(sin), rot, _ptr(batch.pos), _ptr(batch.tok_seg), _ptr(kv.block_table), kv.block_table.stride(0),
        kv.page_size, _ptr(kv.k), _ptr(kv.v), _ptr(q_out), dtype_code(proj.dtype), T, num_heads, num_kv_heads, dim, vdim,
        head_dim, 1 if write_kv else 0, _stream()), "attention_prepare")


def attention_gate(o, gate, g_off: int, per_head: bool, num_heads: int, vdim: int, head_dim: int) -> None:
    """o [T, heads * head_dim] in place: a head's first ``vdim`` elements times the logistic of their gate, taken from the
    rows of ``gate`` from column ``g_off``: one gate a head (``per_head``) or one per value element."""
    T = o.shape[0]
    assert o.is_contiguous() and gate.stride(1) == 1 and gate.dtype == o.dtype and o.shape[1] == num_heads * head_dim
    _check(core().rb_attn_gate(_ptr(o), _ptr(gate), gate.stride(0), g_off, 1 if per_head else 0, dtype_code(o.dtype), T,
                               num_heads, vdim, head_dim, _stream()), "attention_gate")


# ------------------------------------------------------------------------------- mixers with a matrix state

_recurrent = None
_RECURRENT_SOURCES = ["recurrent.cu"]
SCAN_DECAY, SCAN_MEMORY, SCAN_DELTA, SCAN_BONUS, SCAN_SSM, SCAN_DELTA_HEAD = 0, 1, 2, 3, 4, 5
SCAN_MAX_KEY_DIM = 256


def recurrent_lib() -> ctypes.CDLL:
    """The kernels of the mixers that keep a matrix state per head (csrc/recurrent.cu); compiled when a model
    that has such a mixer is first run."""
    global _recurrent
    if _recurrent is None:
        lib = build.load("return_recurrent", _RECURRENT_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I, F, L = c_void_p, c_int, c_float, ctypes.c_longlong
        lib.rb_linear_scan.argtypes = [I, P, P, P, I, I, I, I, I, I, P, P, P, F, F, P, L, I, I, I, I, P, P, P, I, I, I, I, I, P]
        lib.rb_token_shift_mix.argtypes = [P, I, P, I, I, P, L, I, P, P, P, P, I, I, I, P]
        lib.rb_ssm_prep.argtypes = [P, I, I, I, P, P, I, I, P, L, I, P, P, P, P, I, I, P, P, I, P, P, I, I, P]
        lib.rb_gated_part_norm.argtypes = [P, P, I, P, I, F, P, I, I, I, I, P]
        lib.rb_rotary_to_f32.argtypes = [P, I, I, I, P, P, I, P, P, P, I, I, I, I, F, F, P]
        lib.rb_scan_pieces_combine.argtypes = [P, L, P, L, I, P, P, P, P, I, I, I, P]
        lib.rb_scan_pieces_combine.restype = c_int
        lib.rb_scan_pieces_combine_sums.argtypes = [P, L, P, L, I, P, P, I, I, I, I, P, P, P, I, I, I, I, P]
        lib.rb_scan_pieces_combine_sums.restype = c_int
        lib.rb_memory_pieces_combine.argtypes = [P, L, P, L, I, I, I, I, P, P, I, I, I, I, P]
        lib.rb_memory_pieces_combine.restype = c_int
        lib.rb_rotary_inplace.argtypes = [P, I, P, P, I, P, I, I, I, I, P]
        lib.rb_rotary_inplace.restype = c_int
        lib.rb_delta_prep.argtypes = [P, I, P, I, I, P, L, I, P, P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, P]
        lib.rb_gated_conv.argtypes = [P, I, P, P, P, I, I, P, L, I, P, P, P, P, P, I, I, I, P]
        lib.rb_gated_recurrence.argtypes = [P, P, I, P, P, P, I, F, P, I, P, P, L, I, P, P, P, I, I, I, I, P, P]
        lib.rb_gated_pieces_combine.argtypes = [P, P, P, L, I, P, P, I, I, P]
        lib.rb_gated_conv.restype = lib.rb_gated_recurrence.restype = lib.rb_gated_pieces_combine.restype = c_int
        lib.rb_conv_state_update.argtypes = [P, I, I, P, L, I, P, P, I, I, I, P]
        lib.rb_head_norm_gate.argtypes = [P, P, I, P, I, I, I, F, P, I, I, I, I, P]
        lib.rb_add_dual_norm.argtypes = [P, P, I, F, P, I, F, P, P, P, I, F, F, P, P, I, I, I, P]
        lib.rb_scaled_sum.argtypes = [P, I, F, P, I, F, P, I, L, P]
        for name in ("rb_linear_scan", "rb_rotary_to_f32", "rb_delta_prep", "rb_conv_state_update",
                     "rb_head_norm_gate", "rb_add_dual_norm", "rb_scaled_sum", "rb_token_shift_mix", "rb_ssm_prep",
                     "rb_gated_part_norm"):
            getattr(lib, name).restype = c_int
        _recurrent = lib
    return _recurrent


def _is_f32(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise KernelError(f"the kernels take float32 and bfloat16, not {t.dtype}")


def linear_scan(mode: int, q, k, v, gate_a, gate_b, state, offsets, batch, out, heads: int, kv_heads: int,
                dim: int, vdim: int, q_scale: float = 1.0, cap: float = 0.0, forgot_offset: int = -1, extra=None) -> None:
    """The recurrence of a mixer with a [dim, vdim] state per head, over every segment of the step, token by token.

    q, k: [T, >= kv_heads * dim] views (float32 or bfloat16, unit stride along a row), v: [T, >= heads * vdim];
    ``state``: float32 [slots, n], the row of a segment is ``batch.seg_slot``; ``offsets`` = (S, n, m): where the
    matrix, the normaliser and the running maximum start inside a row (the last two for ``SCAN_MEMORY`` only).
    ``gate_a`` / ``gate_b`` by mode: SCAN_DECAY: [heads] decays / None; SCAN_MEMORY: [T, 2 heads] gate
    pre-activations (input, forget) / [2 heads] biases; SCAN_DELTA: [T, heads, dim] row decays / [T, heads] beta;
    SCAN_DELTA_HEAD: [T, heads] decays / [T, heads] beta;
    SCAN_BONUS (o = (S + diag(u) k v^T)^T q, then S <- g * S + k v^T): [T, heads, dim] row decays / None, ``extra`` = u
    [heads, dim]; SCAN_SSM (S <- a S + dt k v^T, o = S^T q + d v): [T, heads] decays / [T, heads] steps, ``extra`` = d
    [heads].
    out: float32 [T, heads * vdim].  ``forgot_offset`` (SCAN_MEMORY): where in a row the sum of the segment's log forget
    gates is left per head, or -1."""
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == heads * vdim
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and dim <= SCAN_MAX_KEY_DIM
    assert gate_a.dtype == torch.float32 and gate_a.is_contiguous()
    if gate_b is not None:
        assert gate_b.dtype == torch.float32 and gate_b.is_contiguous()
    if mode in (SCAN_BONUS, SCAN_SSM):
        assert extra is not None and extra.dtype == torch.float32 and extra.is_contiguous()
        assert extra.numel() == (heads * dim if mode == SCAN_BONUS else heads)
    _check(recurrent_lib().rb_linear_scan(
        mode, _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _is_f32(q), _is_f32(k), _is_f32(v),
        _ptr(gate_a), _ptr(gate_b), _ptr(extra), cap, q_scale, _ptr(state), state.stride(0), offsets[0], offsets[1], offsets[2],
        forgot_offset, _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(out), heads, kv_heads, dim, vdim, batch.num_segments, _stream()),
        "linear_scan")


def scan_pieces_combine(pieces, state, s_off: int, decay, cu_piece, seg_first, seg_slot, per_head: int, total: int,
                        segments: int) -> None:
    """For a fixed-decay state whose long segments were scanned in pieces from zero: per segment, in order,
    ``pieces[p] <- carry; carry <- decay^len(p) * carry + pieces[p]``, starting from the request's state and leaving the
    last carry there.  pieces: float32 [n_pieces, >= total]; per_head: state elements of one head."""
    assert pieces.dtype == state.dtype == decay.dtype == torch.float32 and pieces.is_contiguous() and state.is_contiguous()
    assert cu_piece.dtype == seg_first.dtype == seg_slot.dtype == torch.int32
    _check(recurrent_lib().rb_scan_pieces_combine(_ptr(pieces), pieces.stride(0), _ptr(state), state.stride(0), s_off,
                                                  _ptr(decay), _ptr(cu_piece), _ptr(seg_first), _ptr(seg_slot), per_head,
                                                  total, segments, _stream()), "scan_pieces_combine")


def scan_pieces_combine_sums(pieces, state, s_off: int, decay, sums, by_row: bool, dim: int, vdim: int, cu_piece, seg_first,
                             seg_slot, per_head: int, total: int, segments: int) -> None:
    """``scan_pieces_combine`` for decays that differ from token to token: ``decay`` float32 [T, n] holds one per head
    (n = heads) or, with ``by_row``, one per head and key row (n = heads * dim); a piece's factor is the product of its
    tokens' decays, left as sums of logarithms in ``sums`` (float32 scratch [pieces, n])."""
    n_pieces = cu_piece.numel() - 1
    assert pieces.dtype == state.dtype == decay.dtype == sums.dtype == torch.float32
    assert pieces.is_contiguous() and state.is_contiguous() and decay.is_contiguous() and sums.is_contiguous()
    assert decay.dim() == 2 and sums.shape == (n_pieces, decay.shape[1])
    assert cu_piece.dtype == seg_first.dtype == seg_slot.dtype == torch.int32
    _check(recurrent_lib().rb_scan_pieces_combine_sums(
        _ptr(pieces), pieces.stride(0), _ptr(state), state.stride(0), s_off, _ptr(decay), _ptr(sums), decay.shape[1],
        1 if by_row else 0, dim, vdim, _ptr(cu_piece), _ptr(seg_first), _ptr(seg_slot), per_head, total, n_pieces, segments,
        _stream()), "scan_pieces_combine_sums", 2)


def memory_pieces_combine(pieces, state, offsets, forgot_offset: int, seg_first, seg_slot, per_head_s: int, per_head_n: int,
                          heads: int, segments: int) -> None:
    """The matrix memory's counterpart of ``scan_pieces_combine``: pieces scanned from (0, 0, -inf) hold S', n', m' and
    the sum F of their log forget gates; per segment, in order, every piece gets the state it starts from and the
    request's slot the state behind the last one.  offsets = (S, n, m) inside a row."""
    assert pieces.dtype == state.dtype == torch.float32 and pieces.is_contiguous() and state.is_contiguous()
    _check(recurrent_lib().rb_memory_pieces_combine(_ptr(pieces), pieces.stride(0), _ptr(state), state.stride(0), offsets[0],
                                                    offsets[1], offsets[2], forgot_offset, _ptr(seg_first), _ptr(seg_slot),
                                                    per_head_s, per_head_n, heads, segments, _stream()),
           "memory_pieces_combine", 2)


def rotary_to_f32(x, q_off: int, k_off: int, cos, sin, rot: int, pos, q32, k32, heads: int, dim: int,
                  q_scale: float = 1.0, k_scale: float = 1.0) -> None:
    """q and k heads of the projection rows ``x`` (q at column q_off, k at k_off), turned by their positions on the
    first ``rot`` elements (element i with i + rot/2) and scaled, into float32 q32, k32 [T, heads * dim]."""
    T = x.shape[0]
    assert x.stride(1) == 1 and q32.dtype == k32.dtype == torch.float32 and q32.is_contiguous() and k32.is_contiguous()
    if rot:
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] * 2 == rot and cos.is_contiguous() and sin.is_contiguous()
    else:
        cos = sin = q32
    _check(recurrent_lib().rb_rotary_to_f32(_ptr(x), x.stride(0), q_off, k_off, _ptr(cos), _ptr(sin), rot, _ptr(pos),
                                            _ptr(q32), _ptr(k32), dtype_code(x.dtype), T, heads, dim, q_scale, k_scale,
                                            _stream()), "rotary_to_f32")


def rotary_inplace(x, cos, sin, rot: int, pos, heads: int, dim: int) -> None:
    """The first ``heads`` heads of every row of ``x`` turned in place by their positions (first ``rot`` elements of a
    head, element i with i + rot/2); any even ``rot``."""
    assert x.stride(1) == 1 and cos.dtype == sin.dtype == torch.float32 and cos.shape[1] * 2 == rot
    _check(recurrent_lib().rb_rotary_inplace(_ptr(x), x.stride(0), _ptr(cos), _ptr(sin), rot, _ptr(pos),
                                             dtype_code(x.dtype), x.shape[0], heads, dim, _stream()), "rotary_inplace")


def delta_prep(x, taps, state, conv_off: int, batch, q32, k32, v32, a, A_log, dt_bias, b, heads: int, kv_heads: int,
               dim: int, vdim: int, q_scale: float, head_decay: bool = False) -> None:
    """What the delta rule needs of every token: the short causal convolution and silu of the q, k, v channels of
    ``x`` (what lies before a segment comes from the request's conv state), unit q and k heads, the row decays (in
    place over ``a``) and beta (in place over ``b``).  ``head_decay``: ``a`` holds one number a token and head
    ([T, heads], ``dt_bias`` [heads]) instead of one a key row."""
    T = x.shape[0]
    K = taps.shape[1]
    assert x.stride(1) == 1 and taps.is_contiguous() and taps.shape[0] == 2 * kv_heads * dim + heads * vdim
    assert a.dtype == b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
    assert A_log.dtype == dt_bias.dtype
    for t in (q32, k32, v32):
        assert t.dtype == torch.float32 and t.is_contiguous()
    _check(recurrent_lib().rb_delta_prep(
        _ptr(x), x.stride(0), _ptr(taps), dtype_code(taps.dtype), K, _ptr(state), state.stride(0), conv_off,
        _ptr(batch.tok_seg), _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(q32), _ptr(k32), _ptr(v32), _ptr(a),
        _ptr(A_log), _ptr(dt_bias), dtype_code(A_log.dtype), _ptr(b), dtype_code(x.dtype), T, heads, kv_heads, dim, vdim,
        q_scale, 1 if head_decay else 0, _stream()), "delta_prep")


def gated_conv(x, x_bias, taps, conv_bias, state, conv_off: int, batch, out) -> None:
    """out[t, c] = conv_bias[c] + sum_j taps[c, K - 1 - j] * (x[t - j, c] + x_bias[c]) over the tokens t - j at positions
    >= 0 (what lies before the step comes from the request's held inputs: ``state`` row of its slot from ``conv_off``,
    [channel][K - 1], kept without the bias).  x: a view [T, channels] with unit stride along a row; out [T, channels]."""
    T, W = out.shape
    K = taps.shape[1]
    assert x.stride(1) == 1 and x.shape[1] >= W and out.is_contiguous() and out.dtype == x.dtype and taps.is_contiguous()
    assert taps.shape[0] == W and state.dtype == torch.float32
    for t in (x_bias, conv_bias):
        assert t is None or (t.dtype == taps.dtype and t.numel() == W)
    _check(recurrent_lib().rb_gated_conv(_ptr(x), x.stride(0), _ptr(x_bias), _ptr(taps), _ptr(conv_bias), dtype_code(taps.dtype),
                                         K, _ptr(state), state.stride(0), conv_off, _ptr(batch.pos), _ptr(batch.tok_seg),
                                         _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(out), dtype_code(x.dtype), T, W, _stream()),
           "gated_conv")


def gated_recurrence(u, gates, block: int, r_bias, i_bias, lam, c_decay: float, y, y_bias, state, s_off: int, batch, out,
                     log_decay=None) -> None:
    """Per channel c and segment, token by token: r = sigmoid(gates[0, b, t, o] + r_bias[c]), i = sigmoid(gates[1, b, t, o]
    + i_bias[c]) with b = c // block, o = c % block (gates float32 [2, W / block, T, block]); log f = -c_decay r
    softplus(lam[c]); s <- f s + sqrt(1 - f^2) i u[t, c]; out[t, c] = s * gelu_tanh(y[t, c] + y_bias[c]).  s is the float32
    ``state`` row of the request's slot from ``s_off``.  ``log_decay`` (float32 [segments, W]): receives the sum of a
    segment's log f per channel."""
    T, W = u.shape
    assert log_decay is None or (log_decay.dtype == torch.float32 and log_decay.is_contiguous()
                                 and tuple(log_decay.shape) == (batch.num_segments, W))
    assert u.is_contiguous() and out.is_contiguous() and out.shape == (T, W) and out.dtype == u.dtype == y.dtype
    assert gates.dtype == torch.float32 and gates.is_contiguous() and gates.numel() == T * 2 * W and y.stride(1) == 1
    assert r_bias.dtype == i_bias.dtype == lam.dtype and r_bias.numel() == i_bias.numel() == lam.numel() == W
    assert y_bias is None or (y_bias.dtype == lam.dtype and y_bias.numel() == W)
    _check(recurrent_lib().rb_gated_recurrence(_ptr(u), _ptr(gates), block, _ptr(r_bias), _ptr(i_bias), _ptr(lam),
                                               dtype_code(lam.dtype), c_decay, _ptr(y), y.stride(0), _ptr(y_bias), _ptr(state),
                                               state.stride(0), s_off, _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(out),
                                               dtype_code(u.dtype), W, T, batch.num_segments, _ptr(log_decay), _stream()),
           "gated_recurrence")


def gated_pieces_combine(pieces, log_decay, state, s_off: int, seg_first, seg_slot, segments: int) -> None:
    """For a channel recurrence whose long segments were walked in pieces from zero: per segment, in order,
    ``pieces[p] <- carry; carry <- exp(log_decay[p]) * carry + pieces[p]``, starting from the request's state (``state`` row
    of its slot from ``s_off``) and leaving the last carry there.  pieces, log_decay: float32 [n_pieces, W]."""
    assert pieces.dtype == log_decay.dtype == state.dtype == torch.float32 and pieces.is_contiguous() and log_decay.is_contiguous()
    assert pieces.shape == log_decay.shape and seg_first.dtype == seg_slot.dtype == torch.int32
    _check(recurrent_lib().rb_gated_pieces_combine(_ptr(pieces), _ptr(log_decay), _ptr(state), state.stride(0), s_off,
                                                   _ptr(seg_first), _ptr(seg_slot), pieces.shape[1], segments, _stream()),
           "gated_pieces_combine")


def conv_state_update(x, taps_count: int, state, conv_off: int, batch, channels: int) -> None:
    """The conv state of every segment's request after this step: the last ``taps_count - 1`` inputs of each of the
    first ``channels`` columns of ``x``."""
    _check(recurrent_lib().rb_conv_state_update(_ptr(x), x.stride(0), taps_count, _ptr(state), state.stride(0), conv_off,
                                                _ptr(batch.cu_q), _ptr(batch.seg_slot), dtype_code(x.dtype), channels,
                                                batch.num_segments, _stream()), "conv_state_update")


def token_shift_mix(x, mu, state, shift_off: int, batch, out) -> None:
    """out[n, t] = x[t] + (x[t - 1] - x[t]) * mu[n] for each of the N rows of ``mu`` [N, W]; the predecessor of a segment's
    first token is the row the request kept (``state`` row of its slot from ``shift_off``; zero for a new request).
    x [T, W] with unit stride along a row; out [N, T, W] of x's type."""
    T, W = x.shape
    N = mu.shape[0]
    assert x.stride(1) == 1 and mu.is_contiguous() and mu.shape[1] == W and out.shape == (N, T, W) and out.is_contiguous()
    assert out.dtype == x.dtype and state.dtype == torch.float32
    _check(recurrent_lib().rb_token_shift_mix(_ptr(x), x.stride(0), _ptr(mu), dtype_code(mu.dtype), N, _ptr(state),
                                              state.stride(0), shift_off, _ptr(batch.tok_seg), _ptr(batch.cu_q),
                                              _ptr(batch.seg_slot), _ptr(out), dtype_code(x.dtype), T, W, _stream()),
           "token_shift_mix")


def ssm_prep(x, c_off: int, channels: int, taps, bias, state, conv_off: int, batch, conv_out, dt_off: int, heads: int,
             dt_bias, A_log, dt, decay) -> None:
    """What a state-space scan needs of every token: ``channels`` columns of ``x`` from ``c_off`` through a causal
    convolution (taps [channels, K], last column the token's own; before a segment the request's conv state), plus
    ``bias``, then silu, into float32 conv_out [T, channels]; dt = softplus(x[:, dt_off + h] + dt_bias[h]) and
    decay = exp(-exp(A_log[h]) dt), float32 [T, heads]."""
    T = x.shape[0]
    K = taps.shape[1]
    assert x.stride(1) == 1 and taps.is_contiguous() and taps.shape[0] == channels and bias.numel() == channels
    assert bias.dtype == taps.dtype and dt_bias.dtype == A_log.dtype and dt_bias.numel() == A_log.numel() == heads
    for t, cols in ((conv_out, channels), (dt, heads), (decay, heads)):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, cols)
    _check(recurrent_lib().rb_ssm_prep(
        _ptr(x), x.stride(0), c_off, channels, _ptr(taps), _ptr(bias), dtype_code(taps.dtype), K, _ptr(state), state.stride(0),
        conv_off, _ptr(batch.tok_seg), _ptr(batch.cu_q), _ptr(batch.seg_slot), _ptr(conv_out), dt_off, heads, _ptr(dt_bias),
        _ptr(A_log), dtype_code(A_log.dtype), _ptr(dt), _ptr(decay), dtype_code(x.dtype), T, _stream()), "ssm_prep")


def gated_part_norm(y, gate, weight, parts: int, eps: float, out) -> None:
    """v = y * silu(gate); out = v / rms(v) * weight, the root mean square taken over each of ``parts`` equal parts of a
    row.  y float32 [T, n]; gate: a view [T, n] of the activation type; weight [n]; out [T, n] of the activation type."""
    T, n = y.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and out.is_contiguous() and out.shape == (T, n) and n % parts == 0
    assert gate.stride(1) == 1 and gate.dtype == out.dtype and gate.shape == (T, n) and weight.numel() == n
    _check(recurrent_lib().rb_gated_part_norm(_ptr(y), _ptr(gate), gate.stride(0), _ptr(weight), dtype_code(weight.dtype), eps,
                                              _ptr(out), dtype_code(out.dtype), T, parts, n // parts, _stream()),
           "gated_part_norm")


def head_norm_gate(o, gate, weight, weight_mode: int, gate_act: int, eps: float, out, heads: int, vdim: int) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * act(gate[t, h]).  o float32 [T, heads * vdim]; gate: a view
    [T, heads * vdim] of the activation type.  weight_mode 0: none, 1: [vdim] shared by the heads, 2: [heads * vdim].
    gate_act 0: silu, 1: sigmoid."""
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous() and gate.stride(1) == 1
    assert gate.dtype == out.dtype
    wd = dtype_code(weight.dtype) if weight is not None else F32
    _check(recurrent_lib().rb_head_norm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), wd, weight_mode, gate_act,
                                             eps, _ptr(out), dtype_code(out.dtype), T, heads, vdim, _stream()),
           "head_norm_gate")


def add_dual_norm(stream, deltas, w1, w2, eps: float, offset: float, out1, out2, rows=None, scales=(1.0, 1.0)) -> None:
    """stream (float32) += the deltas (up to two tensors of the stream's shape, float32 or bfloat16; written back
    unless ``rows``), then out1 = norm(stream) * (offset + w1) and, if given, out2 likewise with w2: two norms of the
    same row share its mean square.  out1 None: the add only.  ``rows`` (int32): only these rows are normed.
    ``scales``: a factor on each delta as it is added."""
    H = stream.shape[1]
    assert stream.dtype == torch.float32 and stream.is_contiguous()
    ds = [d for d in (deltas or ()) if d is not None]
    assert len(ds) <= 2
    for d in ds:
        assert d.shape == stream.shape and d.is_contiguous()
    d1 = ds[0] if ds else None
    d2 = ds[1] if len(ds) > 1 else None
    n = stream.shape[0] if rows is None else rows.numel()
    if out1 is not None:
        assert out1.is_contiguous() and out1.shape == (n, H) and w1.numel() == H
        if out2 is not None:
            assert out2.dtype == out1.dtype and out2.shape == out1.shape and w2.dtype == w1.dtype and out2.is_contiguous()
    elif not ds:
        return
    _check(recurrent_lib().rb_add_dual_norm(
        _ptr(stream), _ptr(d1), _is_f32(d1) if d1 is not None else 1, float(scales[0]), _ptr(d2),
        _is_f32(d2) if d2 is not None else 1, float(scales[1]), _ptr(rows), _ptr(w1), _ptr(w2), dtype_code(w1.dtype) if w1 is not None else F32, eps, offset, _ptr(out1),
        _ptr(out2), dtype_code(out1.dtype) if out1 is not None else F32, n, H, _stream()), "add_dual_norm")


def scaled_sum(a, s1: float, b, s2: float, out) -> None:
    """out = s1 * a + s2 * b, elementwise; each of a, b and out float32 or bfloat16."""
    assert a.shape == b.shape == out.shape
    assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
    _check(recurrent_lib().rb_scaled_sum(_ptr(a), _is_f32(a), s1, _ptr(b), _is_f32(b), s2, _ptr(out), _is_f32(out),
                                         a.numel(), _stream()), "scaled_sum")


# ------------------------------------------------------------------------------- attention over cached latents

_latent = None
_LATENT_SOURCES = ["latent.cu"]
LATENT_MAX_RANK = 1024           # numbers of a latent that the attention kernels take


def latent_lib() -> ctypes.CDLL:
    """The kernels of the attention over a paged cache of latents (csrc/latent.cu); compiled when a model that has
    such a mixer is first run."""
    global _latent
    if _latent is None:
        lib = build.load("return_latent", _LATENT_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I, F, L = c_void_p, c_int, c_float, ctypes.c_longlong
        lib.rb_latent_write.argtypes = [P, I, I, P, I, F, I, I, P, P, P, P, P, I, I, P, I, I, P, I, I, I, I, P, I, I, P]
        lib.rb_latent_attention_simt.argtypes = [P, P, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, P]
        lib.rb_head_gate.argtypes = [P, P, I, I, I, I, I, P]
        lib.rb_gemm_f32_heads.argtypes = [P, P, P, I, I, I, I, I, I, I, L, L, L, P]
        lib.rb_latent_expand_scatter.argtypes = [P, I, P, I, I, I, P, I, P, P, I, I, I, I, I, P]
        lib.rb_latent_expand_query.argtypes = [P, I, P, I, I, P, I, I, I, I, I, P]
        lib.rb_latent_take_values.argtypes = [P, P, P, P, I, I, I, I, P]
        lib.rb_latent_gather_rows.argtypes = [P, L, P, P, I, I, P]
        lib.rb_latent_gather_rows.restype = c_int
        for name in ("rb_latent_write", "rb_latent_attention_simt", "rb_head_gate", "rb_gemm_f32_heads",
                     "rb_latent_expand_scatter", "rb_latent_expand_query", "rb_latent_take_values"):
            getattr(lib, name).restype = c_int
        _latent = lib
    return _latent


def latent_write(x, c_off: int, norm_w, eps: float, rank: int, rot: int, cos, sin, batch, block_table, page_size: int,
                 pool, write_cache: bool, xq, q_off: int, heads: int, dim: int, q_abs) -> None:
    """Every token's latent into its page: columns [c_off, c_off + rank) of ``x`` normed with ``norm_w``, the ``rot``
    columns behind them rotated by the position (element i with i + rot/2), zeros up to the pool's width.
    pool: [pages, page_size, width].  Also the rotated parts of the queries (heads of [dim | rot] from column q_off of
    ``xq``) rotated into columns [rank, rank + rot) of every head of q_abs [T, heads * width], zeros behind them."""
    T = x.shape[0]
    width = pool.shape[-1]
    assert x.stride(1) == 1 and pool.dtype == x.dtype and pool.is_contiguous() and width >= rank + rot
    assert q_abs.is_contiguous() and q_abs.dtype == x.dtype and q_abs.shape == (T, heads * width)
    if rot:
        assert cos.dtype == sin.dtype == torch.float32 and cos.shape[1] * 2 == rot and cos.is_contiguous() and sin.is_contiguous()
        assert xq.stride(1) == 1 and xq.dtype == x.dtype
    else:
        cos = sin = batch.pos          # never read
    _check(latent_lib().rb_latent_write(_ptr(x), x.stride(0), c_off, _ptr(norm_w), dtype_code(norm_w.dtype), eps, rank, rot,
                                        _ptr(cos), _ptr(sin), _ptr(batch.pos), _ptr(batch.tok_seg), _ptr(block_table),
                                        block_table.stride(0), page_size, _ptr(pool), width, 1 if write_cache else 0, _ptr(xq),
                                        xq.stride(0), q_off, heads, dim, _ptr(q_abs), dtype_code(x.dtype), T, _stream()),
           "latent_write")


def latent_attention_simt(q_abs, pool, batch, block_table, page_size: int, sink, out, heads: int, rank: int, rot: int,
                          scale: float, window=None) -> None:
    """Attention of every token of the step over its request's cached latents, on the CUDA cores: a head's query
    q_abs[t, h] (``rank`` numbers in the latent's space, then ``rot`` rotated ones) against the cached vectors; the first
    ``rank`` columns of out[t, h] get the weighted mean of the latents.  ``sink``: float32 [heads] or None."""
    T = q_abs.shape[0]
    width = pool.shape[-1]
    assert q_abs.is_contiguous() and out.is_contiguous() and out.shape == q_abs.shape == (T, heads * width) and out.dtype == q_abs.dtype
    assert pool.dtype == q_abs.dtype and pool.is_contiguous()
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.numel() == heads and sink.is_contiguous()
    _check(latent_lib().rb_latent_attention_simt(_ptr(q_abs), _ptr(pool), _ptr(batch.pos), _ptr(batch.tok_seg),
                                                 _ptr(block_table), block_table.stride(0), page_size, _ptr(sink), _ptr(out),
                                                 dtype_code(q_abs.dtype), T, heads, rank, rot, width, scale, int(window or 0),
                                                 _stream()), "latent_attention_simt")


LATENT_TC_MAX_WIDTH = 256        # widest cached vector that the tensor-core attention kernels take as a head


def latent_on_tensor_cores(dtype, width: int) -> bool:
    """Whether the attention over latents of this (padded) width runs on the engine's tensor-core attention kernels."""
    return dtype == torch.bfloat16 and width % 16 == 0 and width <= LATENT_TC_MAX_WIDTH


def latent_attention(q_abs, pool, batch, block_table, page_size: int, sink, out, heads: int, rank: int, rot: int,
                     scale: float, window=None) -> None:
    """Attention of every token of the step over its request's cached latents (its own included).

    bfloat16 with a cached vector of up to 256 numbers: the engine's paged attention kernels (tcgen05 or mma.sync for
    prompt portions, split over the keys for decoded tokens) with one key/value head for all query heads, whose keys and
    values are both the cached vector: a head's output row then holds the weighted mean of the latents in its first
    ``rank`` columns (and that of the rotated key parts behind them, which nobody reads).  Otherwise, and in float32:
    the CUDA-core kernel, whose result does not depend on how the work was cut."""
    width = pool.shape[-1]
    if latent_on_tensor_cores(q_abs.dtype, width):
        as_heads = pool.unsqueeze(1)                       # [pages, 1 kv head, page_size, width]
        paged_attention(q_abs, as_heads, as_heads, batch, block_table, page_size, out, heads, 1, width, scale, window, sink)
        return
    latent_attention_simt(q_abs, pool, batch, block_table, page_size, sink, out, heads, rank, rot, scale, window)


def gather_rows(x, index, out) -> None:
    """out[i] = x[index[i]] for rows of whole 16-byte pieces (x [rows, K] with any row stride, out contiguous)."""
    n, K = out.shape
    assert x.dtype == out.dtype and x.stride(1) == 1 and out.is_contiguous() and x.shape[1] == K
    assert index.dtype == torch.int32 and index.numel() == n
    size = x.element_size()
    _check(latent_lib().rb_latent_gather_rows(_ptr(x), x.stride(0) * size, _ptr(index), _ptr(out), K * size, n, _stream()),
           "gather_rows")


def latent_expand_scatter(kv, lat, rank: int, rot: int, slots, page_size: int, kx, vx, heads: int, dim: int, vdim: int) -> None:
    """Row i of ``kv`` ([U; V] applied to gathered latent i: heads x dim key numbers, then heads x vdim value numbers)
    and the rotated part of ``lat`` row i into the scratch pools kx, vx [pages, heads, page_size, head] at
    slots[i] = page * page_size + row: key [U_h c | rotated part | 0], value [V_h c | 0]."""
    n = slots.numel()
    head = kx.shape[-1]
    assert kv.dtype == lat.dtype == kx.dtype == vx.dtype == torch.bfloat16 and kv.stride(1) == 1 and lat.stride(1) == 1
    assert kx.is_contiguous() and vx.is_contiguous() and kx.shape == vx.shape and kx.shape[1] == heads and kx.shape[2] == page_size
    assert kv.shape == (n, heads * (dim + vdim)) and lat.shape[0] == n and slots.dtype == torch.int32
    _check(latent_lib().rb_latent_expand_scatter(_ptr(kv), kv.stride(0), _ptr(lat), lat.stride(0), rank, rot, _ptr(slots),
                                                 page_size, _ptr(kx), _ptr(vx), heads, dim, vdim, head, n, _stream()),
           "latent_expand_scatter")


def latent_expand_query(q, q_abs, width: int, rank: int, qx, heads: int, dim: int, rot: int) -> None:
    """qx[t, h] = [q[t, h, :dim] | the rotated part that lies in q_abs[t, h, rank : rank + rot] | 0]."""
    T = q.shape[0]
    head = qx.shape[1] // heads
    assert q.dtype == q_abs.dtype == qx.dtype == torch.bfloat16 and q.stride(1) == 1 and q_abs.is_contiguous() and qx.is_contiguous()
    _check(latent_lib().rb_latent_expand_query(_ptr(q), q.stride(0), _ptr(q_abs), width, rank, _ptr(qx), heads, dim, rot, head,
                                               T, _stream()), "latent_expand_query")


def latent_take_values(ox, batch, out, heads: int, vdim: int) -> None:
    """out[t, h * vdim + e] = ox[t, h * head + e] for the tokens of segments of several tokens."""
    T = out.shape[0]
    assert ox.is_contiguous() and out.is_contiguous() and ox.dtype == out.dtype == torch.bfloat16
    _check(latent_lib().rb_latent_take_values(_ptr(ox), _ptr(batch.tok_seg), _ptr(batch.cu_q), _ptr(out), heads, vdim,
                                              ox.shape[1] // heads, T, _stream()), "latent_take_values")


def head_gate(x, gate, heads: int) -> None:
    """x[t, h * vdim + e] *= sigmoid(gate[t, h]), in place (gate: a [T, heads] view of unit stride along a row)."""
    T, HV = x.shape
    assert x.is_contiguous() and gate.dtype == x.dtype and gate.stride(1) == 1 and gate.shape == (T, heads) and HV % heads == 0
    _check(latent_lib().rb_head_gate(_ptr(x), _ptr(gate), gate.stride(0), dtype_code(x.dtype), T, heads, HV // heads,
                                     _stream()), "head_gate")


def linear_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[h] = x[h] @ w[h]^T for every head: x [heads, T, K] (any strides with unit stride along K), w [heads, N, K],
    out [heads, T, N].  float32: the engine's own FFMA kernel, every sum in one order.  bfloat16: the library's batched
    product with float32 accumulation."""
    Hh, T, K = x.shape
    N = w.shape[1]
    assert w.shape == (Hh, N, K) and out.shape == (Hh, T, N) and x.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1
    if x.dtype == torch.float32:
        assert w.dtype == out.dtype == torch.float32
        _check(latent_lib().rb_gemm_f32_heads(_ptr(x), _ptr(w), _ptr(out), Hh, T, N, K, x.stride(1), w.stride(1), out.stride(1),
                                              x.stride(0), w.stride(0), out.stride(0), _stream()), "gemm_f32_heads")
        return
    if not x.is_cuda:
        raise KernelError("the engine's kernels run on a CUDA device only; got a CPU tensor")
    if out.dtype == torch.float32:
        torch.bmm(x, w.transpose(1, 2), out_dtype=torch.float32, out=out)
    else:
        torch.bmm(x, w.transpose(1, 2), out=out)


# ------------------------------------------------------------------------------- mixture of experts

_moe = None
_MOE_SOURCES = ["moe.cu"]


def moe_lib() -> ctypes.CDLL:
    """The kernels of a mixture of experts (csrc/moe.cu); compiled when a model that has one is first run."""
    global _moe
    if _moe is None:
        lib = build.load("return_moe", _MOE_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I, F = c_void_p, c_int, c_float
        lib.rb_moe_route.argtypes = [P, I, P, P, P, I, I, I, I, I, F, I, I, F, P]
        lib.rb_moe_pair_linear.argtypes = [P, I, I, P, P, P, I, I, I, I, I, P]
        lib.rb_clamped_glu.argtypes = [P, I, P, I, I, I, I, F, F, F, P]
        lib.rb_moe_combine.argtypes = [P, P, P, P, P, I, I, I, I, P]
        lib.rb_moe_sort.argtypes = [P, I, I, P, P, P, P]
        lib.rb_moe_grouped_gemm.argtypes = [P, I, P, I, P, P, I, P, I, I, I, I, P]
        lib.rb_moe_gather_rows.argtypes = [P, ctypes.c_longlong, P, I, P, I, I, P]
        for name in ("rb_moe_route", "rb_moe_pair_linear", "rb_clamped_glu", "rb_moe_combine", "rb_moe_sort",
                     "rb_moe_grouped_gemm", "rb_moe_gather_rows"):
            getattr(lib, name).restype = c_int
        _moe = lib
    return _moe


def moe_route(logits, expert_of, weight, top: int, groups: int = 1, keep: int = 1, tiny: float = 1e-20, bias=None,
              score: str = "softmax", group_top: int = 1, scale: float = 1.0) -> None:
    """The router's choice per token from float32 logits [T, E] (plus ``bias``, float32 [E], if given): softmax over all
    experts; with ``groups`` > 1 only the
    experts of the ``keep`` groups (equal runs of neighbours) with the largest best score can be chosen; the ``top``
    largest scores among them, in falling order, into expert_of (int32 [T, top]) with weight = score / (sum + tiny).
    ``score`` "sigmoid": every expert's score is the logistic of its own logit.  ``group_top`` 2: a group scores as the sum
    of its two best.  ``scale``: a factor on the weights."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert expert_of.dtype == torch.int32 and expert_of.shape == (T, top) and expert_of.is_contiguous()
    assert weight.dtype == torch.float32 and weight.shape == (T, top) and weight.is_contiguous()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous()
    _check(moe_lib().rb_moe_route(_ptr(logits), logits.stride(0), _ptr(bias), _ptr(expert_of), _ptr(weight), T, E, top, groups,
                                  keep, tiny, {"softmax": 0, "sigmoid": 1}[score], group_top, scale, _stream()), "moe_route")


def moe_pair_linear(x, in_div: int, w, expert_of, out) -> None:
    """out[i] = x[i // in_div] @ w[expert_of[i]]^T for every (token, chosen expert) pair i; w [E, N, K]."""
    E, N, K = w.shape
    pairs = expert_of.numel()
    assert x.dtype == w.dtype == out.dtype and x.stride(1) == 1 and w.is_contiguous() and out.stride(1) == 1
    assert x.shape[1] == K and out.shape == (pairs, N) and x.shape[0] * in_div == pairs
    _check(moe_lib().rb_moe_pair_linear(_ptr(x), x.stride(0), in_div, _ptr(w), _ptr(expert_of), _ptr(out), out.stride(0),
                                        dtype_code(x.dtype), pairs, N, K, _stream()), "moe_pair_linear")


def clamped_glu(gate_up, out, limit: float, alpha: float, shift: float = 1.0) -> None:
    """gate_up [rows, 2F] = [gate | up]: out = g * sigmoid(alpha g) * (u + shift) with g = min(gate, limit) and
    u = clamp(up, -limit, limit).  An infinite limit, alpha = 1 and shift = 0 give silu(gate) * up."""
    rows, F2 = gate_up.shape
    assert out.shape == (rows, F2 // 2) and out.dtype == gate_up.dtype and gate_up.stride(1) == 1 and out.stride(1) == 1
    _check(moe_lib().rb_clamped_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), out.stride(0), dtype_code(out.dtype), rows,
                                    F2 // 2, float(limit), float(alpha), float(shift), _stream()), "clamped_glu")


def moe_combine(y, weight, shared, out, row_of=None) -> None:
    """out[t] = sum_k weight[t, k] * y[row of pair t * top + k] (+ shared[t]); sums in float32 in the order of k."""
    T, top = weight.shape
    H = out.shape[1]
    assert y.shape == (T * top, H) and y.is_contiguous() and out.is_contiguous() and out.dtype == y.dtype
    if shared is not None:
        assert shared.shape == out.shape and shared.is_contiguous() and shared.dtype == y.dtype
    _check(moe_lib().rb_moe_combine(_ptr(y), _ptr(row_of), _ptr(weight), _ptr(shared), _ptr(out), dtype_code(y.dtype), T, H, top,
                                    _stream()), "moe_combine")


def moe_sort(expert_of, num_experts: int, offsets, pair_at, place_of) -> None:
    """The (token, chosen expert) pairs in the order of their experts: offsets int32 [E + 1] (an expert's run of places),
    pair_at[place] and its inverse place_of[pair], int32 [pairs]."""
    pairs = expert_of.numel()
    assert expert_of.dtype == offsets.dtype == pair_at.dtype == place_of.dtype == torch.int32
    assert offsets.numel() == num_experts + 1 and pair_at.numel() == pairs and place_of.numel() == pairs
    _check(moe_lib().rb_moe_sort(_ptr(expert_of), pairs, num_experts, _ptr(offsets), _ptr(pair_at), _ptr(place_of), _stream()),
           "moe_sort")


def moe_grouped_gemm(x, pair_at, in_div: int, w, offsets, out) -> None:
    """out[place] = x[row(place)] @ w[expert of the place]^T on the tensor cores, bfloat16: row(place) = pair_at[place] //
    in_div, or the place itself with pair_at None.  w [E, N, K]; offsets int32 [E + 1]."""
    E, N, K = w.shape
    places = out.shape[0]
    assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous() and out.stride(1) == 1
    assert x.shape[1] == K and out.shape[1] == N
    _check(moe_lib().rb_moe_grouped_gemm(_ptr(x), x.stride(0), _ptr(pair_at), in_div, _ptr(w), _ptr(offsets), E, _ptr(out),
                                         out.stride(0), places, N, K, _stream()), "moe_grouped_gemm")


_moe_tc5 = None
_MOE_TC5_SOURCES = ["moe_tc5.cu"]


def moe_tc5_lib() -> ctypes.CDLL:
    """The experts' products of a prompt on tcgen05 (csrc/moe_tc5.cu); compiled when a prompt first needs it."""
    global _moe_tc5
    if _moe_tc5 is None:
        lib = build.load("return_moe_tc5", _MOE_TC5_SOURCES, {"RB_PDL_MODE": PDL_MODE})
        P, I = c_void_p, c_int
        lib.rb_moe_tc5_gemm.argtypes = [P, I, P, P, I, P, I, I, I, I, P, P]
        lib.rb_moe_tc5_gemm.restype = c_int
        _moe_tc5 = lib
    return _moe_tc5


def moe_gather_rows(x, pair_at, in_div: int, out) -> None:
    """out[place] = x[pair_at[place] // in_div]: the tokens' rows in the order of the places."""
    places, K = out.shape
    assert x.dtype == out.dtype and x.stride(1) == 1 and out.is_contiguous() and x.shape[1] == K and pair_at.numel() == places
    size = x.element_size()
    _check(moe_lib().rb_moe_gather_rows(_ptr(x), x.stride(0) * size, _ptr(pair_at), in_div, _ptr(out), K * size, places,
                                        _stream()), "moe_gather_rows")


def moe_tc5_gemm(x_sorted, w, offsets, out) -> None:
    """out[place] = x_sorted[place] @ w[expert of the place]^T on tcgen05 (TMA-fed), bfloat16; w [E, N, K]."""
    E, N, K = w.shape
    places = out.shape[0]
    assert x_sorted.dtype == w.dtype == out.dtype == torch.bfloat16 and x_sorted.stride(1) == 1 and w.is_contiguous()
    assert x_sorted.shape == (places, K) and out.shape[1] == N and out.stride(1) == 1
    _tc5_launched.add(x_sorted.device)
    _check(moe_tc5_lib().rb_moe_tc5_gemm(_ptr(x_sorted), x_sorted.stride(0), _ptr(w), _ptr(offsets), E, _ptr(out), out.stride(0),
                                         places, N, K, _ptr(tc5_status(x_sorted.device)), _stream()), "moe_tc5_gemm")


# From this many (token, expert) pairs on, a step's experts run as tiles on the tensor cores over the pairs sorted by
# expert; below, every pair streams its expert's weights (a step of decoded tokens: few pairs, most on experts of their own).
MOE_GROUPED_MIN_PAIRS = 64
# From this many pairs on the tiles are those of the tcgen05 kernel (128 places x 256 columns, operands by TMA, the
# tokens' rows gathered into the order of the places first); between the two, mma.sync tiles of 64 x 128.
MOE_TC5_MIN_PAIRS = 1024


def moe_experts(x, gate_up, down, expert_of, weight, shared, out, limit: float, alpha: float, ctx=None,
                shift: float = 1.0) -> None:
    """out[t] = sum_k weight[t, k] * expert_{expert_of[t, k]}(x[t]) (+ shared[t]); gate_up [E, 2F, H], down [E, H, F];
    an expert is down(g sigmoid(alpha g) (u + shift)) with the gate capped at ``limit`` and the up part clamped to it."""
    E, F2, H = gate_up.shape
    T, top = expert_of.shape
    pairs = T * top

    def buf(name, shape, dtype=None):
        if ctx is not None:
            return ctx.buffer(name, shape, dtype or x.dtype, x.device)
        return torch.empty(shape, dtype=dtype or x.dtype, device=x.device)

    gu = buf("moe.pair_gate_up", (pairs, F2))
    act = buf("moe.pair_act", (pairs, F2 // 2))
    y = buf("moe.pair_y", (pairs, H))
    if (x.dtype == torch.bfloat16 and pairs >= MOE_GROUPED_MIN_PAIRS and H % 8 == 0 and F2 % 16 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        offsets = buf("moe.offsets", (E + 1,), torch.int32)
        pair_at = buf("moe.pair_at", (pairs,), torch.int32)
        place_of = buf("moe.place_of", (pairs,), torch.int32)
        moe_sort(expert_of, E, offsets, pair_at, place_of)
        if pairs >= MOE_TC5_MIN_PAIRS and E <= 1024:
            rows = buf("moe.pair_rows", (pairs, H))
            moe_gather_rows(x, pair_at, top, rows)
            moe_tc5_gemm(rows, gate_up, offsets, gu)
            clamped_glu(gu, act, limit, alpha, shift)
            moe_tc5_gemm(act, down, offsets, y)
        else:
            moe_grouped_gemm(x, pair_at, top, gate_up, offsets, gu)
            clamped_glu(gu, act, limit, alpha, shift)
            moe_grouped_gemm(act, None, 1, down, offsets, y)
        moe_combine(y, weight, shared, out, row_of=place_of)
        return
    moe_pair_linear(x, top, gate_up, expert_of, gu)
    clamped_glu(gu, act, limit, alpha, shift)
    moe_pair_linear(act, 1, down, expert_of, y)
    moe_combine(y, weight, shared, out)


# ------------------------------------------------------------------------------- sampling

def sample(logits, temperature, top_k, top_p, uniform, tokens_out, logprobs_out=None, one_cta: bool = False) -> None:
    """One token per row of float32 logits [n, V]; per-row temperature, top_k, top_p and uniform draw.
    A cluster of eight CTAs takes a row (its parts in their shared memories); ``one_cta``: the kernel with one CTA
    a row, which takes rows of any length and is what rows too long for eight shared memories fall back to."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert top_k.dtype == torch.int32 and tokens_out.dtype == torch.int32
    _check(core().rb_sample(_ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                            _ptr(uniform), _ptr(tokens_out), _ptr(logprobs_out), 1 if one_cta else 0, _stream()), "sample")


def argmax(logits, tokens_out) -> None:
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens_out.dtype == torch.int32
    _check(core().rb_argmax(_ptr(logits), logits.stride(0), n, V, _ptr(tokens_out), _stream()), "argmax")
