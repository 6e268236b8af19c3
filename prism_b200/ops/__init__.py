"""Python face of the hand-written CUDA kernels (``prism_b200/csrc``).

Every function takes CUDA tensors, checks what the kernel assumes (dtype,
contiguity, sizes), and launches on torch's current stream.  There is no CPU
path, and nothing steps in for a missing kernel: if the shared library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
(The one library call is by design, not a fallback: the bf16 matrix product
of more than a few tokens, see ``linear``.)

Which of andre-fu/prism's call sites each op replaces:

==================  ==========================================================
``embed``           ``F.embedding`` (engine/executor.py:74-75)
``add_rmsnorm``     residual add + ``fused_rms_norm`` (executor.py:108,122-124,130)
``linear``          ``F.linear`` (executor.py:109,122,125,127,130)
``rope_kv_write``   eager RoPE (executor.py:117-118) + the cache append inside
                    ``flash_attn_with_kvcache`` (executor.py:119-120)
``attention``       ``flash_attn_with_kvcache`` (executor.py:119-120)
``swiglu``          ``F.silu(gate) * up`` (executor.py:127)
``sample``          argmax / softmax + multinomial (engine/scheduler.py:266-272)
==================  ==========================================================
"""

from __future__ import annotations

import ctypes
import math
import os
import threading
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A kernel refused its arguments or a launch failed."""


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def lib():
    """The loaded shared library; built at the first call if it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.build(verbose=True)
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the prism_b200 CUDA kernels from {path}: {e}") from e
        for name in dir(_Sig):
            if name.startswith("prism_"):
                fn = getattr(_lib, name)
                fn.restype = ctypes.c_int
                fn.argtypes = getattr(_Sig, name)
        _lib.prism_set_pdl(0 if os.environ.get("PRISM_PDL", "1") == "0" else 1)
    return _lib


def library_file() -> Optional[str]:
    return _build.library_path()


_p, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class _Sig:
    prism_embed = [_p, _p, _i, _p, _i, _i, _i, _f, _p, _p, _p, _p]
    prism_add_rmsnorm = [_p, _p, _i, _i, _ll, _p, _i, _f, _p, _i, _p, _i, _i, _p]
    prism_rope_table = [_p, _p, _i, _i, _p, _p]
    prism_rope_kv_write_partial = [_p, _i, _p, _i, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i,
                                   _i, _p, _p]
    prism_rope_kv_write = [_p, _p, _p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i,
                           _i, _i, _p, _p]
    prism_attention_generic = [_p, _i, _p, _i, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i,
                               _i, _f, _p, _p]
    prism_attention_masked_generic = [_p, _i, _i, _p, _i, _p, _ll, _i, _p, _ll, _i, _i, _p, _i, _p, _p, _i, _i, _i,
                                      _i, _i, _i, _i, _i, _i, _i, _f, _p, _i, _p, _p, _i, _p]
    prism_attention_masked_supported = [_i, _i, _i, _i]
    prism_attention_masked_bf16 = [_p, _ll, _i, _p, _ll, _p, _ll, _i, _p, _ll, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i,
                                   _i, _i, _i, _i, _i, _f, _p, _i, _i, _i, _p, _p, _p, _p, _i, _p]
    prism_scale_add_rmsnorm = [_p, _f, _p, _i, _i, _ll, _p, _i, _f, _p, _i, _i, _i, _p]
    prism_gated_product = [_p, _ll, _p, _ll, _p, _ll, _i, _i, _i, _i, _f, _i, _p]
    prism_qk_norm_rope_store = [_p, _p, _p, _ll, _p, _i, _p, _i, _f, _p, _i, _p, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i,
                                _i, _i, _i, _i, _p, _i, _i, _p]
    prism_conv_unit_gates = [_p, _ll, _i, _i, _p, _i, _i, _p, _p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p, _p, _i, _p]
    prism_state_tail = [_p, _ll, _i, _p, _i, _p, _p, _i, _p]
    prism_shift_mix = [_p, _i, _p, _p, _i, _i, _p, _p, _p, _i, _p, _i, _ll, _i, _p]
    prism_headnorm_gate = [_p, _p, _ll, _p, _i, _i, _f, _f, _i, _i, _i, _p, _i, _ll, _i, _p]
    prism_recurrent_scan = [_i, _p, _ll, _ll, _ll, _ll, _p, _p, _ll, _p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _i, _p, _ll, _p]
    prism_unit_removal = [_p, _p, _ll, _p, _i, _f, _i, _i, _i, _p, _p]
    prism_decay_from_exponent = [_p, _ll, _p, _i, _i, _i, _p]
    prism_lowrank_decay = [_p, _ll, _i, _p, _p, _i, _i, _i, _p, _ll, _i, _i, _p, _i, _i, _f, _p]
    prism_rglru_scan_chunked = [_p, _p, _ll, _p, _ll, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _i, _ll, _p]
    prism_moe_route = [_p, _ll, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _i, _i, _i, _f, _f, _p]
    prism_moe_place = [_p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p]
    prism_moe_route_place = [_p, _ll, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _f, _f, _p]
    prism_moe_tcgen05_supported = [_i, _i]
    prism_moe_gather = [_p, _ll, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _p]
    prism_moe_gemm_tcgen05 = [_p, _ll, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _ll, _p, _p]
    prism_moe_gemm = [_p, _ll, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _ll, _i, _p]
    prism_hyper_norm = [_p, _ll, _p, _ll, _p, _i, _i, _ll, _p, _i, _p, _i, _p, _i, _i, _p, _i, _f, _i, _p, _i, _p, _i, _i, _p]
    prism_causal_conv = [_p, _ll, _p, _i, _p, _i, _i, _i, _p, _p, _p, _p, _i, _p, _i, _ll, _i, _i, _p, _p]
    prism_block_gates = [_p, _ll, _p, _p, _i, _p, _p, _i, _p, _i, _f, _i, _i, _i, _p, _p, _ll, _p]
    prism_rglru_scan = [_p, _p, _ll, _p, _ll, _p, _p, _p, _i, _i, _i, _p, _i, _ll, _p]
    prism_cache_store = [_p, _ll, _p, _i, _i, _p, _ll, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _p, _p]
    prism_latent_kv_store = [_p, _ll, _p, _i, _f, _i, _i, _i, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _p, _p, _i, _p, _i,
                             _p, _ll, _p]
    prism_rotate_slice = [_p, _ll, _i, _p, _ll, _i, _i, _i, _i, _p, _p, _i, _i, _p]
    prism_activation = [_p, _ll, _p, _ll, _i, _i, _i, _i, _p]
    prism_glu = [_p, _ll, _p, _ll, _i, _i, _i, _i, _p]
    prism_gather_gate = [_p, _ll, _p, _p, _i, _ll, _i, _i, _p, _i, _ll, _i, _i, _i, _p, _p]
    prism_softcap = [_p, _ll, _f, _p]
    prism_add_rows = [_p, _p, _i, _i, _ll, _p, _i, _i, _i, _p]
    prism_rms_rows = [_p, _ll, _p, _i, _f, _p, _ll, _i, _i, _i, _p]
    prism_attention_bf16_supported = [_i, _i, _i]
    prism_attention_decode_bf16 = [_p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f,
                                   _p, _p, _i, _p, _p, _i, _p, _p]
    prism_attention_decode_qkv_bf16 = [_p, _i, _p, _i, _p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i,
                                       _i, _f, _p, _p, _i, _p, _p, _i, _p, _p]
    prism_attention_prefill_bf16 = [_p, _i, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i,
                                    _f, _p, _p]
    prism_attention_prefill_tc_supported = [_i, _i, _i, _i]
    prism_attention_prefill_tc = [_p, _i, _i, _p, _i, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i,
                                  _f, _p, _i, _p, _p, _p]
    prism_attention_merge_bf16 = [_p, _p, _i, _p, _i, _i, _i, _i, _p]
    prism_swiglu = [_p, _p, _i, _i, _i, _p]
    prism_sgemm_nt = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _p]
    prism_sample = [_p, _i, _i, _i, _p, _p, _p, _p]
    prism_argmax_split = [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p]
    prism_set_pdl = [_i]
    prism_gemm_tcgen05_supported = [_i, _i, _i]
    prism_gemm_tcgen05 = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _i, _i, _p]
    prism_gemv_bf16_supported = [_i, _i, _i]
    prism_gemv_bf16 = [_p, _i, _p, _i, _p, _i, _p, _i, _i, _i, _i, _i, _p]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("prism_b200 kernels run on CUDA tensors only; there is no CPU path")


launch_count = 0      # kernels of this library launched (or captured) by this process


def _check(code: int, what: str):
    global launch_count
    launch_count += 1
    if code != 0:
        if code == 1:       # cudaErrorInvalidValue: the launcher refused the sizes
            raise KernelError(f"{what}: sizes not supported by this kernel")
        raise KernelError(f"{what}: CUDA error {code}")


# --------------------------------------------------------------------------

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor, scale: float = 1.0,
          positions: Optional[torch.Tensor] = None, sin_freq: Optional[torch.Tensor] = None):
    """``out[t] = table[ids[t]] * scale`` as float32.  ids int32 [T]; table [V, H].  ``sin_freq`` (float32 ``[(H + 1) //
    2]``) with ``positions`` (int32 ``[T]``): entry 2i of the row at position p also gets ``sin(p * sin_freq[i])`` and
    entry 2i + 1 the cosine."""
    _cuda(ids, table, out, positions, sin_freq)
    if sin_freq is not None:
        assert sin_freq.dtype == torch.float32 and sin_freq.is_contiguous() and sin_freq.shape[0] == (table.shape[1] + 1) // 2
        assert positions is not None and positions.dtype == torch.int32 and positions.shape[0] == ids.shape[0]
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous()
    T, (V, H) = ids.shape[0], table.shape
    assert out.shape == (T, H)
    _check(lib().prism_embed(_ptr(ids), _ptr(table), _dt(table), _ptr(out), T, H, V, float(scale),
                             _ptr(err), _ptr(positions) if sin_freq is not None else None, _ptr(sin_freq), _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """``residual += delta`` in place (float32; ``delta`` None, ``[T, H]`` or a
    stack ``[k, T, H]`` of partial sums), then ``out = rmsnorm(residual) * weight``
    for every row, or for the rows listed in ``rows`` (int32)."""
    _cuda(residual, delta, weight, out, rows)
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    T, H = residual.shape
    nsplit, stride = 0, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, H)
        nsplit = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * H
    n = T if rows is None else rows.shape[0]
    assert out.shape == (n, H) and weight.shape == (H,)
    _check(lib().prism_add_rmsnorm(_ptr(residual), _ptr(delta), F32 if delta is None else _dt(delta),
                                   nsplit, stride, _ptr(weight), _dt(weight), float(eps), _ptr(out),
                                   _dt(out), _ptr(rows), n, H, _stream()), "add_rmsnorm")


def sgemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor):
    """True float32 ``out = x @ w.T + bias`` on CUDA cores."""
    _cuda(x, w, bias, out)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32
    assert x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    _check(lib().prism_sgemm_nt(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                F32 if bias is None else _dt(bias), _ptr(out), out.stride(0), M, N, K,
                                _stream()), "sgemm")


USE_GEMV = os.environ.get("PRISM_GEMV", "1") != "0"
GEMV_MAX_M = int(os.environ.get("PRISM_GEMV_MAX_M", "16"))      # above 16 tokens it streams at half the bandwidth
EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2


def gemv_supported(M: int, N: int, K: int) -> bool:
    return USE_GEMV and bool(lib().prism_gemv_bf16_supported(M, N, K))


def gemv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epi: int = EPI_BF16):
    """Weight-streaming product for a few tokens: ``out = x @ w.T (+ bias)`` in
    bf16 (``EPI_BF16``) or float32 (``EPI_F32``); or, with ``w`` the fused
    ``[2I, K]`` gate/up weight, ``out[M, I] = silu(x @ gate.T) * (x @ up.T)``
    (``EPI_SWIGLU``)."""
    _cuda(x, w, bias, out)
    M, K = x.shape
    N = out.shape[1]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M
    assert w.shape[0] == (2 * N if epi == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epi == EPI_F32 else torch.bfloat16)
    _check(lib().prism_gemv_bf16(_ptr(w), w.stride(0), _ptr(x), x.stride(0) if M > 1 else K, _ptr(bias),
                                 F32 if bias is None else _dt(bias), _ptr(out), out.stride(0) if M > 1 else N,
                                 M, N, K, epi, _stream()), "gemv_bf16")


EPI_PARTIAL = 3
EPI_GEGLU = 4          # the paired epilogue with the gate through gelu_tanh instead of silu
_tc_err = {}


def _tc_err_word(device) -> torch.Tensor:
    """Device error word for the tensor-core GEMM's bounded waits (one per device)."""
    key = torch.device(device).index or 0
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


_tc_ws = {}
_tc_ws_retired = []       # outgrown workspaces: never freed, a captured graph may still hold their addresses


def _tc_workspace(device, floats: int, tiles: int):
    """Split-K workspace of the tensor-core GEMM: partial sums and one counter per
    tile.  Grown outside graph capture only; kernels leave the counters at zero.
    A workspace that a later call outgrows is kept alive for the life of the process:
    decode graphs captured earlier replay with its addresses, and memory given back to
    the allocator could by then hold somebody's activations."""
    key = torch.device(device).index or 0
    ws = _tc_ws.get(key)
    if ws is None or ws[0].numel() < floats or ws[1].numel() < tiles:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the split-K workspace must be sized before graph capture (run one step eagerly first)")
        if ws is not None:
            _tc_ws_retired.append(ws)
        ws = (torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
              torch.zeros(max(tiles, 4096), dtype=torch.int32, device=device))
        _tc_ws[key] = ws
    return ws


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epi: int = EPI_BF16, ksplit: int = 1, err: Optional[torch.Tensor] = None, group_rows: int = 0):
    """tcgen05 + TMA weight-streaming product for up to 64 tokens.  ``epi``:
    ``EPI_BF16`` / ``EPI_F32`` (``out [M, N]``, + bias), ``EPI_SWIGLU`` (``w`` is
    the fused ``[2N, K]`` gate/up weight), ``EPI_PARTIAL`` (``out`` float32
    ``[ksplit, M, N]`` partial sums over K for the next kernel to add).  ``group_rows`` (a multiple of 128):
    ``x`` is ``[groups, M, K]`` and the weight rows ``[g group_rows, (g + 1) group_rows)`` read ``x[g]``."""
    _cuda(x, w, bias, out)
    group_tokens = 0
    if group_rows:
        assert x.dim() == 3 and x.is_contiguous() and x.shape[0] == -(-w.shape[0] // group_rows) and group_rows % 128 == 0
        group_tokens = x.shape[1]
        x = x.view(-1, x.shape[2])[:group_tokens]
    M, K = x.shape
    N = out.shape[-1]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.is_contiguous()
    assert w.shape[0] == (2 * N if epi in (EPI_SWIGLU, EPI_GEGLU) else N)
    if epi == EPI_PARTIAL:
        assert out.dtype == torch.float32 and out.shape == (ksplit, M, N) and bias is None
    else:
        assert out.shape == (M, N) and (ksplit == 1 or epi not in (EPI_SWIGLU, EPI_GEGLU))
        assert out.dtype == (torch.float32 if epi == EPI_F32 else torch.bfloat16)
    err = err if err is not None else _tc_err_word(x.device)
    ws = cnt = None
    if ksplit > 1 and epi != EPI_PARTIAL:
        ws, cnt = _tc_workspace(x.device, ksplit * M * N, (N + 127) // 128)
    _check(lib().prism_gemm_tcgen05(_ptr(w), w.stride(0), _ptr(x), x.stride(0) if M > 1 else K, _ptr(bias),
                                    F32 if bias is None else _dt(bias), _ptr(out), N, M, N, K, epi, ksplit,
                                    _ptr(ws), _ptr(cnt), _ptr(err), int(group_rows), int(group_tokens), _stream()),
           "gemm_tcgen05")


USE_TC_GEMM = os.environ.get("PRISM_TC_GEMM", "1") != "0"
TC_GEMM_MAX_M = int(os.environ.get("PRISM_TC_GEMM_MAX_M", "16"))


# products with a long K (the down projection) stay on the tcgen05 kernel up to more tokens
# the fused gate/up + SwiGLU product stays on it up to 64 tokens: 14B layer sizes at batch 32, 8 layers + head:
# 1.66 ms against 1.67 ms with the library product + SwiGLU kernel (and 2.00 ms with the mma.sync small-M GEMM)
TC_GEMM_MAX_M_SWIGLU = int(os.environ.get("PRISM_TC_GEMM_MAX_M_SWIGLU", "64"))
TC_KSPLIT_FORCED = int(os.environ.get("PRISM_TC_KSPLIT", "0"))       # experiments: a fixed K-split
TC_GEMM_LONG_K = int(os.environ.get("PRISM_TC_GEMM_LONG_K", "8192"))
TC_GEMM_MAX_M_LONG_K = int(os.environ.get("PRISM_TC_GEMM_MAX_M_LONG_K", "64"))    # batch 64 decode step: 4.79 -> 4.66 ms


def tc_gemm_ok(x: torch.Tensor, w: torch.Tensor, max_m: Optional[int] = None) -> bool:
    """Whether the tcgen05 weight-streaming product takes this call (``max_m``: a caller's own
    limit on the tokens, instead of the general one)."""
    M, K = x.shape
    limit = TC_GEMM_MAX_M if max_m is None else max_m
    if K >= TC_GEMM_LONG_K:
        limit = max(limit, TC_GEMM_MAX_M_LONG_K)
    return (USE_TC_GEMM and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= limit
            and x.stride(1) == 1 and w.stride(1) == 1 and (M == 1 or x.stride(0) % 8 == 0) and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().prism_gemm_tcgen05_supported(M, w.shape[0], K)))


def tc_ksplit(N: int, K: int, sms: Optional[int] = None, M: Optional[int] = None) -> int:
    """CTAs that share one 128-row tile's K range: about one CTA per SM in all (``sms``: the device's
    count), at least 8 blocks of 64 k each.  With up to 16 tokens (``M``) two of the kernel's CTAs fit on an
    SM, so the count is rounded to the nearest instead of down (14B qkv projection, 56 tiles: 3 splits = 168
    CTAs instead of 2 = 112: 6.003 -> 5.880 ms a step at batch 8), and a product with a long K (the down
    projection) is shared half as finely again, 32 blocks each at least: the CTAs that double up have twice
    the weights on their way before the dependency wait (7B down projection, 5 -> 7 splits: 3.008 -> 2.992 ms
    a step at batch 8, 2.831 -> 2.804 at batch 1, 3.218 -> 3.181 at batch 16; 14B and 32B steps 1.9 % shorter).
    With 32 tokens and more one CTA fills an SM's shared memory: never more CTAs than SMs."""
    tiles = (N + 127) // 128
    if TC_KSPLIT_FORCED:
        return TC_KSPLIT_FORCED
    n_sms = sms or num_sms()
    kblocks = (K + 63) // 64
    few = M is not None and M <= 16
    ks = max(1, min((2 * n_sms + tiles) // (2 * tiles) if few else n_sms // tiles, kblocks // 8))
    if few and kblocks // ks >= 48:
        ks = max(ks, min((3 * n_sms // 2) // tiles, kblocks // 32))
    return ks


def check_tc_errors():
    """Raise if a bounded wait of the tensor-core GEMM ran out (synchronises)."""
    for word in _tc_err.values():
        code = int(word.item())
        if code:
            word.zero_()
            raise KernelError(f"tensor-core GEMM: device error {code} (a bounded wait ran out)")


def linear_delta(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, f32: bool = False) -> torch.Tensor:
    """A projection whose result will be added to the residual stream by the
    next norm: like ``linear``, but it may return a float32 stack ``[k, M, N]``
    of partial sums over K, which the fused add + norm kernel adds up.  ``f32``: the
    result is float32 in any case (never rounded to 16 bits before the residual sum)."""
    if bias is None and tc_gemm_ok(x, w):
        N, K = w.shape
        ks = tc_ksplit(N, K, M=x.shape[0])
        if ks > 1:
            out = torch.empty((ks, x.shape[0], N), dtype=torch.float32, device=x.device)
            gemm_tc(x, w, None, out, EPI_PARTIAL, ksplit=ks)
            return out
    return linear(x, w, bias, out_dtype=torch.float32 if f32 else None)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ w.T + bias`` with ``w`` in the ``[out, in]`` layout of the model
    file.  float32 activations, or a float32 weight under bf16 activations
    (a tensor the model file stores in 32-bit), go through the true-float32
    kernel; bf16 x bf16 goes to the library matrix product (cuBLAS through
    torch), as in andre-fu/prism (executor.py:109)."""
    _cuda(x, w, bias)
    M, N = x.shape[0], w.shape[0]
    want = out_dtype or (out.dtype if out is not None else x.dtype)
    if x.dtype == torch.float32 or w.dtype == torch.float32:
        x32 = x if x.dtype == torch.float32 else x.float()
        w32 = w if w.dtype == torch.float32 else w.float()
        o32 = out if (out is not None and out.dtype == torch.float32) else \
            torch.empty((M, N), dtype=torch.float32, device=x.device)
        sgemm(x32, w32, bias, o32)
        if want == torch.float32:
            return o32
        if out is not None:
            out.copy_(o32)
            return out
        return o32.to(want)
    if want in (torch.float32, torch.bfloat16) and tc_gemm_ok(x, w) and (out is None or out.is_contiguous()):
        if out is None or out.dtype != want:
            out = torch.empty((M, N), dtype=want, device=x.device)
        gemm_tc(x, w, bias, out, EPI_F32 if want == torch.float32 else EPI_BF16, ksplit=tc_ksplit(N, x.shape[1]))
        return out
    # bf16 x bf16, library product with float32 accumulation
    if want == torch.float32:
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            res += bias.float()
        if out is not None:
            out.copy_(res)
            return out
        return res
    b = bias if (bias is None or bias.dtype == torch.bfloat16) else bias.to(torch.bfloat16)
    if out is None:
        return torch.nn.functional.linear(x, w, b)
    if b is None:
        return torch.mm(x, w.t(), out=out)
    return torch.addmm(b, x, w.t(), out=out)


def linear_grouped(xs: torch.Tensor, w: torch.Tensor, rows, out_dtype: torch.dtype = torch.float32):
    """Projections of the same tokens that each read an input of their own: ``xs [G, T, K]``; the first ``rows[0]``
    rows of ``w [N, K]`` are applied to ``xs[0]``, the next ``rows[1]`` to ``xs[1]`` and so on.  Returns one ``[T,
    rows[g]]`` result per group, all with the same row stride where the groups are of one size.  One launch of the
    weight-streaming kernel where it takes the sizes (a decode step, groups of one size that is a multiple of 128,
    the last one no larger: the results are column blocks of one buffer), else one product per group."""
    G, T, K = xs.shape
    N = w.shape[0]
    rows = [int(r) for r in rows]
    assert G == len(rows) and sum(rows) == N and w.shape[1] == K and min(rows) > 0
    size = rows[0]
    bounds = [sum(rows[:g]) for g in range(G + 1)]
    if (xs.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and size % 128 == 0 and all(r == size for r in rows[:-1])
            and rows[-1] <= size and xs.is_contiguous() and tc_gemm_ok(xs[0], w)
            and out_dtype in (torch.float32, torch.bfloat16)):
        out = torch.empty((T, N), dtype=out_dtype, device=xs.device)
        gemm_tc(xs, w, None, out, EPI_F32 if out_dtype == torch.float32 else EPI_BF16, ksplit=tc_ksplit(N, K),
                group_rows=size)
        return [out[:, bounds[g]:bounds[g + 1]] for g in range(G)]
    return [linear(xs[g], w[bounds[g]:bounds[g + 1]], None, out_dtype=out_dtype) for g in range(G)]


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor):
    """``out[t, j] = (cos, sin)(positions[t] * inv_freq[j])`` in float32, shared
    by every layer and head of a step."""
    _cuda(positions, inv_freq, out)
    T, half = positions.shape[0], inv_freq.shape[0]
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, half, 2)
    _check(lib().prism_rope_table(_ptr(positions), _ptr(inv_freq), half, T, _ptr(out), _stream()), "rope_table")


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                  tok_seg: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  block_table: Optional[torch.Tensor], num_pages: int, max_pos: int,
                  err: torch.Tensor, table: Optional[torch.Tensor] = None):
    """Rotate ``q [T, nh, hd]`` and ``k [T, nkv, hd]`` in place (views of one
    row-strided buffer) and store k, v at their positions in the paged cache
    ``[pages, P, nkv, hd]``.  ``k_cache`` None: rotate only.  ``table``: the
    step's cos/sin table from ``rope_table`` (lets the vector kernel run)."""
    _cuda(q, k, v, positions, tok_seg, inv_freq, k_cache, v_cache, block_table)
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rs = q.stride(0)
    assert T == 1 or (k.stride(0) == rs and v.stride(0) == rs), "q, k, v must be views of one buffer"
    assert q.stride(2) == 1 and q.stride(1) == hd and k.stride(1) == hd and v.stride(1) == hd
    assert positions.dtype == torch.int32 and tok_seg.dtype == torch.int32
    P = W = 0
    if k_cache is not None:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == q.dtype
        assert k_cache.shape[2:] == (nkv, hd) and block_table.dtype == torch.int32
        P, W = k_cache.shape[1], block_table.shape[1]
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape[0] * 2 == rotary_dim
    if T == 1:
        rs = 0                  # a single row: its stride is never used
    if table is not None:
        assert table.dtype == torch.float32 and table.shape == (T, rotary_dim // 2, 2)
    _check(lib().prism_rope_kv_write(_ptr(q), _ptr(k), _ptr(v), _dt(q), rs, _ptr(positions),
                                     _ptr(tok_seg), _ptr(inv_freq), _ptr(table), rotary_dim, _ptr(k_cache),
                                     _ptr(v_cache), _ptr(block_table), W, P, num_pages, T, nh, nkv,
                                     hd, max_pos, _ptr(err), _stream()), "rope_kv_write")


def rope_kv_write_partial(parts: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                          positions: torch.Tensor, tok_seg: torch.Tensor, table: torch.Tensor, rotary_dim: int,
                          k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                          block_table: Optional[torch.Tensor], num_pages: int, max_pos: int, nkv: int,
                          err: torch.Tensor):
    """``rope_kv_write`` for a qkv projection that arrives as float32 partial
    sums ``parts [k, T, (nh + 2 nkv) * hd]`` (+ ``bias``): the sum, the bias, the
    rotation and the cache store in one kernel; rotated q goes to ``q_out [T, nh, hd]``."""
    _cuda(parts, bias, q_out, positions, tok_seg, table, k_cache, v_cache, block_table)
    ks, T, D = parts.shape
    _, nh, hd = q_out.shape
    assert parts.dtype == torch.float32 and parts.is_contiguous() and D == (nh + 2 * nkv) * hd
    assert q_out.is_contiguous() and table.dtype == torch.float32 and table.shape == (T, rotary_dim // 2, 2)
    P = W = 0
    if k_cache is not None:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == q_out.dtype
        assert k_cache.shape[2:] == (nkv, hd)
        P, W = k_cache.shape[1], block_table.shape[1]
    _check(lib().prism_rope_kv_write_partial(_ptr(parts), ks, _ptr(bias), F32 if bias is None else _dt(bias),
                                             _ptr(q_out), nh * hd, _dt(q_out), _ptr(positions), _ptr(tok_seg),
                                             _ptr(table), rotary_dim, _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
                                             W, P, num_pages, T, nh, nkv, hd, max_pos, _ptr(err), _stream()),
           "rope_kv_write_partial")


# The qkv projection of a few tokens: K-split tcgen05 GEMM -> float32 partial sums -> one kernel that adds them and
# the bias, rotates and stores (several CTAs per token).  PRISM_QKV_LIBRARY=1 (with PRISM_QKV_PARTIAL=0): the
# library product and the rotary kernel, for comparison.
QKV_LIBRARY = os.environ.get("PRISM_QKV_LIBRARY", "0") == "1"


def qkv_rotate_store(ctx, x: torch.Tensor, qkv_w: torch.Tensor, qkv_b: Optional[torch.Tensor], nh: int, nkv: int,
                     hd: int, rot, cache) -> torch.Tensor:
    """The front half of an attention layer: qkv projection (+ bias), rotary
    encoding of q and k (``rot``: RotaryParams or None), store of k, v into the
    cache plane.  Returns q ``[T, nh, hd]``.  For a few tokens the projection runs
    K-split on the tensor-core GEMM and its partial sums are added, biased,
    rotated and stored by one kernel."""
    T = x.shape[0]
    qs, kvs = nh * hd, nkv * hd
    table = None
    if rot is not None and rot.rotary_dim:
        key = ("rotary_table", rot.inv_freq.data_ptr())          # one table per step for all layers
        table = ctx.scratch.get(key)
        if table is None:
            table = ctx.scratch[key] = ctx.alloc((T, rot.rotary_dim // 2, 2), torch.float32)
            rope_table(ctx.positions, rot.inv_freq, table)
    kc, vc = (cache.k, cache.v) if cache.write else (None, None)
    rd = rot.rotary_dim if rot is not None else 0
    if QKV_PARTIAL and table is not None and tc_gemm_ok(x, qkv_w) and hd % 8 == 0 and rot.rotary_dim % 16 == 0:
        ks = tc_ksplit(qkv_w.shape[0], qkv_w.shape[1], M=T)
        if ks > 1:
            parts = ctx.alloc((ks, T, qs + 2 * kvs), torch.float32)
            gemm_tc(x, qkv_w, None, parts, EPI_PARTIAL, ksplit=ks)
            q = ctx.alloc((T, nh, hd), x.dtype)
            rope_kv_write_partial(parts, qkv_b, q, ctx.positions, ctx.tok_seg, table, rot.rotary_dim, kc, vc,
                                  cache.block_table, cache.num_pages, ctx.max_positions, nkv, ctx.err)
            return q
    if QKV_LIBRARY and x.dtype == torch.bfloat16:
        b = qkv_b if (qkv_b is None or qkv_b.dtype == torch.bfloat16) else qkv_b.to(torch.bfloat16)
        qkv = torch.nn.functional.linear(x, qkv_w, b)
    else:
        qkv = linear(x, qkv_w, qkv_b)
    q = qkv[:, :qs].view(T, nh, hd)
    k = qkv[:, qs:qs + kvs].view(T, nkv, hd)
    v = qkv[:, qs + kvs:].view(T, nkv, hd)
    rope_kv_write(q, k, v, ctx.positions, ctx.tok_seg, rot.inv_freq if rot else None, rot.rotary_dim if rot else 0,
                  kc, vc, cache.block_table, cache.num_pages, ctx.max_positions, ctx.err, table=table)
    return q


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                      tok_seg: torch.Tensor, num_pages: int, window: Optional[int], scale: float,
                      err: torch.Tensor):
    """Shape-generic paged causal GQA attention; ``q [T, nh, hd]`` row-strided,
    ``out [T, nh*hd]``."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, tok_seg)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1
    assert k_cache.dtype == q.dtype and out.dtype == q.dtype
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} > 256 is not supported")
    _check(lib().prism_attention_generic(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                         _ptr(k_cache), _ptr(v_cache), _dt(q), _ptr(block_table),
                                         block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, nh,
                                         nkv, hd, P, num_pages, int(window or 0), float(scale),
                                         _ptr(err), _stream()), "attention_generic")


def swiglu(gu: torch.Tensor, out: torch.Tensor):
    """``out = silu(gu[:, :I]) * gu[:, I:]``."""
    _cuda(gu, out)
    T, I2 = gu.shape
    assert gu.is_contiguous() and out.is_contiguous() and out.shape == (T, I2 // 2) and out.dtype == gu.dtype
    _check(lib().prism_swiglu(_ptr(gu), _ptr(out), _dt(gu), T, I2 // 2, _stream()), "swiglu")


_argmax_ws = {}


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor):
    """Per row: argmax if its temperature <= 0, else inverse-CDF sampling of
    ``softmax(logits / temperature)`` at the uniform number ``u``."""
    _cuda(logits, temperature, u, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    R, V = logits.shape
    if temperature is None and V >= 8192 and R <= 4096 and not torch.cuda.is_current_stream_capturing():
        # greedy over a large vocabulary: many blocks per row
        key = torch.device(logits.device).index or 0
        ws = _argmax_ws.get(key)
        nb = 32
        if ws is None or ws[0].numel() < R * nb:
            n = max(R * nb, 4096 * nb)
            ws = _argmax_ws[key] = (torch.empty(n, dtype=torch.float32, device=logits.device),
                                    torch.empty(n, dtype=torch.int32, device=logits.device),
                                    torch.zeros(4096, dtype=torch.int32, device=logits.device))
        _check(lib().prism_argmax_split(_ptr(logits), logits.stride(0), R, V, nb, _ptr(ws[0]), _ptr(ws[1]),
                                        _ptr(ws[2]), _ptr(out), _stream()), "argmax_split")
        return
    _check(lib().prism_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(u),
                              _ptr(out), _stream()), "sample")


# --------------------------------------------------------------------------
# composites: the places where a faster kernel is chosen for a shape
# --------------------------------------------------------------------------

_num_sms = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked of the driver
    once per device.  The grid shapes below (K-splits, attention splits) are sized by it."""
    if not torch.cuda.is_available():
        raise KernelError("the number of SMs is a property of a CUDA device; pass sms= to size a grid without one")
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _num_sms.get(idx)
    if n is None:
        n = _num_sms[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


FORCE_GENERIC_ATTENTION = os.environ.get("PRISM_ATTENTION", "") == "generic"


QKV_PARTIAL = os.environ.get("PRISM_QKV_PARTIAL", "1") != "0"


def _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml):
    slots = T * nsplit                                   # partial results: one per (token, split) ...
    if items is not None:                                # ... or one per work item
        assert starts is not None and items.dtype == torch.int32 and starts.dtype == torch.int32
        assert items.dim() == 2 and items.shape[1] == 4 and items.is_contiguous() and items.data_ptr() % 16 == 0
        assert starts.numel() == T and starts.is_contiguous() and items.shape[0] <= 65535
        slots = items.shape[0]
    if nsplit > 1:
        assert part_o.dtype == torch.float32 and part_o.numel() >= slots * nh * hd
        assert part_ml.dtype == torch.float32 and part_ml.numel() >= slots * nh * 2


def attention_decode_bf16(q, out, k_cache, v_cache, block_table, positions, tok_seg, num_pages, window,
                          scale, nsplit, part_o, part_ml, err, items: Optional[torch.Tensor] = None,
                          starts: Optional[torch.Tensor] = None):
    """Tensor-core decode attention (one token per request) with the keys split
    over ``nsplit`` CTAs per (token, kv head); ``part_o [T, nh, nsplit, hd]`` and
    ``part_ml [T, nh, nsplit, 2]`` are float32 scratch for the partial results.
    With ``items`` (device int32 ``[n, 4]``) and ``starts`` (``[T]``), the step's work items
    (``decode_work_items``), every token's keys are shared among the CTAs chosen for it; ``nsplit``
    is then the most items of a token and the scratch ``[n, nh, hd]`` and ``[n, nh, 2]``."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, tok_seg, part_o, part_ml, items, starts)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1
    _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml)
    _check(lib().prism_attention_decode_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache),
                                             _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                             _ptr(positions), _ptr(tok_seg), T, nh, nkv, hd, P, num_pages,
                                             int(window or 0), float(scale), _ptr(part_o), _ptr(part_ml),
                                             int(nsplit), _ptr(items), _ptr(starts), 0 if items is None else items.shape[0],
                                             _ptr(err), _stream()), "attention_decode_bf16")
    if nsplit > 1:
        global launch_count
        launch_count += 1          # the merge kernel


def attention_decode_qkv_bf16(parts, bias, table, max_pos, out, k_cache, v_cache, block_table, positions, tok_seg,
                              num_pages, nh, window, scale, nsplit, part_o, part_ml, err,
                              items: Optional[torch.Tensor] = None, starts: Optional[torch.Tensor] = None):
    """Decode attention that finishes the qkv projection itself: ``parts [ks, T, (nh + 2 nkv) * hd]`` are the
    projection's float32 partial sums, ``bias`` its bias or None, ``table [T, hd / 2, 2]`` the step's cos/sin.
    Every CTA adds, biases and rotates the query rows it needs; the CTA that holds a token's own position
    does the same for the token's key and value, stores them in the cache and uses them.  The whole head is
    rotated (rotary_dim == hd)."""
    _cuda(parts, bias, table, out, k_cache, v_cache, block_table, positions, tok_seg, part_o, part_ml)
    ks, T, D = parts.shape
    nkv, P, hd = k_cache.shape[2], k_cache.shape[1], k_cache.shape[3]
    assert parts.dtype == torch.float32 and parts.is_contiguous() and D == (nh + 2 * nkv) * hd
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape == (T, hd // 2, 2)
    assert k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (T, nh * hd)
    _cuda(items, starts)
    _check_decode_scratch(items, starts, T, nh, hd, nsplit, part_o, part_ml)
    _check(lib().prism_attention_decode_qkv_bf16(_ptr(parts), ks, _ptr(bias), F32 if bias is None else _dt(bias),
                                                 _ptr(table), int(max_pos), _ptr(out), out.stride(0), _ptr(k_cache),
                                                 _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                                 _ptr(positions), _ptr(tok_seg), T, nh, nkv, hd, P, num_pages,
                                                 int(window or 0), float(scale), _ptr(part_o), _ptr(part_ml),
                                                 int(nsplit), _ptr(items), _ptr(starts),
                                                 0 if items is None else items.shape[0], _ptr(err), _stream()),
           "attention_decode_qkv_bf16")
    if nsplit > 1:
        global launch_count
        launch_count += 1          # the merge kernel


def attention_prefill_bf16(q, out, k_cache, v_cache, block_table, seg_start, cached_len, max_q_len,
                           num_pages, window, scale, err):
    """Tensor-core attention for segments of any length (portions of prompts,
    and single tokens among them)."""
    _cuda(q, out, k_cache, v_cache, block_table, seg_start, cached_len)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    S = cached_len.shape[0]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1 and seg_start.shape[0] == S + 1
    _check(lib().prism_attention_prefill_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache),
                                              _ptr(v_cache), _ptr(block_table), block_table.shape[1],
                                              _ptr(seg_start), _ptr(cached_len), S, int(max_q_len), nh, nkv, hd,
                                              P, num_pages, int(window or 0), float(scale), _ptr(err),
                                              _stream()), "attention_prefill_bf16")


PREFILL_SPLIT_MIN_TILES = 16      # key tiles (of 64) a split CTA should keep
PREFILL_SPLIT_FROM_TILES = 64     # fewer key tiles than this are not split: the merge costs as much as it saves ...
PREFILL_SPLIT_FROM_TILES_FEW_CTAS = 32    # ... unless the query tiles fill under a quarter of the GPU


def prefill_splits(S: int, max_q_len: int, nh: int, max_kv_len: int, window: Optional[int],
                   sms: Optional[int] = None) -> int:
    """CTAs that share the key tiles of one (head, 128 query rows) in the tcgen05 prefill kernel: 1 unless
    the query tiles alone leave most of the GPU idle and the keys are many (a short portion against a
    long cache); then as many as fill the two CTAs per SM, each with at least PREFILL_SPLIT_MIN_TILES.
    (Measured at the 7B head counts, 128 new tokens: 2,048 cached 42 -> 34 us in 2 splits, 8,192 cached
    127 -> 46 us in 8, 32,768 cached 471 -> 86 us in 10; 512 new tokens after 2,048: 48 us whole, 55 us in 2.)"""
    if os.environ.get("PRISM_PREFILL_SPLITS"):
        return int(os.environ["PRISM_PREFILL_SPLITS"])
    NUM_SMS = sms or num_sms()
    ctas = S * nh * ((max_q_len + 127) // 128)
    span = min(max_kv_len, window + max_q_len) if window else max_kv_len
    tiles = (span + 63) // 64
    if tiles < (PREFILL_SPLIT_FROM_TILES_FEW_CTAS if 4 * ctas <= 2 * NUM_SMS else PREFILL_SPLIT_FROM_TILES):
        return 1
    return max(1, min((2 * NUM_SMS) // max(1, ctas), tiles // PREFILL_SPLIT_MIN_TILES, 16))


def attention_merge(part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor):
    """``out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)`` over the splits' partial results
    ``part_o [T, nh, nsplit, hd]`` / ``part_ml [T, nh, nsplit, 2]`` (float32); ``out`` bf16 ``[T, nh * hd]``."""
    _cuda(part_o, part_ml, out)
    T, nh, ns, hd = part_o.shape
    assert part_o.is_contiguous() and part_ml.is_contiguous() and part_ml.shape == (T, nh, ns, 2)
    assert part_o.dtype == torch.float32 and part_ml.dtype == torch.float32 and out.dtype == torch.bfloat16
    assert out.stride(1) == 1 and out.shape == (T, nh * hd)
    _check(lib().prism_attention_merge_bf16(_ptr(part_o), _ptr(part_ml), ns, _ptr(out), out.stride(0), T, nh, hd,
                                            _stream()), "attention_merge")


def attention_prefill_tc(q, out, k_cache, v_cache, block_table, seg_start, cached_len, max_q_len,
                         num_pages, window, scale, err, nsplit: int = 1, first_token: int = 0):
    """The same on the 5th-generation tensor cores (tcgen05, TMA, tensor memory): 128 query
    rows per CTA.  Head size 64 or 128, pages of a multiple of 64 tokens.  ``nsplit`` > 1: that many
    CTAs share a query tile's keys and a second kernel merges their partial results (of the tokens
    from ``first_token`` on: the segments given must cover exactly those)."""
    _cuda(q, out, k_cache, v_cache, block_table, seg_start, cached_len)
    T, nh, hd = q.shape
    nkv, P = k_cache.shape[2], k_cache.shape[1]
    S = cached_len.shape[0]
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and q.stride(1) == hd and out.stride(1) == 1 and seg_start.shape[0] == S + 1
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
    po = pml = None
    if nsplit > 1:
        po = torch.empty((T, nh, nsplit, hd), dtype=torch.float32, device=q.device)
        pml = torch.empty((T, nh, nsplit, 2), dtype=torch.float32, device=q.device)
    _check(lib().prism_attention_prefill_tc(_ptr(q), q.stride(0), T, _ptr(out), out.stride(0), _ptr(k_cache),
                                            _ptr(v_cache), k_cache.shape[0], _ptr(block_table), block_table.shape[1],
                                            _ptr(seg_start), _ptr(cached_len), S, int(max_q_len), nh, nkv, hd,
                                            P, num_pages, int(window or 0), float(scale), _ptr(err), int(nsplit),
                                            _ptr(po), _ptr(pml), _stream()), "attention_prefill_tc")
    if nsplit > 1:
        attention_merge(po[first_token:], pml[first_token:], out[first_token:])


def attention_prefill_tc_supported(hd: int, nh: int, nkv: int, page_size: int) -> bool:
    return bool(lib().prism_attention_prefill_tc_supported(hd, nh, nkv, page_size))


ATTENTION_TC = os.environ.get("PRISM_ATTN_TC", "1") != "0"
ATTENTION_TC_MIN_Q = int(os.environ.get("PRISM_ATTN_TC_MIN_Q", "64"))     # shorter portions: 64-row mma.sync tiles


LONG_CONTEXT = int(os.environ.get("PRISM_LONG_CONTEXT", "4096"))      # keys from which a lone CTA per query tile is too slow


def prefill_on_tc(max_q_len: int, max_kv_len: int, window: Optional[int]) -> bool:
    """Portions of 64 tokens and more go to the tcgen05 kernel (128-row query tiles), shorter ones to the
    mma.sync kernel (64-row tiles, cheaper to start) - unless the cache is long: the tcgen05 kernel can share
    a query tile's keys among CTAs, the mma.sync kernel walks them with one CTA per head (128 tokens behind
    32,768: 86 us against 729 us), and a prompt's last portion can be a few tokens behind all the others."""
    span = min(max_kv_len, window + max_q_len) if window else max_kv_len
    return max_q_len >= ATTENTION_TC_MIN_Q or span >= LONG_CONTEXT


def decoders_apart(n_leading_single: int, their_max_kv_len: int, window: Optional[int]) -> bool:
    """In a mixed step: whether the decoding requests at the head of the batch go to the decode kernel.  Worth
    a launch of its own from ``MIXED_SPLIT_MIN`` of them on - or from one, if their contexts are long: as
    one-token segments of the prefill kernel each would be a single CTA per head walking all its keys."""
    if n_leading_single <= 0:
        return False
    span = min(their_max_kv_len, window + 64) if window else their_max_kv_len
    return n_leading_single >= MIXED_SPLIT_MIN or span >= LONG_CONTEXT


def attention_bf16_shape_ok(hd: int, nh: int, nkv: int) -> bool:
    """The rule of ``prism_attention_bf16_supported`` (csrc/attention_bf16.cu), for callers that have no
    library loaded (a model built on a host without a GPU)."""
    return 16 <= hd <= 128 and hd % 16 == 0 and nkv > 0 and nh % nkv == 0 and nh // nkv <= 16


def attention_bf16_supported(hd: int, nh: int, nkv: int) -> bool:
    return bool(lib().prism_attention_bf16_supported(hd, nh, nkv))


def decode_tiles(position: int, window: Optional[int]) -> int:
    """64-key tiles the token at ``position`` sees (its own key included)."""
    lo = max(0, position - window + 1) if window else 0
    return position // 64 - lo // 64 + 1


def decode_used_splits(tiles: int, target_x16: int, cap: int) -> int:
    """CTAs that share one request's keys under a target of ``target_x16 / 16`` tiles per CTA: as many as keep
    each at or below the target, none with fewer than ``DECODE_MIN_TILES`` tiles, at most ``cap``."""
    target = max(target_x16, DECODE_MIN_TILES * 16)
    return min(max(min(-(-tiles * 16 // target), tiles // DECODE_MIN_TILES), 1), cap)


# Where one wave leaves a quarter of the CTAs or more at less than half the longest CTA's length (many requests too
# short to be split hold a place each and leave it early), the plan goes to CTAs of about half the size in two
# waves: the second wave moves into the places the short CTAs have left.  Equal contexts never qualify (all CTAs are
# the longest), and there two waves lose: batch 48 at 2,100 keys 4.19 -> 4.28 ms a step, batch 56 4.40 -> 4.64 ms.
DECODE_SHORT_CTA = 0.5
DECODE_SECOND_WAVE_FROM_SHARE = 0.25


def _tiles_of(positions, window: Optional[int]):
    pos = np.asarray(positions, dtype=np.int64)
    lo = np.maximum(pos - window + 1, 0) if window else 0
    return pos // 64 - lo // 64 + 1


def _used_splits(tiles, target_x16: int, cap: int = 64):
    """``decode_used_splits`` for an array of requests."""
    target = max(target_x16, DECODE_MIN_TILES * 16)
    used = np.minimum((tiles * 16 + (target - 1)) // target, np.minimum(tiles // DECODE_MIN_TILES, cap))
    return np.maximum(used, 1, out=used)


def _smallest_target(tiles, nkv: int, places: int) -> int:
    """The smallest target (tiles per CTA, in sixteenths), from the tiles divided by the places on, with which
    the requests' CTAs fit into ``places``.  It is seldom much more than that: the search widens from there."""
    tiles16, most = tiles * 16, np.minimum(tiles // DECODE_MIN_TILES, 64)

    def fits(target):
        used = np.minimum((tiles16 + (target - 1)) // target, most)
        return (int(used.sum()) + int(np.count_nonzero(used == 0))) * nkv <= places
    lo = max(DECODE_MIN_TILES * 16, -(-int(tiles.sum()) * nkv * 16 // places))
    if fits(lo):
        return lo
    top = max(lo, int(tiles.max()) * 16)                      # one CTA each: fits, or nothing does
    step = max(1, lo // 8)
    hi = min(top, lo + step)
    while hi < top and not fits(hi):
        lo, step = hi, step * 2
        hi = min(top, lo + step)
    lo += 1                                                   # lo does not fit, hi does
    while lo < hi:
        mid = (lo + hi) // 2
        if fits(mid):
            hi = mid
        else:
            lo = mid + 1
    return lo


# Splitting has to pay: where even the best plan leaves the longest CTA above this fraction of the longest request
# (many requests of about the same length and only a few places to spare), every request keeps a single CTA and
# the step needs no merge kernel (64 requests of 1,024 to 1,536 keys on 8 kv heads: ten of them could be halved,
# the eleventh decides the kernel's time all the same).
DECODE_SPLIT_GAIN = 0.75


def decode_split_target(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                        n_real: Optional[int] = None) -> int:
    """The decode kernel's plan for a step: 64-key tiles per CTA, in sixteenths - the smallest target with which
    the CTAs of the step's decoding requests (``decode_used_splits`` for each, times the kv heads) still fit on
    the GPU at once, two per SM.  A long context among short ones is then shared among many CTAs while the short
    ones take one each, and no CTA runs much longer than the rest.  For equal contexts this is the rule measured
    before: 11 CTAs per (token, kv head) at batch 1 and 2,100 keys, 9 at batch 8, 4 at batch 16, 1 from batch 48
    on.  Where many short requests hold most of the places, so that many CTAs are far shorter than the
    longest (``DECODE_SECOND_WAVE_FROM_SHARE``), the target is the one that fits into twice the places: the short
    CTAs end early and the second wave takes their places (64 requests of 128 to 4,096 keys, 4 kv heads: 5.31 ->
    4.93 ms a step; 32 requests, 8 kv heads: 9.28 -> 8.74 ms; 8 requests, whose CTAs are all about as long:
    3.03 -> 3.16 ms, which is why it is no general rule).  A batch so large that one CTA per (token, kv head) is
    more than fits at once: the same, from the waves that this takes.  ``n_real``: the requests after the first
    ``n_real`` are padding (rows of a captured graph's bucket): they take a place each, but say nothing about
    how unequal the step's CTAs are."""
    slots = 2 * (sms or num_sms())
    tiles = _tiles_of(positions, window)
    real = slice(0, len(tiles) if n_real is None else n_real)
    places = slots * max(1, -(-len(tiles) * nkv // slots))       # the waves that one CTA each needs in any case
    target = _smallest_target(tiles, nkv, places)
    used = _used_splits(tiles, target)
    per = tiles[real] / used[real]
    if used[real][per < DECODE_SHORT_CTA * per.max()].sum() >= DECODE_SECOND_WAVE_FROM_SHARE * used[real].sum():
        target = _smallest_target(tiles, nkv, places + slots)
        used = _used_splits(tiles, target)
    if (tiles / used).max() > DECODE_SPLIT_GAIN * tiles.max():
        target = int(tiles.max()) * 16                           # one CTA each
    return target


def decode_plan_for(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                    n_real: Optional[int] = None):
    """``(target_x16, cap)`` for a step's decoding requests: the plan and the most CTAs any request gets under
    it.  Many requests (a third of a wave of CTAs or more) with long contexts of about one length
    (``DECODE_LONG_FROM_TILES``) get equal splits chosen by how they fill whole waves, see below; the older
    rule for one CTA each at 16,384 keys and more (``DECODE_BALANCE_FROM_TILES``) remains for what that leaves."""
    n_sms = sms or num_sms()
    target = decode_split_target(positions, nkv, window, n_sms, n_real)
    tiles = _tiles_of(positions, window)
    cap = int(_used_splits(tiles, target).max())
    real = tiles if n_real is None else tiles[:n_real]
    least, most = int(real.min()), int(real.max())
    slots = 2 * n_sms
    if least >= DECODE_LONG_FROM_TILES and 4 * least >= 3 * most and 3 * len(tiles) * nkv >= slots:
        # many requests with long contexts of about one length: all get the same number of CTAs - one that
        # fills its last wave to 85 % or more, and among those the one that makes about two waves (measured at
        # 8,192 and 16,384 keys on 4 kv heads: 32 requests best in 4 CTAs each, 40 in 5, 48 in 4 or 3, 64 in 2
        # or 3; up to 11 % of the kernel's time against one wave's worth)
        def waves(k):
            return len(tiles) * nkv * k / slots
        ks = [k for k in range(1, 9) if k == 1 or least // k >= 16]
        full = [k for k in ks if waves(k) / -(-waves(k) // 1) >= 0.85]
        k = min(full, key=lambda k: abs(waves(k) - 2.0)) if full else max(ks, key=lambda k: waves(k) / -(-waves(k) // 1))
        target = -(-most * 16 // k)
        cap = int(_used_splits(tiles, target).max())
    elif cap == 1 and least >= DECODE_BALANCE_FROM_TILES:
        def fill(k):
            m = len(tiles) * nkv * k / n_sms
            return m / -(-m // 1)
        for k in range(2, 9):
            if least // k < 16:
                break
            if fill(k) >= 0.95 > fill(1):
                target = max(DECODE_MIN_TILES * 16, -(-least * 16 // k))
                cap = int(_used_splits(tiles, target).max())
                break
    return target, cap


def decode_work_items(positions, nkv: int, window: Optional[int], sms: Optional[int] = None,
                      n_real: Optional[int] = None, memo: Optional[dict] = None):
    """The decode attention kernel's work for a step: ``(items [n, 4], starts [B], most)`` as int32 arrays
    and the most items any request has.  Request b (at ``positions[b]``, token and segment b of the step) gets
    ``decode_plan_for``'s number of CTAs per kv head, less where fewer already leave each the same number of
    tiles: ``used`` items ``{b, split | used << 16, position, b}`` from item ``first`` on, ``starts[b] = first |
    used << 16``.  The requests whose CTAs are longest come first, so that when the items are more than fit on
    the GPU at once the short ones run last.  ``n_real``: the requests after these are a graph bucket's padding.
    ``memo``: a dict the caller keeps between steps; the items depend on the positions only through the
    requests' tile counts, which change once in 64 steps, so the step before has usually left all but the
    position column."""
    pos = np.asarray(positions, dtype=np.int64)
    tiles = _tiles_of(pos, window)
    key = None
    if memo is not None:
        key = (tiles.tobytes(), n_real, nkv, window, sms)
        if memo.get("key") == key:
            items, tok, starts, most = memo["value"]
            items = items.copy()
            items[:, 2] = pos[tok]
            return items, starts, most
    target, cap = decode_plan_for(positions, nkv, window, sms, n_real)
    used = _used_splits(tiles, target, cap)
    per = -(-tiles // used)
    used = -(-tiles // per)                                # no CTA without a tile
    order = np.argsort(-per, kind="stable")
    first = np.empty(len(pos), dtype=np.int64)
    first[order] = np.cumsum(used[order]) - used[order]
    tok = np.repeat(order, used[order])
    split = np.arange(len(tok)) - first[tok]
    items = np.stack([tok, split | (used[tok] << 16), pos[tok], tok], axis=1).astype(np.int32)
    starts, most = (first | (used << 16)).astype(np.int32), int(used.max())
    if memo is not None:
        memo["key"], memo["value"] = key, (items, tok, starts, most)
    return items, starts, most


DECODE_LONG_FROM_TILES = 128         # 8,192 keys
DECODE_MIN_TILES = 3                # 64-key tiles a split CTA keeps at least (csrc/attention_bf16.cuh: DEC_MIN_TILES)
DECODE_BALANCE_FROM_TILES = 256     # 16,384 keys: below, the merge costs what the balance gains (batch 64: 8,192 keys
                                    # 203 -> 201 us in 4 splits, 32,768 keys 717 -> 673 us)


def decode_splits(T: int, nkv: int, max_kv_len: int, window: Optional[int], balance: bool = True,
                  sms: Optional[int] = None) -> int:
    """How many CTAs share one (token, kv head)'s keys: as many as fill one wave
    of two CTAs per SM, at most one per ``DECODE_MIN_TILES`` 64-key tiles.  More, shorter CTAs lose:
    each pays the same fixed latencies (position, block table, first bytes, merge), and the merge grows
    with them (batch 1 at 2,100 keys: 33 splits of one tile 2.90 ms a step, 12 splits 2.81, 8 splits 2.87).
    ``max_kv_len`` is the longest context of the batch, or, when a graph is captured, the longest the
    graph may ever see - the kernel itself keeps ``DECODE_MIN_TILES`` tiles per CTA for the context it
    finds and leaves the splits it does not need empty.  ``balance`` (the few splits of a large batch
    against long contexts) is for the former only: a bound of 32,768 says nothing about the contexts a
    replay will meet."""
    if os.environ.get("PRISM_DECODE_SPLITS", "0") != "0":
        return int(os.environ["PRISM_DECODE_SPLITS"])
    NUM_SMS = sms or num_sms()
    span = min(max_kv_len, window + 64) if window else max_kv_len
    tiles = max(1, (span + 63) // 64)
    fill = (2 * NUM_SMS) // max(1, T * nkv)
    n = max(1, min(-(-tiles // DECODE_MIN_TILES), 64, fill))
    if balance and n == 1 and tiles >= DECODE_BALANCE_FROM_TILES:
        # A large batch against long contexts: one CTA per (token, kv head) fills the GPU, but unevenly (256
        # CTAs are two on 108 SMs and one on 40, and the kernel lasts as long as the pairs).  A few splits
        # make the CTAs small enough to spread evenly: the fewest (each keeping 16 tiles or more) that
        # load every SM to within 5 % of the busiest.
        def balance(k):
            m = T * nkv * k / NUM_SMS
            return m / -(-m // 1)
        for k in range(1, 9):
            if k > 1 and tiles // k < 16:
                break
            if balance(k) >= 0.95:
                return k
    return n


# A mixed step hands its leading single-token segments to the decode kernel when there are at least
# this many (measured on 7B shapes, 512-token portion beside them: 8 decoders 1.72 vs 1.65 ms per
# 4 layers with / without the split, 64 decoders 2.09 vs 2.90 ms).
MIXED_SPLIT_MIN = int(os.environ.get("PRISM_MIXED_SPLIT_MIN", "12"))


def _leading_single_token_segments(ctx) -> int:
    """How many segments at the start of the batch bring exactly one token (the scheduler
    puts the decoding requests first).  Known on the host only; 0 inside a captured graph."""
    if ctx.host is None:
        return 0
    n = ctx.scratch.get("lead_single")
    if n is None:
        n = 0
        for q in ctx.host["q_len"]:
            if q != 1:
                break
            n += 1
        ctx.scratch["lead_single"] = n
    return n


def _attention_portions(ctx, q, out, cache, window, scale, first_seg: int):
    """Segments ``first_seg ..`` of the batch with the prefill kernels."""
    T, nh, hd = q.shape
    nkv = cache.k.shape[2]
    seg_start, cached_len, bt = ctx.seg_start[first_seg:], ctx.cached_len[first_seg:], cache.block_table[first_seg:]
    if (ATTENTION_TC and prefill_on_tc(ctx.max_q_len, ctx.max_kv_len, window) and scale > 0 and cache.k.is_contiguous()
            and cache.v.is_contiguous() and attention_prefill_tc_supported(hd, nh, nkv, cache.k.shape[1])):
        ns = prefill_splits(cached_len.shape[0], ctx.max_q_len, nh, ctx.max_kv_len, window)
        attention_prefill_tc(q, out, cache.k, cache.v, bt, seg_start, cached_len, ctx.max_q_len, cache.num_pages,
                             window, scale, ctx.err, nsplit=ns, first_token=first_seg)
    else:
        attention_prefill_bf16(q, out, cache.k, cache.v, bt, seg_start, cached_len, ctx.max_q_len, cache.num_pages,
                               window, scale, ctx.err)


def _decode_scratch(ctx, cache, nd: int, nh: int, nkv: int, hd: int, window: Optional[int]):
    """``(nsplit, part_o, part_ml, items, starts)`` for the decode kernel.  A step whose descriptor carries work
    items for this cache group (the runner makes them from the requests' real contexts) runs on them; otherwise
    the splits are equal for all requests and chosen from the longest context."""
    work = getattr(ctx, "decode_work", {}).get(getattr(cache, "group", None))
    if work is not None and work[3] == nd:
        items, starts, most = work[0], work[1][:nd], work[2]
        n = items.shape[0]
        return most, ctx.alloc((n, nh, hd), torch.float32), ctx.alloc((n, nh, 2), torch.float32), items, starts
    nsplit = decode_splits(nd, nkv, ctx.max_kv_len, window, balance=ctx.host is not None)
    return nsplit, ctx.alloc((nd, nh, nsplit, hd), torch.float32), ctx.alloc((nd, nh, nsplit, 2), torch.float32), None, None


def attention(ctx, q: torch.Tensor, out: torch.Tensor, cache, window: Optional[int], scale: float):
    """Attention of the step's tokens over one cache plane.  ``cache`` is a
    ``PagedCacheView``; the kernel is chosen by dtype and shape, and the
    shape-generic kernel takes whatever the faster ones refuse.  In a mixed
    step the decoding requests at the head of the batch go to the decode kernel
    (one CTA set per kv head, GQA-packed) and only the prompt portions to the
    prefill kernel, whose query tiles a single token would leave almost empty."""
    T, nh, hd = q.shape
    nkv = cache.k.shape[2]
    if q.dtype == torch.bfloat16 and not FORCE_GENERIC_ATTENTION and attention_bf16_supported(hd, nh, nkv):
        nd = T if ctx.decode_only else _leading_single_token_segments(ctx)
        if not ctx.decode_only:
            longest = max(ctx.host["cached_len"][:nd]) + 1 if nd else 0      # keys of the longest decoding request
            if not decoders_apart(nd, longest, window):
                nd = 0
        if nd > 0:
            nsplit, part_o, part_ml, items, starts = _decode_scratch(ctx, cache, nd, nh, nkv, hd, window)
            attention_decode_bf16(q[:nd], out[:nd], cache.k, cache.v, cache.block_table, ctx.positions[:nd],
                                  ctx.tok_seg[:nd], cache.num_pages, window, scale, nsplit, part_o, part_ml, ctx.err,
                                  items=items, starts=starts)
        if nd < ctx.S:
            _attention_portions(ctx, q, out, cache, window, scale, nd)
        return
    attention_generic(q, out, cache.k, cache.v, cache.block_table, ctx.positions, ctx.tok_seg,
                      cache.num_pages, window, scale, ctx.err)


# PRISM_QKV_IN_ATTENTION=1: in a pure decode step the qkv projection's partial sums go straight to the decode
# attention kernel, which adds, biases, rotates and stores (no kernel between the projection and attention).
# Off by default: one launch fewer, the same step time (3.08 ms both ways at batch 8).  The attention CTAs then
# become resident beside the projection's CTAs, of which only one fits per SM next to them, so half of them start
# after the projection has ended and ask for their keys only then; with the small rotary kernel in between all of
# them are resident and have their first tiles on the way before they are released.
QKV_IN_ATTENTION = os.environ.get("PRISM_QKV_IN_ATTENTION", "0") == "1"


def qkv_attention(ctx, x: torch.Tensor, qkv_w: torch.Tensor, qkv_b: Optional[torch.Tensor], nh: int, nkv: int, hd: int,
                  rot, cache, window: Optional[int], scale: float, out: torch.Tensor):
    """An attention layer between its input and its output projection: qkv projection (+ bias), rotary
    encoding of q and k, store of k and v, attention over the cache plane into ``out [T, nh * hd]``.
    ``qkv_rotate_store`` followed by ``attention``; with ``QKV_IN_ATTENTION`` a pure decode step of a few
    tokens runs as two kernels (K-split projection, attention that finishes the projection)."""
    T = x.shape[0]
    if (QKV_IN_ATTENTION and QKV_PARTIAL and ctx.decode_only and cache.write and rot is not None
            and rot.rotary_dim == hd and x.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
            and not FORCE_GENERIC_ATTENTION and tc_gemm_ok(x, qkv_w)
            and cache.k.is_contiguous() and cache.v.is_contiguous() and attention_bf16_supported(hd, nh, nkv)):
        ks = tc_ksplit(qkv_w.shape[0], qkv_w.shape[1], M=T)
        if ks > 1:
            key = ("rotary_table", rot.inv_freq.data_ptr())          # one table per step for all layers
            table = ctx.scratch.get(key)
            if table is None:
                table = ctx.scratch[key] = ctx.alloc((T, hd // 2, 2), torch.float32)
                rope_table(ctx.positions, rot.inv_freq, table)
            parts = ctx.alloc((ks, T, (nh + 2 * nkv) * hd), torch.float32)
            gemm_tc(x, qkv_w, None, parts, EPI_PARTIAL, ksplit=ks)
            nsplit, part_o, part_ml, items, starts = _decode_scratch(ctx, cache, T, nh, nkv, hd, window)
            attention_decode_qkv_bf16(parts, qkv_b, table, ctx.max_positions, out, cache.k, cache.v, cache.block_table,
                                      ctx.positions, ctx.tok_seg, cache.num_pages, nh, window, scale, nsplit,
                                      part_o, part_ml, ctx.err, items=items, starts=starts)
            return
    q = qkv_rotate_store(ctx, x, qkv_w, qkv_b, nh, nkv, hd, rot, cache)
    attention(ctx, q, out, cache, window, scale)


def feed_forward_swiglu(ctx, x: torch.Tensor, gate_up_w: torch.Tensor, down_w: torch.Tensor):
    """``down(silu(gate(x)) * up(x))`` with the fused gate/up weight."""
    M, I = x.shape[0], gate_up_w.shape[0] // 2
    if tc_gemm_ok(x, gate_up_w, TC_GEMM_MAX_M_SWIGLU):
        act = ctx.alloc((M, I), x.dtype)
        gemm_tc(x, gate_up_w, None, act, EPI_SWIGLU)       # gate/up product with the SwiGLU in its epilogue
        return linear_delta(act, down_w)
    if x.dtype == torch.bfloat16 and gate_up_w.dtype == torch.bfloat16 and M <= GEMV_MAX_M \
            and gemv_supported(M, I, x.shape[1]) and (M == 1 or x.stride(0) % 8 == 0):
        act = ctx.alloc((M, I), x.dtype)
        gemv(x, gate_up_w, None, act, EPI_SWIGLU)        # gate/up product with the SwiGLU in its epilogue
        return linear_delta(act, down_w)
    gu = linear(x, gate_up_w)
    act = ctx.alloc((x.shape[0], gate_up_w.shape[0] // 2), x.dtype)
    swiglu(gu, act)
    return linear_delta(act, down_w)


# --------------------------------------------------------------------------
# attention with a key mask, a softmax sink and keys and values of different sizes
# --------------------------------------------------------------------------

MASK_CAUSAL, MASK_WINDOW, MASK_CHUNK = 0, 1, 2      # csrc/common.cuh: PRISM_MASK_*


class KeyMask:
    """Which keys a position sees; every kind is causal.  ``causal``: all keys
    from 0; ``window(n)``: the last n (itself and the n - 1 before it);
    ``chunk(n)``: those of its own block of n positions, blocks counted from
    position 0 of the sequence.  ``window(n, keep_first=m)``: the last n and,
    however far back, the first m positions of the sequence."""

    __slots__ = ("kind", "size", "keep")

    def __init__(self, kind: int = MASK_CAUSAL, size: int = 0, keep: int = 0):
        if kind not in (MASK_CAUSAL, MASK_WINDOW, MASK_CHUNK):
            raise ValueError(f"unknown mask kind {kind}")
        if kind != MASK_CAUSAL and int(size) < 1:
            raise ValueError(f"a window or chunk needs a size of at least 1, got {size}")
        if int(keep) < 0 or (keep and kind != MASK_WINDOW):
            raise ValueError("only a window keeps first positions visible, and not a negative number of them")
        self.kind, self.size, self.keep = int(kind), int(size) if kind != MASK_CAUSAL else 0, int(keep)

    @classmethod
    def causal(cls):
        return cls()

    @classmethod
    def window(cls, n: Optional[int], keep_first: int = 0):
        return cls() if not n else cls(MASK_WINDOW, n, keep_first)

    @classmethod
    def chunk(cls, n: Optional[int]):
        return cls() if not n else cls(MASK_CHUNK, n)

    def first_key(self, pos: int) -> int:
        """The first key the token at ``pos`` sees (the last is ``pos`` itself)."""
        if self.kind == MASK_WINDOW:
            return max(0, pos - self.size + 1)
        if self.kind == MASK_CHUNK:
            return pos // self.size * self.size
        return 0

    def sees(self, pos: int, key: int) -> bool:
        return key <= pos and (key >= self.first_key(pos) or key < self.keep)

    def most_keys(self, max_kv_len: int) -> int:
        return max_kv_len if self.kind == MASK_CAUSAL else min(max_kv_len, self.size + self.keep)

    def __repr__(self):
        return f"KeyMask({('causal', 'window', 'chunk')[self.kind]}, {self.size}" + (f", keep_first={self.keep})" if self.keep else ")")


def _plane_strides(plane: torch.Tensor):
    """``(elements between consecutive slots, elements between kv heads)`` of a cache plane
    ``[pages, P, nkv, d]`` (or a slice of its last axis); slots of a page and pages follow one another."""
    assert plane.dim() == 4 and plane.stride(3) == 1 and plane.stride(0) == plane.shape[1] * plane.stride(1)
    return plane.stride(1), plane.stride(2)


def _check_dist_bias(dist_bias: Optional[torch.Tensor], nh: int):
    if dist_bias is not None:
        assert dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.dim() == 2
        assert dist_bias.shape[0] == nh and dist_bias.shape[1] >= 1


def attention_masked_generic(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                             block_table: torch.Tensor, positions: torch.Tensor, tok_seg: torch.Tensor,
                             num_pages: int, mask: KeyMask, scale: float, sink: Optional[torch.Tensor],
                             err: torch.Tensor, dist_bias: Optional[torch.Tensor] = None):
    """Shape-generic paged attention: ``q [T, nh, dk]`` (token and head strides free), keys ``[pages, P, nkv,
    dk]``, values ``[pages, P, nkv, dv]`` (may be a slice of the key plane), ``out [T, nh * dv]``; ``sink
    [nh]``: one more term ``exp(sink_h)`` in head h's softmax denominator.  float32 or bf16 storage, all
    arithmetic float32.  ``dist_bias [nh, D + 1]`` float32: the key n positions back has ``dist_bias[h, min(n, D)]``
    added to its scaled score."""
    _cuda(q, out, k_plane, v_plane, block_table, positions, tok_seg, sink, dist_bias)
    _check_dist_bias(dist_bias, q.shape[1])
    T, nh, dk = q.shape
    P, nkv, dv = k_plane.shape[1], k_plane.shape[2], v_plane.shape[3]
    assert k_plane.shape[3] == dk and v_plane.shape[:3] == k_plane.shape[:3]
    assert q.stride(2) == 1 and out.stride(1) == 1 and out.shape == (T, nh * dv)
    assert k_plane.dtype == q.dtype and v_plane.dtype == q.dtype and out.dtype == q.dtype
    assert positions.dtype == torch.int32 and tok_seg.dtype == torch.int32 and block_table.dtype == torch.int32
    krs, khs = _plane_strides(k_plane)
    vrs, vhs = _plane_strides(v_plane)
    if sink is not None:
        assert sink.shape == (nh,) and sink.is_contiguous()
    _check(lib().prism_attention_masked_generic(
        _ptr(q), q.stride(0) if T > 1 else nh * dk, q.stride(1) if nh > 1 else dk, _ptr(out),
        out.stride(0) if T > 1 else nh * dv, _ptr(k_plane), krs, khs, _ptr(v_plane), vrs, vhs, _dt(q),
        _ptr(block_table), block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, nh, nkv, dk, dv, P, num_pages,
        mask.kind, mask.size, mask.keep, float(scale), _ptr(sink), F32 if sink is None else _dt(sink), _ptr(err),
        _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[1] - 1, _stream()), "attention_masked_generic")


def cache_store(src: torch.Tensor, plane: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                tok_seg: torch.Tensor, num_pages: int, max_pos: int, err: torch.Tensor,
                src2: Optional[torch.Tensor] = None, plane2: Optional[torch.Tensor] = None):
    """Rows ``src [T, width]`` (row stride free) into the paged plane ``[pages, P, ...]`` (``width`` entries a
    slot), each at its token's position; ``src2`` into ``plane2`` (a plane of another width with the same pages:
    a layer's values beside its keys) in the same launch."""
    _cuda(src, plane, block_table, positions, tok_seg, src2, plane2)
    T, width = src.shape
    P = plane.shape[1]
    assert plane.is_contiguous() and plane[0, 0].numel() == width and plane.dtype == src.dtype and src.stride(1) == 1
    width2 = 0
    if plane2 is not None:
        width2 = src2.shape[1]
        assert plane2.is_contiguous() and plane2[0, 0].numel() == width2 and plane2.dtype == src.dtype
        assert src2.stride(1) == 1 and src2.shape[0] == T and plane2.shape[:2] == plane.shape[:2]
    _check(lib().prism_cache_store(_ptr(src), src.stride(0) if T > 1 else width, _ptr(plane), _dt(src), width,
                                   _ptr(src2), 0 if src2 is None else (src2.stride(0) if T > 1 else width2), _ptr(plane2),
                                   width2, _ptr(block_table), block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, P,
                                   num_pages, int(max_pos), _ptr(err), _stream()), "cache_store")


def latent_kv_store(x: torch.Tensor, weight: torch.Tensor, eps: float, rank: int, rot_dims: int,
                    inv_freq: Optional[torch.Tensor], plane: torch.Tensor, block_table: torch.Tensor,
                    positions: torch.Tensor, tok_seg: torch.Tensor, num_pages: int, max_pos: int, err: torch.Tensor,
                    xq: Optional[torch.Tensor] = None, q_weight: Optional[torch.Tensor] = None,
                    q_out: Optional[torch.Tensor] = None):
    """The cache row of latent attention from its down projection ``x [T, rank + r]`` (float32): the first
    ``rank`` entries RMS-normed with ``weight``, the last ``r`` with their first ``rot_dims`` entries rotated
    by the token's position; stored at the token's slot of ``plane [pages, P, 1, rank + r]``.  ``xq [T, q_rank]``
    (float32, another column block of the same matrix as ``x``): RMS-normed with ``q_weight`` into ``q_out`` by the
    same launch."""
    _cuda(x, weight, inv_freq, plane, block_table, positions, tok_seg, xq, q_weight, q_out)
    T, width = x.shape
    r = width - rank
    assert x.dtype == torch.float32 and x.stride(1) == 1 and weight.shape == (rank,) and weight.is_contiguous()
    assert plane.is_contiguous() and plane[0, 0].numel() == width
    if rot_dims:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape[0] * 2 == rot_dims
    q_rank = 0
    if q_out is not None:
        q_rank = xq.shape[1]
        assert xq.dtype == torch.float32 and xq.stride(1) == 1 and xq.shape[0] == T and (T == 1 or xq.stride(0) == x.stride(0))
        assert q_weight.shape == (q_rank,) and q_weight.is_contiguous() and q_out.shape == (T, q_rank)
        assert q_out.stride(1) == 1 and q_out.dtype == plane.dtype
    _check(lib().prism_latent_kv_store(_ptr(x), x.stride(0) if T > 1 else width, _ptr(weight), _dt(weight), float(eps),
                                       rank, r, int(rot_dims), _ptr(inv_freq), _ptr(plane), _dt(plane), _ptr(block_table),
                                       block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, plane.shape[1], num_pages,
                                       int(max_pos), _ptr(err), _ptr(xq), q_rank, _ptr(q_weight),
                                       F32 if q_weight is None else _dt(q_weight), _ptr(q_out),
                                       0 if q_out is None else q_out.stride(0), _stream()), "latent_kv_store")


def rotate_slice(src: torch.Tensor, dst: torch.Tensor, rot_dims: int, inv_freq: Optional[torch.Tensor],
                 positions: torch.Tensor):
    """``dst[t, h, :] = src[t, h, :]`` with the first ``rot_dims`` entries rotated by token t's position (entry
    i paired with i + rot_dims / 2).  ``src`` and ``dst`` are ``[T, nh, width]`` views with token and head
    strides of their own."""
    _cuda(src, dst, inv_freq, positions)
    T, nh, width = src.shape
    assert dst.shape == src.shape and dst.dtype == src.dtype and src.stride(2) == 1 and dst.stride(2) == 1
    _check(lib().prism_rotate_slice(_ptr(src), src.stride(0), src.stride(1), _ptr(dst), dst.stride(0), dst.stride(1),
                                    _dt(src), width, int(rot_dims), _ptr(inv_freq), _ptr(positions), T, nh, _stream()),
           "rotate_slice")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "tanh": 4, "sigmoid": 5}      # csrc/activation.cu: PRISM_ACT_*


def activation(x: torch.Tensor, out: torch.Tensor, kind: str):
    """``out = act(x)`` elementwise for ``[rows, cols]`` tensors with row strides of their own."""
    _cuda(x, out)
    rows, cols = x.shape
    assert out.shape == x.shape and out.dtype == x.dtype and x.stride(1) == 1 and out.stride(1) == 1
    _check(lib().prism_activation(_ptr(x), x.stride(0), _ptr(out), out.stride(0), _dt(x), rows, cols,
                                  ACTIVATIONS[kind], _stream()), "activation")


def glu(gu: torch.Tensor, out: torch.Tensor, kind: str):
    """``out[t, i] = act(gu[t, i]) * gu[t, I + i]``: the hidden layer of a gated feed-forward whose gate and up
    projections are one product (gate columns first).  ``kind``: ``silu`` or ``gelu_tanh``."""
    _cuda(gu, out)
    rows, I = out.shape
    assert gu.shape == (rows, 2 * I) and gu.dtype == out.dtype and gu.stride(1) == 1 and out.stride(1) == 1
    _check(lib().prism_glu(_ptr(gu), gu.stride(0), _ptr(out), out.stride(0), _dt(gu), rows, I, ACTIVATIONS[kind], _stream()),
           "glu")


def gather_gate(z: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, offset: int, out: torch.Tensor, kind: str,
                err: torch.Tensor):
    """``out[t, c] = act(z[t, c]) * table[ids[t], offset + c]``: a gate on a slice of a row gathered per token.
    ``z [T, cols]`` float32, ``table [V, *]`` (float32 or bf16), ``out [T, cols]`` in the compute dtype."""
    _cuda(z, ids, table, out)
    T, cols = z.shape
    assert z.dtype == torch.float32 and z.stride(1) == 1 and ids.dtype == torch.int32 and ids.shape[0] == T
    assert table.dim() == 2 and table.stride(1) == 1 and 0 <= offset and offset + cols <= table.shape[1]
    assert out.shape == (T, cols) and out.stride(1) == 1
    _check(lib().prism_gather_gate(_ptr(z), z.stride(0), _ptr(ids), _ptr(table), _dt(table), table.stride(0), int(offset),
                                   table.shape[0], _ptr(out), _dt(out), out.stride(0), T, cols, ACTIVATIONS[kind], _ptr(err),
                                   _stream()), "gather_gate")


def softcap(x: torch.Tensor, cap: float):
    """``x <- cap * tanh(x / cap)`` in place on a contiguous float32 tensor."""
    _cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().prism_softcap(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


def add_rows(residual: torch.Tensor, delta: Optional[torch.Tensor], copy: Optional[torch.Tensor]):
    """``residual += delta`` in place (float32 ``[T, H]``; ``delta`` None, ``[T, H]`` or a stack ``[k, T, H]`` of
    partial sums) and ``copy`` (``[T, H]`` in the compute dtype, or None) receives the new rows: the residual sum
    alone, for a sublayer that reads the stream itself."""
    _cuda(residual, delta, copy)
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    T, H = residual.shape
    nsplit = 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, H)
        nsplit = 1 if delta.dim() == 2 else delta.shape[0]
    if copy is not None:
        assert copy.shape == (T, H) and copy.is_contiguous()
    _check(lib().prism_add_rows(_ptr(residual), _ptr(delta), F32 if delta is None else _dt(delta), nsplit, T * H, _ptr(copy),
                                F32 if copy is None else _dt(copy), T, H, _stream()), "add_rows")


def feed_forward_glu(ctx, x: torch.Tensor, gate_up_w: torch.Tensor, down_w: torch.Tensor, kind: str):
    """``down(act(gate(x)) * up(x))`` with the fused gate/up weight and ``act`` one of ``silu``, ``gelu_tanh``; silu
    takes the path with the activation in the product's epilogue (``feed_forward_swiglu``)."""
    if kind == "silu":
        return feed_forward_swiglu(ctx, x, gate_up_w, down_w)
    if tc_gemm_ok(x, gate_up_w, TC_GEMM_MAX_M_SWIGLU):
        act = ctx.alloc((x.shape[0], gate_up_w.shape[0] // 2), x.dtype)
        gemm_tc(x, gate_up_w, None, act, EPI_GEGLU)        # gate/up product with the gated activation in its epilogue
        return linear_delta(act, down_w)
    gu = linear(x, gate_up_w)
    act = ctx.alloc((x.shape[0], gate_up_w.shape[0] // 2), x.dtype)
    glu(gu, act, kind)
    return linear_delta(act, down_w)


def masked_attention(ctx, q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                     block_table: torch.Tensor, num_pages: int, mask: KeyMask, scale: float,
                     sink: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None):
    """Attention of the step's tokens over one cache plane whose keys and values may differ in size, under a
    ``KeyMask`` and with an optional softmax sink.  The kernel is chosen by dtype and shape; the shape-generic
    one takes what the tensor-core kernel refuses."""
    T, nh, dk = q.shape
    nkv, dv = k_plane.shape[2], v_plane.shape[3]
    if (q.dtype == torch.bfloat16 and MASKED_TC and not FORCE_GENERIC_ATTENTION
            and attention_masked_tc_ok(q, k_plane, v_plane, nh, nkv, dk, dv)):
        few = ctx.decode_only
        ns = masked_decode_splits(ctx.S, nkv * (-(-(nh // nkv) // 16)), mask.most_keys(ctx.max_kv_len)) if few else 1
        attention_masked_bf16(q, out, k_plane, v_plane, block_table, ctx.seg_start, ctx.cached_len, ctx.S,
                              ctx.max_q_len, num_pages, mask, scale, sink, few, ctx.err, nsplit=ns, dist_bias=dist_bias)
        return
    attention_masked_generic(q, out, k_plane, v_plane, block_table, ctx.positions, ctx.tok_seg, num_pages, mask,
                             scale, sink, ctx.err, dist_bias)


MASKED_TC = os.environ.get("PRISM_MASKED_TC", "1") != "0"


MASKED_DECODE_MIN_TILES = 2       # 64-key tiles a CTA keeps at least when a request's keys are shared among CTAs


def masked_decode_splits(S: int, nkv: int, most_keys: int, sms: Optional[int] = None) -> int:
    """CTAs that share one (request, kv head)'s keys (``nkv``: kv heads times the groups of 16 query heads that
    share one) in a decode step of the masked attention kernel: as many as
    fill one wave of two CTAs per SM, none with fewer than ``MASKED_DECODE_MIN_TILES`` tiles.  ``most_keys``:
    the most keys a request of the step can see (its mask's size, or the longest context)."""
    if os.environ.get("PRISM_MASKED_SPLITS"):
        return int(os.environ["PRISM_MASKED_SPLITS"])
    tiles = most_keys // 64 + 1
    fill = (2 * (sms or num_sms())) // max(1, S * nkv)
    return max(1, min(fill, tiles // MASKED_DECODE_MIN_TILES, 64))


def _values_in_keys(k_plane: torch.Tensor, v_plane: torch.Tensor) -> bool:
    """Whether the values are the leading entries of the key rows (one plane, read once)."""
    return v_plane.data_ptr() == k_plane.data_ptr() and v_plane.stride()[:3] == k_plane.stride()[:3]


def attention_masked_tc_ok(q, k_plane, v_plane, nh: int, nkv: int, dk: int, dv: int) -> bool:
    """The rule of ``prism_attention_masked_bf16`` (csrc/attention_masked.cu): whole 16-byte pieces everywhere,
    values of up to 256 entries."""
    if not lib().prism_attention_masked_supported(dk, dv, nh, nkv):
        return False
    krs, khs = _plane_strides(k_plane)
    ok = (q.stride(0) % 8 == 0 or q.shape[0] == 1) and (q.stride(1) % 8 == 0 or nh == 1) and q.data_ptr() % 16 == 0 \
        and krs % 8 == 0 and khs % 8 == 0 and k_plane.data_ptr() % 16 == 0
    if _values_in_keys(k_plane, v_plane):
        return ok and dv <= dk
    vrs, vhs = _plane_strides(v_plane)
    return ok and dv % 8 == 0 and vrs % 8 == 0 and vhs % 8 == 0 and v_plane.data_ptr() % 16 == 0


def attention_masked_bf16(q, out, k_plane, v_plane, block_table, seg_start, cached_len, S: int, max_q_len: int,
                          num_pages: int, mask: KeyMask, scale: float, sink: Optional[torch.Tensor], few_rows: bool,
                          err: torch.Tensor, nsplit: int = 1, dist_bias: Optional[torch.Tensor] = None):
    """Tensor-core attention under a ``KeyMask`` with an optional sink; ``few_rows``: a decode step (one token
    per segment), where a CTA takes up to 16 query heads of a kv head, its four warps share the keys and
    ``nsplit`` CTAs the key tiles of one (segment, kv head), merged by a second kernel."""
    _cuda(q, out, k_plane, v_plane, block_table, seg_start, cached_len, sink, dist_bias)
    T, nh, dk = q.shape
    _check_dist_bias(dist_bias, nh)
    P, nkv, dv = k_plane.shape[1], k_plane.shape[2], v_plane.shape[3]
    assert q.dtype == torch.bfloat16 and k_plane.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(2) == 1 and out.stride(1) == 1 and out.shape == (T, nh * dv) and seg_start.shape[0] == S + 1
    krs, khs = _plane_strides(k_plane)
    vrs, vhs = _plane_strides(v_plane)
    vin = _values_in_keys(k_plane, v_plane)
    po = pml = None
    if few_rows and nsplit > 1:
        po = torch.empty((S, nh, nsplit, dv), dtype=torch.float32, device=q.device)
        pml = torch.empty((S, nh, nsplit, 2), dtype=torch.float32, device=q.device)
    _check(lib().prism_attention_masked_bf16(
        _ptr(q), q.stride(0) if T > 1 else nh * dk, q.stride(1) if nh > 1 else dk, _ptr(out),
        out.stride(0) if T > 1 else nh * dv, _ptr(k_plane), krs, khs, None if vin else _ptr(v_plane), vrs, vhs,
        _ptr(block_table), block_table.shape[1], _ptr(seg_start), _ptr(cached_len), S, int(max_q_len), nh, nkv, dk, dv,
        P, num_pages, mask.kind, mask.size, mask.keep, float(scale), _ptr(sink), F32 if sink is None else _dt(sink),
        1 if few_rows else 0, int(nsplit) if few_rows else 1, _ptr(po), _ptr(pml), _ptr(err), _ptr(dist_bias),
        0 if dist_bias is None else dist_bias.shape[1] - 1, _stream()),
        "attention_masked_bf16")
    if few_rows and nsplit > 1:
        global launch_count
        launch_count += 1          # the merge kernel


def feed_forward_hidden(ctx, x: torch.Tensor, up_w: Optional[torch.Tensor], kind: str, out: torch.Tensor,
                        hidden: Optional[torch.Tensor] = None):
    """``out = act(up(x))``; ``hidden``: the up projection if another product has made it already.  ``out``
    may be a column block of a wider buffer."""
    if hidden is None:
        hidden = linear(x, up_w)
    activation(hidden, out, kind)


def feed_forward_act(ctx, x: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor, kind: str):
    """``down(act(up(x)))``."""
    act = ctx.alloc((x.shape[0], up_w.shape[0]), x.dtype)
    feed_forward_hidden(ctx, x, up_w, kind, act)
    return linear_delta(act, down_w)


def stack_deltas(ctx, deltas):
    """Several results that are to be added to the residual stream together, as one float32 stack ``[k, T,
    H]`` for the fused add + norm kernel.  Each is ``[T, H]`` in any dtype or already a float32 stack of
    partial sums."""
    parts = [d if d.dim() == 3 else d.unsqueeze(0) for d in deltas]
    if all(p.dtype == torch.float32 for p in parts):
        return torch.cat(parts, 0)
    out = ctx.alloc((sum(p.shape[0] for p in parts),) + tuple(parts[0].shape[1:]), torch.float32)
    o = 0
    for p in parts:
        out[o:o + p.shape[0]].copy_(p)
        o += p.shape[0]
    return out


def rms_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor):
    """``out = x / sqrt(mean(x^2) + eps) * weight`` row by row; ``x [rows, width]`` float32 and ``out`` (the
    compute dtype) with row strides of their own."""
    _cuda(x, weight, out)
    rows, width = x.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1 and out.shape == x.shape
    assert weight.shape == (width,) and weight.is_contiguous()
    _check(lib().prism_rms_rows(_ptr(x), x.stride(0), _ptr(weight), _dt(weight), float(eps), _ptr(out), out.stride(0),
                                _dt(out), rows, width, _stream()), "rms_rows")


def matmul_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """Per head h: ``out[:, h, :] = x[:, h, :] @ w[h].T`` for ``x [T, H, K]``, ``w [H, N, K]`` and ``out [T, H,
    N]`` (views with token and head strides of their own, last axis dense).  float32: the true-float32 kernel
    head by head; bf16: the library's batched product with float32 accumulation."""
    _cuda(x, w, out)
    T, H, K = x.shape
    assert w.shape[0] == H and w.shape[2] == K and out.shape == (T, H, w.shape[1])
    if x.dtype == torch.float32:
        for h in range(H):
            sgemm(x[:, h], w[h], None, out[:, h])
        return
    torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))


# --------------------------------------------------------------------------
# norm after the sum, query/key norm with interleaved rotation, gates, recurrent mixers
# --------------------------------------------------------------------------

def scale_add_rmsnorm(x: torch.Tensor, alpha: float, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                      copy: Optional[torch.Tensor] = None):
    """``x <- rmsnorm(alpha * x + delta) * weight`` in place on the float32 rows ``x [T, H]``; ``delta``: None,
    ``[T, H]`` or a stack ``[k, T, H]`` of partial sums (any dtype of the kernels).  ``copy [T, H]``: receives the
    new rows in its own dtype (what a bf16 matrix product reads next)."""
    _cuda(x, delta, weight, copy)
    assert x.dtype == torch.float32 and x.is_contiguous() and weight.shape == (x.shape[1],) and weight.is_contiguous()
    T, H = x.shape
    nsplit = 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, H)
        nsplit = 1 if delta.dim() == 2 else delta.shape[0]
    if copy is not None:
        assert copy.shape == (T, H) and copy.is_contiguous()
    _check(lib().prism_scale_add_rmsnorm(_ptr(x), float(alpha), _ptr(delta), F32 if delta is None else _dt(delta), nsplit,
                                         T * H, _ptr(weight), _dt(weight), float(eps), _ptr(copy),
                                         F32 if copy is None else _dt(copy), T, H, _stream()), "scale_add_rmsnorm")


def gated_product(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, kind: str = "sigmoid", scale: float = 1.0):
    """``out = x * act(gate) * scale``; ``x`` and ``out`` ``[rows, cols]`` in the compute dtype, ``gate`` float32
    ``[rows, cols / group]`` (one gate entry for ``group`` neighbouring columns: a gate per head), each with a row
    stride of its own; ``kind``: ``sigmoid`` or ``silu``."""
    _cuda(x, gate, out)
    rows, cols = x.shape
    assert gate.dtype == torch.float32 and gate.shape[0] == rows and out.shape == x.shape and out.dtype == x.dtype
    assert x.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1
    assert gate.shape[1] > 0 and cols % gate.shape[1] == 0
    _check(lib().prism_gated_product(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _ptr(out), out.stride(0), _dt(x),
                                     rows, cols, ACTIVATIONS[kind], float(scale), cols // gate.shape[1], _stream()),
           "gated_product")


def qk_norm_rope_store(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       freq: Optional[torch.Tensor], rot: int, q_out: torch.Tensor, k_plane: Optional[torch.Tensor],
                       v_plane: Optional[torch.Tensor], block_table: torch.Tensor, positions: torch.Tensor,
                       tok_seg: torch.Tensor, num_pages: int, max_pos: int, err: torch.Tensor, whole: bool = False,
                       halves: bool = False, nkv: Optional[int] = None):
    """From float32 column blocks ``q [T, nh * dk]``, ``k [T, nkv * dk]``, ``v [T, nkv * dv]`` of one product (one
    row stride): RMS norm of every q and k head with ``q_weight`` / ``k_weight`` (``[dk]``, None: no norm) - or,
    with ``whole``, of the whole projection at once (weights ``[nh * dk]`` and ``[nkv * dk]``); rotation of the
    first ``rot`` entries by ``position * freq[i]``, in interleaved pairs or (``halves``) entry i with entry
    ``i + rot / 2``; q into ``q_out [T, nh, dk]``, k and v into their cache planes at the token's slot.  ``k``, ``v``
    and the planes None: the layer has no keys and values of its own, only q is made."""
    _cuda(q, k, v, q_weight, k_weight, freq, q_out, k_plane, v_plane, block_table, positions, tok_seg)
    T, nh, dk = q_out.shape
    assert q.dtype == torch.float32 and q.stride(1) == 1 and q.shape == (T, nh * dk) and q_out.is_contiguous()
    if k_plane is None:
        assert k is None and v is None and v_plane is None
        nkv, dv, P = int(nkv or 1), 1, 1
        k = v = q                       # never read
    else:
        nkv, dv, P = k_plane.shape[2], v_plane.shape[3], k_plane.shape[1]
        assert k.dtype == v.dtype == torch.float32 and k.stride(1) == v.stride(1) == 1
        assert k.shape == (T, nkv * dk) and v.shape == (T, nkv * dv)
        assert T == 1 or q.stride(0) == k.stride(0) == v.stride(0)
        assert k_plane.is_contiguous() and v_plane.is_contiguous()
        assert k_plane.dtype == q_out.dtype == v_plane.dtype and k_plane.shape[3] == dk and k_plane.shape[:3] == v_plane.shape[:3]
    if rot:
        assert freq.dtype == torch.float32 and freq.shape == (rot // 2,) and freq.is_contiguous()
    for w, n in ((q_weight, nh), (k_weight, nkv)):
        assert w is None or (w.shape == ((n * dk,) if whole else (dk,)) and w.is_contiguous())
    _check(lib().prism_qk_norm_rope_store(
        _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(q_weight), F32 if q_weight is None else _dt(q_weight), _ptr(k_weight),
        F32 if k_weight is None else _dt(k_weight), float(eps), _ptr(freq), int(rot), _ptr(q_out), _ptr(k_plane),
        _ptr(v_plane), _dt(q_out), _ptr(block_table), block_table.shape[1], _ptr(positions), _ptr(tok_seg), T, nh, nkv, dk,
        dv, P, num_pages, int(max_pos), _ptr(err), 1 if whole else 0, 1 if halves else 0, _stream()), "qk_norm_rope_store")


def conv_unit_gates(proj: torch.Tensor, b_off: int, a_off: int, taps: torch.Tensor, tail: torch.Tensor,
                    a_log: torch.Tensor, dt_bias: torch.Tensor, ctx, G: int, H: int, dk: int, dv: int, unit_eps: float,
                    qkv: torch.Tensor, bg: torch.Tensor, move_tail: bool = False):
    """The input side of the gated delta rule from the float32 projection rows ``proj`` (columns ``[0, C)``: the q
    | k | v channels, ``C = 2 G dk + H dv``; ``b_off``/``a_off``: first column of the beta / decay projections):
    short causal convolution over time with ``taps [C, K]`` (the ``K - 1`` inputs before the step in ``tail
    [slots, K - 1, C]``) and silu; q and k heads made unit vectors (q also times ``dk^-1/2``) into ``qkv [T, C]``;
    ``bg [T, 2 H]`` = sigmoid(b) | exp(-exp(a_log) softplus(a + dt_bias)).  ``move_tail``: every request of the step
    brings one token, and the kernel moves the tail up by it itself (else ``state_tail`` follows)."""
    _cuda(proj, taps, tail, a_log, dt_bias, qkv, bg)
    T = proj.shape[0]
    C, K = taps.shape
    assert C == 2 * G * dk + H * dv and proj.dtype == torch.float32 and proj.stride(1) == 1 and taps.is_contiguous()
    assert tail.dtype == torch.float32 and tail.is_contiguous() and tuple(tail.shape[1:]) == (max(K - 1, 0), C)
    assert qkv.shape == (T, C) and qkv.is_contiguous() and bg.is_contiguous()
    assert qkv.dtype == torch.float32 and bg.dtype == torch.float32
    if a_log is None:               # the decay is formed elsewhere (one per key channel): bg holds beta alone
        assert bg.shape == (T, H)
    else:
        assert bg.shape == (T, 2 * H) and a_log.shape == (H,) and dt_bias.shape == (H,)
    _check(lib().prism_conv_unit_gates(_ptr(proj), proj.stride(0), int(b_off), int(a_off), _ptr(taps), _dt(taps), K,
                                       _ptr(tail), _ptr(a_log), F32 if a_log is None else _dt(a_log), _ptr(dt_bias),
                                       F32 if dt_bias is None else _dt(dt_bias), _ptr(ctx.tok_seg),
                                       _ptr(ctx.seg_start), _ptr(ctx.state_slots), T, G, H, dk, dv, float(unit_eps),
                                       _ptr(qkv), _ptr(bg), 1 if move_tail else 0, _stream()), "conv_unit_gates")


def state_tail(src: torch.Tensor, tail: torch.Tensor, ctx):
    """Per request of the step: the last ``rows`` rows of its input so far (``src [T, width]`` float32, row stride
    free, holds this step's) into ``tail [slots, rows, width]``; rows the step does not reach back to move up from
    the tail as it was."""
    _cuda(src, tail)
    rows, width = tail.shape[1], tail.shape[2]
    if rows == 0:
        return
    assert src.dtype == torch.float32 and tail.dtype == torch.float32 and tail.is_contiguous() and src.stride(1) == 1
    assert src.shape[1] >= width
    _check(lib().prism_state_tail(_ptr(src), src.stride(0), width, _ptr(tail), rows, _ptr(ctx.seg_start),
                                  _ptr(ctx.state_slots), ctx.S, _stream()), "state_tail")


def shift_mix(x: torch.Tensor, prev: torch.Tensor, mu: torch.Tensor, ctx, out: torch.Tensor, keep_prev: bool = False):
    """``out[s] = x + (x_prev - x) * mu[s]`` for ``mu [n, D]``; ``x [T, D]`` float32, ``x_prev`` the row before in
    the same request (``prev [slots, 1, D]`` for a step's first token); ``out [n, T, D]`` in the compute dtype.
    ``keep_prev``: every request of the step brings one token, and the kernel leaves it in ``prev`` itself (else
    ``state_tail`` follows)."""
    _cuda(x, prev, mu, out)
    T, D = x.shape
    n = mu.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and prev.dtype == torch.float32 and prev.is_contiguous()
    assert prev[0].numel() == D and mu.shape == (n, D) and mu.is_contiguous() and out.shape == (n, T, D) and out.is_contiguous()
    _check(lib().prism_shift_mix(_ptr(x), D, _ptr(prev), _ptr(mu), _dt(mu), n, _ptr(ctx.tok_seg), _ptr(ctx.seg_start),
                                 _ptr(ctx.state_slots), T, _ptr(out), _dt(out), T * D, 1 if keep_prev else 0, _stream()),
           "shift_mix")


def headnorm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, scale: float, out: torch.Tensor,
                  gate_act: str = "silu"):
    """``out[t, h] = o[t, h] / rms(o[t, h]) * weight * act(gate[t, h]) * scale``, ``gate_act``: ``silu``, ``sigmoid`` or
    ``none`` (the gate holds the factor itself); ``o [T, H, dv]`` float32, ``gate
    [T, H * dv]`` float32 and ``out [T, H * dv]`` (compute dtype) with row strides of their own; ``weight [dv]`` (one
    for all heads) or ``[H * dv]``."""
    _cuda(o, gate, weight, out)
    T, H, dv = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1
    assert gate.shape == (T, H * dv) and out.shape == (T, H * dv) and out.stride(1) == 1 and weight.is_contiguous()
    assert weight.shape in ((dv,), (H * dv,))
    per_head = 1 if (weight.shape[0] == H * dv and H > 1) else 0
    _check(lib().prism_headnorm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _dt(weight), per_head, float(eps),
                                     float(scale), T, H, dv, _ptr(out), _dt(out), out.stride(0),
                                     {"silu": 0, "sigmoid": 1, "none": 2}[gate_act], _stream()), "headnorm_gate")


SCAN_DELTA, SCAN_BONUS, SCAN_CHANNEL, SCAN_GENERAL = 0, 1, 2, 3      # csrc/recurrent.cu: PRISM_SCAN_*


def recurrent_scan(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, ctx, H: int,
                   rep: int, dk: int, dv: int, out: torch.Tensor, bg: Optional[torch.Tensor] = None,
                   ww: Optional[torch.Tensor] = None, w0: Optional[torch.Tensor] = None, u: Optional[torch.Tensor] = None,
                   decay_ready: bool = False, ex: Optional[torch.Tensor] = None):
    """The step's tokens through a matrix-state recurrence, request by request, token after token, from and
    into ``state [slots, H, dv, dk]`` (float32).  ``q`` (or r), ``k``, ``v``: float32 rows ``[T, heads * size]`` with
    one row stride - column blocks of one product, or products of their own.  ``SCAN_DELTA``: delta rule with ``bg
    [T, 2 H]`` (beta | scalar decay), ``rep`` heads share a q/k head.  ``SCAN_BONUS``: per-channel decay ``exp(-exp(ww
    + w0))`` (``ww [T, H * dk]``) and bonus ``u [H * dk]`` for the current token; ``decay_ready``: ``ww`` holds the decay
    itself (``lowrank_decay``, ``decay_from_exponent``).  ``SCAN_CHANNEL``: delta rule whose decay is a vector over the
    key channels, ``ww [T, H * dk]`` (the decay itself), with ``bg [T, H]`` (beta).  ``SCAN_GENERAL``: the generalized
    delta rule ``S <- diag(w) S - c (e^T S) + k v^T; o = S^T r`` with the decay ``ww [T, H * dk]`` and ``ex [T, 2 H dk]``
    = unit key e | removal rate times e (``unit_removal``); every head has its own r and k.  ``out [T, H, dv]`` float32."""
    _cuda(q, k, v, state, out, bg, ww, w0, u, ex)
    T = q.shape[0]
    for t in (q, k, v):
        assert t.dtype == torch.float32 and t.dim() == 2 and t.shape[0] == T and t.stride(1) == 1
        assert T == 1 or t.stride(0) == q.stride(0), "q, k and v rows must be equally far apart"
    assert q.shape[1] == k.shape[1] == (H // rep) * dk and v.shape[1] == H * dv
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dv, dk)
    assert out.shape == (T, H, dv) and out.is_contiguous() and out.dtype == torch.float32
    if mode == SCAN_DELTA:
        assert bg is not None and bg.shape == (T, 2 * H) and bg.is_contiguous() and bg.dtype == torch.float32
    elif mode == SCAN_CHANNEL:
        assert bg is not None and bg.shape == (T, H) and bg.is_contiguous() and bg.dtype == torch.float32
        assert ww.dtype == torch.float32 and ww.shape == (T, H * dk) and ww.stride(1) == 1
    elif mode == SCAN_GENERAL:
        assert rep == 1 and ww.dtype == torch.float32 and ww.shape == (T, H * dk) and ww.stride(1) == 1
        assert ex is not None and ex.dtype == torch.float32 and ex.shape == (T, 2 * H * dk) and ex.is_contiguous()
    else:
        assert ww.dtype == torch.float32 and ww.shape == (T, H * dk) and ww.stride(1) == 1
        assert w0.numel() == H * dk and u.numel() == H * dk and w0.is_contiguous() and u.is_contiguous()
    # the kernel addresses k and v from q's first element; the three may be separate allocations
    k_off, v_off = (k.data_ptr() - q.data_ptr()) // 4, (v.data_ptr() - q.data_ptr()) // 4
    stride = q.stride(0) if T > 1 else max(q.shape[1], 4) // 4 * 4
    _check(lib().prism_recurrent_scan(
        int(mode), _ptr(q), stride, 0, k_off, v_off, _ptr(bg), _ptr(ww),
        0 if ww is None else ww.stride(0), _ptr(w0), F32 if w0 is None else _dt(w0), _ptr(u), F32 if u is None else _dt(u),
        _ptr(state), _ptr(ctx.seg_start), _ptr(ctx.state_slots), ctx.S, int(getattr(ctx, "max_q_len", None) or T), H, rep, dk, dv,
        _ptr(out), 1 if decay_ready else 0, _ptr(ex), 0 if ex is None else ex.stride(0), _stream()),
        "recurrent_scan")


def unit_removal(k: torch.Tensor, a: torch.Tensor, a_bias: Optional[torch.Tensor], unit_eps: float, H: int, dk: int,
                 ex: torch.Tensor):
    """What the generalized delta rule takes out of its state, per token and head: ``ex[:, h dk + i] = e_i = k_i /
    sqrt(sum k^2 + unit_eps)`` and ``ex[:, (H + h) dk + i] = sigmoid(a_i + a_bias_i) e_i``.  ``k``, ``a``: float32
    column blocks ``[T, H * dk]`` of one product (one row stride); ``ex [T, 2 H dk]`` float32."""
    _cuda(k, a, a_bias, ex)
    T = k.shape[0]
    assert k.dtype == a.dtype == torch.float32 and k.shape == a.shape == (T, H * dk) and k.stride(1) == a.stride(1) == 1
    assert T == 1 or k.stride(0) == a.stride(0)
    assert ex.dtype == torch.float32 and ex.shape == (T, 2 * H * dk) and ex.is_contiguous()
    assert a_bias is None or (a_bias.numel() == H * dk and a_bias.is_contiguous())
    _check(lib().prism_unit_removal(_ptr(k), _ptr(a), k.stride(0), _ptr(a_bias), F32 if a_bias is None else _dt(a_bias),
                                    float(unit_eps), T, H, dk, _ptr(ex), _stream()), "unit_removal")


LR_EXPEXP, LR_SOFTPLUS, LR_SIGMOID, LR_EXPSIG = 0, 1, 2, 3      # csrc/recurrent.cu: PRISM_LR_*


def lowrank_decay(low: torch.Tensor, w2t: torch.Tensor, w0: Optional[torch.Tensor], out: torch.Tensor, inner_tanh: bool = True,
                  epilogue: int = LR_EXPEXP, rate_log: Optional[torch.Tensor] = None, per: int = 1, rate: float = 1.0):
    """``out = epi(inner(low) @ w2t + w0)``: the second half of a low-rank product with what follows it, in one launch
    and in float32 throughout.  ``inner``: tanh or nothing.  ``epilogue``: ``LR_EXPEXP`` ``exp(-exp(z))`` (a per-channel
    decay from its double exponent), ``LR_SOFTPLUS`` ``exp(-exp(rate_log[n // per]) softplus(z))`` (a per-channel decay
    with one rate per ``per`` channels), ``LR_SIGMOID`` (a gate), ``LR_EXPSIG`` ``exp(-rate sigmoid(z))`` (a per-channel
    decay that stays above ``exp(-rate)``).  ``low [T, R]`` float32 (row stride free), ``w2t [R,
    N]`` float32 (the second matrix, transposed), ``w0 [N]`` or None, ``out [T, N]`` float32."""
    _cuda(low, w2t, w0, out, rate_log)
    T, R = low.shape
    N = w2t.shape[1]
    assert low.dtype == torch.float32 and low.stride(1) == 1 and w2t.dtype == torch.float32 and w2t.is_contiguous()
    assert w2t.shape[0] == R and out.shape == (T, N) and out.dtype == torch.float32 and out.stride(1) == 1
    assert w0 is None or (w0.numel() == N and w0.is_contiguous())
    if epilogue == LR_SOFTPLUS:
        assert rate_log is not None and rate_log.is_contiguous() and rate_log.numel() * per == N
    _check(lib().prism_lowrank_decay(_ptr(low), low.stride(0), R, _ptr(w2t), _ptr(w0), F32 if w0 is None else _dt(w0), N, T,
                                     _ptr(out), out.stride(0), 1 if inner_tanh else 0, int(epilogue), _ptr(rate_log),
                                     F32 if rate_log is None else _dt(rate_log), int(per), float(rate), _stream()), "lowrank_decay")


def decay_from_exponent(ww: torch.Tensor, w0: torch.Tensor):
    """``ww <- exp(-exp(ww + w0))`` in place (``ww [T, A]`` float32, row stride free): the per-channel decay of the
    decayed-sum scan, formed once where a step has many tokens."""
    _cuda(ww, w0)
    T, A = ww.shape
    assert ww.dtype == torch.float32 and ww.stride(1) == 1 and w0.numel() == A and w0.is_contiguous()
    _check(lib().prism_decay_from_exponent(_ptr(ww), ww.stride(0), _ptr(w0), _dt(w0), T, A, _stream()), "decay_from_exponent")


def hyper_norm(x: torch.Tensor, streams: int, x_out: Optional[torch.Tensor], delta: Optional[torch.Tensor],
               mix: Optional[torch.Tensor], out_w: Optional[torch.Tensor], in_w: Optional[torch.Tensor],
               weight: Optional[torch.Tensor], eps: float, h: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
               rms: bool = False):
    """Hyper-connections around a sublayer, in one launch: the update that the previous sublayer left open, ``x_j <-
    sum_i mix[i, j] x_i + out_w[j] delta`` for all ``streams`` copies at once, then the read-in ``u = sum_j in_w[j]
    x_j`` and its norm ``h = norm(u) * weight`` (layer norm without bias, or RMS norm).  ``x``: ``[streams, T, W]``
    float32, or ``[T, W]`` read as ``streams`` equal copies; ``x_out [streams, T, W]`` (may be ``x``; None: not written);
    ``delta [T, W]`` or a stack ``[k, T, W]`` of partial sums, float32 or bf16 (None: nothing left open); ``mix`` None:
    identity, ``out_w`` / ``in_w`` None: ones; ``weight`` None: the update alone.  ``rows``: only these tokens are
    normed into ``h [len(rows), W]``, and the streams are not written."""
    _cuda(x, x_out, delta, mix, out_w, in_w, weight, h, rows)
    s = int(streams)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() in (2, 3)
    T, W = x.shape[-2], x.shape[-1]
    in_ss = T * W if x.dim() == 3 else 0
    assert x.dim() == 2 or x.shape[0] == s
    if x_out is not None:
        assert x_out.dtype == torch.float32 and x_out.shape == (s, T, W) and x_out.is_contiguous()
    nsplit = 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, W)
        nsplit = delta.shape[0] if delta.dim() == 3 else 1
    for t, n in ((mix, s * s), (out_w, s), (in_w, s)):
        assert t is None or (t.numel() == n and t.is_contiguous())
    n = T if rows is None else rows.shape[0]
    if weight is not None:
        assert weight.shape == (W,) and weight.is_contiguous() and h.shape == (n, W) and h.is_contiguous()
    dt = lambda t: F32 if t is None else _dt(t)
    _check(lib().prism_hyper_norm(_ptr(x), in_ss, _ptr(x_out), T * W, _ptr(delta), dt(delta), nsplit, T * W, _ptr(mix), dt(mix),
                                  _ptr(out_w), dt(out_w), _ptr(in_w), dt(in_w), s, _ptr(weight), dt(weight), float(eps),
                                  1 if rms else 0, _ptr(h), dt(h), _ptr(rows), n, W, _stream()), "hyper_norm")


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], tail: torch.Tensor, ctx, out: torch.Tensor,
                move_tail: bool = False, add_input: bool = False, taps_t: Optional[torch.Tensor] = None):
    """``out[t, c] = bias[c] + sum_j taps[c, K-1-j] x[t-j, c]``: a short causal convolution over time per channel,
    float32; ``x [T, C]`` (row stride free), ``taps [C, K]`` (last column: the current token's), ``tail [slots, K - 1,
    C]`` the request's last inputs before this step.  ``move_tail``: every request brings one token, and the kernel
    moves the tail up itself (else ``state_tail`` follows).  ``add_input``: ``out = x + conv(x)``.  ``out``: float32
    or the compute dtype (rounded once).  ``taps_t``: the same taps as float32 ``[K, C]`` (made once by the caller), read
    128 bits at a time where the sizes allow."""
    _cuda(x, taps, bias, tail, out, taps_t)
    assert taps_t is None or (taps_t.dtype == torch.float32 and taps_t.is_contiguous() and taps_t.shape == (taps.shape[1], taps.shape[0]))
    T = x.shape[0]
    C, K = taps.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[1] == C and taps.is_contiguous()
    assert tail.dtype == torch.float32 and tail.is_contiguous() and tuple(tail.shape[1:]) == (max(K - 1, 0), C)
    assert out.shape == (T, C) and out.stride(1) == 1
    assert bias is None or (bias.shape == (C,) and bias.is_contiguous())
    _check(lib().prism_causal_conv(_ptr(x), x.stride(0), _ptr(taps), _dt(taps), _ptr(bias), F32 if bias is None else _dt(bias),
                                   K, C, _ptr(tail), _ptr(ctx.tok_seg), _ptr(ctx.seg_start), _ptr(ctx.state_slots), T, _ptr(out),
                                   _dt(out), out.stride(0), 1 if move_tail else 0, 1 if add_input else 0, _ptr(taps_t), _stream()), "causal_conv")


def block_gates(u: torch.Tensor, wr: torch.Tensor, wi: torch.Tensor, br: torch.Tensor, bi: torch.Tensor, lam: torch.Tensor,
                cdecay: float, a_out: torch.Tensor, g_out: torch.Tensor):
    """The gates of a real-gated linear recurrent unit and the recurrence's coefficients from them: per block b of
    channels ``r = sigmoid(wr[b] u_b + br[b])``, ``i = sigmoid(wi[b] u_b + bi[b])``; ``a = exp(-cdecay r softplus(lam))``
    into ``a_out`` and ``sqrt(1 - a^2) i u`` into ``g_out``.  ``u [T, blocks * bs]`` float32 (row stride free), ``wr``,
    ``wi [blocks, bs, bs]`` ([out, in]); float32 arithmetic throughout."""
    _cuda(u, wr, wi, br, bi, lam, a_out, g_out)
    T, C = u.shape
    blocks, bs = wr.shape[0], wr.shape[1]
    assert u.dtype == torch.float32 and u.stride(1) == 1 and blocks * bs == C and wr.shape == wi.shape == (blocks, bs, bs)
    assert wr.is_contiguous() and wi.is_contiguous() and wr.dtype == wi.dtype and br.dtype == bi.dtype
    assert br.numel() == C and bi.numel() == C and lam.numel() == C and br.is_contiguous() and bi.is_contiguous() and lam.is_contiguous()
    for t in (a_out, g_out):
        assert t.dtype == torch.float32 and t.shape == (T, C) and t.stride(1) == 1 and t.stride(0) == a_out.stride(0)
    _check(lib().prism_block_gates(_ptr(u), u.stride(0), _ptr(wr), _ptr(wi), _dt(wr), _ptr(br), _ptr(bi), _dt(br), _ptr(lam),
                                   _dt(lam), float(cdecay), T, blocks, bs, _ptr(a_out), _ptr(g_out), a_out.stride(0), _stream()),
           "block_gates")


RGLRU_CHUNKED_FROM = 128       # a request's tokens in one step from which the scan runs in chunks (csrc/rglru.cu)


def rglru_scan(a: torch.Tensor, g: torch.Tensor, y: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor,
               gelu: bool = True):
    """``S <- a S + g`` per channel, token after token of each request of the step, from and into ``state [slots, C]``
    (float32); ``out = S * gelu_tanh(y)`` (or ``S * y``) in the compute dtype.  ``a``, ``g [T, C]`` float32 with one
    row stride, ``y [T, C]`` float32 (row stride free)."""
    _cuda(a, g, y, state, out)
    T, C = a.shape
    assert a.dtype == g.dtype == y.dtype == torch.float32 and a.stride(1) == g.stride(1) == y.stride(1) == 1
    assert g.shape == (T, C) and y.shape == (T, C) and a.stride(0) == g.stride(0) and out.shape == (T, C) and out.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state[0].numel() == C
    longest = int(getattr(ctx, "max_q_len", None) or T)
    if longest >= RGLRU_CHUNKED_FROM:
        # long stretches: chunks of 64 tokens side by side, their carries combined afterwards (two launches)
        ws = ctx.alloc((T // 64 + ctx.S + 1, 2, C), torch.float32)
        ws0 = ctx.alloc((ctx.S, C), torch.float32)
        _check(lib().prism_rglru_scan_chunked(_ptr(a), _ptr(g), a.stride(0), _ptr(y), y.stride(0), _ptr(state),
                                              _ptr(ctx.seg_start), _ptr(ctx.state_slots), ctx.S, C, longest, 1 if gelu else 0,
                                              _ptr(ws), _ptr(ws0), _ptr(out), _dt(out), out.stride(0), _stream()),
               "rglru_scan_chunked")
        return
    _check(lib().prism_rglru_scan(_ptr(a), _ptr(g), a.stride(0), _ptr(y), y.stride(0), _ptr(state), _ptr(ctx.seg_start),
                                  _ptr(ctx.state_slots), ctx.S, C, 1 if gelu else 0, _ptr(out), _dt(out), out.stride(0),
                                  _stream()), "rglru_scan")


MOE_ACTS = {"silu": 0, "gelu_tanh": 1, "relu": 2, "relu2": 3}      # csrc/moe.cu: moe_act
moe_tensor_cores = True                                 # bf16 experts on tcgen05 (csrc/moe_tcgen05.cu); False: CUDA cores


MOE_ONE_CTA_TOKENS = 16       # steps of up to this many tokens are routed and placed by one CTA in one launch (a warp a token at a time: 64 tokens take longer than the three launches)


class MoeChoice:
    """How a router's scores become a choice beyond "the largest": ``correction [E]`` is added to every score for
    the choice only (the weights use the scores without it); the experts form ``groups`` equal groups of
    neighbours, a group's score is its largest choice score, and only experts of the best ``keep`` groups can be
    chosen; a choice's weight is divided by the sum of the chosen plus ``sum_eps`` (with renorm) and multiplied by
    ``scale``."""

    __slots__ = ("correction", "groups", "keep", "scale", "sum_eps")

    def __init__(self, correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, scale: float = 1.0,
                 sum_eps: float = 0.0):
        self.correction, self.groups, self.keep = correction, int(groups), int(keep)
        self.scale, self.sum_eps = float(scale), float(sum_eps)


def _moe_route_place(L, logits, T, E, top, softmax, renorm, pad, counts, offs, sel_e, sel_w, sel_rank, row_tok, row_w, row_dst,
                     choice: Optional[MoeChoice] = None):
    sm, rn = 1 if softmax else 0, 1 if renorm else 0
    ch = choice or MoeChoice()
    corr = ch.correction
    if corr is not None:
        _cuda(corr)
        assert corr.shape == (E,) and corr.is_contiguous()
    assert ch.groups >= 1 and E % ch.groups == 0 and 1 <= ch.keep <= ch.groups and ch.keep * (E // ch.groups) >= top
    extra = (_ptr(corr), F32 if corr is None else _dt(corr), ch.groups, ch.keep, ch.scale, ch.sum_eps)
    if T <= MOE_ONE_CTA_TOKENS and 8 * (2 * E + 2 * ch.groups) * 4 + (2 * E + 1) * 4 <= 48 * 1024:
        _check(L.prism_moe_route_place(_ptr(logits), logits.stride(0), T, E, int(top), sm, rn, int(pad), _ptr(counts), _ptr(offs),
                                       _ptr(sel_e), _ptr(sel_w), _ptr(sel_rank), _ptr(row_tok), _ptr(row_w), _ptr(row_dst),
                                       *extra, _stream()), "moe_route_place")
        return
    counts.zero_()
    _check(L.prism_moe_route(_ptr(logits), logits.stride(0), T, E, int(top), sm, rn, _ptr(counts), _ptr(sel_e), _ptr(sel_w),
                             _ptr(sel_rank), *extra, _stream()), "moe_route")
    _check(L.prism_moe_place(_ptr(counts), _ptr(sel_e), _ptr(sel_w), _ptr(sel_rank), T, E, int(top), int(pad), _ptr(offs),
                             _ptr(row_tok), _ptr(row_w), _ptr(row_dst), _stream()), "moe_place")


def moe_feed_forward(ctx, x: torch.Tensor, logits: torch.Tensor, gate_up_w: torch.Tensor, down_w: torch.Tensor, top: int,
                     softmax: bool = False, renorm: bool = False, scale_input: bool = True, act: str = "silu",
                     gated: bool = True, choice: Optional[MoeChoice] = None, extra_planes: int = 0) -> torch.Tensor:
    """Mixture of experts on the step's rows: ``x [T, W]`` (compute dtype), router ``logits [T, E]`` float32,
    ``gate_up_w [E, 2 F, W]`` (an expert's gate rows, then its up rows), ``down_w [E, W, F]``.  Each token takes the
    ``top`` experts with the largest scores (sigmoid of the logits, or their softmax); a choice's weight is its score
    (``renorm``: over the sum of the chosen) and multiplies the expert's input (``scale_input``) or its output.
    ``gated`` False: experts without a gate, ``down(act(up(a)))``, and ``gate_up_w`` is ``[E, F, W]``.  ``choice``: a
    ``MoeChoice`` (correction, groups, weight scale).  ``extra_planes``: the stack gets that many more planes after the
    choices' for the caller to fill (a shared expert's result), so that nothing is copied together afterwards.
    Returns float32 ``[top, T, W]``: one plane per choice, which the next norm adds up.  The rows are sorted by
    expert on the device and run as grouped products; the host never learns the counts.  bf16 with rows of 16-byte
    multiples: tcgen05 tiles of one expert each (``csrc/moe_tcgen05.cu``); otherwise CUDA cores (``csrc/moe.cu``)."""
    _cuda(x, logits, gate_up_w, down_w)
    T, W = x.shape
    E, F2, _ = gate_up_w.shape
    F = F2 // 2 if gated else F2
    gt = 1 if gated else 0
    assert logits.dtype == torch.float32 and logits.shape == (T, E) and logits.stride(1) == 1 and x.stride(1) == 1
    assert gate_up_w.shape == (E, (2 if gated else 1) * F, W) and down_w.shape == (E, W, F) and gate_up_w.is_contiguous() and down_w.is_contiguous()
    assert gate_up_w.dtype == x.dtype and down_w.dtype == x.dtype and 1 <= top <= E
    rows = T * top
    dev = x.device
    L = lib()
    si = 1 if scale_input else 0
    if x.dtype == torch.bfloat16 and moe_tensor_cores and L.prism_moe_tcgen05_supported(W, F) and x.stride(0) % 8 == 0:
        # tensor cores: every expert's rows start at a multiple of the token tile, one tile has one expert
        ntok = 16 if T <= 16 else (32 if T <= 32 else 64)
        tiles = min(rows, (rows + E * (ntok - 1)) // ntok)          # no more tiles than this, whatever the choice
        padded = tiles * ntok
        ints = torch.empty(E + (E + 1) + 2 * rows + padded, dtype=torch.int32, device=dev)
        counts, offs = ints[:E], ints[E:2 * E + 1]
        o = 2 * E + 1
        sel_e, sel_rank, row_dst = ints[o:o + rows], ints[o + rows:o + 2 * rows], ints[o + 2 * rows:]
        flt = torch.empty(rows + padded, dtype=torch.float32, device=dev)
        sel_w, row_w = flt[:rows], flt[rows:]
        err = _tc_err_word(dev)
        _moe_route_place(L, logits, T, E, top, softmax, renorm, ntok, counts, offs, sel_e, sel_w, sel_rank, None, None, None, choice)
        xs = ctx.alloc((padded, W), x.dtype)
        _check(L.prism_moe_gather(_ptr(x), x.stride(0), _ptr(offs), _ptr(sel_e), _ptr(sel_w), _ptr(sel_rank), T, int(top), W, si,
                                  _ptr(xs), _ptr(row_dst), _ptr(row_w), _stream()), "moe_gather")
        hidden = ctx.alloc((padded, F), x.dtype)
        _check(L.prism_moe_gemm_tcgen05(_ptr(xs), W, _ptr(gate_up_w), _ptr(offs), _ptr(counts), None, None, ntok, tiles, E, F, W,
                                        gt, MOE_ACTS[act], _ptr(hidden), F, _ptr(err), _stream()), "moe_gemm_tcgen05")
        y = ctx.alloc((top + extra_planes, T, W), torch.float32)
        _check(L.prism_moe_gemm_tcgen05(_ptr(hidden), F, _ptr(down_w), _ptr(offs), _ptr(counts), _ptr(row_dst),
                                        None if scale_input else _ptr(row_w), ntok, tiles, E, W, F, 0, 0, _ptr(y), W, _ptr(err),
                                        _stream()), "moe_gemm_tcgen05")
        return y
    ints = torch.empty(E + (E + 1) + 4 * rows, dtype=torch.int32, device=dev)
    counts, offs = ints[:E], ints[E:2 * E + 1]
    o = 2 * E + 1
    sel_e, sel_rank, row_tok, row_dst = (ints[o + i * rows:o + (i + 1) * rows] for i in range(4))
    flt = torch.empty(2 * rows, dtype=torch.float32, device=dev)
    sel_w, row_w = flt[:rows], flt[rows:]
    _moe_route_place(L, logits, T, E, top, softmax, renorm, 1, counts, offs, sel_e, sel_w, sel_rank, row_tok, row_w, row_dst, choice)
    hidden = ctx.alloc((rows, F), x.dtype)
    _check(L.prism_moe_gemm(_ptr(x), x.stride(0), _ptr(gate_up_w), _dt(x), _ptr(offs), _ptr(row_tok), _ptr(row_w), _ptr(row_dst),
                            rows, E, F, W, 1, si, MOE_ACTS[act], _ptr(hidden), F, gt, _stream()), "moe_gemm")
    y = ctx.alloc((top + extra_planes, T, W), torch.float32)
    _check(L.prism_moe_gemm(_ptr(hidden), F, _ptr(down_w), _dt(x), _ptr(offs), _ptr(row_tok), _ptr(row_w), _ptr(row_dst),
                            rows, E, W, F, 0, si, 0, _ptr(y), W, 1, _stream()), "moe_gemm")
    return y
