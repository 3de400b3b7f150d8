"""ctypes bindings of the package's CUDA kernels, taking torch tensors.

Every function launches on torch's current stream and raises ``KernelError`` when
the launch fails.  There is no CPU fallback: without a CUDA device or without the
compiled extension these functions raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_libs: Dict[Tuple, ctypes.CDLL] = {}


def _lib(name: str, source: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    key = (name, source, tuple(sorted((defines or {}).items())))
    lib = _libs.get(key)
    if lib is None:
        path = build.compile_module(name, source, defines)
        lib = ctypes.CDLL(path)
        _libs[key] = lib
    return lib


def _fn(lib: ctypes.CDLL, name: str, argtypes):
    f = getattr(lib, name)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = c_int
    return f


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


LAUNCHES = 0   # kernels of this package launched (or captured into a graph) so far


def _check(code: int, what: str, n: int = 1) -> None:
    global LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    LAUNCHES += n


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32, bfloat16)") from None


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("redline_b200 kernels run on CUDA tensors only; there is no CPU fallback")


# ------------------------------------------------------------------ elementwise

def _ew() -> ctypes.CDLL:
    return _lib("elementwise", "elementwise.cu")


def resolve_ids(ids: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> None:
    """ids[i] = sampled[src[i]] where src[i] >= 0."""
    _need_cuda(ids, src, sampled)
    f = _fn(_ew(), "rl_resolve_ids", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(src), _ptr(sampled), n, _stream()), "resolve_ids")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
              scale: float = 1.0) -> None:
    """out[t] = float(table[ids[t]]) * scale; out is the float32 residual stream [T, H]."""
    _need_cuda(ids, table, out)
    f = _fn(_ew(), "rl_embedding", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                                     c_void_p])
    _check(f(_ptr(ids), _ptr(table), _code(table.dtype), _ptr(out), ids.numel(), table.shape[1],
             table.shape[0], float(scale), _ptr(status), _stream()), "embedding")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows_idx: Optional[torch.Tensor] = None,
                rows: Optional[int] = None) -> None:
    """residual += delta (if given); out = rmsnorm(residual) * weight.  With
    ``rows_idx`` only those rows are normalised (out row i <- row rows_idx[i]) and
    residual is left as it is."""
    _need_cuda(residual, weight, out)
    n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else residual.shape[0])
    f = _fn(_ew(), "rl_add_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                       c_int, c_int, c_float, c_void_p])
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_rmsnorm: delta and out must have the same dtype")
    _check(f(_ptr(residual), _ptr(delta), _ptr(weight), _code(weight.dtype), _ptr(out), _code(out.dtype),
             _ptr(rows_idx), n, residual.shape[-1], float(eps), _stream()), "add_rmsnorm")


def add_residual(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    f = _fn(_ew(), "rl_add_residual", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _code(delta.dtype), delta.numel(), _stream()), "add_residual")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(gate_up, out)
    f = _fn(_ew(), "rl_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _code(out.dtype), gate_up.shape[0], out.shape[1], _stream()), "swiglu")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    _need_cuda(x, bias)
    f = _fn(_ew(), "rl_add_bias", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x.dtype), _ptr(bias), _code(bias.dtype), x.shape[0], x.shape[1], _stream()), "add_bias")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor],
                  cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                  vcache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  page_size: int, status: torch.Tensor, tokens: Optional[int] = None) -> None:
    """Rotates q and k heads of qkv [T, (Hq + 2 Hkv) D] in place and writes k, v to
    the cache slot of each token (``slots`` None or negative: no write; a slot beyond the pool is
    not written and sets bit 4 of ``status``)."""
    _need_cuda(qkv, positions)
    f = _fn(_ew(), "rl_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p,
                                         c_void_p])
    max_pos = cos.shape[0] if cos is not None else 2 ** 31 - 1
    num_slots = kcache.shape[0] * page_size if kcache is not None else 0
    _check(f(_ptr(qkv), _code(qkv.dtype), _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(kcache),
             _ptr(vcache), tokens if tokens is not None else qkv.shape[0], num_heads, num_kv_heads, head_dim,
             page_size, max_pos, num_slots, _ptr(status), _stream()), "rope_kv_write")


# ------------------------------------------------------------------------ gemm

def gemm_tn_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T, float accumulation on the CUDA cores."""
    _need_cuda(x, w, out)
    f = _fn(_lib("gemm_simt", "gemm_simt.cu"), "rl_gemm_tn_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    M = rows if rows is not None else x.shape[0]
    N, K = w.shape
    if x.shape[1] != K or out.shape[1] != N or x.stride(1) != 1 or out.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"gemm_tn_simt: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(f(_ptr(x), _code(x.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype), M, N, K,
             x.stride(0), out.stride(0), _stream()), "gemm_tn_simt")



# ---------------------------------------------------------------- skinny gemm

SKINNY_MAX_ROWS = 16
SKINNY_UNSTAGED_ROWS = 8    # up to here bfloat16 activations are read from global memory, not staged
EPI_BF16, EPI_F32, EPI_ADD_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
EPI_GEGLU_TANH = 4     # gemm_tc and gemm_skinny: as EPI_SWIGLU with the tanh form of GELU on the gate
_sm_count: Dict[int, int] = {}


def sm_count(device: torch.device) -> int:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _sm_count:
        _sm_count[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _sm_count[i]


def skinny_ok(rows: int, w: torch.Tensor, x_dtype: torch.dtype) -> bool:
    """Whether gemm_skinny takes this product: few rows, bfloat16 operands, K a multiple of 8."""
    return (rows <= SKINNY_MAX_ROWS and w.dtype == torch.bfloat16 and x_dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.is_contiguous())


def norm_handover_buffers(rows: int, width: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Buffers for a norm handed over between two skinny products: xw [rows, width] bfloat16 and the
    per-tile sums of squares [rows, ceil(width / 16)] float32."""
    return (torch.zeros((rows, width), dtype=torch.bfloat16, device=device),
            torch.zeros((rows, (width + 15) // 16), dtype=torch.float32, device=device))


def gemm_skinny(w: torch.Tensor, y: torch.Tensor, epilogue: int, rows: int, x: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                eps: float = 0.0, rows_idx: Optional[torch.Tensor] = None,
                hand_out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                hand_in: Optional[torch.Tensor] = None) -> None:
    """y = epilogue(x @ w^T) for at most 16 rows on the tensor cores (csrc/gemm_skinny.cu).

    x given: bfloat16 activations [rows, K].  residual + norm_w given instead: x is
    bfloat16(rmsnorm(residual[rows_idx]) * norm_w) formed inside the kernel.
    epilogue EPI_BF16 / EPI_F32: store into y; EPI_ADD_RESIDUAL: y (float32 stream) += product;
    EPI_SWIGLU: w is [2 N, K] (gate rows, then up rows), y = silu(gate) * up, [rows, N]; EPI_GEGLU_TANH: the
    same with the tanh form of GELU on the gate.

    The RMSNorm between a product that ends in ``residual +=`` and the product after it can be handed
    over instead of run as a kernel: with ``hand_out = (next_norm_weight, xw, sums)`` (EPI_ADD_RESIDUAL)
    the product also leaves xw = bfloat16(residual * next_norm_weight) and per-tile sums of residual^2
    (buffers of ``norm_handover_buffers``); the next product is then called with ``x = xw``,
    ``hand_in = sums`` and the norm's ``eps`` (at most 8 rows) and scales its rows by
    rsqrt(sum / K + eps): the same norm, with the rounding to bfloat16 before the scaling."""
    _need_cuda(w, y)
    f = _fn(_lib("gemm_skinny", "gemm_skinny.cu"), "rl_gemm_skinny_handover",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_void_p])
    K = w.shape[1]
    N = w.shape[0] // 2 if epilogue in (EPI_SWIGLU, EPI_GEGLU_TANH) else w.shape[0]
    norm = residual is not None
    if norm:
        if norm_w is None or residual.dtype != torch.float32 or residual.shape[1] != K or residual.stride(0) != K:
            raise KernelError("gemm_skinny: the fused norm needs a contiguous float32 residual [*, K] and a weight")
        ldx = 0
    else:
        if x is None or x.dtype != torch.bfloat16 or x.shape[1] != K or x.stride(1) != 1:
            raise KernelError("gemm_skinny: x must be bfloat16 [rows, K]")
        ldx = x.stride(0)
    want = {EPI_BF16: torch.bfloat16, EPI_F32: torch.float32, EPI_ADD_RESIDUAL: torch.float32,
            EPI_SWIGLU: torch.bfloat16, EPI_GEGLU_TANH: torch.bfloat16}[epilogue]
    if y.dtype != want or y.shape[1] != N or y.stride(1) != 1:
        raise KernelError(f"gemm_skinny: output must be {want} [rows, {N}]")
    next_w = xw = ss_out = None
    ldxw = ss_n = 0
    if hand_out is not None:
        next_w, xw, ss_out = hand_out
        tiles = (N + 15) // 16
        if (epilogue != EPI_ADD_RESIDUAL or xw.dtype != torch.bfloat16 or xw.shape[1] != N or xw.stride(1) != 1
                or xw.shape[0] < rows or ss_out.dtype != torch.float32 or not ss_out.is_contiguous()
                or ss_out.shape[1] != tiles or ss_out.shape[0] < rows or next_w.numel() != N
                or next_w.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("gemm_skinny: hand_out needs EPI_ADD_RESIDUAL, a norm weight [N], xw bfloat16 "
                              "[rows, N] and sums float32 [rows, ceil(N / 16)]")
        ldxw = xw.stride(0)
    if hand_in is not None:
        if (norm or rows > SKINNY_UNSTAGED_ROWS or epilogue == EPI_ADD_RESIDUAL or hand_in.dtype != torch.float32
                or not hand_in.is_contiguous() or hand_in.shape[0] < rows):
            raise KernelError("gemm_skinny: hand_in needs bfloat16 x of at most 8 rows and sums float32 [rows, n]")
        ss_n = hand_in.shape[1]
    _check(f(_ptr(w), _ptr(x), ldx, _ptr(residual), _ptr(norm_w),
             1 if (norm_w is not None and norm_w.dtype == torch.float32) else 0, _ptr(rows_idx), float(eps),
             1 if norm else 0, _ptr(y), y.stride(0), epilogue, rows, N, K, _ptr(next_w),
             1 if (next_w is not None and next_w.dtype == torch.float32) else 0, _ptr(xw), ldxw, _ptr(ss_out),
             _ptr(hand_in), ss_n, sm_count(w.device), _stream()),
           "gemm_skinny")


# ------------------------------------------------------------ tcgen05 gemm

_tc_status: Dict[int, torch.Tensor] = {}


def tc_status(device: torch.device) -> torch.Tensor:
    """The device word in which the tcgen05 kernels report a wait that ran out (bit 0: gemm_tc,
    bit 2: prompt-portion attention, bit 3: gemm_mid)."""
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _tc_status:
        _tc_status[i] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[i]


def gemm_tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_tc takes this product: bfloat16 operands, K a multiple of 8, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.is_contiguous()
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, epilogue: int = EPI_BF16, tile_n: int = 0) -> None:
    """y = epilogue(x @ w^T) with tcgen05 tensor cores, TMEM accumulators and TMA loads
    (csrc/gemm_tc.cu): bfloat16 x [M, K], w [N, K] (EPI_SWIGLU and EPI_GEGLU_TANH: [2 N, K], gate rows then
    up rows).
    Epilogues as gemm_skinny's.  tile_n: 0 lets the kernel choose its tiling; 128 or 256 force one CTA per
    128-row tile of that width, 512 forces CTA pairs (tcgen05.mma.cta_group::2) on 256 x 256 tiles."""
    _need_cuda(x, w, y)
    f = _fn(_lib("gemm_tc", "gemm_tc.cu"), "rl_gemm_tc",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    M, K = x.shape
    N = w.shape[0] // 2 if epilogue in (EPI_SWIGLU, EPI_GEGLU_TANH) else w.shape[0]
    want = {EPI_BF16: torch.bfloat16, EPI_F32: torch.float32, EPI_ADD_RESIDUAL: torch.float32,
            EPI_SWIGLU: torch.bfloat16, EPI_GEGLU_TANH: torch.bfloat16}[epilogue]
    if w.shape[1] != K or y.dtype != want or y.shape[1] != N or y.stride(1) != 1 or not gemm_tc_ok(x, w):
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} y{tuple(y.shape)} {y.dtype}")
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(y), y.stride(0), epilogue, M, N, K, _ptr(tc_status(x.device)),
             sm_count(x.device), tile_n, _stream()), "gemm_tc")


# ------------------------------------------------- tcgen05 gemm for 17 to 128 rows

MID_MAX_ROWS = 128


def gemm_mid_ok(rows: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_mid takes this product: at most 128 rows, bfloat16 operands, K a multiple of 8,
    16-byte aligned rows."""
    return 0 < rows <= MID_MAX_ROWS and gemm_tc_ok(x, w)


MID_ROUTED_ROWS = 64


def mid_rows(rows: int, *weights: torch.Tensor) -> bool:
    """Whether a part should take ``rows`` rows with gemm_mid products over these weights: at most 64 rows
    (measured on a B200 with 1B-model weights, decode steps of 32 / 48 / 64 sequences: 1.21 / 1.33 / 1.253 ms
    against 1.23 / 1.36 / 1.267 with the library's products and separate norm and SwiGLU kernels; at 96 and
    128 rows 1.72 / 1.91 against 1.67 / 1.90, so those stay with the library), bfloat16 weights with 16-byte
    aligned rows.  ``REDLINE_MID_PRODUCTS=0`` says no (for comparisons)."""
    if rows <= 0 or rows > MID_ROUTED_ROWS or os.environ.get("REDLINE_MID_PRODUCTS", "1") == "0":
        return False
    return all(w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0
               for w in weights)


def mid_handover_buffers(width: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Buffers for a norm handed over between two gemm_mid products: xw [128, width] bfloat16 and the
    per-feature-tile sums of squares [128, ceil(width / 128)] float32."""
    return (torch.zeros((MID_MAX_ROWS, width), dtype=torch.bfloat16, device=device),
            torch.zeros((MID_MAX_ROWS, mid_sum_columns(width)), dtype=torch.float32, device=device))


def mid_sum_columns(width: int) -> int:
    return (width + 127) // 128


def gemm_mid(x: torch.Tensor, w: torch.Tensor, y: Optional[torch.Tensor], epilogue: int = EPI_BF16,
             residual: Optional[torch.Tensor] = None,
             hand_out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
             hand_in: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """epilogue(x @ w^T) for up to 128 rows with tcgen05 tensor cores (csrc/gemm_mid.cu): the weight rows
    are the 128-row operand, the tokens the narrow one, K is split over the CTAs of a thread-block cluster
    and the partial tiles are added through distributed shared memory in a fixed order.  bfloat16 x [M, K],
    w [N, K] (EPI_SWIGLU: [2 N, K], gate rows then up rows).

    EPI_BF16 / EPI_SWIGLU: y bfloat16 [M, N].  EPI_ADD_RESIDUAL: ``residual`` float32 [M, N] += the product
    (y is not used); with ``hand_out = (next_norm_weight, xw, sums)`` (buffers of ``mid_handover_buffers``)
    it also leaves xw = bfloat16(residual * weight) and the sums of residual^2 per feature tile.  A product
    called with ``x = xw``, ``hand_in = sums`` and the norm's ``eps`` scales row m of its result by
    rsqrt(sums[m].sum() / K + eps): the product of the normed stream."""
    lib = _lib("gemm_mid", "gemm_mid.cu")
    f = _fn(lib, "rl_gemm_mid",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
             c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p])
    M, K = x.shape
    gated = epilogue == EPI_SWIGLU
    N = w.shape[0] // 2 if gated else w.shape[0]
    if epilogue not in (EPI_BF16, EPI_SWIGLU, EPI_ADD_RESIDUAL) or w.shape[1] != K or not gemm_mid_ok(M, x, w):
        raise KernelError(f"gemm_mid: shapes x{tuple(x.shape)} w{tuple(w.shape)} epilogue {epilogue}")
    if epilogue == EPI_ADD_RESIDUAL:
        _need_cuda(x, w, residual)
        if (residual is None or residual.dtype != torch.float32 or residual.shape[0] < M or residual.shape[1] != N
                or residual.stride(1) != 1 or residual.stride(0) % 4 != 0):
            raise KernelError("gemm_mid: EPI_ADD_RESIDUAL needs residual float32 [M, N] with 16-byte aligned rows")
    else:
        _need_cuda(x, w, y)
        if (y is None or y.dtype != torch.bfloat16 or y.shape[0] < M or y.shape[1] != N or y.stride(1) != 1
                or hand_out is not None):
            raise KernelError(f"gemm_mid: y must be bfloat16 [M, {N}] (and only EPI_ADD_RESIDUAL hands a norm out)")
    norm_w = xw = sums_out = None
    if hand_out is not None:
        norm_w, xw, sums_out = hand_out
        if (norm_w.numel() != N or norm_w.dtype not in (torch.bfloat16, torch.float32) or not norm_w.is_contiguous()
                or xw.dtype != torch.bfloat16 or xw.shape[0] < M or xw.shape[1] != N or xw.stride(1) != 1
                or sums_out.dtype != torch.float32 or sums_out.shape[0] < M or sums_out.stride(1) != 1
                or sums_out.shape[1] < mid_sum_columns(N)):
            raise KernelError("gemm_mid: hand_out needs a norm weight [N], xw bfloat16 [M, N] and sums float32 "
                              "[M, ceil(N / 128)]")
    if hand_in is not None:
        if hand_in.dtype != torch.float32 or hand_in.shape[0] < M or hand_in.stride(1) != 1 or hand_in.shape[1] < 1:
            raise KernelError("gemm_mid: hand_in must be float32 [M, n]")
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(y) if y is not None else None, y.stride(0) if y is not None else 0,
             epilogue, M, N, K, _ptr(residual) if residual is not None else None,
             residual.stride(0) if residual is not None else 0,
             _ptr(norm_w) if norm_w is not None else None,
             1 if (norm_w is not None and norm_w.dtype == torch.float32) else 0,
             _ptr(xw) if xw is not None else None, xw.stride(0) if xw is not None else 0,
             _ptr(sums_out) if sums_out is not None else None, sums_out.stride(0) if sums_out is not None else 0,
             _ptr(hand_in) if hand_in is not None else None, hand_in.stride(0) if hand_in is not None else 0,
             hand_in.shape[1] if hand_in is not None else 0, float(eps), _ptr(tc_status(x.device)), _stream()),
           "gemm_mid")


# ------------------------------------------------------------------- attention

MAX_HEAD_DIM = 256


def _attn(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or head_dim < 16 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to "
                          f"{MAX_HEAD_DIM}; got {head_dim}")
    return _lib(f"attention_d{head_dim}", "attention.cu", {"RL_HEAD_DIM": head_dim})


DECODE_PARTITION = 128
PREFILL_TILE_ROWS = 128


def attn_decode(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                block_table: torch.Tensor, items: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                max_parts: int, counters: Optional[torch.Tensor], out: torch.Tensor, nitems: int,
                num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                impl: int = 0) -> None:
    """One query token per item over the paged cache.

    items     int32 [nitems, 4]: (token index of the query, sequence index, context length, 0)
    counters  int32 [nitems * num_kv_heads], zero (the tensor-core kernel needs and keeps them zero)
    impl      0: the best kernel that applies (streaming tensor-core for launches with many partitions,
              one-partition tensor-core, CUDA-core); 1: CUDA-core; 2: one-partition tensor-core or error;
              3: streaming tensor-core or error; 4: one cluster per (item, kv head), partial results
              merged through distributed shared memory (few rows of similar length) or error
    """
    _need_cuda(q, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_decode",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    need = nitems * num_heads * max_parts
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise KernelError("attn_decode: partition workspace too small")
    if counters is not None and counters.numel() < nitems * num_kv_heads:
        raise KernelError("attn_decode: counter workspace too small")
    if items.data_ptr() % 16 != 0:
        raise KernelError("attn_decode: items must be 16-byte aligned")
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table),
             block_table.shape[1], _ptr(items), _ptr(part_o), _ptr(part_ml), max_parts, _ptr(counters), _ptr(out),
             out.stride(0), nitems, num_heads, num_kv_heads, page_size, window, float(scale), impl, _stream()),
           "attn_decode", 2)


def attn_decode_streams(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                        part_o: torch.Tensor, counters: Optional[torch.Tensor], out: torch.Tensor, max_parts: int,
                        nitems: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                        impl: int = 0) -> bool:
    """Whether ``attn_decode`` with these arguments runs the streaming kernel."""
    if not q.is_cuda or q.dtype != torch.bfloat16 or head_dim not in (64, 128):
        return False
    f = _fn(_attn(head_dim), "rl_attn_decode_streams",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int])
    return bool(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(part_o), _ptr(counters),
                  _ptr(out), out.stride(0), max_parts, nitems, num_heads, num_kv_heads, page_size, impl))


_rows_cluster: Dict[Tuple[int, int, int], Tuple[int, int]] = {}
_rows_warps: Dict[int, int] = {}


def attn_decode_rows_cluster(nitems: int, num_kv_heads: int, head_dim: int, device: torch.device) -> Tuple[int, int]:
    """(CTAs per row, clusters resident at once) that ``attn_decode`` with impl 4 would use for a launch of
    ``nitems`` items; (0, 0) if it does not take such a launch (no tensor-core decode kernel for this head
    size).  With fewer resident clusters than rows a cluster takes several rows, one after another."""
    if device.type != "cuda" or head_dim not in (64, 128) or nitems <= 0:
        return 0, 0
    key = (device.index if device.index is not None else torch.cuda.current_device(), nitems * num_kv_heads, head_dim)
    if key not in _rows_cluster:
        f = _fn(_attn(head_dim), "rl_attn_decode_rows_cluster", [c_int, c_int, c_void_p])
        resident = ctypes.c_int(0)
        with torch.cuda.device(key[0]):
            csize = int(f(nitems, num_kv_heads, ctypes.byref(resident)))
        _rows_cluster[key] = (csize, resident.value)
    return _rows_cluster[key]


def attn_decode_rows_pays(nitems: int, num_kv_heads: int, head_dim: int, max_ctx: int, sum_ctx: int, window: int,
                          device: torch.device) -> bool:
    """Whether the decode kernel of one cluster per (item, kv head) (impl 4) is expected to beat the others for
    a launch of ``nitems`` rows of at most ``max_ctx`` and together ``sum_ctx`` keys.  Its time goes with the
    longest row (a row has its cluster's SMs only) times the rows a cluster takes in turn, the streaming
    kernel's with all keys plus the count and merge of its pieces.  The constants are fitted to times on a
    B200 (head size 64, 8 kv heads, batches 1 to 128 at 512 to 8,192 keys): 4.4 us plus, per row a group of
    warps takes, 1.7 us per 32-key sub-block of a warp's run (and 0.7 + 0.25 x turns when it takes more than
    one), but no less than the keys' bytes at 6.2 TB/s; against 8 us plus the keys' bytes at 5.3 TB/s."""
    csize, resident = attn_decode_rows_cluster(nitems, num_kv_heads, head_dim, device)
    if csize <= 0 or resident <= 0 or max_ctx <= 0:
        return False
    if window > 0:
        max_ctx, sum_ctx = min(max_ctx, window), min(sum_ctx, nitems * window)
    if head_dim not in _rows_warps:
        _rows_warps[head_dim] = int(_fn(_attn(head_dim), "rl_attn_decode_rows_warps", [])())
    warps = _rows_warps[head_dim]
    rows = nitems * num_kv_heads
    groups = 1                      # (as the launcher chooses them)
    if rows > resident:
        groups = next((d for d in range(2, warps) if warps % d == 0 and resident * d >= rows), warps)
    turns = (rows + resident * groups - 1) // (resident * groups)
    sub_blocks = (max_ctx + 31) // 32
    per_row = csize * (warps // groups)
    nbytes = sum_ctx * num_kv_heads * head_dim * 4
    per_turn = 1.7 * (head_dim / 64.0) * ((sub_blocks + per_row - 1) // per_row) + (0.7 + 0.25 * turns if turns > 1 else 0.0)
    t_rows = 4.4 + max(turns * per_turn, nbytes / 6.2e6)
    t_stream = 8.0 + nbytes / 5.3e6
    return t_rows < t_stream


def attn_decode_rope_ok(qkv: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                        part_o: torch.Tensor, counters: Optional[torch.Tensor], out: torch.Tensor, max_parts: int,
                        nitems: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                        k_col: int, v_col: int) -> bool:
    """Whether ``attn_decode_rope`` takes a launch with these arguments: bfloat16, head size 64 or 128,
    and one of the two tensor-core decode kernels applies."""
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or head_dim not in (64, 128):
        return False
    f = _fn(_attn(head_dim), "rl_attn_decode_rope_ok",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int])
    return bool(f(_ptr(qkv), q_stride, _ptr(kcache), _ptr(vcache), _ptr(part_o), _ptr(counters), _ptr(out),
                  out.stride(0), max_parts, nitems, num_heads, num_kv_heads, page_size, k_col, v_col))


def attn_decode_rope(qkv: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_table: torch.Tensor, items: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                     max_parts: int, counters: torch.Tensor, out: torch.Tensor, nitems: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                     cos: torch.Tensor, sin: torch.Tensor, k_col: int, v_col: int, status: torch.Tensor,
                     impl: int = 0) -> None:
    """``attn_decode`` by a tensor-core kernel with the rotary encoding and the cache write done in the
    kernel: ``qkv`` holds the UNROTATED rows [q | k | v] of the query tokens (k at column ``k_col``, v at
    ``v_col``); a token's position is its context length - 1; its rotated k and its v are written into the
    cache there.  Only where ``attn_decode_rope_ok`` says so.  impl 0 or 4 as for ``attn_decode``."""
    _need_cuda(qkv, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_decode_rope",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
             c_void_p, c_int, c_void_p])
    need = nitems * num_heads * max_parts
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise KernelError("attn_decode_rope: partition workspace too small")
    if counters.numel() < nitems * num_kv_heads:
        raise KernelError("attn_decode_rope: counter workspace too small")
    if cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2 or not cos.is_contiguous() or not sin.is_contiguous():
        raise KernelError("attn_decode_rope: cos / sin must be contiguous float32 [positions, head_dim / 2]")
    _check(f(_ptr(qkv), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table), block_table.shape[1], _ptr(items),
             _ptr(part_o), _ptr(part_ml), max_parts, _ptr(counters), _ptr(out), out.stride(0), nitems, num_heads,
             num_kv_heads, page_size, window, float(scale), _ptr(cos), _ptr(sin), cos.shape[0], k_col, v_col,
             _ptr(status), impl, _stream()), "attn_decode_rope")


def attn_prefill(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_table: torch.Tensor, tile_seq: torch.Tensor, tile_tok: torch.Tensor,
                 tile_rows: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, tiles: int,
                 num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                 scale: float, impl: int = 0) -> None:
    """Tiles of up to 128 consecutive query tokens of one sequence (tile_seq, tile_tok, tile_rows) over the
    paged cache.  impl 0: the best kernel that applies (bfloat16: tcgen05 at head size 64, mma.sync at
    head size 128; else CUDA cores); 1: CUDA cores; 2: the mma.sync kernel or an error; 3: the tcgen05
    kernel or an error."""
    _need_cuda(q, kcache, out)
    f = _fn(_attn(head_dim), "rl_attn_prefill",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table),
             block_table.shape[1], _ptr(tile_seq), _ptr(tile_tok), _ptr(tile_rows), _ptr(positions),
             _ptr(out), out.stride(0), tiles, num_heads, num_kv_heads, page_size, window, float(scale), impl,
             _ptr(tc_status(q.device)), _stream()), "attn_prefill")


# ------------------------------------------- row-wise kernels of blocks with norms on both sides

ACT_NONE, ACT_RELU_SQ, ACT_GELU_ERF, ACT_SILU, ACT_GELU_TANH, ACT_SIGMOID = 0, 1, 2, 3, 4, 5
ACT_CLAMPED_SWISH = 6      # gated_act only: min / clamp of gate and up, g * sigmoid(slope * g) * (up + 1)
ACTIVATIONS = {"none": ACT_NONE, "relu_squared": ACT_RELU_SQ, "gelu": ACT_GELU_ERF, "silu": ACT_SILU,
               "gelu_tanh": ACT_GELU_TANH}
NORM_LAYER, NORM_RMS = 0, 1


def _rw() -> ctypes.CDLL:
    return _lib("rowwise", "rowwise.cu")


def sandwich_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                  pre_w: Optional[torch.Tensor], out: Optional[torch.Tensor], eps: float, kind: int = NORM_LAYER,
                  rows_idx: Optional[torch.Tensor] = None, rows: Optional[int] = None) -> None:
    """residual (float32 stream) += norm(delta) * post_w (delta given; without post_w delta is added as it
    is), then out = norm(residual) * pre_w (out given).  ``kind``: layer norm (mean removed, variance as the
    mean of squared deviations) or RMS norm, both with a weight and no bias.  ``out`` without ``pre_w``
    receives the (new) stream rows as they are, in its own type.  With ``rows_idx`` out row i comes from
    stream row rows_idx[i] and nothing is added."""
    _need_cuda(residual, delta, out)
    n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else residual.shape[0])
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("sandwich_norm: the stream must be contiguous float32")
    if rows_idx is not None and delta is not None:
        raise KernelError("sandwich_norm: gathered rows take no addend")
    act = out if out is not None else delta
    if act is None:
        return
    ws = [w for w in (post_w, pre_w) if w is not None]
    if any(w.dtype != ws[0].dtype for w in ws):
        raise KernelError("sandwich_norm: the weights must have one type")
    if delta is not None and out is not None and delta.dtype != out.dtype:
        raise KernelError("sandwich_norm: delta and out must have the same dtype")
    f = _fn(_rw(), "rl_sandwich_norm", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                         c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), delta.stride(0) if delta is not None else 0, _ptr(post_w), _ptr(pre_w),
             _code(ws[0].dtype) if ws else 0, _ptr(out), out.stride(0) if out is not None else 0, _code(act.dtype),
             _ptr(rows_idx), n, residual.shape[-1], float(eps), kind, _stream()), "sandwich_norm")


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], act: int, cols: Optional[int] = None,
             rows: Optional[int] = None) -> None:
    """In place: x[r, c] = act(x[r, c] + bias[c]) for c < cols (x may be a row-strided view; bias float32)."""
    _need_cuda(x, bias)
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous()):
        raise KernelError("bias_act: the bias must be contiguous float32")
    if x.stride(1) != 1:
        raise KernelError("bias_act: rows must be contiguous")
    f = _fn(_rw(), "rl_bias_act", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x.dtype), x.stride(0), _ptr(bias), rows if rows is not None else x.shape[0],
             cols if cols is not None else x.shape[1], act, _stream()), "bias_act")


def cache_store(src: torch.Tensor, col: int, heads: int, dim: int, slots: torch.Tensor, cache: torch.Tensor,
                page_size: int, status: torch.Tensor, tokens: Optional[int] = None) -> None:
    """cache [pages, heads, page_size, dim] <- columns [col, col + heads * dim) of src's rows, each token at
    its slot (page * page_size + offset; negative: not written; beyond the pool: bit 2 of ``status``)."""
    _need_cuda(src, slots, cache)
    if src.dtype != cache.dtype or src.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("cache_store: source and cache must have one type, contiguous rows")
    f = _fn(_rw(), "rl_cache_store", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                       c_longlong, c_int, c_void_p, c_void_p])
    _check(f(_ptr(src), _code(src.dtype), src.stride(0), col, heads, dim, _ptr(slots), _ptr(cache), page_size,
             cache.shape[0] * page_size, tokens if tokens is not None else src.shape[0], _ptr(status), _stream()),
           "cache_store")


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                  rows: Optional[int] = None) -> None:
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate): o float32 [T, n] contiguous, gate a
    (row-strided) view [T, n] of the activation type."""
    _need_cuda(o, gate, weight, out)
    if o.dtype != torch.float32 or not o.is_contiguous() or gate.stride(1) != 1 or not out.is_contiguous() \
            or gate.dtype != out.dtype:
        raise KernelError("gated_rmsnorm: o float32 contiguous, gate and out of the activation type")
    f = _fn(_rw(), "rl_gated_rmsnorm", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                         c_float, c_void_p])
    _check(f(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _code(weight.dtype), _ptr(out), _code(out.dtype),
             rows if rows is not None else o.shape[0], o.shape[1], float(eps), _stream()), "gated_rmsnorm")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: int, limit: float = 0.0, slope: float = 1.0,
              bias: Optional[torch.Tensor] = None) -> None:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i], I = out.shape[1].  ``ACT_CLAMPED_SWISH``: with
    g = min(gate, limit) and u = clamp(up, -limit, limit), out = g * sigmoid(slope * g) * (u + 1).  ``bias``
    (float32 [2 I], gate's then up's) is added to gate and up on the way in."""
    _need_cuda(gate_up, out, bias)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != gate_up.shape[1] or not bias.is_contiguous()):
        raise KernelError("gated_act: the bias is contiguous float32 [gate | up]")
    if gate_up.stride(1) != 1 or not out.is_contiguous() or gate_up.dtype != out.dtype \
            or gate_up.shape[1] != 2 * out.shape[1]:
        raise KernelError("gated_act: [gate | up] rows of the output's type and twice its width")
    f = _fn(_rw(), "rl_gated_act", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p,
                                     c_void_p])
    _check(f(_ptr(gate_up), gate_up.stride(0), _ptr(out), _code(out.dtype), out.shape[0], out.shape[1], act,
             float(limit), float(slope), _ptr(bias), _stream()), "gated_act")


HEAD_NORM_NONE, HEAD_NORM_EACH, HEAD_NORM_WHOLE = 0, 1, 2
VALUE_MIX_NONE, VALUE_MIX_KEEP, VALUE_MIX_BLEND = 0, 1, 2


def head_prep(x: torch.Tensor, positions: torch.Tensor, tokens: int, q_col: int, q_heads: int, k_col: int,
              k_heads: int, dim: int, status: torch.Tensor, q_weight: Optional[torch.Tensor] = None,
              k_weight: Optional[torch.Tensor] = None, norm_mode: int = HEAD_NORM_NONE, eps: float = 0.0,
              cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, v_col: int = 0, v_size: int = 0,
              v_first: Optional[torch.Tensor] = None, mix_mode: int = VALUE_MIX_NONE, lam: float = 0.0,
              slots: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
              v_cache: Optional[torch.Tensor] = None, page_size: int = 0, halves: bool = False) -> None:
    """In place on the rows of a projection buffer (csrc/rowwise.cu: head_prep_kernel): the query heads at
    ``q_col`` and the key heads at ``k_col`` are RMS-normed (per head with weights [dim], or over the whole
    section with weights [heads * dim]) and their first 2 * cos.shape[1] entries rotated in neighbouring
    pairs (``halves``: entry i paired with entry i + cos.shape[1]) by the tables' angles at each token's position; the values at ``v_col`` are kept in ``v_first``
    [tokens, v_size] or blended with it, v <- (1 - lam) v + lam v_first.  All in float32.  With ``slots`` the
    finished keys and values are also written to their paged caches ([pages, k_heads, page_size, dim] and
    [pages, v_heads, page_size, vdim]; a slot beyond the pool is not written and sets bit 2 of ``status``)."""
    _need_cuda(x, positions, q_weight, k_weight, cos, sin, v_first)
    if x.stride(1) != 1:
        raise KernelError("head_prep: rows must be contiguous")
    if norm_mode != HEAD_NORM_NONE:
        want = (dim, dim) if norm_mode == HEAD_NORM_EACH else (q_heads * dim, k_heads * dim)
        if q_weight is None or k_weight is None or (q_weight.numel(), k_weight.numel()) != want \
                or q_weight.dtype != k_weight.dtype:
            raise KernelError(f"head_prep: norm weights of {want} entries and one type")
    pairs = 0
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
                or not cos.is_contiguous() or not sin.is_contiguous() or 2 * cos.shape[1] > dim:
            raise KernelError("head_prep: cos and sin are contiguous float32 [positions, pairs], 2 * pairs <= dim")
        pairs = cos.shape[1]
    if mix_mode != VALUE_MIX_NONE and (v_first is None or v_first.dtype != x.dtype or not v_first.is_contiguous()
                                       or v_first.shape[0] < tokens or v_first.shape[1] != v_size):
        raise KernelError("head_prep: v_first must be [tokens, v_size] of the buffer's type")
    v_heads, num_slots = 1, 0
    if slots is not None:
        if (k_cache is None or v_cache is None or k_cache.dtype != x.dtype or v_cache.dtype != x.dtype
                or not k_cache.is_contiguous() or not v_cache.is_contiguous() or page_size <= 0
                or tuple(k_cache.shape[1:]) != (k_heads, page_size, dim) or v_cache.shape[2] != page_size
                or v_cache.shape[1] * v_cache.shape[3] != v_size or v_cache.shape[0] != k_cache.shape[0]):
            raise KernelError("head_prep: caches [pages, heads, page_size, size] of the buffer's type")
        v_heads, num_slots = v_cache.shape[1], k_cache.shape[0] * page_size
    f = _fn(_rw(), "rl_head_prep", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int,
                                     c_int, c_longlong, c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), _code(x.dtype), x.stride(0), _ptr(positions), tokens, q_col, q_heads, k_col, k_heads, dim,
             _ptr(q_weight), _ptr(k_weight), _code(q_weight.dtype) if q_weight is not None else 0, norm_mode,
             float(eps), _ptr(cos), _ptr(sin), pairs, cos.shape[0] if cos is not None else 0, v_col, v_size,
             _ptr(v_first), mix_mode, float(lam), _ptr(slots), _ptr(k_cache), _ptr(v_cache), v_heads, page_size,
             num_slots, _ptr(status), 1 if halves else 0, _stream()), "head_prep")


# ------------------------------------ attention with score maps, a capped score and kept first tokens

MAPS_MAX_DIM, MAPS_MAX_VDIM = 576, 512      # (the tensor-core kernel takes sizes up to 256; longer rows run on CUDA cores)


def _maps(dim: int, vdim: int, maps: int, v_stride: int = 0) -> ctypes.CDLL:
    """``v_stride``: the length of a row of the value cache when it is longer than a value (a mixer whose
    values are the leading entries of its keys hands the key cache in as the value cache); 0: ``vdim``."""
    if not (1 <= dim <= MAPS_MAX_DIM and 1 <= vdim <= MAPS_MAX_VDIM and maps in (1, 2)):
        raise KernelError(f"attention_maps takes key sizes up to {MAPS_MAX_DIM}, value sizes up to {MAPS_MAX_VDIM} and one "
                          f"or two maps; got {dim}, {vdim}, {maps}")
    if v_stride in (0, vdim):
        return _lib(f"attention_maps_d{dim}_v{vdim}_m{maps}", "attention_maps.cu",
                    {"RL_QK_DIM": dim, "RL_V_DIM": vdim, "RL_MAPS": maps})
    if v_stride < vdim:
        raise KernelError(f"attention_maps: a value row of {v_stride} entries cannot hold a value of {vdim}")
    return _lib(f"attention_maps_d{dim}_v{vdim}_m{maps}_s{v_stride}", "attention_maps.cu",
                {"RL_QK_DIM": dim, "RL_V_DIM": vdim, "RL_MAPS": maps, "RL_V_STRIDE": v_stride})


def maps_attn_decode(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_table: torch.Tensor, items: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                     max_parts: int, out: torch.Tensor, nitems: int, heads: int, kv_heads: int, dim: int, vdim: int,
                     maps: int, page_size: int, window: int, keep_first: int, scale: float, softcap: float,
                     lam: float, post_scale: float, eps: float, unit_norm: bool,
                     sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                     gate_mode: int = 0, slopes: Optional[torch.Tensor] = None, v_stride: int = 0) -> None:
    """One query token per item (``items`` as for ``attn_decode``) over the paged cache, ``maps`` score maps
    per head over shared values (csrc/attention_maps.cu): q rows (head, map) of ``dim``, key cache
    [pages, kv_heads * maps, page, dim], value cache [pages, kv_heads, page, vdim], out heads of ``vdim``.
    ``sink`` (float32 [heads], one map only) joins every head's softmax denominator; ``gate`` (a row-strided
    view of q's type) multiplies the output by its sigmoid, per head (``gate_mode`` 1, [tokens, heads]) or
    per entry (2, [tokens, heads * vdim]); ``post_scale`` multiplies the output too.  ``slopes`` (float32
    [heads]): slope_h times the distance between query and key is taken off every score of head h.
    ``v_stride``: see ``_maps``."""
    _need_cuda(q, kcache, vcache, out, sink, gate, slopes)
    _check_tail(maps, heads, vdim, q, sink, gate, gate_mode, slopes)
    f = _fn(_maps(dim, vdim, maps, v_stride), "rl_maps_decode",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_float, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    need = nitems * heads * maps * max_parts
    if part_o.numel() < need * vdim or part_ml.numel() < need * 2:
        raise KernelError("maps_attn_decode: partition workspace too small")
    if items.data_ptr() % 16 != 0:
        raise KernelError("maps_attn_decode: items must be 16-byte aligned")
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table), block_table.shape[1],
             _ptr(items), _ptr(part_o), _ptr(part_ml), max_parts, _ptr(out), out.stride(0), nitems, heads, kv_heads,
             page_size, window, keep_first, float(scale), float(softcap), float(lam), float(post_scale), float(eps),
             1 if unit_norm else 0, _ptr(sink), _ptr(slopes), _ptr(gate), gate.stride(0) if gate is not None else 0,
             gate_mode if gate is not None else 0, _stream()), "maps_attn_decode", 2)


def _check_tail(maps: int, heads: int, vdim: int, q: torch.Tensor, sink: Optional[torch.Tensor],
                gate: Optional[torch.Tensor], gate_mode: int, slopes: Optional[torch.Tensor] = None) -> None:
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != heads or not slopes.is_contiguous()):
        raise KernelError("attention_maps: the distance slopes are float32 [heads]")
    if sink is not None and (maps != 1 or sink.dtype != torch.float32 or sink.numel() != heads
                             or not sink.is_contiguous()):
        raise KernelError("attention_maps: a sink is float32 [heads] and goes with one score map")
    if gate is not None and (gate_mode not in (1, 2) or gate.dtype != q.dtype or gate.stride(1) != 1
                             or gate.shape[1] != (heads if gate_mode == 1 else heads * vdim)):
        raise KernelError("attention_maps: a gate has the queries' type and one entry per head or per output entry")


def maps_attn_prefill(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                      block_table: torch.Tensor, tile_seq: torch.Tensor, tile_tok: torch.Tensor,
                      tile_rows: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, tiles: int,
                      tile_rows_max: int, heads: int, kv_heads: int, dim: int, vdim: int, maps: int, page_size: int,
                      window: int, keep_first: int, scale: float, softcap: float, lam: float, post_scale: float,
                      eps: float, unit_norm: bool, sink: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, gate_mode: int = 0, impl: int = 0,
                      slopes: Optional[torch.Tensor] = None, v_stride: int = 0) -> None:
    """Tiles of up to ``tile_rows_max`` consecutive query tokens of one sequence; otherwise as
    ``maps_attn_decode``.  impl 0: the best kernel that applies (bfloat16 with sizes that are multiples of
    16: mma.sync tensor cores; else CUDA cores); 1: CUDA cores; 2: the tensor-core kernel or an error."""
    _need_cuda(q, kcache, vcache, out, sink, gate, slopes)
    _check_tail(maps, heads, vdim, q, sink, gate, gate_mode, slopes)
    f = _fn(_maps(dim, vdim, maps, v_stride), "rl_maps_prefill",
            [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
             c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_code(q.dtype), _ptr(q), q_stride, _ptr(kcache), _ptr(vcache), _ptr(block_table), block_table.shape[1],
             _ptr(tile_seq), _ptr(tile_tok), _ptr(tile_rows), _ptr(positions), _ptr(out), out.stride(0), tiles,
             tile_rows_max, heads, kv_heads, page_size, window, keep_first, float(scale), float(softcap), float(lam),
             float(post_scale), float(eps), 1 if unit_norm else 0, _ptr(sink), _ptr(slopes), _ptr(gate),
             gate.stride(0) if gate is not None else 0, gate_mode if gate is not None else 0, impl, _stream()),
           "maps_attn_prefill")


# ------------------------------------------------------- attention over a cached latent

def _latent() -> ctypes.CDLL:
    return _lib("latent", "latent.cu")


def latent_prep(proj: torch.Tensor, positions: torch.Tensor, tokens: int, heads: int, dn: int, dr: int, rank: int,
                rot_dims: int, norm_w: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                qa: torch.Tensor, slots: Optional[torch.Tensor], cache: torch.Tensor, page_size: int,
                status: torch.Tensor) -> None:
    """Rows of ``proj``: per head a query [dn unrotated | dr rotated], then [latent of ``rank`` | key part of dr].
    The latent is RMS-normed (float32, weight ``norm_w``); the key part and every head's rotated query part turn
    by the token's position (the first ``rot_dims`` rotated entries, entry i with i + rot_dims/2; cos / sin
    float32 [positions, rot_dims/2]); [latent | key part] goes into ``cache`` [pages, 1, page, rank + dr] at the
    token's slot (negative: not written), the rotated query parts into columns [rank, rank + dr) of every
    head of ``qa`` [tokens, heads * (rank + dr)] (csrc/latent.cu)."""
    _need_cuda(proj, positions, norm_w, cos, sin, qa, slots, cache)
    if proj.dtype != qa.dtype or proj.dtype != cache.dtype or proj.stride(1) != 1 or qa.stride(1) != 1 \
            or not cache.is_contiguous() or norm_w.numel() != rank:
        raise KernelError("latent_prep: projection, query rows and cache have one type and contiguous rows")
    if dr > 0 and (cos is None or sin is None or cos.dtype != torch.float32 or cos.shape[1] * 2 != rot_dims
                   or rot_dims > dr or not cos.is_contiguous() or not sin.is_contiguous()):
        raise KernelError("latent_prep: cos / sin are float32 [positions, rot_dims / 2], rot_dims at most dr")
    if proj.shape[1] < heads * (dn + dr) + rank + dr or qa.shape[1] < heads * (rank + dr):
        raise KernelError("latent_prep: rows too short for the heads and the latent")
    f = _fn(_latent(), "rl_latent_prep",
            [c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
             c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(_code(proj.dtype), _code(norm_w.dtype), _ptr(proj), proj.stride(0), _ptr(positions), tokens, heads, dn, dr,
             rank, rot_dims if dr > 0 else 0, _ptr(norm_w), float(eps), _ptr(cos), _ptr(sin),
             cos.shape[0] if cos is not None else 0, _ptr(qa), qa.stride(0), _ptr(slots), _ptr(cache), page_size,
             cache.shape[0] * page_size, _ptr(status), _stream()), "latent_prep")


def head_linear(x: torch.Tensor, x_col: int, x_head: int, w: torch.Tensor, y: torch.Tensor, y_col: int, y_head: int,
                tokens: Optional[int] = None, impl: int = 0) -> None:
    """y[t, y_col + h * y_head + j] = sum_k w[h, j, k] * x[t, x_col + h * x_head + k] for every head h:
    w [heads, n, k]; float32 sums in ascending k.  impl 1: CUDA cores also where the tensor cores apply."""
    _need_cuda(x, w, y)
    heads, n, k = w.shape
    if x.dtype != y.dtype or x.stride(1) != 1 or y.stride(1) != 1 or not w.is_contiguous() \
            or (x.dtype == torch.float32 and w.dtype != torch.float32):
        raise KernelError("head_linear: x and y have one type and contiguous rows; w contiguous [heads, n, k]")
    if x_col + (heads - 1) * x_head + k > x.shape[1] or y_col + (heads - 1) * y_head + n > y.shape[1]:
        raise KernelError("head_linear: the heads do not fit the rows")
    f = _fn(_latent(), "rl_head_linear", [c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int,
                                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_code(x.dtype), _code(w.dtype), _ptr(x), x.stride(0), x_col, x_head, _ptr(w), heads, n, k, _ptr(y),
             y.stride(0), y_col, y_head, tokens if tokens is not None else x.shape[0], impl, _stream()), "head_linear")


# ------------------------------------------------------- linear attention with a decaying state

LINEAR_ATTN_CHUNK_FROM = 256       # sequences that bring at least so many tokens are cut into chunks
LINEAR_ATTN_MAX_CHUNKS = 64


def linear_attention_chunks(longest: int) -> Tuple[int, int]:
    """(chunk length, most chunks) for a step whose longest sequence brings ``longest`` tokens; (0, 1) when
    every sequence is run as one chain."""
    if longest < LINEAR_ATTN_CHUNK_FROM:
        return 0, 1
    chunk = max(64, (longest + LINEAR_ATTN_MAX_CHUNKS - 1) // LINEAR_ATTN_MAX_CHUNKS)
    return chunk, (longest + chunk - 1) // chunk


def linear_attention(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, seq_of_token: torch.Tensor,
                     state_slot: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                     tokens: int, sequences: int, heads: int, dim: int, vdim: int,
                     chunk_state: Optional[torch.Tensor] = None, chunk: int = 0, max_chunks: int = 1) -> None:
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head over every sequence of the step, from and
    into the sequences' state slots (csrc/linear_attention.cu).  qkv [tokens, *] holds q, k (heads x dim)
    and v (heads x vdim) at the given columns; state float32 [slots, heads, dim, vdim]; out float32
    [tokens, heads * vdim].  With ``chunk_state`` (float32, sequences * max_chunks * heads * dim * vdim)
    sequences are cut into chunks of ``chunk`` tokens that run side by side."""
    _need_cuda(qkv, state, out)
    if state.dtype != torch.float32 or out.dtype != torch.float32 or decay.dtype != torch.float32 \
            or not state.is_contiguous() or not out.is_contiguous() or qkv.stride(1) != 1:
        raise KernelError("linear_attention: state, decay and out are contiguous float32")
    if not 1 <= dim <= 256:
        raise KernelError(f"linear_attention takes key sizes up to 256; got {dim}")
    if chunk_state is not None and max_chunks > 1 and \
            chunk_state.numel() < sequences * max_chunks * heads * dim * vdim:
        raise KernelError("linear_attention: chunk workspace too small")
    f = _fn(_lib(f"linear_attention_d{dim}", "linear_attention.cu", {"RL_LIN_DIM": dim}), "rl_linear_attention",
            [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    chunked = chunk_state is not None and max_chunks > 1
    _check(f(_code(qkv.dtype), _ptr(qkv), qkv.stride(0), q_col, k_col, v_col, _ptr(seq_of_token), _ptr(state_slot),
             _ptr(decay), _ptr(state), _ptr(out), _ptr(chunk_state) if chunked else None, tokens, sequences, heads,
             vdim, chunk, max_chunks if chunked else 1, _stream()), "linear_attention", 3 if chunked else 1)


# ------------------------------------------------------- matrix memory with exponential gates

def _mm(dim: int) -> ctypes.CDLL:
    if not 1 <= dim <= 256:
        raise KernelError(f"matrix_memory takes key sizes up to 256; got {dim}")
    return _lib(f"matrix_memory_d{dim}", "matrix_memory.cu", {"RL_MM_DIM": dim})


def matrix_memory_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of one request's state: [heads, dim, vdim + 1] (the matrix and, as one more column, the
    normaliser) followed by [heads] stabilisers."""
    return heads * dim * (vdim + 1) + heads


def matrix_memory(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, q_scale: float, gates: torch.Tensor,
                  bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor], cap: float,
                  seq_of_token: torch.Tensor, state_slot: torch.Tensor, state: torch.Tensor, stab: torch.Tensor,
                  num: torch.Tensor, qn: torch.Tensor, tokens: int, sequences: int, heads: int, dim: int,
                  vdim: int, chunk_state: Optional[torch.Tensor] = None, chunk: int = 0, max_chunks: int = 1) -> None:
    """The recurrence of csrc/matrix_memory.cu over every sequence of the step, from and into the sequences'
    state slots.  qkv [tokens, *] holds q, k (heads x dim) and v (heads x vdim) at the given columns;
    ``gates`` float32 [tokens, 2 heads] holds the input-gate and forget-gate projections and is overwritten;
    ``stab`` [tokens, heads], ``num`` [tokens, heads * vdim] and ``qn`` [tokens, heads] (float32) receive the
    stabiliser, S^T q and n . q of every token.  With ``chunk_state`` (float32, sequences * max_chunks * heads *
    dim * (vdim + 1)) sequences are cut into chunks of ``chunk`` tokens that run side by side
    (``linear_attention_chunks`` says how a step is cut)."""
    _need_cuda(qkv, gates, state, stab, num, qn)
    for t in (gates, state, stab, num, qn, bias_i, bias_f):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError("matrix_memory: gates, biases, state and outputs are contiguous float32")
    if qkv.stride(1) != 1 or gates.shape[1] != 2 * heads \
            or state.shape[1] != matrix_memory_state_floats(heads, dim, vdim):
        raise KernelError("matrix_memory: bad shapes")
    chunked = chunk_state is not None and max_chunks > 1
    if chunked and (chunk_state.dtype != torch.float32
                    or chunk_state.numel() < sequences * max_chunks * heads * dim * (vdim + 1)):
        raise KernelError("matrix_memory: chunk workspace too small")
    lib = _mm(dim)
    f = _fn(lib, "rl_memory_gates", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gates), _ptr(bias_i), _ptr(bias_f), float(cap), _ptr(seq_of_token), _ptr(state_slot), _ptr(state),
             _ptr(stab), tokens, sequences, heads, vdim, _stream()), "matrix_memory gates")
    f = _fn(lib, "rl_memory_recurrence", [c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_void_p])
    _check(f(_code(qkv.dtype), _ptr(qkv), qkv.stride(0), q_col, k_col, v_col, float(q_scale), _ptr(gates),
             _ptr(seq_of_token), _ptr(state_slot), _ptr(state), _ptr(num), _ptr(qn),
             _ptr(chunk_state) if chunked else None, tokens, sequences, heads, vdim, chunk,
             max_chunks if chunked else 1, _stream()), "matrix_memory recurrence", 3 if chunked else 1)


def matrix_memory_output(num: torch.Tensor, qn: torch.Tensor, stab: torch.Tensor, gate: Optional[torch.Tensor],
                         weight: torch.Tensor, out: torch.Tensor, tokens: int, heads: int, dim: int, vdim: int,
                         eps: float, floor: float, out_scale: float = 1.0) -> None:
    """out = unit_rms_per_head(num / (max(|qn|, exp(-stab)) + floor)) * weight * sigmoid(gate) * out_scale;
    ``gate`` and ``out`` are row-strided views of the activation type."""
    _need_cuda(num, qn, stab, gate, weight, out)
    if out.stride(1) != 1 or (gate is not None and (gate.stride(1) != 1 or gate.dtype != out.dtype)) \
            or weight.numel() != heads * vdim:
        raise KernelError("matrix_memory_output: bad shapes")
    f = _fn(_mm(dim), "rl_memory_output", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                           c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(_ptr(num), _ptr(qn), _ptr(stab), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight),
             _code(weight.dtype), _ptr(out), out.stride(0), _code(out.dtype), tokens, heads, vdim, float(eps),
             float(floor), float(out_scale), _stream()), "matrix_memory_output")


# ------------------------------------------- several residual streams, normed pairs, short convolutions

MAX_STREAMS = 8
MAX_CONV_TAPS = 8


def _so() -> ctypes.CDLL:
    return _lib("stream_ops", "stream_ops.cu")


def streams_step(streams: torch.Tensor, tokens: int, init: Optional[torch.Tensor] = None,
                 y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                 out_w: Optional[torch.Tensor] = None, read_in: Optional[torch.Tensor] = None,
                 norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, normed: Optional[torch.Tensor] = None,
                 total: Optional[torch.Tensor] = None) -> None:
    """One sublayer's boundary on the float32 streams [tokens, n, width] (csrc/stream_ops.cu): with ``init``
    [tokens, width] every stream becomes a copy of it; with ``y`` (the sublayer's output, activation type) the
    streams are mixed, X_t <- sum_s mix[s, t] X_s + out_w[t] y; with ``read_in`` the next sublayer's input is
    formed, normed = rmsnorm(sum_s read_in[s] X_s) * norm_w; with ``total`` the sum of the streams is written.
    mix, out_w and read_in are float32."""
    _need_cuda(streams, init, y, mix, out_w, read_in, norm_w, normed, total)
    n, width = streams.shape[1], streams.shape[2]
    if streams.dtype != torch.float32 or not streams.is_contiguous() or not 1 <= n <= MAX_STREAMS:
        raise KernelError(f"streams_step: contiguous float32 [tokens, n <= {MAX_STREAMS}, width]")
    for t in (init, total):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.shape[1] != width):
            raise KernelError("streams_step: init and total are contiguous float32 [tokens, width]")
    if y is not None and (mix is None or out_w is None or mix.numel() != n * n or out_w.numel() != n
                          or mix.dtype != torch.float32 or out_w.dtype != torch.float32 or y.stride(1) != 1):
        raise KernelError("streams_step: a sublayer's output comes with float32 mix [n, n] and out [n]")
    if read_in is not None and (norm_w is None or normed is None or read_in.numel() != n
                                or read_in.dtype != torch.float32 or normed.stride(1) != 1
                                or (y is not None and y.dtype != normed.dtype)):
        raise KernelError("streams_step: read_in float32 [n] comes with a norm weight and a buffer for the normed rows")
    act = normed if normed is not None else y
    f = _fn(_so(), "rl_streams_step", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(streams), _ptr(init), _ptr(y), y.stride(0) if y is not None else 0,
             _ptr(mix.contiguous()) if mix is not None else None, _ptr(out_w), _ptr(read_in), _ptr(norm_w),
             _code(norm_w.dtype) if norm_w is not None else 0, _ptr(normed),
             normed.stride(0) if normed is not None else 0, _code(act.dtype) if act is not None else 0, _ptr(total),
             tokens, n, width, float(eps), _stream()), "streams_step")


def pair_norm_mean(a: torch.Tensor, wa: torch.Tensor, ca: float, b: torch.Tensor, wb: torch.Tensor, cb: float,
                   out: torch.Tensor, eps: float, rows: Optional[int] = None, bias_a: Optional[torch.Tensor] = None,
                   bias_b: Optional[torch.Tensor] = None) -> None:
    """out = ca * rmsnorm(a + bias_a) * wa + cb * rmsnorm(b + bias_b) * wb over rows of the activation type; the
    biases (float32 [width]) are optional (csrc/stream_ops.cu)."""
    _need_cuda(a, b, wa, wb, out, bias_a, bias_b)
    for bias in (bias_a, bias_b):
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != a.shape[1] or not bias.is_contiguous()):
            raise KernelError("pair_norm_mean: a bias is contiguous float32 [width]")
    if a.dtype != b.dtype or a.dtype != out.dtype or wa.dtype != wb.dtype or a.shape[1] != b.shape[1] \
            or a.stride(1) != 1 or b.stride(1) != 1 or out.stride(1) != 1 or wa.numel() != a.shape[1]:
        raise KernelError("pair_norm_mean: two inputs and an output of one type and width, weights of one type")
    f = _fn(_so(), "rl_pair_norm_mean", [c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_float,
                                         c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    _check(f(_code(a.dtype), _ptr(a), a.stride(0), _ptr(wa), float(ca), _ptr(b), b.stride(0), _ptr(wb), float(cb),
             _code(wa.dtype), _ptr(out), out.stride(0), rows if rows is not None else a.shape[0], a.shape[1],
             float(eps), _ptr(bias_a), _ptr(bias_b), _stream()), "pair_norm_mean")


def short_conv(x: torch.Tensor, col_x: int, w: torch.Tensor, bias: Optional[torch.Tensor], y: torch.Tensor, col_y: int,
               act: int, seq_of_token: torch.Tensor, state_slot: torch.Tensor, state: torch.Tensor, tokens: int,
               single: bool = False) -> None:
    """Causal convolution over time on ``w.shape[0]`` channels of x's rows, from column ``col_x``, into y's from
    ``col_y`` (another buffer): y_t = act(sum_j w[c, j] (x_(t - taps + 1 + j) + bias_c)) within a token's own
    sequence; what lies before the step's portion comes from the sequence's slot of ``state`` (float32
    [slots, (taps - 1) * channels]: the last inputs, zeros for a new request), which is then moved on
    (csrc/stream_ops.cu).  ``act``: ACT_NONE or ACT_SILU.  ``single``: every sequence of the step has exactly one
    token (one launch instead of two)."""
    _need_cuda(x, w, bias, y, state)
    channels, taps = w.shape
    if x.dtype != y.dtype or x.stride(1) != 1 or y.stride(1) != 1 or not w.is_contiguous() \
            or x.data_ptr() == y.data_ptr() or not 1 <= taps <= MAX_CONV_TAPS or act not in (ACT_NONE, ACT_SILU):
        raise KernelError(f"short_conv: two buffers of one type, contiguous weights [channels, taps <= {MAX_CONV_TAPS}]")
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < (taps - 1) * channels:
        raise KernelError("short_conv: the state is float32 [slots, (taps - 1) * channels]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != channels or not bias.is_contiguous()):
        raise KernelError("short_conv: the bias is contiguous float32 [channels]")
    f = _fn(_so(), "rl_short_conv", [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p])
    _check(f(_code(x.dtype), _ptr(x), x.stride(0), col_x, _ptr(w), _code(w.dtype), _ptr(bias), _ptr(y), y.stride(0),
             col_y, channels, taps, act, _ptr(seq_of_token), _ptr(state_slot), _ptr(state), state.stride(0), tokens,
             1 if single else 0, _stream()), "short_conv", 2 if (taps > 1 and not single) else 1)


# ------------------------------------------------------------------- the gated delta rule

def _delta(dim: int) -> ctypes.CDLL:
    if not 1 <= dim <= 256:
        raise KernelError(f"delta_rule takes key sizes up to 256; got {dim}")
    return _lib(f"delta_rule_d{dim}", "delta_rule.cu", {"RL_DELTA_DIM": dim})


def delta_prep(x: torch.Tensor, q_col: int, k_col: int, qk_heads: int, heads: int, dim: int, q_scale: float,
               unit_floor: float, zb: torch.Tensor, za: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
               q: torch.Tensor, k: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, tokens: int) -> None:
    """What the delta rule's recurrence is fed (csrc/delta_rule.cu), all float32: q and k heads of x's rows as
    unit vectors x / sqrt(sum x^2 + unit_floor) (q times ``q_scale``), beta = sigmoid(zb) per head, and per head
    and key channel decay = exp(-exp(a_log_h) * softplus(za + dt_bias))."""
    _need_cuda(x, zb, za, dt_bias, a_log, q, k, beta, decay)
    for t in (zb, za, dt_bias, a_log, q, k, beta, decay):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("delta_prep: projections, constants and outputs are contiguous float32")
    if x.stride(1) != 1 or zb.shape[1] != heads or za.shape[1] != heads * dim or dt_bias.numel() != heads * dim \
            or a_log.numel() != heads or q.shape[1] != qk_heads * dim or heads % qk_heads != 0:
        raise KernelError("delta_prep: bad shapes")
    f = _fn(_delta(dim), "rl_delta_prep", [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_void_p])
    _check(f(_code(x.dtype), _ptr(x), x.stride(0), q_col, k_col, qk_heads, heads, float(q_scale), float(unit_floor),
             _ptr(zb), _ptr(za), _ptr(dt_bias), _ptr(a_log), _ptr(q), _ptr(k), _ptr(beta), _ptr(decay), tokens,
             _stream()), "delta_prep")


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor,
               seq_of_token: torch.Tensor, state_slot: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
               tokens: int, sequences: int, heads: int, qk_heads: int, dim: int, vdim: int) -> None:
    """Per head S <- diag(decay) S; d = beta (v - S^T k); S <- S + k d^T; o = S^T q over every sequence of the
    step, from and into the sequences' state slots (csrc/delta_rule.cu).  q, k float32 [tokens, qk_heads * dim],
    v a row-strided view [tokens, heads * vdim] of the activation type, beta [tokens, heads], decay
    [tokens, heads * dim], state float32 [slots, heads * dim * vdim], out float32 [tokens, heads * vdim]."""
    _need_cuda(q, k, v, beta, decay, state, out)
    for t in (q, k, beta, decay, out):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("delta_rule: q, k, beta, decay and out are contiguous float32")
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < heads * dim * vdim or v.stride(1) != 1 \
            or v.shape[1] != heads * vdim or heads % qk_heads != 0:
        raise KernelError("delta_rule: bad shapes")
    f = _fn(_delta(dim), "rl_delta_rule", [c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p])
    _check(f(_code(v.dtype), _ptr(q), _ptr(k), _ptr(v), v.stride(0), _ptr(beta), _ptr(decay), _ptr(seq_of_token),
             _ptr(state_slot), _ptr(state), state.stride(0), _ptr(out), tokens, sequences, heads, qk_heads, vdim,
             _stream()), "delta_rule")


def head_gated_norm(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                    tokens: int, heads: int, vdim: int, eps: float, dim: int = 64) -> None:
    """out = o / sqrt(mean over a head (o^2) + eps) * weight * sigmoid(gate): o float32 [tokens, heads * vdim],
    weight [vdim] (one for all heads) or [heads * vdim], gate and out row-strided views of the activation type."""
    _need_cuda(o, gate, weight, out)
    if o.dtype != torch.float32 or not o.is_contiguous() or out.stride(1) != 1 \
            or (gate is not None and (gate.stride(1) != 1 or gate.dtype != out.dtype)) \
            or weight.numel() not in (vdim, heads * vdim):
        raise KernelError("head_gated_norm: bad shapes")
    f = _fn(_delta(dim), "rl_head_gated_norm", [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                                c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_code(out.dtype), _ptr(o), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight),
             _code(weight.dtype), 1 if weight.numel() == heads * vdim and heads > 1 else 0, _ptr(out), out.stride(0),
             tokens, heads, vdim, float(eps), _stream()), "head_gated_norm")


# ------------------------------------------------------------------- routed feed-forward

def _moe() -> ctypes.CDLL:
    return _lib("moe", "moe.cu")


MOE_TILE_ROWS = 64
MOE_FEW_PAIRS = 64        # up to so many (token, expert) pairs the products stream the weights per pair


def moe_max_tiles(pairs: int, experts: int) -> int:
    return pairs // MOE_TILE_ROWS + experts


def moe_route(x: torch.Tensor, router: Optional[torch.Tensor], choice: torch.Tensor, weight: torch.Tensor, tokens: int,
              groups: int, keep: int, group_top: int, top: int, softmax: bool = False, renorm: bool = False,
              bias: Optional[torch.Tensor] = None, choice_bias: Optional[torch.Tensor] = None,
              weight_scale: float = 1.0, renorm_floor: float = 0.0) -> None:
    """Per token: scores of the experts (float32 sums; sigmoid, or softmax), the best ``keep`` of ``groups``
    groups of neighbouring experts by the sum of their ``group_top`` best scores, the ``top`` best experts
    of those into choice [tokens, top] int32 with their scores in weight [tokens, top] float32.  With
    ``router`` None, ``x`` holds the logits themselves, float32 [tokens, experts].  ``bias`` (float32
    [experts]) is added to the logits before they are scored.  ``choice_bias`` (float32 [experts]) is added to
    the scores for the choice only: the weights are the scores without it.  With ``renorm`` the chosen scores
    are divided by their sum + ``renorm_floor``; every weight is multiplied by ``weight_scale``."""
    _need_cuda(x, router, choice, weight, bias, choice_bias)
    if choice_bias is not None and (choice_bias.dtype != torch.float32 or not choice_bias.is_contiguous()):
        raise KernelError("moe_route: the choice bias is contiguous float32 [experts]")
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != x.shape[1] and router is None):
        raise KernelError("moe_route: the bias is contiguous float32 [experts]")
    if router is None:
        if x.dtype != torch.float32:
            raise KernelError("moe_route: logits handed in must be float32")
        experts, width = x.shape[1], 0
    else:
        experts, width = router.shape
    if experts % max(groups, 1) != 0 or choice.dtype != torch.int32 or weight.dtype != torch.float32 \
            or x.stride(1) != 1 or (router is not None and not router.is_contiguous()):
        raise KernelError("moe_route: experts must divide into the groups; choice int32, weight float32")
    if choice_bias is not None and choice_bias.numel() != experts:
        raise KernelError("moe_route: one choice bias per expert")
    f = _fn(_moe(), "rl_moe_route", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                                      c_void_p])
    _check(f(_ptr(x), _code(x.dtype), x.stride(0), _ptr(router), _code(router.dtype) if router is not None else 0,
             tokens, width, experts,
             max(groups, 1), keep, group_top, top, 1 if softmax else 0, 1 if renorm else 0, _ptr(bias),
             _ptr(choice_bias), float(weight_scale), float(renorm_floor), _ptr(choice), _ptr(weight), _stream()),
           "moe_route")


def moe_group(choice: torch.Tensor, pairs: int, experts: int, order: torch.Tensor, tile_expert: torch.Tensor,
              tile_begin: torch.Tensor, tile_rows: torch.Tensor, meta: torch.Tensor, tiled: Optional[int] = None) -> None:
    """Lists the (token, slot) pairs expert by expert (``order``) and cuts every expert's list into tiles of
    up to 64 pairs (``tile_*``, their number in meta[0]); all int32, the tile lists ``moe_max_tiles`` long.
    ``tiled``: only the first so many experts get tiles (the others have no matrices: identity experts)."""
    _need_cuda(choice, order, tile_expert, tile_begin, tile_rows, meta)
    f = _fn(_moe(), "rl_moe_group", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p])
    _check(f(_ptr(choice), pairs, experts, experts if tiled is None else tiled, _ptr(order), _ptr(tile_expert),
             _ptr(tile_begin), _ptr(tile_rows), _ptr(meta), _stream()), "moe_group")


def moe_gemm(src: torch.Tensor, src_div: int, w: torch.Tensor, dst: torch.Tensor, order: torch.Tensor,
             tile_expert: torch.Tensor, tile_begin: torch.Tensor, tile_rows: torch.Tensor, meta: torch.Tensor,
             max_tiles: int, act: int = ACT_NONE, few_pairs: Optional[bool] = None) -> None:
    """dst[pair] = act(w[expert of the pair] @ src[pair // src_div]) for every listed pair: w [experts, n, k]
    (or [experts * n, k]) with ``n = dst.shape[1]``, src [*, k], dst [pairs, n].  ``few_pairs`` chooses the
    kernel that streams the weights for a handful of pairs (default: up to MOE_FEW_PAIRS rows of dst)."""
    _need_cuda(src, w, dst)
    n, k = dst.shape[1], src.shape[1]
    if w.shape[-1] != k or not w.is_contiguous() or src.stride(1) != 1 or dst.stride(1) != 1 or src.dtype != dst.dtype \
            or w.dtype != src.dtype:
        raise KernelError(f"moe_gemm: shapes src{tuple(src.shape)} w{tuple(w.shape)} dst{tuple(dst.shape)}, one type")
    f = _fn(_moe(), "rl_moe_gemm", [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    if few_pairs is None:
        few_pairs = dst.shape[0] <= MOE_FEW_PAIRS
    _check(f(_code(src.dtype), _ptr(src), src.stride(0), src_div, _ptr(w), n, k, _ptr(dst), dst.stride(0), _ptr(order),
             _ptr(tile_expert), _ptr(tile_begin), _ptr(tile_rows), _ptr(meta), max_tiles, 1 if few_pairs else 0, act,
             _stream()), "moe_gemm")


def moe_combine(y: torch.Tensor, weight: torch.Tensor, shared: Optional[torch.Tensor], out: torch.Tensor,
                tokens: int, top: int, choice: Optional[torch.Tensor] = None, real_experts: int = 0,
                x: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k weight[t, k] * y[t * top + k] (+ shared[t]), k in order; y, shared and out contiguous.
    With ``choice`` and ``x`` (the experts' input [tokens, width]) a pair whose chosen index is at least
    ``real_experts`` stands for the identity: its term is weight[t, k] * x[t]."""
    _need_cuda(y, weight, out, choice, x)
    if not (y.is_contiguous() and out.is_contiguous() and (shared is None or shared.is_contiguous())):
        raise KernelError("moe_combine: contiguous tensors")
    if (choice is None) != (x is None) or (x is not None and (x.dtype != out.dtype or x.stride(1) != 1)):
        raise KernelError("moe_combine: identity experts need the choices and the experts' input in out's type")
    f = _fn(_moe(), "rl_moe_combine", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_int, c_void_p, c_int, c_void_p])
    _check(f(_code(out.dtype), _ptr(y), _ptr(weight), _ptr(shared), _ptr(out), tokens, out.shape[1], top, _ptr(choice),
             real_experts, _ptr(x), x.stride(0) if x is not None else 0, _stream()), "moe_combine")


# -------------------------------------------------------------------- sampling

SAMPLE_CHUNKS = 64


def sample(logits: torch.Tensor, rows: int, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed_lo: torch.Tensor, seed_hi: torch.Tensor, position: torch.Tensor,
           out_token: torch.Tensor, out_logprob: Optional[torch.Tensor], stream_id: int = 0,
           scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits.  ``scratch`` (float32, rows * SAMPLE_CHUNKS * 4) lets greedy
    rows use a two-stage arg max over the whole GPU."""
    _need_cuda(logits, out_token)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    f = _fn(_lib("sampling", "sampling.cu"), "rl_sample",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_uint, c_void_p, c_void_p, c_void_p, c_void_p])
    if scratch is not None and scratch.numel() < rows * SAMPLE_CHUNKS * 4:
        raise KernelError("sample: scratch too small")
    _check(f(_ptr(logits), rows, logits.shape[1], logits.stride(0), _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(position), stream_id, _ptr(out_token),
             _ptr(out_logprob), _ptr(scratch), _stream()), "sample", 2 if scratch is not None else 1)


def gather_logprob(logits: torch.Tensor, rows: int, target: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(logits, target, out)
    f = _fn(_lib("sampling", "sampling.cu"), "rl_gather_logprob",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), rows, logits.shape[1], logits.stride(0), _ptr(target), _ptr(out), _stream()),
           "gather_logprob")


def build_all(head_dims=(64, 128), maps_dims=((64, 128, 2), (128, 128, 1)), linear_dims=(64,), memory_dims=(64,),
              delta_dims=(128,), verbose: bool = True) -> None:
    """Compiles every kernel family (attention for the given head sizes, attention with score maps for the
    given (key size, value size, maps), linear attention and the matrix memory for the given key sizes) and
    removes built files of these modules that belong to other versions of the sources."""
    built = [
        build.compile_module("elementwise", "elementwise.cu", verbose=verbose),
        build.compile_module("gemm_simt", "gemm_simt.cu", verbose=verbose),
        build.compile_module("gemm_skinny", "gemm_skinny.cu", verbose=verbose),
        build.compile_module("gemm_tc", "gemm_tc.cu", verbose=verbose),
        build.compile_module("gemm_mid", "gemm_mid.cu", verbose=verbose),
        build.compile_module("sampling", "sampling.cu", verbose=verbose),
        build.compile_module("rowwise", "rowwise.cu", verbose=verbose),
        build.compile_module("moe", "moe.cu", verbose=verbose),
        build.compile_module("latent", "latent.cu", verbose=verbose),
        build.compile_module("stream_ops", "stream_ops.cu", verbose=verbose),
        build.compile_module("host_core", "host_core.cpp", verbose=verbose),   # host-only: cache manager, batch filler
    ]
    for d in head_dims:
        built.append(build.compile_module(f"attention_d{d}", "attention.cu", {"RL_HEAD_DIM": d}, verbose=verbose))
    for d, v, m, *stride in maps_dims:         # (key size, value size, maps[, length of a value row if longer])
        if stride and stride[0] not in (0, v):
            built.append(build.compile_module(f"attention_maps_d{d}_v{v}_m{m}_s{stride[0]}", "attention_maps.cu",
                                              {"RL_QK_DIM": d, "RL_V_DIM": v, "RL_MAPS": m, "RL_V_STRIDE": stride[0]},
                                              verbose=verbose))
            continue
        built.append(build.compile_module(f"attention_maps_d{d}_v{v}_m{m}", "attention_maps.cu",
                                          {"RL_QK_DIM": d, "RL_V_DIM": v, "RL_MAPS": m}, verbose=verbose))
    for d in linear_dims:
        built.append(build.compile_module(f"linear_attention_d{d}", "linear_attention.cu", {"RL_LIN_DIM": d},
                                          verbose=verbose))
    for d in memory_dims:
        built.append(build.compile_module(f"matrix_memory_d{d}", "matrix_memory.cu", {"RL_MM_DIM": d}, verbose=verbose))
    for d in delta_dims:
        built.append(build.compile_module(f"delta_rule_d{d}", "delta_rule.cu", {"RL_DELTA_DIM": d}, verbose=verbose))
    build.remove_other_versions(built)
