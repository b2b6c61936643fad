"""Local tcgen05 GEMM: ``C = alpha * A @ B.T`` with A [M,K], B [N,K] (nn.Linear weight layout).

bf16 inputs, or fp8 e4m3 inputs with per-tensor scales folded into ``alpha``;
fp32 accumulation in tensor memory; bf16 output.  This is the single-GPU
building block of every fused tensor-parallel op (reference counterpart:
``matmul::kernel`` in datasets/example053_thunderkitten_gemm_ar_easy/nv/
empty_thunderkitten_gemm_ar.cu:84-191).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N


class GemmError(RuntimeError):
    pass


def _check(t: torch.Tensor, name: str):
    if not (t.is_cuda and t.is_contiguous() and t.dim() == 2 and t.data_ptr() % 16 == 0):
        raise GemmError(f"{name} must be a contiguous, 16-byte aligned 2-D CUDA tensor")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, alpha: float = 1.0,
         bn: int = 0, max_ctas: int = 0, status_ptr: int = 0, stream=None) -> torch.Tensor:
    """``out[M,N] = alpha * a[M,K] @ b[N,K].T`` on the tcgen05 kernel (no library GEMM)."""
    lib = N.load()
    _check(a, "a")
    _check(b, "b")
    M, K = a.shape
    Nn, K2 = b.shape
    if K != K2:
        raise GemmError(f"inner dimensions differ: {K} vs {K2}")
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a.device)
    _check(out, "out")
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, Nn):
        raise GemmError("out must be bf16 [M, N]")
    if a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16:
        fn = lib.cb_gemm_bf16
    elif a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn:
        fn = lib.cb_gemm_fp8
    else:
        raise GemmError(f"unsupported dtypes {a.dtype} x {b.dtype}")
    rc = fn(N.ptr(a), N.ptr(b), N.ptr(out), M, Nn, K, C.c_float(alpha), bn, max_ctas,
            C.c_void_p(status_ptr), N.stream_ptr(stream))
    if rc != 0:
        raise GemmError(f"gemm launch failed: {N.last_error()}")
    return out


def gemm_role_trace(a: torch.Tensor, b: torch.Tensor, bn: int = 512) -> dict:
    """Runs one bf16 GEMM with the kernel's role trace on and returns, per role, the mean
    share of its time spent waiting (SM clock cycles, averaged over the CTAs that had work):
    ``mma_wait_operands``, ``mma_wait_accumulator``, ``producer_wait_slots``,
    ``epilogue_wait_accumulator``, plus ``mma_cycles`` (mean total of the MMA thread)."""
    lib = N.load()
    _check(a, "a")
    _check(b, "b")
    M, K = a.shape
    Nn = b.shape[0]
    out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a.device)
    nsm = torch.cuda.get_device_properties(a.device).multi_processor_count
    trace = torch.zeros(nsm * 8, dtype=torch.int64, device=a.device)
    rc = lib.cb_gemm_bf16_traced(N.ptr(a), N.ptr(b), N.ptr(out), M, Nn, K, C.c_float(1.0), bn,
                                 N.ptr(trace), C.c_void_p(0), N.stream_ptr())
    if rc != 0:
        raise GemmError(f"gemm launch failed: {N.last_error()}")
    torch.cuda.synchronize()
    t = trace.view(nsm, 8).double().cpu()
    mma = t[t[:, 2] > 0]
    prod = t[t[:, 4] > 0]
    epi = t[t[:, 6] > 0]
    return {
        "mma_cycles": float(mma[:, 2].mean()) if len(mma) else 0.0,
        "mma_wait_operands": float((mma[:, 0] / mma[:, 2]).mean()) if len(mma) else 0.0,
        "mma_wait_accumulator": float((mma[:, 1] / mma[:, 2]).mean()) if len(mma) else 0.0,
        "producer_wait_slots": float((prod[:, 3] / prod[:, 4]).mean()) if len(prod) else 0.0,
        "epilogue_wait_accumulator": float((epi[:, 5] / epi[:, 6]).mean()) if len(epi) else 0.0,
    }


# ------------------------------------------------------------- block-scaled fp8 operands
def quantize_blockscaled(x: torch.Tensor, row_block: int = 1):
    """bf16 [rows, K] -> (e4m3 [rows, K], fp32 scales).  ``row_block=1``: one scale per row and
    128 columns (activations, "1x128"); ``row_block=128``: one per 128x128 block (weights)."""
    lib = N.load()
    _check(x, "x")
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows + row_block - 1) // row_block, K // 128, dtype=torch.float32,
                    device=x.device)
    rc = lib.cb_quant_blockscaled(N.ptr(x), N.ptr(q), N.ptr(s), C.c_longlong(rows), K, row_block,
                                  N.stream_ptr())
    if rc != 0:
        raise GemmError(N.last_error())
    return q, s


def quantize_blockscaled_pow2(x: torch.Tensor, row_block: int = 1):
    """As :func:`quantize_blockscaled` with every scale rounded up to a power of two, the form
    the tensor cores can apply themselves.  Returns ``(q, scales fp32, sf)`` where ``sf`` is an
    int32 tensor ``[ceil(K/512), rows]``: word ``[kg, r]`` packs the exponent bytes (value
    ``2 ** (byte - 127)``) of K blocks ``4 kg .. 4 kg + 3`` of row ``r``, lowest byte first
    (missing blocks: 127).  For ``row_block=128`` every row of a block carries the block's
    byte, so ``sf`` has one column per row of ``x`` either way - what :func:`gemm_fp8_mx` takes."""
    lib = N.load()
    _check(x, "x")
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows + row_block - 1) // row_block, K // 128, dtype=torch.float32,
                    device=x.device)
    sf = torch.full(((K // 128 + 3) // 4, rows), 0x7f7f7f7f, dtype=torch.int32, device=x.device)
    rc = lib.cb_quant_blockscaled_pow2(N.ptr(x), N.ptr(q), N.ptr(s), N.ptr(sf), rows,
                                       C.c_longlong(rows), K, row_block, N.stream_ptr())
    if rc != 0:
        raise GemmError(N.last_error())
    return q, s, sf


def sf_exponents(sf: torch.Tensor, kblocks: int) -> torch.Tensor:
    """Unpacks :func:`quantize_blockscaled_pow2`'s words to exponent bytes ``[rows, kblocks]``."""
    kg, rows = sf.shape
    b = sf.view(torch.uint8).view(kg, rows, 4).permute(1, 0, 2).reshape(rows, kg * 4)
    return b[:, :kblocks]


def gemm_fp8_mx(a_q, a_sf, b_q, b_sf, out=None, alpha: float = 1.0, pair: bool = True,
                status_ptr: int = 0, stream=None):
    """``out = (a_q * 2^(a_sf-127)) @ (b_q * 2^(b_sf-127)).T`` with the power-of-two block scales
    applied by the tensor cores (``tcgen05.mma.kind::mxf8f6f4.block_scale``): ``a_sf``
    [ceil(K/512), M], ``b_sf`` [ceil(K/512), N] int32 from :func:`quantize_blockscaled_pow2`."""
    lib = N.load()
    _check(a_q, "a_q")
    _check(b_q, "b_q")
    M, K = a_q.shape
    Nn = b_q.shape[0]
    if a_q.dtype != torch.float8_e4m3fn or b_q.dtype != torch.float8_e4m3fn:
        raise GemmError("operands must be float8_e4m3fn")
    if K % 128 or b_q.shape[1] != K:
        raise GemmError("K must be a multiple of 128 and equal for both operands")
    kg = (K // 128 + 3) // 4
    for t, rows, name in ((a_sf, M, "a_sf"), (b_sf, Nn, "b_sf")):
        if not (t.dtype == torch.int32 and t.is_contiguous() and tuple(t.shape) == (kg, rows)):
            raise GemmError(f"{name} must be a contiguous int32 tensor [{kg}, {rows}]")
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a_q.device)
    _check(out, "out")
    # pair: a CTA pair per 256 x 192 tile (default, fastest); otherwise one CTA per 128 x 192
    rc = lib.cb_gemm_fp8_mx(N.ptr(a_q), N.ptr(a_sf), N.ptr(b_q), N.ptr(b_sf), N.ptr(out), M, Nn, K,
                            C.c_float(alpha), 0 if pair else -1, C.c_void_p(status_ptr),
                            N.stream_ptr(stream))
    if rc != 0:
        raise GemmError(f"gemm launch failed: {N.last_error()}")
    return out


def dequantize_blockscaled(q: torch.Tensor, s: torch.Tensor, row_block: int = 1,
                           out: torch.Tensor | None = None) -> torch.Tensor:
    lib = N.load()
    rows, K = q.shape
    if out is None:
        out = torch.empty(rows, K, dtype=torch.bfloat16, device=q.device)
    rc = lib.cb_dequant_blockscaled(N.ptr(q), N.ptr(s), N.ptr(out), C.c_longlong(rows), K,
                                    row_block, N.stream_ptr())
    if rc != 0:
        raise GemmError(N.last_error())
    return out


def gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, out=None, alpha: float = 1.0, pair: bool | None = None,
                         max_ctas: int = 0, status_ptr: int = 0, stream=None):
    """``out = (a_q * a_s [1x128 blocks]) @ (b_q * b_s [128x128 blocks]).T`` on the fp8 tensor
    cores: the quantised operands are the MMA operands, and every 128-wide K block's partial sum
    is multiplied by its two scales and accumulated in fp32 registers inside the kernel."""
    lib = N.load()
    _check(a_q, "a_q")
    _check(b_q, "b_q")
    M, K = a_q.shape
    Nn = b_q.shape[0]
    if a_q.dtype != torch.float8_e4m3fn or b_q.dtype != torch.float8_e4m3fn:
        raise GemmError("operands must be float8_e4m3fn")
    if K % 128 or b_q.shape[1] != K:
        raise GemmError("K must be a multiple of 128 and equal for both operands")
    if tuple(a_s.shape) != (M, K // 128) or tuple(b_s.shape) != ((Nn + 127) // 128, K // 128):
        raise GemmError("scales must be [M, K/128] and [ceil(N/128), K/128]")
    if not (a_s.is_contiguous() and b_s.is_contiguous() and a_s.dtype == torch.float32
            and b_s.dtype == torch.float32):
        raise GemmError("scales must be contiguous fp32 tensors")
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a_q.device)
    _check(out, "out")
    if pair is None:
        nsm = torch.cuda.get_device_properties(a_q.device).multi_processor_count
        pair = ((M + 255) // 256) * ((Nn + 255) // 256) * 2 >= nsm
    rc = lib.cb_gemm_fp8_blockscaled(N.ptr(a_q), N.ptr(a_s), N.ptr(b_q), N.ptr(b_s), N.ptr(out), M,
                                     Nn, K, C.c_float(alpha), int(bool(pair)), max_ctas,
                                     C.c_void_p(status_ptr), N.stream_ptr(stream))
    if rc != 0:
        raise GemmError(f"gemm launch failed: {N.last_error()}")
    return out


def gemm_fp8_blockscaled_expanded(a_q, a_s, b_q, b_s, out=None, b_cache: dict | None = None):
    """The same product through bf16: both operands are expanded by a bandwidth-bound kernel and
    multiplied on the bf16 path.  Kept as the slow cross-check of :func:`gemm_fp8_blockscaled`.
    ``b_cache`` (a dict) keeps the expanded weight across calls."""
    a = dequantize_blockscaled(a_q, a_s, 1)
    key = (b_q.data_ptr(), b_s.data_ptr())
    if b_cache is not None and key in b_cache:
        b = b_cache[key]
    else:
        b = dequantize_blockscaled(b_q, b_s, 128)
        if b_cache is not None:
            b_cache[key] = b
    return gemm(a, b, out=out)
