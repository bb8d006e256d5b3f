"""CPU oracle for the MXFP8 quantise + AllGather-Matmul path (TEST INFRASTRUCTURE ONLY).

Only the tests, the smoke check and the benchmark's CPU-baseline / reference legs may import
this module; the shipped library never does.

Three restatements of the same arithmetic live here so that they can check one another:

* ``C`` - ctypes wrappers over ``mx_oracle.c`` (fast, threaded): the checker used at size.
* ``*_np`` - an independent vectorised numpy restatement (bit operations only).
* ``golden_*_torch`` - a step-by-step torch-CPU port of the reference's golden generator
  (examples/utils/gen_mx_quant_allgather_data.py:168-189,255-324 with the "native" backend and
  examples/utils/gen_data_fp8_mx_allgather_matmul.py:643-658); this is the leg timed as the
  CPU baseline because it is what the reference itself runs on the host.

Parity is pinned against outputs of the reference generator itself, stored in tests/golden/.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmx_oracle.so")

MODE_GOLDEN = 0  # tiny-block rule of the CPU golden (amax < 1e-12 -> scale byte 0x7F)
MODE_DEVICE = 1  # tiny-block rule of the device kernel (byte = max(E - 8, 0))

_lib = None


def build() -> str:
    """Compile mx_oracle.c into libmx_oracle.so (no-op when it is up to date)."""
    src = os.path.join(_HERE, "mx_oracle.c")
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libmx_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        L.mxo_quantize_rows.argtypes = [vp, sz, sz, vp, vp, ci]
        L.mxo_quantize_rows.restype = ci
        L.mxo_quantize_weight.argtypes = [vp, sz, sz, vp, vp, ci]
        L.mxo_quantize_weight.restype = ci
        L.mxo_dequant_rows.argtypes = [vp, vp, sz, sz, vp]
        L.mxo_dequant_rows.restype = None
        L.mxo_dequant_weight.argtypes = [vp, vp, sz, sz, vp]
        L.mxo_dequant_weight.restype = None
        L.mxo_gemm_f32.argtypes = [vp, vp, vp, sz, sz, sz]
        L.mxo_gemm_f32.restype = None
        L.mxo_e4m3_from_f32.argtypes = [ctypes.c_float]
        L.mxo_e4m3_from_f32.restype = ctypes.c_uint8
        L.mxo_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.mxo_e4m3_to_f32.restype = ctypes.c_float
        L.mxo_quantize_rows_e5m2.argtypes = [vp, sz, sz, vp, vp, ci]
        L.mxo_quantize_rows_e5m2.restype = ci
        L.mxo_dequant_rows_e5m2.argtypes = [vp, vp, sz, sz, vp]
        L.mxo_dequant_rows_e5m2.restype = None
        L.mxo_e5m2_from_f32.argtypes = [ctypes.c_float]
        L.mxo_e5m2_from_f32.restype = ctypes.c_uint8
        L.mxo_e5m2_to_f32.argtypes = [ctypes.c_uint8]
        L.mxo_e5m2_to_f32.restype = ctypes.c_float
        L.mxo_quantize_rows_e2m1.argtypes = [vp, sz, sz, vp, vp, ci]
        L.mxo_quantize_rows_e2m1.restype = ci
        L.mxo_dequant_rows_e2m1.argtypes = [vp, vp, sz, sz, vp]
        L.mxo_dequant_rows_e2m1.restype = None
        L.mxo_e2m1_from_f32.argtypes = [ctypes.c_float, ci]
        L.mxo_e2m1_from_f32.restype = ctypes.c_uint8
        L.mxo_e2m1_to_f32.argtypes = [ctypes.c_uint8]
        L.mxo_e2m1_to_f32.restype = ctypes.c_float
        L.mxo_quantize_rows_e1m2.argtypes = [vp, sz, sz, vp, vp, ci]
        L.mxo_quantize_rows_e1m2.restype = ci
        L.mxo_dequant_rows_e1m2.argtypes = [vp, vp, sz, sz, vp]
        L.mxo_dequant_rows_e1m2.restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


# --------------------------------------------------------------------------------------
# bf16 helpers (bit patterns are carried as uint16)
# --------------------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# --------------------------------------------------------------------------------------
# C oracle wrappers
# --------------------------------------------------------------------------------------
FMT_E4M3, FMT_E5M2 = 0, 1


def quantize_rows(x_bits: np.ndarray, mode: int = MODE_GOLDEN, fmt: int = FMT_E4M3):
    """bf16 bits [rows, K] -> (codes uint8 [rows, K], scales uint8 [rows, K/32]); codes E4M3 or E5M2."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, K = x_bits.shape
    codes = np.empty((rows, K), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    fn = lib().mxo_quantize_rows_e5m2 if fmt == FMT_E5M2 else lib().mxo_quantize_rows
    if fn(_p(x_bits), rows, K, _p(codes), _p(scales), mode) != 0:
        raise ValueError("K must be a multiple of 32")
    return codes, scales


def quantize_rows_e2m1(x_bits: np.ndarray, mode: int = MODE_GOLDEN):
    """bf16 bits [rows, K] -> (packed E2M1 codes uint8 [rows, K/2], low nibble = even column; scales [rows, K/32]).

    The FP4 variant of the operators; oracle and fixtures only, no CUDA kernel reads these yet."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, K = x_bits.shape
    packed = np.empty((rows, K // 2), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    if lib().mxo_quantize_rows_e2m1(_p(x_bits), rows, K, _p(packed), _p(scales), mode) != 0:
        raise ValueError("K must be a multiple of 32")
    return packed, scales


def dequant_rows_e2m1(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, half = packed.shape
    out = np.empty((rows, 2 * half), np.float32)
    lib().mxo_dequant_rows_e2m1(_p(packed), _p(scales), rows, 2 * half, _p(out))
    return out


def quantize_rows_e1m2(x_bits: np.ndarray, mode: int = MODE_GOLDEN):
    """The E1M2 form of quantize_rows_e2m1 (emax 0, max 1.75); oracle only."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, K = x_bits.shape
    packed = np.empty((rows, K // 2), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    if lib().mxo_quantize_rows_e1m2(_p(x_bits), rows, K, _p(packed), _p(scales), mode) != 0:
        raise ValueError("K must be a multiple of 32")
    return packed, scales


def dequant_rows_e1m2(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, half = packed.shape
    out = np.empty((rows, 2 * half), np.float32)
    lib().mxo_dequant_rows_e1m2(_p(packed), _p(scales), rows, 2 * half, _p(out))
    return out


def quantize_weight(b_bits: np.ndarray, mode: int = MODE_GOLDEN):
    """bf16 bits [K, N] -> (codes uint8 [K, N], scales uint8 [K/64, N, 2]) blocks along K."""
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    K, N = b_bits.shape
    codes = np.empty((K, N), np.uint8)
    scales = np.empty((K // 64, N, 2), np.uint8)
    if lib().mxo_quantize_weight(_p(b_bits), K, N, _p(codes), _p(scales), mode) != 0:
        raise ValueError("K must be a multiple of 64")
    return codes, scales


def dequant_rows(codes: np.ndarray, scales: np.ndarray, fmt: int = FMT_E4M3) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, K = codes.shape
    out = np.empty((rows, K), np.float32)
    (lib().mxo_dequant_rows_e5m2 if fmt == FMT_E5M2 else lib().mxo_dequant_rows)(_p(codes), _p(scales), rows, K, _p(out))
    return out


def dequant_weight(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    K, N = codes.shape
    out = np.empty((K, N), np.float32)
    lib().mxo_dequant_weight(_p(codes), _p(scales), K, N, _p(out))
    return out


def gemm_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.empty((M, N), np.float32)
    lib().mxo_gemm_f32(_p(a), _p(b), _p(c), M, N, K)
    return c


def allgather_matmul(a_codes_per_rank, a_scales_per_rank, b_codes, b_scales, rows=None, a_fmt: int = FMT_E4M3) -> np.ndarray:
    """Golden C for one rank: concat over ranks of dequant(A_r), times dequant(B); fp32.

    ``rows`` optionally selects rows of the gathered A (sampled parity at benchmark sizes).
    """
    a_codes = np.concatenate(a_codes_per_rank, axis=0)
    a_scales = np.concatenate(a_scales_per_rank, axis=0)
    if rows is not None:
        a_codes, a_scales = a_codes[rows], a_scales[rows]
    return gemm_f32(dequant_rows(a_codes, a_scales, a_fmt), dequant_weight(b_codes, b_scales))


# --------------------------------------------------------------------------------------
# independent numpy restatement (cross-check of the C code)
# --------------------------------------------------------------------------------------
def _e4m3_rne_np(y: np.ndarray) -> np.ndarray:
    """fp32 (|y| <= 448, finite) -> E4M3FN codes, RNE, via integer arithmetic on the bits."""
    u = y.view(np.uint32)
    sign = ((u >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
    a = u & np.uint32(0x7FFFFFFF)
    av = a.view(np.float32)
    sub = av < np.float32(2.0 ** -6)
    q_sub = np.rint(av * np.float32(512.0)).astype(np.uint32)  # numpy rint is nearest-even
    e = (a >> np.uint32(23)).astype(np.int64) - 127
    man = a & np.uint32(0x7FFFFF)
    keep = man >> np.uint32(20)
    rem = man & np.uint32(0xFFFFF)
    up = (rem > np.uint32(0x80000)) | ((rem == np.uint32(0x80000)) & ((keep & np.uint32(1)) == 1))
    q_norm = (((e + 7).astype(np.uint32) << np.uint32(3)) | keep) + up.astype(np.uint32)
    q = np.where(sub, q_sub, q_norm).astype(np.uint8)
    return sign | q


def quantize_rows_np(x_bits: np.ndarray, mode: int = MODE_GOLDEN):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, K = x_bits.shape
    nb = K // 32
    blk = x_bits.reshape(rows, nb, 32)
    amax = (blk & np.uint16(0x7FFF)).max(axis=-1)
    E = (amax >> np.uint16(7)).astype(np.int64)
    nonfinite = E == 255
    if mode == MODE_GOLDEN:
        zero = amax <= np.uint16(0x2B8C)
        byte = np.where(zero, 127, E - 8)
    else:
        byte = np.maximum(E - 8, 0)
        zero = byte == 0
    byte = np.where(nonfinite, 255, byte)
    mul_exp = np.clip(127 - byte, -126, 127)
    mul = ((mul_exp + 127).astype(np.uint32) << np.uint32(23)).view(np.float32)
    y = bf16_bits_to_f32(blk).reshape(rows, nb, 32) * mul[..., None]
    y = np.clip(y, np.float32(-448.0), np.float32(448.0)).astype(np.float32)
    codes = _e4m3_rne_np(np.ascontiguousarray(y))
    signed_zero = ((blk >> np.uint16(8)) & np.uint16(0x80)).astype(np.uint8)
    codes = np.where(zero[..., None], signed_zero, codes)
    codes = np.where(nonfinite[..., None], np.uint8(0x7F), codes)
    return codes.reshape(rows, K).astype(np.uint8), byte.astype(np.uint8)


# --------------------------------------------------------------------------------------
# torch-CPU port of the reference golden (the timed CPU baseline)
# --------------------------------------------------------------------------------------
def golden_quantize_torch(x_f32):
    """Port of _quantize_axis_last_fp8(x, "E4M3") with the "native" backend.

    Returns (codes uint8 tensor [M, K], scale bytes uint8 [M, K/32], dequant fp32 [M, K]).
    """
    import torch

    M, N = x_f32.shape
    nb = N // 32
    blocks = x_f32.view(M, nb, 32)
    max_abs = blocks.abs().amax(dim=-1)
    zero_mask = max_abs < 1e-12
    safe = torch.where(zero_mask, torch.ones_like(max_abs), max_abs)
    bits = safe.contiguous().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) - 127 - 8
    exp = exp.clamp(-128, 127)
    exp = torch.where(zero_mask, torch.zeros_like(exp), exp)
    scale = torch.exp2(exp.to(torch.float32))
    scaled = (blocks / scale.unsqueeze(-1)).clamp(-448.0, 448.0)
    q = scaled.to(torch.float8_e4m3fn)
    deq = (q.to(torch.float32) * scale.unsqueeze(-1)).reshape(M, N)
    codes = q.reshape(M, N).view(torch.uint8)
    scale_bytes = scale.to(torch.float8_e8m0fnu).view(torch.uint8)
    return codes, scale_bytes, deq


def golden_allgather_matmul_torch(a_f32_per_rank, b_deq_f32):
    """Port of the golden GEMM: quantise every rank's A, concat the dequantised rows, fp32 matmul."""
    import torch

    deq = [golden_quantize_torch(a)[2] for a in a_f32_per_rank]
    return torch.matmul(torch.cat(deq, dim=0), b_deq_f32)


# --------------------------------------------------------------------------------------
# tolerance rules
# --------------------------------------------------------------------------------------
def check_close(out_f32: np.ndarray, gold_f32: np.ndarray, rtol: float = 1e-2, atol: float = 1e-3):
    """The stated bar for the bf16 GEMM output: |out - gold| <= atol + rtol * |gold| everywhere."""
    diff = np.abs(out_f32.astype(np.float64) - gold_f32.astype(np.float64))
    bound = atol + rtol * np.abs(gold_f32.astype(np.float64))
    bad = int((diff > bound).sum())
    return bad, float(diff.max())


def check_reference_rule(out_f32: np.ndarray, gold_f32: np.ndarray, k: int, bf16: bool = True):
    """examples/utils/utils.py:97-105 + verify_result.py:213-241: every element within
    rtol * max(1, |gold|), rtol = 2^-7 (K < 2048) or 2^-6 for bf16 (2^-8 / 2^-7 for fp16);
    mean bias |mean(diff / max(1,|gold|))| reported beside it."""
    if bf16:
        rtol = 2.0 ** -7 if k < 2048 else 2.0 ** -6
    else:
        rtol = 2.0 ** -8 if k < 2048 else 2.0 ** -7
    tmax = np.maximum(1.0, np.abs(gold_f32.astype(np.float64)))
    diff = out_f32.astype(np.float64) - gold_f32.astype(np.float64)
    bad = int((np.abs(diff) > rtol * tmax).sum())
    eb = float(abs((diff / tmax).mean()))
    return bad, eb
