"""ctypes binding of libcatccos_b200.so (the C ABI declared in include/catccos_b200.h).

This is the host harness the tests and the benchmark drive the library through; torch is used only
for device memory and streams.  There is no fallback: when the shared library is missing or a call
fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# CATCCOS_B200_TRACE=1 in the environment selects the library built with the device-side timeline
# (python -m catccos_b200.build --trace); everything else is the same C ABI.
TRACE = os.environ.get("CATCCOS_B200_TRACE", "") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "libcatccos_b200_trace.so" if TRACE else "libcatccos_b200.so")

EXPORTS = [
    "catccos_b200_init",
    "catccos_b200_init_local",
    "catccos_b200_set_rank",
    "catccos_b200_finalize",
    "catccos_b200_symm_alloc",
    "catccos_b200_symm_free",
    "catccos_b200_symm_bytes_needed",
    "catccos_b200_mx_quant_allgather",
    "catccos_b200_fp8_mx_allgather_matmul",
    "catccos_b200_fp4_mx_allgather_matmul",
    "catccos_b200_mx_quant_allgather_matmul",
    "catccos_b200_mx_quant",
    "catccos_b200_mx_quant_fp4",
    "catccos_b200_mx_gemm",
    "catccos_b200_mx_gemm_quant_out",
    "catccos_b200_packed_row_bytes",
    "catccos_b200_mx_quant_scatter_packed",
    "catccos_b200_mxfp8_matmul_reduce_scatter",
    "catccos_b200_mx_quant_matmul_static",
    "catccos_b200_mx_quant_matmul_static_status",
    "catccos_b200_last_status",
    "catccos_b200_set_option",
    "catccos_b200_launch_count",
]


class Tiling(ctypes.Structure):
    """CocTilingParams (utils/info.h:97-115): 17 x uint32, same order."""

    _fields_ = [
        (n, ctypes.c_uint32)
        for n in (
            "m", "k", "n", "transA", "transB", "m0", "k0", "n0", "commTileM", "commInterval", "commNpuSplit",
            "commDataSplit", "commBlockM", "rankSize", "epSize", "expertNum", "topK",
        )
    ]


class CatccosError(RuntimeError):
    def __init__(self, fn: str, code: int):
        super().__init__(f"{fn} failed with code {code}")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library; raises if it has not been built (python -m catccos_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m catccos_b200.build` (nvcc, sm_100a). "
            "There is no CPU or PyTorch fallback for this path.")
    L = ctypes.CDLL(LIB_PATH)
    vp, u32, i32, sz, i64 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
    tp = ctypes.POINTER(Tiling)
    L.catccos_b200_init.argtypes = [i32, i32, i32, ctypes.c_char_p]
    L.catccos_b200_init_local.argtypes = [i32, ctypes.POINTER(i32)]
    L.catccos_b200_set_rank.argtypes = [i32]
    L.catccos_b200_finalize.argtypes = []
    L.catccos_b200_symm_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    L.catccos_b200_symm_free.argtypes = [vp]
    L.catccos_b200_symm_bytes_needed.argtypes = [tp, i32]
    L.catccos_b200_symm_bytes_needed.restype = sz
    L.catccos_b200_mx_quant_allgather.argtypes = [vp, vp, vp, vp, vp, tp, u32]
    L.catccos_b200_fp8_mx_allgather_matmul.argtypes = [vp, vp, vp, vp, vp, vp, vp, tp, u32]
    L.catccos_b200_fp4_mx_allgather_matmul.argtypes = [vp, vp, vp, vp, vp, vp, vp, tp, u32]
    L.catccos_b200_mx_quant_allgather_matmul.argtypes = [vp, vp, vp, vp, vp, vp, tp, u32]
    L.catccos_b200_mx_quant.argtypes = [vp, vp, u32, u32, vp, vp]
    L.catccos_b200_mx_quant_fp4.argtypes = [vp, vp, u32, u32, vp, vp]
    L.catccos_b200_mx_gemm.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, u32]
    L.catccos_b200_mx_gemm_quant_out.argtypes = [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]
    L.catccos_b200_packed_row_bytes.argtypes = [u32]
    L.catccos_b200_packed_row_bytes.restype = sz
    L.catccos_b200_mx_quant_scatter_packed.argtypes = [vp, vp, vp, vp, u32, u32, u32]
    L.catccos_b200_mxfp8_matmul_reduce_scatter.argtypes = [vp, vp, vp, vp, vp, vp, vp, tp, u32]
    L.catccos_b200_mx_quant_matmul_static.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32]
    L.catccos_b200_last_status.argtypes = [ctypes.POINTER(u32)]
    L.catccos_b200_mx_quant_matmul_static_status.argtypes = [ctypes.POINTER(u32)]
    L.catccos_b200_set_option.argtypes = [ctypes.c_char_p, i64]
    L.catccos_b200_launch_count.argtypes = []
    L.catccos_b200_launch_count.restype = ctypes.c_uint64
    for name in EXPORTS:
        if name not in ("catccos_b200_symm_bytes_needed", "catccos_b200_launch_count", "catccos_b200_packed_row_bytes"):
            getattr(L, name).restype = i32
    if TRACE:
        L.catccos_b200_trace_arm.argtypes = []
        L.catccos_b200_trace_arm.restype = i32
        L.catccos_b200_trace_read.argtypes = [ctypes.POINTER(ctypes.c_uint64), u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]
        L.catccos_b200_trace_read.restype = i32
    _lib = L
    return L


def _check(fn: str, code: int) -> None:
    if code != 0:
        raise CatccosError(fn, code)


def _stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def make_tiling(m: int, k: int, n: int, world: int) -> Tiling:
    """The reference drivers' default tile fields (main.cpp:105-118), with the problem shape filled in."""
    return Tiling(m=m, k=k, n=n, m0=128, k0=256, n0=256, commTileM=64, commInterval=3, commNpuSplit=2,
                  commDataSplit=16, commBlockM=64, rankSize=world, topK=1)


# ---------------------------------------------------------------------------------------------
# set-up
# ---------------------------------------------------------------------------------------------
def init(rank: int, world: int, device: int, ip_port: str | None) -> None:
    _check("catccos_b200_init", load().catccos_b200_init(rank, world, device, ip_port.encode() if ip_port else None))
    # tuning runs: CATCCOS_B200_OPTS="key=value,key=value" sets library options (test hooks included) on every rank
    for kv in filter(None, os.environ.get("CATCCOS_B200_OPTS", "").split(",")):
        key, value = kv.split("=", 1)
        set_option(key.strip(), int(value))


def init_local(world: int, devices) -> None:
    arr = (ctypes.c_int * world)(*devices)
    _check("catccos_b200_init_local", load().catccos_b200_init_local(world, arr))


def set_rank(rank: int) -> None:
    _check("catccos_b200_set_rank", load().catccos_b200_set_rank(rank))


def finalize() -> None:
    _check("catccos_b200_finalize", load().catccos_b200_finalize())


def symm_alloc(nbytes: int) -> int:
    p = ctypes.c_void_p()
    _check("catccos_b200_symm_alloc", load().catccos_b200_symm_alloc(nbytes, ctypes.byref(p)))
    return p.value


class _DeviceSpan:
    """A raw device address range in the form torch.as_tensor understands."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def symm_tensor(ptr: int, nbytes: int, offset: int = 0):
    """A uint8 torch view of [ptr + offset, ptr + offset + nbytes) inside a buffer from symm_alloc (no copy)."""
    import torch

    return torch.as_tensor(_DeviceSpan(ptr + offset, nbytes), device="cuda")


def symm_free(ptr: int) -> None:
    _check("catccos_b200_symm_free", load().catccos_b200_symm_free(ptr))


def symm_bytes_needed(t: Tiling, quant_op) -> int:
    """quant_op: False / 0 = AllGather-Matmul, True / 1 = quantise + AllGather, 2 = Matmul + ReduceScatter."""
    return int(load().catccos_b200_symm_bytes_needed(ctypes.byref(t), int(quant_op)))


def set_option(key: str, value: int) -> None:
    _check("catccos_b200_set_option", load().catccos_b200_set_option(key.encode(), value))


def last_status():
    out = (ctypes.c_uint32 * 4)()
    code = load().catccos_b200_last_status(out)
    return code, tuple(int(v) for v in out)


def static_status():
    """The wait record of the allocation-free entry point's last call on the current device."""
    out = (ctypes.c_uint32 * 4)()
    code = load().catccos_b200_mx_quant_matmul_static_status(out)
    return code, tuple(int(v) for v in out)


def launch_count() -> int:
    return int(load().catccos_b200_launch_count())


def trace_arm() -> None:
    """Trace build only: the next GEMM launch of the acting rank records its device-side timeline."""
    _check("catccos_b200_trace_arm", load().catccos_b200_trace_arm())


def trace_read():
    """Trace build only: the armed launch's timeline as a numpy array [CTAs, slots] of uint64."""
    import numpy as np

    buf = (ctypes.c_uint64 * (256 * 128))()
    grid, slots = ctypes.c_uint32(), ctypes.c_uint32()
    _check("catccos_b200_trace_read",
           load().catccos_b200_trace_read(buf, len(buf), ctypes.byref(grid), ctypes.byref(slots)))
    return np.frombuffer(buf, dtype=np.uint64, count=grid.value * slots.value).reshape(grid.value, slots.value).copy()


# ---------------------------------------------------------------------------------------------
# operators on torch CUDA tensors
# ---------------------------------------------------------------------------------------------
def mx_quant(x_bf16):
    """bf16 [rows, K] -> (codes uint8 [rows, K], scales uint8 [rows, K/32]); no communication."""
    import torch

    rows, k = x_bf16.shape
    assert x_bf16.is_cuda and x_bf16.is_contiguous() and x_bf16.element_size() == 2
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x_bf16.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=x_bf16.device)
    _check("catccos_b200_mx_quant",
           load().catccos_b200_mx_quant(_stream(), x_bf16.data_ptr(), rows, k, codes.data_ptr(), scales.data_ptr()))
    return codes, scales


def mx_quant_fp4(x_bf16):
    """bf16 [rows, K] -> (packed E2M1 codes uint8 [rows, K/2], scales uint8 [rows, K/32]); no communication."""
    import torch

    rows, k = x_bf16.shape
    assert x_bf16.is_cuda and x_bf16.is_contiguous() and x_bf16.element_size() == 2
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x_bf16.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=x_bf16.device)
    _check("catccos_b200_mx_quant_fp4",
           load().catccos_b200_mx_quant_fp4(_stream(), x_bf16.data_ptr(), rows, k, packed.data_ptr(), scales.data_ptr()))
    return packed, scales


def mx_gemm(a_codes, a_scales, b, b_scales, out=None, out_dtype=None):
    """c [M, N] = dequant(a)[M, K] x dequant(b [K, N])."""
    import torch

    m, k = a_codes.shape
    n = b_scales.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or torch.bfloat16, device=a_codes.device)
    _check("catccos_b200_mx_gemm",
           load().catccos_b200_mx_gemm(_stream(), a_codes.data_ptr(), a_scales.data_ptr(), b.data_ptr(),
                                       b_scales.data_ptr(), out.data_ptr(), m, n, k))
    return out


def mx_gemm_quant_out(a_codes, a_scales, b, b_scales):
    """The GEMM whose epilogue MX-quantises its output: (codes uint8 [M, N], scales uint8 [M, N/32])."""
    import torch

    m, k = a_codes.shape
    n = b_scales.shape[1]
    codes = torch.empty((m, n), dtype=torch.uint8, device=a_codes.device)
    scales = torch.empty((m, n // 32), dtype=torch.uint8, device=a_codes.device)
    _check("catccos_b200_mx_gemm_quant_out",
           load().catccos_b200_mx_gemm_quant_out(_stream(), a_codes.data_ptr(), a_scales.data_ptr(), b.data_ptr(),
                                                 b_scales.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, n, k))
    return codes, scales


def packed_row_bytes(n: int) -> int:
    return int(load().catccos_b200_packed_row_bytes(n))


def mx_quant_scatter_packed(x_bf16, expanded_row_idx, packed_out, top_k: int) -> None:
    """Quantises every token (row of x) once and writes its packed row to each of its top_k destination rows."""
    tokens, n = x_bf16.shape
    _check("catccos_b200_mx_quant_scatter_packed",
           load().catccos_b200_mx_quant_scatter_packed(_stream(), x_bf16.data_ptr(), expanded_row_idx.data_ptr(),
                                                       packed_out.data_ptr(), tokens, n, top_k))


def mxfp8_matmul_reduce_scatter(a_codes, a_scales, b, b_scales, d, symm: int, world: int) -> None:
    """d [m / world, n] = this rank's row chunk of the sum over ranks of dequant(a) x dequant(b); m is the whole M."""
    m, k = a_codes.shape
    n = b_scales.shape[1]
    t = make_tiling(m, k, n, world)
    _check("catccos_b200_mxfp8_matmul_reduce_scatter",
           load().catccos_b200_mxfp8_matmul_reduce_scatter(_stream(), a_codes.data_ptr(), b.data_ptr(), a_scales.data_ptr(),
                                                           b_scales.data_ptr(), d.data_ptr(), symm, ctypes.byref(t), 0))


def mx_quant_matmul_static(a_bf16, b, b_scales, c) -> None:
    """The allocation-free single-GPU fused call (scratch is the library's built-in device array)."""
    m, k = a_bf16.shape
    n = b_scales.shape[1]
    _check("catccos_b200_mx_quant_matmul_static",
           load().catccos_b200_mx_quant_matmul_static(_stream(), a_bf16.data_ptr(), b.data_ptr(), b_scales.data_ptr(),
                                                      c.data_ptr(), m, n, k))


def mx_quant_allgather(x_bf16, out_codes, out_scales, symm: int, world: int) -> None:
    m, k = x_bf16.shape
    t = make_tiling(m, 1, k, world)  # the quantised axis is `n` for this operator
    _check("catccos_b200_mx_quant_allgather",
           load().catccos_b200_mx_quant_allgather(_stream(), x_bf16.data_ptr(), out_codes.data_ptr(),
                                                  out_scales.data_ptr(), symm, ctypes.byref(t), 0))


def mx_quant_allgather_matmul(a_bf16, b, b_scales, c, symm: int, world: int) -> None:
    m, k = a_bf16.shape
    n = b_scales.shape[1]
    t = make_tiling(m, k, n, world)
    _check("catccos_b200_mx_quant_allgather_matmul",
           load().catccos_b200_mx_quant_allgather_matmul(_stream(), a_bf16.data_ptr(), b.data_ptr(),
                                                         b_scales.data_ptr(), c.data_ptr(), symm, ctypes.byref(t), 0))


def fp8_mx_allgather_matmul(a_codes, a_scales, b, b_scales, c, symm: int, world: int) -> None:
    m, k = a_codes.shape
    n = b_scales.shape[1]
    t = make_tiling(m, k, n, world)
    _check("catccos_b200_fp8_mx_allgather_matmul",
           load().catccos_b200_fp8_mx_allgather_matmul(_stream(), a_codes.data_ptr(), b.data_ptr(),
                                                       a_scales.data_ptr(), b_scales.data_ptr(), c.data_ptr(), symm,
                                                       ctypes.byref(t), 0))


def fp4_mx_allgather_matmul(a_packed, a_scales, b_packed, b_scales, c, symm: int, world: int) -> None:
    """The FP4 operator: a packed E2M1 [m, k/2], b packed E2M1 [k, n/2]."""
    m, k = a_packed.shape[0], a_packed.shape[1] * 2
    n = b_scales.shape[1]
    t = make_tiling(m, k, n, world)
    _check("catccos_b200_fp4_mx_allgather_matmul",
           load().catccos_b200_fp4_mx_allgather_matmul(_stream(), a_packed.data_ptr(), b_packed.data_ptr(),
                                                       a_scales.data_ptr(), b_scales.data_ptr(), c.data_ptr(), symm,
                                                       ctypes.byref(t), 0))
