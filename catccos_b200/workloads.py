"""Seeded synthetic inputs for the five benchmark configurations of the MXFP8 path.

Every generator is a pure function of (config, world, rank, seed) built on
``numpy.random.default_rng`` so that tests, the benchmark and the CPU baseline see the same
bytes.  Activations are returned as bf16 bit patterns (uint16, round-to-nearest-even from
fp32), which is what the quantise kernel consumes.

Shapes follow the operator convention of the reference: for the matmul operator
``m = M_local, k = K, n = N_local`` (examples/ascend950_fp8_mx_allgather_matmul/main.cpp:105-118);
the quantise operator calls the quantised axis ``n`` (mx_quant_allgather_host.h:30-44).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Config:
    name: str
    m_local: int
    k: int
    n_local: int  # 0 for the standalone quantise + allgather
    worlds: tuple
    dist: str  # "normal" | "student_t3_outlier"
    note: str


CONFIGS = {
    "c1_golden": Config("c1_golden", 256, 1024, 1024, (2,), "normal", "2-rank CPU-golden case"),
    "c2_quant_ag": Config("c2_quant_ag", 4096, 7168, 0, (1, 2, 4, 8), "normal", "standalone MX-quant + AllGather"),
    "c3_prefill": Config("c3_prefill", 1024, 7168, 2304, (1, 2, 4, 8), "normal", "TP prefill AllGather-Matmul"),
    "c4_outlier": Config("c4_outlier", 4096, 5120, 3456, (2, 4, 8), "student_t3_outlier", "outlier stress"),
    "c5_decode": Config("c5_decode", 16, 7168, 4096, (2, 4, 8), "normal", "decode, latency bound"),
}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern with round-to-nearest-even (inputs are finite)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def outlier_channels(k: int, seed: int) -> np.ndarray:
    """The fixed set of ceil(0.1 % of K) channels that are scaled by 100 (same on all ranks)."""
    n = int(np.ceil(0.001 * k))
    return np.sort(np.random.default_rng(seed * 1000 + 999).choice(k, size=n, replace=False))


def activation_bits(cfg: Config, rank: int, seed: int = 0, rows: int | None = None) -> np.ndarray:
    """A_r as bf16 bits [M_local, K] for one rank (``rows`` truncates for sampled checks)."""
    m = cfg.m_local if rows is None else rows
    rng = np.random.default_rng(seed * 1000 + rank)
    if cfg.dist == "normal":
        x = rng.standard_normal((m, cfg.k), dtype=np.float32)
    elif cfg.dist == "student_t3_outlier":
        x = rng.standard_t(3.0, size=(m, cfg.k)).astype(np.float32)
        x[:, outlier_channels(cfg.k, seed)] *= np.float32(100.0)
    else:
        raise ValueError(cfg.dist)
    return f32_to_bf16_bits(x)


def weight_bits(cfg: Config, rank: int, seed: int = 0) -> np.ndarray:
    """B_r ~ N(0, 0.02) as bf16 bits [K, N_local]."""
    rng = np.random.default_rng(seed * 1000 + 500 + rank)
    w = rng.standard_normal((cfg.k, cfg.n_local), dtype=np.float32) * np.float32(0.02)
    return f32_to_bf16_bits(w)


def gemm_flops(cfg: Config, world: int) -> float:
    """Algorithmic FLOP per GPU: 2 * (world * M_local) * K * N_local."""
    return 2.0 * world * cfg.m_local * cfg.k * cfg.n_local


def quant_ag_ingress_bytes(cfg: Config, world: int) -> float:
    """NVLink ingress bytes per GPU: (world - 1) * M_local * (K + K / 32)."""
    return float((world - 1) * cfg.m_local * (cfg.k + cfg.k // 32))


def quant_ag_hbm_bytes(cfg: Config, world: int) -> float:
    """HBM bytes per GPU: read bf16 A_r once, write the gathered codes and scales once."""
    return float(cfg.m_local * cfg.k * 2 + world * cfg.m_local * (cfg.k + cfg.k // 32))
