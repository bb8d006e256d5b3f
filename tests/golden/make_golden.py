"""Generates the golden fixtures in this directory by running the REFERENCE's own CPU golden
code on seeded inputs.  Run it where the reference checkout is available:

    GEN_DATA_QUANT_BACKEND=native python tests/golden/make_golden.py /path/to/reference

It imports examples/utils/gen_mx_quant_allgather_data.py (the quantiser the reference uses to
make golden files, with the round-to-nearest-even "native" backend, which is the device
kernel's rounding) and restates only the file-layout lines of
examples/utils/gen_data_fp8_mx_allgather_matmul.py:618-658 (scale reshapes, rank-order
concat, fp32 matmul).  The fixtures are small .npz files; tests compare the oracle and the
CUDA path against them bit for bit (codes, scales) or within tolerance (GEMM output).
"""
import os
import sys

os.environ["GEN_DATA_QUANT_BACKEND"] = "native"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: GEN_DATA_QUANT_BACKEND=native python tests/golden/make_golden.py /path/to/reference")
REF = sys.argv[1]
sys.path.insert(0, os.path.join(REF, "examples", "utils"))
import gen_mx_quant_allgather_data as ref  # noqa: E402

assert ref._QUANT_BACKEND == "native"


def bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (r >> np.uint32(16)).astype(np.uint16)


def bits_f32(b):
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def ref_quant_rows(bits, fmt="E4M3"):
    """Reference quantiser on bf16 inputs -> (codes u8 [M,K], scale bytes u8 [M,K/32])."""
    x = torch.from_numpy(bits_f32(bits).copy())
    q, scale, _ = ref._quantize_axis_last_fp8(x, fmt)
    codes = q.view(torch.uint8).numpy().copy()
    sb = scale.to(torch.float8_e8m0fnu).view(torch.uint8).numpy().copy()
    return codes, sb[:, : bits.shape[1] // 32]


def save(name, **arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(name, {k: (v.shape, str(v.dtype)) for k, v in arrays.items()}, os.path.getsize(path), "bytes")


def main():
    # 1. N(0,1) activations
    rng = np.random.default_rng(20240)
    x = bf16_bits(rng.standard_normal((48, 256), dtype=np.float32))
    c, s = ref_quant_rows(x)
    save("quant_normal.npz", x=x, codes=c, scales=s)

    # 2. Student-t(3) with one channel in 256 scaled by 100 (saturation / wide exponent spread)
    rng = np.random.default_rng(20241)
    xo = rng.standard_t(3.0, size=(32, 256)).astype(np.float32)
    xo[:, [17, 200]] *= np.float32(100.0)
    xo = bf16_bits(xo)
    c, s = ref_quant_rows(xo)
    assert ((c & 0x7F) == 0x7E).any(), "fixture must contain saturated codes"
    save("quant_outlier.npz", x=xo, codes=c, scales=s)

    # 3. edge sweep: one block per biased exponent 1..254 (amax = 1.5 * 2^(E-127)) with the
    #    other 31 elements spread down 40 binades (ties, subnormal codes, underflow to +-0),
    #    plus all-zero, negative-zero, bf16-subnormal and sub-1e-12 blocks.
    rng = np.random.default_rng(20242)
    blocks = []
    for E in range(1, 255):
        top = np.uint16((E << 7) | 0x40)
        b = np.empty(32, np.uint16)
        b[0] = top | (np.uint16(0x8000) if E % 3 == 0 else np.uint16(0))
        for i in range(1, 32):
            e = max(E - int(rng.integers(0, 40)), 0)
            b[i] = np.uint16((int(rng.integers(0, 2)) << 15) | (e << 7) | int(rng.integers(0, 128)))
        blocks.append(b)
    blocks.append(np.zeros(32, np.uint16))
    blocks.append(np.full(32, 0x8000, np.uint16))
    blocks.append(rng.integers(0, 128, 32).astype(np.uint16))  # bf16 subnormals only
    tiny = np.full(32, 0x2B8C, np.uint16)  # largest bf16 below 1e-12
    tiny[::2] |= 0x8000
    blocks.append(tiny)
    edge = np.full(32, 0x2B8D, np.uint16)  # smallest bf16 above 1e-12
    blocks.append(edge)
    # exact ties in the scaled domain: amax 448-ish block with k + 0.5 ulp patterns
    tie = bf16_bits(np.array([1.0, 1.0625, 1.1875, 1.3125, 0.0009765625 * 1.5, 2.0 ** -10, -(2.0 ** -10),
                              3.0 * 2.0 ** -11, 0.5625, 240.0, 232.0, 248.0, 17.0, 19.0, 21.0, 23.0] * 2,
                             dtype=np.float32))
    tie[15] = bf16_bits(np.array([256.0], np.float32))[0]
    blocks.append(tie)
    while len(blocks) % 4:
        blocks.append(np.zeros(32, np.uint16))
    xe = np.stack(blocks).reshape(-1, 128)
    c, s = ref_quant_rows(xe)
    save("quant_edges.npz", x=xe, codes=c, scales=s)

    # 4. small 2-rank AllGather-Matmul in the reference's file layouts
    rng = np.random.default_rng(20243)
    world, m, k, n = 2, 32, 256, 64
    a_bits = [bf16_bits(rng.standard_normal((m, k), dtype=np.float32)) for _ in range(world)]
    b_bits = bf16_bits(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02))
    a_deq, a_codes, a_scales = [], [], []
    for r in range(world):
        q, scale, deq = ref._quantize_fp8(torch.from_numpy(bits_f32(a_bits[r]).copy()), "E4M3", 1)
        a_codes.append(q.view(torch.uint8).numpy().copy())
        a_scales.append(scale.to(torch.float8_e8m0fnu).view(torch.uint8).numpy().copy())
        a_deq.append(deq)
    qb, sb, b_deq = ref._quantize_fp8(torch.from_numpy(bits_f32(b_bits).copy()), "E4M3", 0)
    sb = sb.to(torch.float8_e8m0fnu)
    sb = sb.reshape(sb.shape[0] // 2, 2, sb.shape[1]).permute(0, 2, 1).contiguous()  # [K/64, N, 2]
    golden = torch.matmul(torch.cat(a_deq, dim=0), b_deq).numpy()
    save(
        "agmm_small.npz",
        a_bits=np.stack(a_bits),
        b_bits=b_bits,
        a_codes=np.stack(a_codes),
        a_scales=np.stack(a_scales),
        b_codes=qb.view(torch.uint8).numpy().copy(),
        b_scales=sb.view(torch.uint8).numpy().copy(),
        golden=golden.astype(np.float32),
    )

    # 5. the E5M2 output type (MX_QUANT_DTYPE = 1: emax 15, max 57344) on the inputs of 1-3, and the same
    #    2-rank AllGather-Matmul with E5M2 activations (weights stay E4M3)
    e5 = {}
    for tag, xin in (("normal", x), ("outlier", xo), ("edges", xe)):
        c5, s5 = ref_quant_rows(xin, "E5M2")
        e5["x_" + tag], e5["codes_" + tag], e5["scales_" + tag] = xin, c5, s5
    a5_deq, a5_codes, a5_scales = [], [], []
    for r in range(world):
        q, scale, deq = ref._quantize_fp8(torch.from_numpy(bits_f32(a_bits[r]).copy()), "E5M2", 1)
        a5_codes.append(q.view(torch.uint8).numpy().copy())
        a5_scales.append(scale.to(torch.float8_e8m0fnu).view(torch.uint8).numpy().copy())
        a5_deq.append(deq)
    e5["agmm_a_codes"], e5["agmm_a_scales"] = np.stack(a5_codes), np.stack(a5_scales)
    e5["agmm_golden"] = torch.matmul(torch.cat(a5_deq, dim=0), b_deq).numpy().astype(np.float32)
    save("quant_e5m2.npz", **e5)

    # 6. the FP4 output type (E2M1: emax 2, max 6, two codes per byte), as gen_data_fp4_e2m1 builds its files:
    #    table rounding, nibble packing, E8M0 scale bytes.  Also on the dequantised tensor, which is what the
    #    reference feeds its kernel (the two rounding rules agree there).
    e4 = {}
    for tag, xin in (("normal", x), ("outlier", xo), ("edges", xe)):
        xf = torch.from_numpy(bits_f32(xin).copy())
        q, scale, deq = ref._quantize(xf, "E2M1", 1)
        _, idx = ref._quantize_to_fp4_lut(q, "E2M1")
        e4["x_" + tag] = xin
        e4["packed_" + tag] = ref._pack_fp4_nibbles(idx).numpy().copy()
        e4["scales_" + tag] = scale.to(torch.float8_e8m0fnu).view(torch.uint8).numpy().copy()[:, : xin.shape[1] // 32]
        e4["dequant_" + tag] = deq.numpy().astype(np.float32)
    save("quant_e2m1.npz", **e4)

    # 7. the same for E1M2 (emax 0, max 1.75), the other FP4 type of the generator
    e1 = {}
    for tag, xin in (("normal", x), ("edges", xe)):
        xf = torch.from_numpy(bits_f32(xin).copy())
        q, scale, deq = ref._quantize(xf, "E1M2", 1)
        _, idx = ref._quantize_to_fp4_lut(q, "E1M2")
        e1["x_" + tag] = xin
        e1["packed_" + tag] = ref._pack_fp4_nibbles(idx).numpy().copy()
        e1["scales_" + tag] = scale.to(torch.float8_e8m0fnu).view(torch.uint8).numpy().copy()[:, : xin.shape[1] // 32]
        e1["dequant_" + tag] = deq.numpy().astype(np.float32)
    save("quant_e1m2.npz", **e1)


if __name__ == "__main__":
    main()
