"""CPU tests of the drop-in boundary: the shared library loads without a GPU and exports every
symbol the header declares; argument checks that need no device."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "catccos_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(catccos_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(capi):
    lib = capi.load()
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(capi.EXPORTS) == names


def test_tiling_struct_matches_reference_layout(capi):
    assert ctypes.sizeof(capi.Tiling) == 17 * 4
    assert [f[0] for f in capi.Tiling._fields_][:3] == ["m", "k", "n"]
    assert capi.Tiling.rankSize.offset == 13 * 4


def test_symm_bytes_needed(capi):
    t = capi.make_tiling(4096, 1, 7168, 8)
    need = capi.symm_bytes_needed(t, True)
    data = 8 * 4096 * (7168 + 224)
    assert 2 * data < need < 2 * data + (2 << 20)
    assert need < 1004 * 1024 * 1024  # fits the reference's SHMEM_BUFF_BYTES (utils/info.h:36)


def test_set_option_rejects_unknown(capi):
    assert capi.load().catccos_b200_set_option(b"no_such_option", 1) == -1
    assert capi.load().catccos_b200_set_option(b"block_n", 192) == -1
    assert capi.load().catccos_b200_set_option(b"block_n", 0) == 0
    for key, bad in ((b"tiny_block_rule", 2), (b"c_dtype", 2), (b"a_dtype", 3), (b"b_dtype", 3)):  # the public keys
        assert capi.load().catccos_b200_set_option(key, 0) == 0
        assert capi.load().catccos_b200_set_option(key, bad) == -1
    assert capi.load().catccos_b200_set_option(b"timeout_ms", 2000) == 0


def test_misaligned_scale_pointers_are_refused_before_any_launch(capi):
    # With k % 128 == 0 a row's scale bytes are written four at a time: a scales pointer carved from a byte
    # pool at an odd offset must come back as EINVAL, not as a misaligned-address fault on the device.
    # The checks run before the library touches CUDA, so made-up addresses do.
    L = capi.load()
    assert L.catccos_b200_mx_quant(None, 0x10000, 8, 128, 0x20000, 0x30001) == -1
    assert L.catccos_b200_mx_quant(None, 0x10000, 8, 128, 0x20008, 0x30000) == -1  # codes not 16-byte aligned
    t = capi.make_tiling(8, 1, 128, 1)
    assert L.catccos_b200_mx_quant_allgather(None, 0x10000, 0x20000, 0x30002, None, ctypes.byref(t), 0) in (-1, -3)
    st = (ctypes.c_uint32 * 4)()
    # the allocation-free entry point refuses bad pointers before it touches its shared array
    assert L.catccos_b200_mx_quant_matmul_static(None, 0x10008, 0x20000, 0x30000, 0x40000, 8, 16, 128) == -1
    assert st[0] == 0
