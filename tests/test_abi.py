"""CPU-side checks of the drop-in boundary: the shared library loads, exports every symbol
include/sfbert_b200.h declares, and rejects bad arguments before touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    if not os.path.exists(os.path.join(ge.PKG_DIR, "libsfbert_b200.so")):
        ge.build()
    path = os.path.join(ge.PKG_DIR, "libsfbert_b200.so")
    lib = C.CDLL(path)
    lib.sfb_last_error.restype = C.c_char_p
    return lib


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sfbert_b200.h")).read()
    return sorted(set(re.findall(r"\b(sfb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), n


def test_package_symbol_list_matches_header():
    import __graft_entry__ as ge
    src = open(os.path.join(ge.PKG_DIR, "__init__.py")).read()
    for n in _declared_symbols():
        assert '"%s"' % n in src, n


def test_version_and_magic(lib, oracle):
    assert lib.sfb_version() >= 100
    for d in (1, 2, 3, 4, 5, 6, 7, 8, 12, 100):
        m, s = C.c_uint32(0), C.c_uint32(0)
        lib.sfb_magicu64(C.c_uint32(d), C.byref(m), C.byref(s))
        assert (m.value, s.value) == oracle.magicu64(d)


def test_bad_arguments_are_rejected_with_a_message(lib):
    vp = C.c_void_p
    one = vp(16)  # never dereferenced: the checks come first
    u = C.c_uint32
    # unsupported block size (the reference silently does nothing, blocksparse.h:448)
    rc = lib.sfb_bst_sgemm_nt(None, one, one, one, one, 0, 1, u(16), u(4), u(1), u(2), u(2), u(1), u(64), u(1), u(4))
    assert rc != 0 and b"block_size" in lib.sfb_last_error()
    # NULL operand
    rc = lib.sfb_bst_sgemm_nt(None, None, one, one, one, 0, 1, u(32), u(4), u(1), u(2), u(2), u(1), u(64), u(1), u(4))
    assert rc != 0 and b"NULL" in lib.sfb_last_error()
    # lut_heads that is neither 1 nor H
    rc = lib.sfb_fused_attention(None, one, one, one, one, one, None, 0, u(32), u(4), u(1), u(2), u(4), u(64), u(3), u(4),
                                 u(1), C.c_float(0.125), u(2))
    assert rc != 0 and b"lut_heads" in lib.sfb_last_error()
    # an op that is neither NN_OP nor TN_OP
    rc = lib.sfb_bst_sgemm_xn(None, one, one, one, one, 1, 0, u(32), u(4), u(1), u(2), u(2), u(1), u(64), u(1), u(6), u(0),
                              u(1), u(0), u(2))
    assert rc != 0 and b"op" in lib.sfb_last_error()
    rc = lib.sfb_mask_pack(None, one, u(1), u(4), u(48), 0, u(0), one, one)
    assert rc != 0 and b"block_size" in lib.sfb_last_error()
    rc = lib.sfb_bias_residual_layernorm(None, one, None, None, None, one, None, None, one, one, u(4), u(100), 0)
    assert rc != 0 and b"multiple of 8" in lib.sfb_last_error()
