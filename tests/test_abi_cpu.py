"""CPU checks of the C-ABI library: it loads, exports every declared symbol, and its pure-host
entry points behave.  No compute call is made here."""
import ctypes as C

import pytest

from hf2q_b200 import _lib, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _lib.declared_symbols()
    assert len(declared) >= 20
    assert set(declared) == set(_lib.SIGNATURES), "header and ctypes table disagree"
    for name in declared:
        assert hasattr(lib, name), name


def test_geometry_matches_ggml_type_rs(lib):
    # ggml_type.rs:60-127
    for t, (be, bb) in {2: (32, 18), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210),
                        3: (32, 20), 6: (32, 22), 7: (32, 24), 20: (32, 18)}.items():
        e, b = C.c_uint32(), C.c_uint32()
        assert lib.hf2q_cuda_block_geometry(t, C.byref(e), C.byref(b)) == 0
        assert (e.value, b.value) == (be, bb)
        out = C.c_uint64()
        assert lib.hf2q_cuda_row_bytes(t, 4096, C.byref(out)) == 0
        assert out.value == 4096 // be * bb
    out = C.c_uint64()
    assert lib.hf2q_cuda_row_bytes(12, 4096 + 32, C.byref(out)) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_row_bytes(10, 4096, C.byref(out)) == _lib.ERR_UNSUPPORTED_TYPE   # Q2_K: not on this path
    assert lib.hf2q_cuda_expert_stride(13, 512, 2048, C.byref(out)) == 0 and out.value == 720896


def test_strerror_and_version(lib):
    assert lib.hf2q_cuda_strerror(0) == b"ok"
    assert b"unsupported" in lib.hf2q_cuda_strerror(_lib.ERR_UNSUPPORTED_TYPE)
    assert b"sm_100a" in lib.hf2q_cuda_version()


def test_ctx_create_without_a_gpu_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.hf2q_cuda_ctx_create(0, C.byref(h)) == _lib.ERR_NO_DEVICE
    import hf2q_b200
    with pytest.raises(hf2q_b200.Hf2qError):
        hf2q_b200.GpuContext(0)


def test_null_context_is_rejected(lib):
    assert lib.hf2q_cuda_qmatmul(None, None, None, 0, None, None, 1, 1, 256, 12, None, 0) == _lib.ERR_INVALID_ARGUMENT
    assert lib.hf2q_cuda_ctx_destroy(None) == _lib.ERR_INVALID_ARGUMENT
