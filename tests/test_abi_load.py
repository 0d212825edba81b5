"""CPU: the C-ABI library loads and exports every symbol include/spyb.h declares; host-only calls behave."""
import ctypes as C
import os

import pytest

from spy_b200 import backend


def test_library_exports_every_declared_symbol():
    if not os.path.exists(backend.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    l = C.CDLL(backend.LIB_PATH)
    declared = backend.exported_symbols()
    assert len(declared) >= 20
    missing = [s for s in declared if not hasattr(l, s)]
    assert not missing, f"declared in spyb.h but not exported: {missing}"


def test_is_support_matches_the_operator_table():
    l = backend.lib()
    for name, op in backend.OP.items():
        assert l.spyb_is_support(op) == 1, name
    for op in (6, 7, 12, 14, 15, 16, 19, 21, 22, 24, 25, 28):   # MaskedCopy .. Quantize: not on the LLaMa path
        assert l.spyb_is_support(op) == 0


def test_create_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(backend.SpybError):
        backend.B200Backend(0)


def test_shared_memory_ledger_is_kept_per_device_and_kernel():
    """cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (device, kernel) pair: the library's record of what it
    has already raised must be kept per pair, or the second device of a process never gets the attribute set."""
    assert backend.lib().spyb_selftest_host() == 0
