"""The C-ABI library loads and exports every symbol the header declares (no compute
calls: this runs without a GPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "peerkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from peerkv_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"libpeerkv.so does not export {n}"
    assert sorted(_lib.EXPORTS) == names, "the ctypes binding and the header list different symbols"


def test_library_reports_version_and_errors_without_a_gpu():
    from peerkv_b200 import _lib
    L = _lib.lib()
    assert L.pkv_abi_version() == 1
    # argument errors are reported before any CUDA call
    rc = L.pkv_merge_partials(0, None, 0, None, 0, 1, 1, 128, None, 4, None, None)
    assert rc == -1 and b"null" in L.pkv_last_error()
    rc = L.pkv_shard_create(None, 0, 1, 1)
    assert rc == -1


def test_structs_match_header_layout():
    from peerkv_b200 import _lib
    assert ctypes.sizeof(_lib.KvView) == 4 * 8 + 4 * 4 + 4 * 8
    assert ctypes.sizeof(_lib.DecodeArgs) == 8 + 16 + ctypes.sizeof(_lib.KvView) + 8 + 8 + 8 + 8


def test_no_cpu_fallback():
    import pytest
    import torch
    from peerkv_b200 import PeerKVError, ops
    q = torch.randn(1, 32, 128).half()
    K = torch.randn(1, 8, 10, 128).half()
    with pytest.raises(PeerKVError):
        ops.decode_contiguous(q, K, K)
