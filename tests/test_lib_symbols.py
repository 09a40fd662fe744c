"""The C-ABI library loads and exports every entry point include/dm_b200.h declares (no GPU needed: nothing is
launched), and the ctypes prototypes cover exactly the declared functions."""
import os
import re

from .conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "dm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(dm_[a-z0-9_]+)\s*\(", text))


def test_header_symbols_exported():
    import __graft_entry__ as entry
    entry.build()                                   # no-op when the in-tree library is current
    from delta_matching_b200 import _lib
    names = _declared()
    assert {"dm_fwd", "dm_delta", "dm_bwd", "dm_quant_qkv", "dm_quant_do", "dm_version"} <= names
    L = _lib.lib()
    for n in names:
        assert hasattr(L, n), n
    assert set(_lib.SIGNATURES) == names
    assert L.dm_version() >= 100
    assert L.dm_numerics() == b"sm100-mx"
    assert os.path.basename(_lib.loaded_library()).startswith("libdm_b200")


def test_argument_checks_without_gpu():
    """Shape validation happens before any CUDA call, so it can be exercised on a machine without a GPU."""
    from delta_matching_b200 import _lib
    L = _lib.lib()
    assert L.dm_quant_qkv_workspace_bytes(4, 4096, 8, 128) == 4 * 8 * 64 * 128 * 4
    assert L.dm_quant_qkv_workspace_bytes(0, 4096, 8, 128) == 0
    rc = L.dm_fwd(None, None, None, None, None, None, 1, 256, 2, 2, 96, 1, None, 0, 0, 0, None, None, None)
    assert rc == -1 and "head_dim" in _lib.last_error()
    rc = L.dm_delta(None, None, None, None, None, None, None, None, None, 1, 256, 3, 2, 128, 1, None, None, None)
    assert rc == -1 and "nheads" in _lib.last_error()
    rc = L.dm_fwd(None, None, None, None, None, None, 70000, 256, 1, 1, 128, 1, None, 0, 0, 0, None, None, None)
    assert rc == -1 and "65535" in _lib.last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from delta_matching_b200 import _lib
    import pytest
    monkeypatch.setenv("DM_SO", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="does not exist"):
        _lib.library_path()
