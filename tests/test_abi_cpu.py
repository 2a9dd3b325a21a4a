"""The C-ABI library loads without a GPU and exports every symbol the header declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "qm_attention.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(qm_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_functions()
    for needed in ("qm_decode_append_rope", "qm_decode_attention", "qm_prefill_append_rope_varlen",
                   "qm_prefill_attention_varlen", "qm_attention_combine", "qm_kv_pool_create", "qm_kv_pool_reset"):
        assert needed in names


def test_library_builds_and_exports_every_declared_symbol(qm):
    lib = qm.load_library()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in qm_attention.h but not exported"
        assert name in qm.ABI, f"{name} has no ctypes prototype"
    assert sorted(qm.ABI) == declared_functions()


def test_every_entry_point_cites_the_reference():
    text = HEADER.read_text()
    # each launcher-replacing entry point names the reference file:line it stands in for
    for name in ("qm_decode_append_rope", "qm_decode_attention", "qm_prefill_append_rope_varlen",
                 "qm_prefill_attention_varlen", "qm_kv_pool_reset", "qm_rope_table_fill", "qm_validate_b200_device"):
        head = text[:text.index(name + "(")]
        comment = head[head.rindex("/*"):]
        assert re.search(r"17\.cu:\d+", comment), name


def test_argument_errors_are_reported_before_any_launch(qm):
    lib = qm.load_library()
    # null pool / null pointers: status codes, no CUDA call needed
    assert lib.qm_kv_pool_reset(None, None) == qm.QM_EINVAL
    assert b"null" in lib.qm_last_error_string()
    assert lib.qm_decode_attention(None, 0, None, None, None, 1, 1, 16, None, None, 0, None) == qm.QM_EINVAL
    assert lib.qm_attention_combine(None, 1, 1, None, None) == qm.QM_EINVAL
    assert lib.qm_kv_pool_create(0, 1, 8, ctypes.byref(ctypes.c_void_p())) == qm.QM_EINVAL
    assert lib.qm_kv_pool_destroy(None) == qm.QM_OK
    assert lib.qm_decode_workspace_bytes(64, 8) > 0


def test_missing_library_fails_loudly(qm, tmp_path):
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        qm.load_library(tmp_path / "absent.so")
