"""Host-side checks that need no GPU: the library loads, exports what the header declares, and
rejects bad arguments with error codes before touching the device."""
import ctypes
import os
import re

import pytest

from sparseattention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(hsa_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    assert names == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_arch():
    lib = _lib.load()
    assert lib.hsa_version() >= 100
    assert lib.hsa_compiled_arch() == 100


def test_span_input_rows():
    lib = _lib.load()
    for n, want in ((2, 1), (4, 3), (12, 10), (16, 15), (4096, 4095), (7, 4)):
        assert lib.hsa_span_input_y_rows(n) == want


def _v(ptr=0x1000):
    return _lib.HsaView(ptr, 0, 0)


def test_bad_arguments_return_codes():
    lib = _lib.load()
    assert lib.hsa_topology_build(3, 1, None, None, None, None) == -1
    assert b"power of two" in lib.hsa_last_error()
    assert lib.hsa_topology_build(0, 1, None, None, None, None) == -1
    # span attention: N not a power of two, null pointers, bad dtype, bad algo
    assert lib.hsa_span_attn_fwd(_v(), _v(), _v(), _v(), None, 1, 12, 1, 16, 1, 1, 0, 0, None) == -1
    assert lib.hsa_span_attn_fwd(_v(0), _v(), _v(), _v(), None, 1, 16, 1, 16, 1, 1, 0, 0, None) == -1
    assert lib.hsa_span_attn_fwd(_v(), _v(), _v(), _v(), None, 1, 16, 1, 16, 1, 1, 7, 0, None) == -3
    assert lib.hsa_span_attn_fwd(_v(), _v(), _v(), _v(), None, 1, 16, 1, 16, 1, 1, 0, 9, None) == -1   # unknown algo
    assert lib.hsa_span_attn_fwd(_v(), _v(), _v(), _v(), None, 1, 16, 1, 16, -1, 1, 0, 0, None) == -1
    assert lib.hsa_span_attn_fwd(_v(), _v(), _v(), _v(), None, 1, 16, 1, 100000, 1, 1, 0, 0, None) == -1
    # parent op: zero parents
    assert lib.hsa_parent_nodes_fwd(_v(), _v(), _v(), _v(), _v(), _v(), None, 1, 0, 1, 16, 0, None) == -1
    # backward: workspace too small
    need = lib.hsa_span_attn_bwd_workspace_bytes(2, 16, 3, 16, 2, 1, 0, 0)
    assert need >= 2 * 16 * 3 * 4
    rc = lib.hsa_span_attn_bwd(_v(), _v(), _v(), _v(), ctypes.c_void_p(0x1000), _v(), _v(), _v(), _v(),
                               ctypes.c_void_p(0x1000), 8, 2, 16, 3, 16, 2, 1, 0, 0, None)
    assert rc == -4 and b"workspace" in lib.hsa_last_error()


def test_ops_refuse_cpu_tensors():
    import torch
    from sparseattention_b200 import build_parent_nodes, hierarchical_attention
    q = torch.zeros(1, 4, 1, 8)
    with pytest.raises(_lib.HsaError):
        build_parent_nodes(q, q, q, torch.zeros(1, 8, 1, 8), torch.zeros(1, 8, 1, 8))
    with pytest.raises(_lib.HsaError):
        hierarchical_attention(q, torch.zeros(1, 7, 1, 8), torch.zeros(1, 7, 1, 8),
                               torch.tensor([[1, 5], [0, 5], [3, 4], [2, 4]], dtype=torch.int32), None, None, 1)
