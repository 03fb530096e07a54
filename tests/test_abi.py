"""The shared library loads, exports every symbol include/redrafter_b200.h declares, and the ctypes
signature table agrees with the header (parameter count and pointer/int/float kinds).  No compute
calls: runs without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "redrafter_b200.h")


def _declarations():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    decls = {}
    for m in re.finditer(r"RD_API\s+([\w\s\*]+?)\b(rd_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        plist = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
        decls[name] = (ret, plist)
    return decls


def _kind(param: str) -> str:
    if "*" in param:
        return "p"
    if param.startswith("float"):
        return "f"
    if param.startswith("int64_t"):
        return "l"
    if param.startswith("int"):
        return "i"
    raise AssertionError(param)


def test_header_declares_the_expected_entry_points():
    decls = _declarations()
    assert len(decls) >= 24
    for name in ("rd_tree_pack", "rd_gemm_bf16_tc", "rd_attention", "rd_accept_commit_greedy", "rd_vocab_topk"):
        assert name in decls


def test_library_exports_every_declared_symbol():
    from recurrent_drafting import _lib

    assert os.path.exists(_lib.LIB_PATH), "build the library first: python ml-recurrent-drafter_b200/build.py"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declarations():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_matches_header():
    from recurrent_drafting import _lib

    decls = _declarations()
    assert set(decls) == set(_lib.SIGNATURES), set(decls) ^ set(_lib.SIGNATURES)
    kinds = {ctypes.c_void_p: "p", ctypes.c_int: "i", ctypes.c_int64: "l", ctypes.c_float: "f"}
    for name, (ret, params) in decls.items():
        res, args = _lib.SIGNATURES[name]
        assert len(args) == len(params), f"{name}: header has {len(params)} parameters, table has {len(args)}"
        for i, (a, p) in enumerate(zip(args, params)):
            assert kinds[a] == _kind(p), f"{name} parameter {i} ({p})"


def test_host_only_calls():
    from recurrent_drafting import _lib

    lib = _lib.load()
    assert lib.rd_abi_version() == 1
    assert lib.rd_strerror(0) == b"ok"
    assert b"dtype" in lib.rd_strerror(-2)
    # argument validation happens on the host before any launch
    assert lib.rd_tree_pack(None, 1, 1, 1, None, None, None, None, None, None, None, None, None, None, None, None, 1, None, None) == -1
    assert lib.rd_gemm_plan_create(None, 0, 0, None, 0, 0, 0) is None


def test_cpu_tensor_is_rejected():
    import torch

    from recurrent_drafting import _lib

    with pytest.raises(_lib.RedrafterError):
        _lib.ptr(torch.zeros(1))
