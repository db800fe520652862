"""The C-ABI library loads without a GPU and exports every function include/fa_b200.h declares;
argument errors are reported through status codes, not exceptions or crashes."""
import ctypes
import os
import re

import fa_b200_capi as capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"^\s*(?:const\s+char\*|int|size_t|void)\s+(fa_\w+)\s*\(", text, flags=re.M)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 17
    for n in names:
        assert hasattr(capi.lib, n), f"{n} missing from libfa_b200.so"
        assert n in capi.EXPORTS, f"{n} has no ctypes binding"
    assert set(capi.EXPORTS) == set(names)


def test_version_and_error_strings():
    assert b"sm_100a" in capi.lib.fa_version()
    assert capi.lib.fa_fwd(None) != 0
    assert b"null" in capi.lib.fa_last_error()


def test_struct_layouts_match_header_sizes():
    # natural alignment on LP64: the header's field order gives these sizes
    assert ctypes.sizeof(capi.FaTensor) == 32
    assert ctypes.sizeof(capi.FwdParams) % 8 == 0
    assert capi.FwdParams.stream.offset + 8 == ctypes.sizeof(capi.FwdParams)
    assert capi.BwdParams.alibi_stride_b.offset + 8 == ctypes.sizeof(capi.BwdParams) == 408


def test_argument_validation_needs_no_gpu():
    p = capi.FwdParams()
    p.dtype, p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv = 1, 1, 8, 8, 3, 2, 64, 64
    assert capi.lib.fa_fwd(p) == 3 and b"divisible" in capi.lib.fa_last_error()
    p.hq = 4
    p.d = 300
    assert capi.lib.fa_fwd(p) == 3
    p.d = 64
    p.dtype = 7
    assert capi.lib.fa_fwd(p) == 2
    p.dtype = 1
    assert capi.lib.fa_fwd(p) == 1 and b"q is null" in capi.lib.fa_last_error()
    p.q.ptr = 0x1004
    assert capi.lib.fa_fwd(p) == 4
    b = capi.BwdParams()
    b.dtype, b.b, b.sq, b.sk, b.hq, b.hkv, b.d, b.dv_dim = 0, 1, 8, 8, 2, 2, 60, 64
    assert capi.lib.fa_bwd(b) == 3


def test_split_planner_is_host_only():
    p = capi.FwdParams()
    p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv, p.dtype = 128, 1, 33024, 32, 8, 128, 128, 1
    p.seqused_k = 0x1000   # never dereferenced by the planner
    p.num_splits = 0
    n = capi.lib.fa_fwd_num_splits(p)
    assert 2 <= n <= 256
    need = capi.lib.fa_fwd_workspace_bytes(p)
    rows = 128 * 32
    assert need >= n * rows * (128 + 1) * 4
    p.num_splits = 1
    assert capi.lib.fa_fwd_num_splits(p) == 1 and capi.lib.fa_fwd_workspace_bytes(p) == 0
    p.num_splits = 4
    assert capi.lib.fa_fwd_num_splits(p) == 4
    assert capi.lib.fa_scheduler_metadata_ints(16) == 8 + 8 * 16


def _header_fields(name):
    """Field names of `typedef struct { ... } name;` in the header, in order."""
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    chunk = [c for c in text.split("typedef struct") if re.search(r"\}\s*%s\s*;" % name, c)][0]
    body = chunk[chunk.index("{") + 1:chunk.index("} " + name)]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        stmt = re.sub(r"^(const\s+)?\w+(\s+const)?[\s\*]*", "", stmt, count=1)       # drop the type
        names += [re.sub(r"[\s\*]|\[.*\]", "", part) for part in stmt.split(",")]
    return names


def test_ctypes_structs_follow_the_header_field_by_field():
    for name, cls in (("fa_fwd_params", capi.FwdParams), ("fa_bwd_params", capi.BwdParams)):
        assert _header_fields(name) == [f[0] for f in cls._fields_], name
