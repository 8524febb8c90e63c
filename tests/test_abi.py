"""The C-ABI library loads without a GPU and exports every symbol that include/tango_b200.h declares; argument
validation that happens before any CUDA call returns the documented error codes."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tango_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tango_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    from tango_b200 import _lib
    names = _declared()
    assert len(names) >= 17
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} declared in tango_b200.h but not exported"
    assert set(_lib.EXPORTED) == set(names), "ctypes signature table out of sync with the header"


def test_version_and_strerror():
    from tango_b200 import _lib
    assert _lib.lib.tango_version() >= 100
    assert _lib.lib.tango_strerror(0) == b"ok"
    assert b"invalid" in _lib.lib.tango_strerror(-1)
    assert b"unknown" in _lib.lib.tango_strerror(-99)


def test_argument_validation_without_gpu():
    from tango_b200 import _lib
    L = _lib.lib
    assert L.tango_quantize(None, -1, 4, 4, None, None, None, 4, 1, 0, 0, None, None) == -1    # negative rows
    assert L.tango_quantize(None, 4, 4, 4, None, None, None, 4, 7, 0, 0, None, None) == -1     # bad mode
    assert L.tango_quantize(None, 4, 8, 4, None, None, None, 8, 1, 0, 0, None, None) == -1     # ld < cols
    assert L.tango_sddmm_elementwise(9, None, None, 1, None, 4, None, 4, 4, None, None, None, None, None) == -1
    assert L.tango_spmm_copy_u(None, None, 4, 0, None, 16, 16, None, None, None, 0, None, 16, None, None, None) == -1
    assert L.tango_qgemm_nt(None, 16, None, 16, 8, 8, 0, None, None, None, None, 8, None, None, None) == -1
    assert L.tango_qgemm_dw_workspace_bytes(256, 602) == 256 * 604 * 4
    # empty problems succeed without touching the device
    assert L.tango_sddmm_dot(None, None, 0, None, 16, None, 16, 1, 16, None, None, None, None, None) == 0
    assert L.tango_spmm_incidence(None, None, 0, None, 4, 4, None, None, 4, None, None) == 0


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "tango_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"


def _prototypes():
    """name -> (return type text, [parameter type texts]) for every function declared in the header."""
    text = open(os.path.join(ROOT, "include", "tango_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(tango_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        plist = [] if params in ("", "void") else [" ".join(p.split()) for p in params.split(",")]
        protos[name] = (ret, plist)
    return protos


def _ctype_of(decl: str):
    """ctypes class the binding must use for a C parameter (or return) declaration."""
    if "*" in decl or decl.startswith("tango_stream_t"):
        return ctypes.c_void_p
    base = decl.replace("const ", "").split()[0]
    return {"int": ctypes.c_int, "int64_t": ctypes.c_int64, "uint64_t": ctypes.c_uint64,
            "float": ctypes.c_float}[base]


def test_ctypes_signatures_match_the_header():
    """Every entry of the ctypes table has the arity and the scalar / pointer classes of its C prototype, so a
    signature change in the header cannot silently shift arguments in the binding."""
    from tango_b200 import _lib
    protos = _prototypes()
    assert set(protos) == set(_lib._SIGS)
    for name, (ret, params) in protos.items():
        argtypes, restype = _lib._SIGS[name]
        assert len(argtypes) == len(params), f"{name}: {len(argtypes)} ctypes arguments, {len(params)} in the header"
        for k, (a, decl) in enumerate(zip(argtypes, params)):
            want = _ctype_of(decl)
            if want is ctypes.c_void_p:          # any pointer class will do (typed struct pointers included)
                assert a is ctypes.c_void_p or issubclass(a, ctypes._Pointer), f"{name}: argument {k} ({decl})"
            else:
                assert a is want, f"{name}: argument {k} ({decl}) bound as {a.__name__}"
        if "char" in ret:
            assert restype is ctypes.c_char_p
        else:
            assert restype is _ctype_of(ret), f"{name}: returns {ret}, bound as {restype.__name__}"


def test_plan_struct_matches_the_header():
    """tango_spmm_plan is passed by pointer from ctypes: its fields must have the names, order and C types of the
    header's struct, or every pointer behind the first mismatch would be read from the wrong offset."""
    from tango_b200 import _lib
    text = open(os.path.join(ROOT, "include", "tango_b200.h")).read()
    body = re.search(r"typedef struct tango_spmm_plan \{(.*?)\} tango_spmm_plan;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if not decl:
            continue
        m = re.match(r"(.*?)(\w+)$", decl)
        ctype, name = m.group(1).strip(), m.group(2)
        if "*" in ctype:
            want = ctypes.c_void_p
        else:
            want = {"int64_t": ctypes.c_int64, "int32_t": ctypes.c_int32, "int": ctypes.c_int}[ctype]
        fields.append((name, want))
    assert [(n, t) for n, t in _lib.SpmmPlan._fields_] == fields


def test_dense_hub_region_arguments_are_validated_before_any_cuda_call():
    from tango_b200 import _lib
    L = _lib.lib
    buf = (ctypes.c_int8 * 4096)()
    base = ctypes.addressof(buf)
    base = (base + 255) // 256 * 256                     # a 256-byte aligned address inside the buffer
    plan = _lib.SpmmPlan()
    plan.heavy_rows, plan.n_heavy, plan.ws, plan.ws_ld = base, 128, base, 16
    plan.row_order, plan.n_long_rows = base, 128
    plan.dense_a, plan.dense_n_tiles, plan.dense_units, plan.dense_n_units = base, 1, base, 1
    plan.dense_rows, plan.dense_cols, plan.dense_n_cols, plan.dense_b = 128, base, 128, base
    plan.n_skip_rows = 64                                # must equal n_heavy with a dense region
    args = (base, base, 256, 1, base, 16, 16, base, None, None, 0, base, 16, None)
    assert L.tango_spmm_copy_u(*args, ctypes.byref(plan), None) == -1
    plan.n_skip_rows = 128
    plan.dense_n_cols = 100                              # not a multiple of 128
    assert L.tango_spmm_copy_u(*args, ctypes.byref(plan), None) == -1
    plan.dense_n_cols = 128
    plan.dense_a = base + 8                              # tiles must be 16-byte aligned
    assert L.tango_spmm_copy_u(*args, ctypes.byref(plan), None) == -2
    # the quantised attention entry point rejects an unknown rounding mode outright
    assert L.tango_gat_edge_softmax_quantized(None, None, None, None, 0, 0, None, None, 4, None, None, 0.2, None, None,
                                              None, None, 7, 0, 0, None, None) == -1
