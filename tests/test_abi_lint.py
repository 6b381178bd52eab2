"""Static check of the boundary between Python and the native libraries: every ``ctypes`` call of an
``extern "C"`` entry point (``ft_*`` of the CUDA library, ``ftref_*`` of the host reference library)
passes as many arguments as the C prototype declares, and every argument that is wrapped in a
``ctypes`` type at the call site has the width and kind of its C parameter (``c_int`` for ``int``,
``c_long`` for ``long``, ``c_uint`` for ``unsigned int``, ``c_ulonglong`` for ``unsigned long long``,
``c_float`` for ``float``, a pointer for a pointer or a stream). A call that drifts from its prototype
would read garbage on the device; this finds it without one."""
import ast
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "forgetrain_b200" / "csrc"


def _c_prototypes() -> dict[str, tuple[str, list[str]]]:
    protos: dict[str, tuple[str, list[str]]] = {}
    for f in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.h")) + list((CSRC / "ref_cpu").glob("*.cpp")):
        text = f.read_text()
        found = list(re.finditer(r'extern "C"\s+[\w\s\*]+?\s+(ft\w+)\s*\(([^)]*)\)', text, re.S))
        # functions inside an `extern "C" { ... }` block: a definition or declaration at line start
        found += list(re.finditer(r'^(?:void|int|float|double)\s+(ft\w+)\s*\(([^)]*)\)', text, re.S | re.M))
        for m in found:
            params = [p.strip() for p in m.group(2).replace("\n", " ").split(",")]
            protos.setdefault(m.group(1), (f.name, [p for p in params if p and p != "void"]))
    return protos


def _c_kind(param: str) -> str:
    p = re.sub(r"\b(const|__restrict__)\b", "", param).strip()
    if "*" in p or p.startswith("cudaStream_t"):
        return "ptr"
    for pattern, kind in ((r"unsigned long long|uint64_t|size_t", "u64"), (r"unsigned int|unsigned\b|uint32_t", "u32"),
                          (r"long long|int64_t|long\b", "i64"), (r"int\b|int32_t", "i32"), (r"float\b", "f32"),
                          (r"double\b", "f64")):
        if re.match(pattern, p):
            return kind
    raise AssertionError(f"parameter {param!r}: a type this check does not know")


_PY_KIND = {"c_int": "i32", "c_float": "f32", "c_long": "i64", "c_longlong": "i64", "c_uint": "u32",
            "c_ull": "u64", "c_ulonglong": "u64", "c_double": "f64", "c_size_t": "u64",
            "c_void_p": "ptr", "P": "ptr", "ptr": "ptr", "_ptr": "ptr", "stream": "ptr", "byref": "ptr"}


def _py_kind(node) -> str | None:
    """Kind of an argument that is visibly typed at the call site, else None (a variable)."""
    if isinstance(node, ast.Call):
        f = node.func
        return _PY_KIND.get(f.attr if isinstance(f, ast.Attribute) else getattr(f, "id", ""))
    return None


def _call_sites():
    files = list((ROOT / "forgetrain_b200").rglob("*.py")) + [ROOT / "bench.py", ROOT / "microbench.py"] + \
        list((ROOT / "tests").glob("*.py"))
    for f in files:
        for n in ast.walk(ast.parse(f.read_text())):
            if isinstance(n, ast.Call) and isinstance(n.func, ast.Attribute) and n.func.attr.startswith("ft"):
                yield f, n


def test_every_native_call_matches_its_c_prototype():
    protos = _c_prototypes()
    assert len(protos) >= 30 and "ft_gemm_bf16" in protos and "ftref_gemm" in protos
    called, compared, problems = set(), 0, []
    for f, n in _call_sites():
        name = n.func.attr
        if name not in protos or any(isinstance(a, ast.Starred) for a in n.args):
            continue
        called.add(name)
        where = f"{f.relative_to(ROOT)}:{n.lineno} {name}"
        params = protos[name][1]
        if len(n.args) != len(params) or n.keywords:
            problems.append(f"{where}: {len(n.args)} arguments for {len(params)} parameters")
            continue
        for i, (a, p) in enumerate(zip(n.args, params)):
            kind = _py_kind(a)
            if kind is None:
                continue
            compared += 1
            if kind != _c_kind(p):
                problems.append(f"{where}: argument {i} is {kind}, parameter `{p}` is {_c_kind(p)}")
    assert not problems, "\n".join(problems)
    assert compared > 300                               # the check did look at the calls
    # every entry point has a caller (the TMA-descriptor cache reset is a debugging aid)
    assert set(protos) - called <= {"ft_tmap_cache_clear"}, sorted(set(protos) - called)


def test_every_return_code_of_the_native_entry_points_has_a_hint():
    """``check_rc`` explains a failed call: each negative code that an entry point can return is in
    its table, so no user is left with a bare number."""
    from forgetrain_b200.ops import _lib
    codes = set()
    for f in CSRC.glob("*.cu"):
        codes |= {int(c) for c in re.findall(r"return (-\d+);", f.read_text())}
    assert codes and codes <= set(_lib._RC_HINTS), sorted(codes - set(_lib._RC_HINTS))
    try:
        _lib.check_rc(-4, "ft_gemm_bf16")
    except RuntimeError as e:
        assert "ft_gemm_bf16 failed with code -4: no TMA descriptor for the first operand" in str(e)
    else:
        raise AssertionError("check_rc did not raise")
    _lib.check_rc(0, "anything")
