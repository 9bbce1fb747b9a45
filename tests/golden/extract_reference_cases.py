"""Extracts the known-answer cases of the reference's own kernel unit tests into tests/golden/reference_cases.json.

The reference's tests build literal matrices with genGivenVals<DT>(numRows, {values...}) and compare a kernel's result
with a literal expected matrix (test/runtime/local/kernels/*Test.cpp).  This script reads those C++ files AS TEXT
(nothing is compiled or executed), pairs every check call with the literals it names, and writes them out as JSON with
the source file and line of each check.  The JSON is the committed fixture; the script is kept so the fixture can be
regenerated from a DAPHNE checkout:

    python tests/golden/extract_reference_cases.py /path/to/daphne > tests/golden/reference_cases.json
"""
from __future__ import annotations

import json
import math
import re
import sys
from pathlib import Path

FILES = ["AggRowTest.cpp", "AggColTest.cpp", "AggAllTest.cpp", "EwBinaryMatTest.cpp", "EwBinaryObjScaTest.cpp",
         "EwUnaryMatTest.cpp", "SyrkTest.cpp", "GemvTest.cpp", "MatMulTest.cpp", "SolveTest.cpp", "CTableTest.cpp",
         "TransposeTest.cpp", "DiagMatrixTest.cpp"]

SCOPE_RE = re.compile(r"^\s*(TEMPLATE_PRODUCT_TEST_CASE|TEMPLATE_TEST_CASE|TEST_CASE|#define\s+\w+TEST_CASE\w*)\b")
GEN_RE = re.compile(r"(?:auto|\w+\s*\*)\s*(\w+)\s*=\s*genGivenVals<([^>]*(?:<[^>]*>)?[^>]*)>\(\s*(\w+)\s*,\s*\{(.*?)\}\s*\)\s*;",
                    re.S)
CHECK_RE = re.compile(r"\b(check\w+)(?:<[^>;()]*>)?\(\s*(?:(\w+OpCode)::(\w+)\s*,\s*)?([^;]*?)\)\s*;")
# assignments inside SECTION blocks (CTableTest, TransposeTest): name = genGivenVals<DT>(rows, {...});
ASSIGN_RE = re.compile(r"(?<![\w*])(\w+)\s*=\s*genGivenVals<([^>]*(?:<[^>]*>)?[^>]*)>\(\s*(\w+)\s*,\s*\{(.*?)\}\s*\)\s*;", re.S)
SECTION_RE = re.compile(r"SECTION\(\s*\"([^\"]*)\"\s*\)\s*\{")
SCALAR_ASSIGN_RE = re.compile(r"\b(weight|resNumRows|resNumCols)\s*=\s*([^;{}]+);")
IGNORED_TOKENS = {"nullptr", "dctx", "dctx.get()", "ctx", "nullptr)"}

_ENV = {"sqrt": math.sqrt, "exp": math.exp, "log": math.log, "sin": math.sin, "cos": math.cos, "tan": math.tan,
        "asin": math.asin, "acos": math.acos, "atan": math.atan, "sinh": math.sinh, "cosh": math.cosh,
        "tanh": math.tanh, "pow": math.pow, "M_PI": math.pi, "M_E": math.e, "inf": math.inf, "nan": math.nan,
        "true": 1, "false": 0}


def _clean(text: str) -> str:
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"/\*.*?\*/", lambda m: "\n" * m.group().count("\n"), text, flags=re.S)  # keeps line numbers
    return text.replace("\\\n", "\n")


def _value(tok: str):
    t = tok.strip()
    if not t:
        return None
    t = re.sub(r"std::numeric_limits<[^>]*>::infinity\(\)", "inf", t)
    t = re.sub(r"std::numeric_limits<[^>]*>::quiet_NaN\(\)", "nan", t)
    t = re.sub(r"\b(?:VT|VTRes|VTArg|typename\s+\w+::VT|double|float|int64_t|size_t|uint32_t)\s*\(([^()]*)\)", r"(\1)", t)
    t = re.sub(r"\((?:VT|VTRes|VTArg|typename\s+\w+::VT|double|float|int64_t|size_t)\)", "", t)
    t = re.sub(r"static_cast<[^>]*>", "", t)
    t = re.sub(r"\bstd::", "", t)
    t = re.sub(r"(?<=[0-9.])[fFlLuU]+\b", "", t)
    try:
        v = eval(t, {"__builtins__": {}}, _ENV)  # literals and a few math calls only
    except Exception:
        raise ValueError(tok)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ValueError(tok)
    return float(v) if isinstance(v, float) else int(v)


def _split_values(body: str):
    out, depth, cur = [], 0, ""
    for ch in body:
        if ch in "([":
            depth += 1
        elif ch in ")]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    out.append(cur)
    return [v for v in (_value(x) for x in out) if v is not None]


def _enc(v):
    if isinstance(v, float) and (math.isnan(v) or math.isinf(v)):
        return "nan" if math.isnan(v) else ("inf" if v > 0 else "-inf")
    return v


def extract(root: Path):
    cases, skipped = [], 0
    for fname in FILES:
        path = root / "test" / "runtime" / "local" / "kernels" / fname
        if not path.exists():
            continue
        raw = path.read_text()
        # keep line numbers: work on the raw text for positions, on a cleaned copy (same length) for parsing
        text = re.sub(r"//[^\n]*", lambda m: " " * len(m.group()), raw)
        text = text.replace("\\\n", " \n")
        lines = text.split("\n")
        starts = [i for i, ln in enumerate(lines) if SCOPE_RE.match(ln)] + [len(lines)]
        offs = [0]
        for ln in lines:
            offs.append(offs[-1] + len(ln) + 1)
        for si in range(len(starts) - 1):
            a, b = offs[starts[si]], offs[starts[si + 1]]
            scope = text[a:b]
            header = lines[starts[si]].strip()
            mats = {}
            for m in GEN_RE.finditer(scope):
                name, dt, nrows, body = m.groups()
                try:
                    vals = _split_values(body)
                    nr = int(nrows) if nrows.isdigit() else None
                except ValueError:
                    continue
                mats[name] = {"dt": re.sub(r"\s+", "", dt), "rows": nr, "values": [_enc(v) for v in vals]}
            for m in CHECK_RE.finditer(scope):
                fn, enum, op, rest = m.groups()
                if fn in ("checkEqApprox", "checkEq"):
                    continue
                line = text.count("\n", 0, a + m.start()) + 1
                args = []
                ok = True
                for tok in [t.strip() for t in re.split(r",(?![^()]*\))", rest) if t.strip()]:
                    if tok in mats and mats[tok]["rows"] is not None:
                        args.append({"matrix": tok, **mats[tok]})
                    elif tok in IGNORED_TOKENS:
                        continue
                    else:
                        try:
                            args.append({"scalar": _enc(_value(tok))})
                        except ValueError:
                            ok = False
                if not ok or not args:
                    skipped += 1
                    continue
                cases.append({"file": f"test/runtime/local/kernels/{fname}", "line": line, "test": header[:120],
                              "check": fn, "op": op, "args": args})
            # SolveTest builds A = t(X) X and b = t(X) (X w) with kernels and checks solve(A, b) against w
            if fname == "SolveTest.cpp" and "X" in mats and "w" in mats and "checkSolve(" in scope:
                line = text.count("\n", 0, a + scope.index("checkSolve(A")) + 1 if "checkSolve(A" in scope else 0
                cases.append({"file": f"test/runtime/local/kernels/{fname}", "line": line, "test": header[:120],
                              "check": "solveNormalEquations", "op": None,
                              "args": [{"matrix": "X", **mats["X"]}, {"matrix": "w", **mats["w"]}]})
            # CTableTest / TransposeTest assign their literals inside SECTION blocks and check once after them
            if fname in ("CTableTest.cpp", "TransposeTest.cpp"):
                secs = list(SECTION_RE.finditer(scope))
                for i, sm in enumerate(secs):
                    body = scope[sm.end(): secs[i + 1].start() if i + 1 < len(secs) else len(scope)]
                    depth, end = 1, len(body)
                    for pos, ch in enumerate(body):
                        depth += ch == "{"
                        depth -= ch == "}"
                        if depth == 0:
                            end = pos
                            break
                    body = body[:end]
                    local = {}
                    for m in ASSIGN_RE.finditer(body):
                        name, dt, nrows, vals = m.groups()
                        try:
                            local[name] = {"matrix": name, "dt": re.sub(r"\s+", "", dt),
                                           "rows": int(nrows) if nrows.isdigit() else None,
                                           "values": [_enc(v) for v in _split_values(vals)]}
                        except ValueError:
                            pass
                    scal = {}
                    for m in SCALAR_ASSIGN_RE.finditer(body):
                        try:
                            scal[m.group(1)] = _enc(_value(m.group(2)))
                        except ValueError:
                            pass
                    line = text.count("\n", 0, a + sm.start()) + 1
                    if fname == "CTableTest.cpp" and {"ys", "xs", "exp"} <= set(local) and len(scal) == 3:
                        cases.append({"file": f"test/runtime/local/kernels/{fname}", "line": line,
                                      "test": sm.group(1)[:120], "check": "ctableSection", "op": None,
                                      "args": [local["ys"], local["xs"], {"scalar": scal["weight"]},
                                               {"scalar": scal["resNumRows"]}, {"scalar": scal["resNumCols"]},
                                               local["exp"]]})
                    elif fname == "TransposeTest.cpp" and {"m", "mt"} <= set(local):
                        cases.append({"file": f"test/runtime/local/kernels/{fname}", "line": line,
                                      "test": sm.group(1)[:120], "check": "transposeSection", "op": None,
                                      "args": [local["m"], local["mt"]]})
    cases += _extract_seq(root)
    cases += _extract_reorg(root)
    cases += _extract_outer(root)
    cases += _extract_aggcum(root)
    cases += _extract_onehot(root)
    cases += _extract_cond(root)
    cases += _extract_slice(root)
    return cases, skipped


ANY_GEN_RE = re.compile(r"(\w+)\s*=\s*genGivenVals<([^;(]*)>\(\s*(\d+)\s*,\s*\{(.*?)\}\s*\)\s*;", re.S)


def _extract_onehot(root: Path):
    """OneHotTest.cpp, numeric test case: one arg, per SECTION an info row and either an expected matrix or an
    expected exception."""
    path = root / "test/runtime/local/kernels/OneHotTest.cpp"
    if not path.exists():
        return []
    text = _clean(path.read_text())
    a = text.find('TEMPLATE_PRODUCT_TEST_CASE("OneHot"')
    b = text.find('TEMPLATE_PRODUCT_TEST_CASE("OneHot"', a + 40)
    scope = text[a:b if b > a else len(text)]
    m = ANY_GEN_RE.search(scope)
    if not m or m.group(1) != "arg":
        return []
    arg = {"matrix": "arg", "dt": "DTArg", "rows": int(m.group(3)), "values": [_enc(v) for v in _split_values(m.group(4))]}
    out = []
    secs = list(SECTION_RE.finditer(scope))
    for i, sm in enumerate(secs):
        body = scope[sm.end(): secs[i + 1].start() if i + 1 < len(secs) else len(scope)]
        local = {}
        for am in ANY_GEN_RE.finditer(body):
            name, dt, nrows, vals = am.groups()
            local[name] = {"matrix": name, "dt": re.sub(r"\s+", "", dt), "rows": int(nrows),
                           "values": [_enc(v) for v in _split_values(vals)]}
        if "info" not in local:
            continue
        line = text.count("\n", 0, a + sm.start()) + 1
        if "REQUIRE_THROWS_AS" in body:
            out.append({"file": "test/runtime/local/kernels/OneHotTest.cpp", "line": line, "test": sm.group(1)[:120],
                        "check": "oneHotThrow", "op": None, "args": [arg, local["info"]]})
        elif "exp" in local:
            out.append({"file": "test/runtime/local/kernels/OneHotTest.cpp", "line": line, "test": sm.group(1)[:120],
                        "check": "oneHot", "op": None, "args": [arg, local["info"], local["exp"]]})
    return out


def _extract_aggcum(root: Path):
    """AggCumTest.cpp: one test case per opcode; every SECTION assigns arg and exp, the check follows the sections."""
    path = root / "test/runtime/local/kernels/AggCumTest.cpp"
    if not path.exists():
        return []
    text = _clean(path.read_text())
    out = []
    starts = [m.start() for m in re.finditer(r"TEMPLATE_PRODUCT_TEST_CASE\(", text)] + [len(text)]
    for a, b in zip(starts, starts[1:]):
        scope = text[a:b]
        om = re.search(r"checkAggCum\(\s*AggOpCode::(\w+)", scope)
        if not om:
            continue
        secs = list(SECTION_RE.finditer(scope))
        for i, sm in enumerate(secs):
            body = scope[sm.end(): secs[i + 1].start() if i + 1 < len(secs) else om.start()]
            local = {}
            for am in ASSIGN_RE.finditer(body):
                name, dt, nrows, vals = am.groups()
                try:
                    local[name] = {"matrix": name, "dt": "DT", "rows": int(nrows),
                                   "values": [_enc(v) for v in _split_values(vals)]}
                except ValueError:
                    pass
            if {"arg", "exp"} <= set(local):
                out.append({"file": "test/runtime/local/kernels/AggCumTest.cpp",
                            "line": text.count("\n", 0, a + sm.start()) + 1, "test": sm.group(1)[:120],
                            "check": "aggCum", "op": om.group(1), "args": [local["arg"], local["exp"]]})
    return out


OUTER_RE = re.compile(r"helper<TestType>\(\s*BinaryOpCode::(\w+)\s*,\s*\{([^}]*)\}\s*,\s*\{([^}]*)\}\s*,\s*\{([^}]*)\}\s*\)\s*;")


def _extract_outer(root: Path):
    """OuterBinaryTest.cpp: helper<TestType>(opcode, {lhs column}, {rhs row}, {expected, row-major})."""
    path = root / "test/runtime/local/kernels/OuterBinaryTest.cpp"
    if not path.exists():
        return []
    text = _clean(path.read_text())
    out = []
    for m in OUTER_RE.finditer(text):
        op, lhs, rhs, exp = m.groups()
        lv, rv, ev = (_split_values(x) for x in (lhs, rhs, exp))
        out.append({"file": "test/runtime/local/kernels/OuterBinaryTest.cpp", "line": text.count("\n", 0, m.start()) + 1,
                    "test": "OuterBinary", "check": "outerBinary", "op": op,
                    "args": [{"matrix": "lhs", "dt": "DT", "rows": len(lv), "values": [_enc(v) for v in lv]},
                             {"matrix": "rhs", "dt": "DT", "rows": 1, "values": [_enc(v) for v in rv]},
                             {"matrix": "exp", "dt": "DT", "rows": len(lv), "values": [_enc(v) for v in ev]}]})
    return out


def _extract_reorg(root: Path):
    """ColBindTest.cpp ("ColBind": m0, m1, exp) and the dense part of ExtractColTest.cpp (one arg, a selection and an
    expected matrix -- or an expected out_of_range -- per SECTION)."""
    out = []
    base = root / "test/runtime/local/kernels"
    path = base / "ColBindTest.cpp"
    if path.exists():
        text = _clean(path.read_text())
        a = text.find('TEMPLATE_PRODUCT_TEST_CASE("ColBind"')
        b = text.find("TEST_CASE(", a + 40)
        scope = text[a:b if b > a else len(text)]
        mats = {}
        for m in GEN_RE.finditer(scope):
            name, dt, nrows, body = m.groups()
            mats[name] = {"matrix": name, "dt": re.sub(r"\s+", "", dt), "rows": int(nrows),
                          "values": [_enc(v) for v in _split_values(body)]}
        if {"m0", "m1", "exp"} <= set(mats):
            out.append({"file": "test/runtime/local/kernels/ColBindTest.cpp",
                        "line": text.count("\n", 0, a + scope.find("colBind<")) + 1, "test": "ColBind",
                        "check": "colBind", "op": None, "args": [mats["m0"], mats["m1"], mats["exp"]]})
    path = base / "ExtractColTest.cpp"
    if path.exists():
        text = _clean(path.read_text())
        a = text.find('TEST_NAME("Dense/Generic Matrix")')
        scope = text[a:]
        m = GEN_RE.search(scope)
        if a >= 0 and m and m.group(1) == "arg":
            arg = {"matrix": "arg", "dt": "DT", "rows": int(m.group(3)), "values": [_enc(v) for v in _split_values(m.group(4))]}
            secs = list(SECTION_RE.finditer(scope))
            for i, sm in enumerate(secs):
                body = scope[sm.end(): secs[i + 1].start() if i + 1 < len(secs) else len(scope)]
                local = {}
                for am in ASSIGN_RE.finditer(body):
                    name, dt, nrows, vals = am.groups()
                    local[name] = {"matrix": name, "dt": "DT", "rows": int(nrows),
                                   "values": [_enc(v) for v in _split_values(vals)]}
                if "sel" not in local and "create<DTEmpty>(0, 1" in body:
                    local["sel"] = {"matrix": "sel", "dt": "DT", "rows": 0, "values": []}
                line = text.count("\n", 0, a + sm.start()) + 1
                if "checkExtractColThrow" in body and "sel" in local:
                    out.append({"file": "test/runtime/local/kernels/ExtractColTest.cpp", "line": line,
                                "test": sm.group(1)[:120], "check": "extractColThrow", "op": None,
                                "args": [arg, local["sel"]]})
                elif "checkExtractCol(" in body and {"sel", "exp"} <= set(local):
                    out.append({"file": "test/runtime/local/kernels/ExtractColTest.cpp", "line": line,
                                "test": sm.group(1)[:120], "check": "extractCol", "op": None,
                                "args": [arg, local["sel"], local["exp"]]})
    return out


SEQ_RE = re.compile(r"(\w+)\s*=\s*genGivenVals<DT>\(\s*(\d+)\s*,\s*\{(.*?)\}\s*\)\s*;\s*checkSeq\(\s*\w+\s*,([^;]*?),\s*\1\s*\)\s*;",
                    re.S)


def _extract_seq(root: Path):
    """SeqTest.cpp assigns the expected column to a variable declared earlier and checks it right away:
    targetMatrix = genGivenVals<DT>(n, {...}); checkSeq(inputMatrix, start, end, inc, targetMatrix);"""
    path = root / "test/runtime/local/kernels/SeqTest.cpp"
    if not path.exists():
        return []
    text = _clean(path.read_text())
    out = []
    for m in SEQ_RE.finditer(text):
        _, nrows, body, scal = m.groups()
        try:
            vals = _split_values(body)
            sc = [_value(t) for t in scal.split(",")]
        except ValueError:
            continue
        if len(sc) != 3:
            continue
        out.append({"file": "test/runtime/local/kernels/SeqTest.cpp", "line": text.count("\n", 0, m.start()) + 1,
                    "test": "Seq", "check": "checkSeq", "op": None,
                    "args": [{"scalar": _enc(v)} for v in sc] +
                            [{"matrix": "targetMatrix", "dt": "DT", "rows": int(nrows), "values": [_enc(v) for v in vals]}]})
    return out


COND_SCALAR_RE = re.compile(r"\b(argThen|argElse)\s*=\s*(VT\([^()]*\))\s*;")


def _extract_cond(root: Path):
    """CondMatMatMatTest.cpp, CondMatMatScaTest.cpp, CondMatScaMatTest.cpp and CondMatScaScaTest.cpp: one SECTION
    ("example 1") assigns argCond and exp as literal 3 x 3 matrices and argThen / argElse as literal matrices or as
    scalars VT(x); the expected literal may name the scalars.  The test is instantiated for int64_t and double, and
    VT(x) truncates for the former, so one case is written per value type."""
    out = []
    for fname in ("CondMatMatMatTest.cpp", "CondMatMatScaTest.cpp", "CondMatScaMatTest.cpp", "CondMatScaScaTest.cpp"):
        path = root / "test/runtime/local/kernels" / fname
        if not path.exists():
            continue
        text = _clean(path.read_text())
        sm = SECTION_RE.search(text)
        if not sm:
            continue
        end = text.find("DT *res = nullptr;", sm.end())
        body = text[sm.end(): end if end > 0 else len(text)]
        line = text.count("\n", 0, text.find(fname[0].lower() + fname[1:-8] + "(res", sm.end())) + 1
        for vt in ("double", "int64_t"):
            conv = (lambda x: float(x)) if vt == "double" else (lambda x: int(x))
            scalars = {n: conv(_value(v)) for n, v in COND_SCALAR_RE.findall(body)}
            local = {}
            for am in ASSIGN_RE.finditer(body):
                name, _, nrows, vals = am.groups()
                toks = re.sub(r"\b(argThen|argElse)\b", lambda m: repr(scalars[m.group(1)]), vals)
                toks = re.sub(r"\bVT\(([^()]*)\)", lambda m: repr(conv(_value(m.group(1)))), toks)
                local[name] = {"matrix": name, "dt": f"DenseMatrix<{vt}>", "rows": int(nrows),
                               "values": [_enc(v) for v in _split_values(toks)]}
            args = []
            for name in ("argCond", "argThen", "argElse", "exp"):
                if name in local:
                    args.append(local[name])
                elif name in scalars:
                    args.append({"scalar": _enc(scalars[name])})
            if len(args) == 4:
                out.append({"file": f"test/runtime/local/kernels/{fname}", "line": line, "test": sm.group(1),
                            "check": "cond", "op": vt, "args": args})
    return out


VECTOR_RE = re.compile(r"std::vector<[^;=]*>\s*(\w+)\s*=\s*\{(.*?)\}\s*;", re.S)
SLICE_CALL_RE = re.compile(r"\b(sliceRow|sliceCol)\(\s*res\s*,\s*arg\s*,\s*([^,]+),\s*([^,]+),\s*nullptr\s*\)")


def _extract_slice(root: Path):
    """SliceRowTest.cpp and SliceColTest.cpp, the numeric DenseMatrix parts: one case that slices [1, 3) of a literal
    4 x 6 matrix and three bound pairs that must raise out_of_range."""
    out = []
    for fname, kernel in (("SliceRowTest.cpp", "sliceRow"), ("SliceColTest.cpp", "sliceCol")):
        path = root / "test/runtime/local/kernels" / fname
        if not path.exists():
            continue
        text = _clean(path.read_text())
        scopes = [m.start() for m in re.finditer(r"TEMPLATE_(?:PRODUCT_)?TEST_CASE\(", text)] + [len(text)]
        for a, b in zip(scopes, scopes[1:]):
            scope = text[a:b]
            if "ALL_STRING_VALUE_TYPES" in scope or "(Frame)" in scope.split("{", 1)[0]:
                continue
            vecs = {n: [_enc(v) for v in _split_values(body)] for n, body in VECTOR_RE.findall(scope)}
            mats = {}
            for m in re.finditer(r"auto\s+(\w+)\s*=\s*genGivenVals<DT>\(\s*(\d+)\s*,\s*(\w+|\{.*?\})\s*\)\s*;", scope, re.S):
                name, nrows, src = m.groups()
                vals = vecs.get(src) if not src.startswith("{") else [_enc(v) for v in _split_values(src[1:-1])]
                if vals is not None:
                    mats[name] = {"matrix": name, "dt": "DT", "rows": int(nrows), "values": vals}
            if "arg" not in mats:
                continue
            for cm in SLICE_CALL_RE.finditer(scope):
                lo, up = (int(_value(t)) for t in cm.group(2, 3))  # VTSel of the throwing calls truncates like VT(x)
                throws = "REQUIRE_THROWS_AS" in scope[max(0, cm.start() - 24): cm.start()]
                if not throws and "exp" not in mats:
                    continue
                out.append({"file": f"test/runtime/local/kernels/{fname}", "line": text.count("\n", 0, a + cm.start()) + 1,
                            "test": kernel, "check": kernel + ("Throw" if throws else ""), "op": None,
                            "args": [mats["arg"], {"scalar": lo}, {"scalar": up}] + ([] if throws else [mats["exp"]])})
    return out


if __name__ == "__main__":
    import os
    root = Path(sys.argv[1] if len(sys.argv) > 1 else
                os.environ.get("DAPHNE_ROOT") or Path(__file__).resolve().parents[3] / "reference")
    cases, skipped = extract(root)
    json.dump({"source": "daphne-eu/daphne test/runtime/local/kernels (literals of the reference's unit tests)",
               "skipped_unparsed_checks": skipped, "cases": cases}, sys.stdout, indent=None, separators=(",", ":"))
    sys.stderr.write(f"{len(cases)} cases, {skipped} skipped\n")
