"""Extracts the known-answer vectors of the reference's own unit tests for the gemm / matmul /
conv2d path into ``reference_goldens.json`` (beside this script).

The reference is C++ and cannot be built in this environment, so its test sources are read as
text: tensor literals, ``range()`` constructors and the ``EXPECT_EQ(matmul(...), ...)`` lines are
parsed out of

    dlf/test/TensorTest.cpp          gemm_test()            (alpha=2, beta=3, 4 transpose combos)
    dlf/test/GPGPUTest.cpp           gemm_test()            (same data through the GPU API)
    dlf/test/MatMulTest.cpp          TYPED_TEST(MatMulTest, *)
    dlf/test/DNNTest.cpp             TEST(Conv2D, *), TEST(MaxPool, *), TEST(DNNTest, GlobalPooling)
    dlf/test/model/PredictTest.cpp   Gemm, Conv (+bias)
    dlf/test/TensorTest.cpp          dot_test()             (v.v, v.M, M.v, M.M)
    dlf/test/UniformTest.cpp         TEST(UniformTest, Dot), TEST(UniformTest, MultiDot*)
    dlf/test/GPGPUTest.cpp           vector_dot_vector_test() ... matrix_dot_matrix_test()
    dlf/test/GPGPUTest.cpp           symm_test(), trmm_test()

Usage:  python tests/golden/make_goldens.py /path/to/dlf-checkout
Only the JSON travels with the repository; the tests never read the reference tree.
"""
import json
import os
import re
import sys


def _ints(s):
    return [int(x) for x in re.findall(r"-?\d+", s)]


def _line_of(text, pos):
    return text.count("\n", 0, pos) + 1


def _block(text, start):
    """Returns (body, end) of the brace block whose '{' is at or after `start`."""
    i = text.index("{", start)
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1:j], j + 1
    raise ValueError("unbalanced braces")


def _split_args(s):
    out, depth, cur, in_str = [], 0, "", False
    for ch in s:
        if ch == '"':
            in_str = not in_str
        if not in_str:
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
            elif ch == "," and depth == 0:
                out.append(cur.strip())
                cur = ""
                continue
        cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


T = r"(?:TypeParam|T|float)"
RE_RANGE = re.compile(r"(?:auto|Tensor<%s>)\s+(\w+)\s*=\s*Tensor<%s>\(\{([\d,\s]+)\}\)\.range\((\d+)\)\s*;" % (T, T))
RE_LIT = re.compile(r"(?:auto\s+(\w+)\s*=\s*Tensor<%s>|Tensor<%s>\s+(\w+))\s*\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)\s*;" % (T, T), re.S)
RE_FILL = re.compile(r"auto\s+(\w+)\s*=\s*Tensor<%s>\(\{([\d,\s]+)\},\s*(\d+)\)\s*;" % T)
RE_SCALAR = re.compile(r"auto\s+(\w+)\s*=\s*(?:Tensor<%s>::scalar|Scalar<%s>)\((\d+)\)\s*;" % (T, T))
RE_MATRIX = re.compile(r"auto\s+(\w+)\s*=\s*Matrix<%s>\(\{(.*?)\}\)\s*;" % T, re.S)
RE_VECTOR = re.compile(r"auto\s+(\w+)\s*=\s*Vector<%s>\(\{([^}]*)\}\)\s*;" % T)
RE_ALIAS = re.compile(r"auto\s+(\w+)\s*=\s*((?:unsqueeze\(|as_strided\(|\w+\[\")[^;]*);")
RE_EMPTY = re.compile(r"auto\s+(\w+)\s*=\s*Tensor<%s>\((?:\{([\d,\s]+)\}|filter\.output_shape\(\))?\)\s*;" % T)


def parse_vars(body):
    vars_ = {}
    for m in RE_RANGE.finditer(body):
        vars_[m.group(1)] = {"shape": _ints(m.group(2)), "range": int(m.group(3))}
    for m in RE_LIT.finditer(body):
        vars_[m.group(1) or m.group(2)] = {"shape": _ints(m.group(3)), "values": _ints(m.group(4))}
    for m in RE_FILL.finditer(body):
        vars_[m.group(1)] = {"shape": _ints(m.group(2)), "fill": int(m.group(3))}
    for m in RE_SCALAR.finditer(body):
        vars_[m.group(1)] = {"shape": [], "values": [int(m.group(2))]}
    for m in RE_MATRIX.finditer(body):
        rows = re.findall(r"\{([^{}]*)\}", m.group(2))
        vals = [_ints(r) for r in rows]
        vars_[m.group(1)] = {"shape": [len(vals), len(vals[0])], "values": sum(vals, [])}
    for m in RE_VECTOR.finditer(body):
        v = _ints(m.group(2))
        vars_[m.group(1)] = {"shape": [len(v)], "values": v}
    for m in RE_ALIAS.finditer(body):
        if m.group(1).startswith("dev"):
            continue
        vars_[m.group(1)] = {"expr": m.group(2).strip()}
    return vars_


def extract_gemm(path, rel):
    text = open(path).read()
    pos = text.index("static void gemm_test()")
    body, _ = _block(text, pos)
    v = parse_vars(body)
    low = {k.lower(): val for k, val in v.items()}
    al = re.search(r"T\(2\)", body) and re.search(r"T\(3\)", body)
    assert al, "alpha/beta literals moved"
    return {"source": "%s:%d" % (rel, _line_of(text, pos)), "alpha": 2, "beta": 3,
            "A": low["a"], "A_t": low.get("t_a") or low["a_t"], "B": low["b"],
            "B_t": low.get("t_b") or low["b_t"], "C": low["c"], "R": low["r"]}


def extract_matmul(path, rel):
    text = open(path).read()
    cases = []
    for m in re.finditer(r"TYPED_TEST\(MatMulTest,\s*(\w+)\)", text):
        name = m.group(1)
        body, _ = _block(text, m.end())
        # tests written as several independent { } scopes
        scopes = []
        stripped = body.strip()
        if stripped.startswith("{"):
            pos = 0
            while True:
                try:
                    pos = body.index("{", pos)
                except ValueError:
                    break
                inner, pos = _block(body, pos)
                scopes.append(inner)
        else:
            scopes.append(body)
        for si, scope in enumerate(scopes):
            vars_ = parse_vars(scope)
            checks = []
            for c in re.finditer(r"EXPECT_EQ\(matmul\((.*)\),\s*([\w\[\]]+)\);", scope):
                args = _split_args(c.group(1))
                if len(args) != 2 or "dev" in c.group(1):
                    continue
                checks.append({"a": args[0], "b": args[1], "expect": c.group(2)})
            if not checks:
                continue
            cases.append({"name": name + ("_%d" % si if len(scopes) > 1 else ""),
                          "source": "%s:%d" % (rel, _line_of(text, m.start())),
                          "vars": vars_, "checks": checks})
    return cases


def extract_conv(path, rel):
    text = open(path).read()
    cases = []
    for m in re.finditer(r"TEST\(Conv2D,\s*(\w+)\)", text):
        body, _ = _block(text, m.end())
        vars_ = parse_vars(body)
        f = re.search(r"dnn::Filter2D\(X\.shape\(\), W\.shape\(\)(?:,\s*(\d+))?\)((?:\.\w+\([\d,\s]*\))*)", body)
        cfg = {"group": int(f.group(1) or 1), "pads": [0, 0, 0, 0], "strides": [1, 1]}
        for call in re.finditer(r"\.(\w+)\(([\d,\s]*)\)", f.group(2)):
            vals = _ints(call.group(2))
            if call.group(1) == "pads":
                cfg["pads"] = vals if len(vals) == 4 else [vals[0], vals[1], vals[0], vals[1]]
            elif call.group(1) == "strides":
                cfg["strides"] = vals
        case = {"name": m.group(1), "source": "%s:%d" % (rel, _line_of(text, m.start())),
                "X": vars_["X"], "W": vars_["W"], "filter": cfg}
        if "R" in vars_:
            case["R"] = vars_["R"]
        cases.append(case)
    return cases


def extract_pool(path, rel):
    """TEST(MaxPool, *) cases that carry a literal result, and TEST(DNNTest, GlobalPooling)."""
    text = open(path).read()
    cases = []
    for m in re.finditer(r"TEST\(MaxPool,\s*(\w+)\)", text):
        body, _ = _block(text, m.end())
        vars_ = parse_vars(body)
        if "R" not in vars_:
            continue
        f = re.search(r"dnn::Filter2D\(X\.shape\(\),\s*(\d+),\s*(\d+)\)((?:\.\w+\([^()]*\))*)", body)
        cfg = {"kernel": [int(f.group(1)), int(f.group(2))], "calls": []}
        for call in re.finditer(r"\.(\w+)\(([^()]*)\)", f.group(3)):
            arg = call.group(2).strip()
            cfg["calls"].append([call.group(1), arg.strip('"') if arg.startswith('"') else _ints(arg)])
        cases.append({"name": m.group(1), "source": "%s:%d" % (rel, _line_of(text, m.start())), "mode": "max",
                      "X": vars_["X"], "R": vars_["R"], "filter": cfg})
    m = re.search(r"TEST\(DNNTest,\s*GlobalPooling\)", text)
    body, _ = _block(text, m.end())
    vars_ = parse_vars(body)
    lits = dict((k, [float(v) for v in vals.split(",")]) for k, vals in
                re.findall(r"auto (\w+_R) = Tensor<float>\(\{2, 3, 1, 1\},\s*\{([^}]*)\}\)", body))
    glob = {"source": "%s:%d" % (rel, _line_of(text, m.start())), "X": vars_["X"],
            "max_R": lits["max_R"], "avg_R": lits["avg_R"]}
    return {"maxpool": cases, "global": glob}


def extract_predict(path, rel):
    text = open(path).read()
    out = {}
    m = re.search(r"TYPED_TEST\(PredictTest,\s*Gemm\)", text)
    body, _ = _block(text, m.end())
    sets = re.findall(r"Tensor<float>\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)", body)
    out["gemm"] = {"source": "%s:%d" % (rel, _line_of(text, m.start())), "alpha": 1, "beta": 1,
                   "A": {"shape": _ints(sets[0][0]), "values": _ints(sets[0][1])},
                   "B": {"shape": _ints(sets[1][0]), "values": _ints(sets[1][1])},
                   "C": {"shape": _ints(sets[2][0]), "values": _ints(sets[2][1])},
                   "Y": {"shape": _ints(sets[3][0]), "values": _ints(sets[3][1])}}
    m = re.search(r"TYPED_TEST\(PredictTest,\s*Conv\)", text)
    body, _ = _block(text, m.end())
    pads = _ints(re.search(r"pads\(\{([\d,\s]+)\}\)", body).group(1))
    bias = re.search(r'TensorData\("B",\s*DataType::FLOAT,\s*\{([\d,\s]+)\},\s*\{([^}]*)\}\)', body)
    vars_ = parse_vars(body)
    y = re.search(r"predictor\.get\(0\),\s*Tensor<float>\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)", body, re.S)
    out["conv"] = {"source": "%s:%d" % (rel, _line_of(text, m.start())), "pads": pads,
                   "X": vars_["X"], "W": vars_["W"],
                   "bias": {"shape": _ints(bias.group(1)), "values": _ints(bias.group(2))},
                   "Y": {"shape": _ints(y.group(1)), "values": _ints(y.group(2))}}
    return out


RE_ANY_TENSOR = re.compile(
    r"(?:auto\s+(\w+)\s*=\s*Tensor<\w+>|Tensor<\w+>\s+(\w+))\s*\(\{?\{([\d,\s]+)\},\s*\{([^}]*)\}\}?\)\s*;", re.S)
RE_ANY_RANGE = re.compile(r"auto\s+(\w+)\s*=\s*Tensor<\w+>\(\{([\d,\s]+)\}\)\.range\((\d*)\)\s*;")


def _dot_vars(body):
    v = {}
    for m in RE_ANY_RANGE.finditer(body):
        v[m.group(1)] = {"shape": _ints(m.group(2)), "range": int(m.group(3) or 0)}
    for m in RE_ANY_TENSOR.finditer(body):
        v[m.group(1) or m.group(2)] = {"shape": _ints(m.group(3)), "values": _ints(m.group(4))}
    m = re.search(r"auto\s+(\w+)\s*=\s*Tensor<\w+>::scalar\((\d+)\)\s*;", body)
    if m:
        v[m.group(1)] = {"shape": [], "values": [int(m.group(2))]}
    return v


def _dot_expected(expr, v):
    expr = expr.strip()
    m = re.fullmatch(r"Tensor<\w+>::scalar\((\d+)\)", expr)
    if m:
        return {"shape": [], "values": [int(m.group(1))]}
    m = re.fullmatch(r"Tensor<\w+>\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)", expr, re.S)
    if m:
        return {"shape": _ints(m.group(1)), "values": _ints(m.group(2))}
    return v[expr]


def extract_dot(tensor_test, uniform_test, gpgpu_test):
    """dot / multi_dot known answers: every case is {source, args: [tensor...], expected}."""
    cases = []
    # TensorTest.cpp dot_test(): four brace scopes, each with a, b and one EXPECT_EQ(dot(a, b), ...)
    path, rel = tensor_test
    text = open(path).read()
    pos = text.index("static void dot_test()")
    body, _ = _block(text, pos)
    i = 0
    while True:
        j = body.find("{", i)
        if j < 0:
            break
        scope, end = _block(body, j)
        i = end
        m = re.search(r"EXPECT_EQ\(dot\((\w+),\s*(\w+)\),\s*(.*?)\);", scope, re.S)
        if not m:
            continue
        v = _dot_vars(scope)
        cases.append({"source": "%s:%d" % (rel, _line_of(text, pos)), "name": "TensorTest.Dot.%d" % len(cases),
                      "args": [v[m.group(1)], v[m.group(2)]], "expected": _dot_expected(m.group(3), v)})
    # UniformTest.cpp: Dot and the MultiDot family
    path, rel = uniform_test
    text = open(path).read()
    for m in re.finditer(r"TEST\(UniformTest,\s*((?:Dot|MultiDot)\w*)\)", text):
        body, _ = _block(text, m.end())
        v = _dot_vars(body)
        call = re.search(r"(?:auto\s+(\w+)\s*=\s*|EXPECT_EQ\()(multi_dot|dot)\(([\w,\s]+)\)", body)
        names = [x.strip() for x in call.group(3).split(",")]
        if call.group(1):  # auto D = multi_dot(A, B, C); EXPECT_EQ(D, <expected>);
            e = re.search(r"EXPECT_EQ\(%s,\s*(.*?)\);" % call.group(1), body, re.S)
            expected = _dot_expected(e.group(1), v)
        else:              # EXPECT_EQ(dot(A, B), C);
            e = re.search(r"EXPECT_EQ\(dot\([\w,\s]+\),\s*(\w+)\);", body)
            expected = v[e.group(1)]
        cases.append({"source": "%s:%d" % (rel, _line_of(text, m.start())), "name": "UniformTest." + m.group(1),
                      "args": [v[n] for n in names], "expected": expected})
    # GPGPUTest.cpp: vector/matrix dot helpers (A, B, R)
    path, rel = gpgpu_test
    text = open(path).read()
    for m in re.finditer(r"static void (\w+_dot_\w+_test)\(\)", text):
        body, _ = _block(text, m.end())
        v = _dot_vars(body)
        cases.append({"source": "%s:%d" % (rel, _line_of(text, m.start())), "name": "GPGPUTest." + m.group(1),
                      "args": [v["A"], v["B"]], "expected": v["R"]})
    return cases


def extract_level3(path, rel):
    """symm_test() and trmm_test() of GPGPUTest.cpp: A = {6,5}.range(1); B = {4,3}.range(1) (symm)
    or the 4x4 identity (trmm); every EXPECT_EQ against a literal is one case."""
    text = open(path).read()
    out = {"symm": [], "trmm": []}
    pos = text.index("void symm_test()")
    body, _ = _block(text, pos)
    for m in re.finditer(r"EXPECT_EQ\(symm\(Side::(\w+),\s*Triangle::(\w+),\s*A,\s*B\),\s*"
                         r"Tensor<T>\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)\)", body, re.S):
        out["symm"].append({"source": "%s:%d" % (rel, _line_of(text, pos)), "side": m.group(1), "triangle": m.group(2),
                            "A": {"shape": [6, 5], "range": 1}, "B": {"shape": [4, 3], "range": 1},
                            "expected": {"shape": _ints(m.group(3)), "values": _ints(m.group(4))}})
    pos = text.index("void trmm_test()")
    body, _ = _block(text, pos)
    for m in re.finditer(r"EXPECT_EQ\(trmm\(Side::(\w+),\s*Triangle::(\w+),\s*Transpose::(\w+),\s*Diagonal::(\w+),"
                         r"\s*A,\s*B\),\s*Tensor<T>\(\{([\d,\s]+)\},\s*\{([^}]*)\}\)\)", body, re.S):
        out["trmm"].append({"source": "%s:%d" % (rel, _line_of(text, pos)), "side": m.group(1), "triangle": m.group(2),
                            "transpose": m.group(3), "diagonal": m.group(4),
                            "A": {"shape": [6, 5], "range": 1}, "B": {"shape": [4, 4], "identity": True},
                            "expected": {"shape": _ints(m.group(5)), "values": _ints(m.group(6))}})
    assert "range(1)" in body and "identity({4, 4})" in body, "trmm_test inputs moved"
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_goldens.py /path/to/dlf-checkout")
    root = sys.argv[1]
    t = os.path.join(root, "dlf", "test")
    g1 = extract_gemm(os.path.join(t, "TensorTest.cpp"), "dlf/test/TensorTest.cpp")
    g2 = extract_gemm(os.path.join(t, "GPGPUTest.cpp"), "dlf/test/GPGPUTest.cpp")
    data = {
        "_comment": "Generated by tests/golden/make_goldens.py from the reference's unit tests; "
                    "do not edit by hand.",
        "gemm": [g1, g2],
        "matmul": extract_matmul(os.path.join(t, "MatMulTest.cpp"), "dlf/test/MatMulTest.cpp"),
        "conv2d": extract_conv(os.path.join(t, "DNNTest.cpp"), "dlf/test/DNNTest.cpp"),
        "pool": extract_pool(os.path.join(t, "DNNTest.cpp"), "dlf/test/DNNTest.cpp"),
        "predict": extract_predict(os.path.join(t, "model", "PredictTest.cpp"),
                                   "dlf/test/model/PredictTest.cpp"),
        "level3": extract_level3(os.path.join(t, "GPGPUTest.cpp"), "dlf/test/GPGPUTest.cpp"),
        "dot": extract_dot((os.path.join(t, "TensorTest.cpp"), "dlf/test/TensorTest.cpp"),
                           (os.path.join(t, "UniformTest.cpp"), "dlf/test/UniformTest.cpp"),
                           (os.path.join(t, "GPGPUTest.cpp"), "dlf/test/GPGPUTest.cpp")),
    }
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_goldens.json")
    with open(out, "w") as f:
        json.dump(data, f, indent=1)
    print("wrote", out, "gemm:", len(data["gemm"]), "matmul:", len(data["matmul"]),
          "conv2d:", len(data["conv2d"]), "dot:", len(data["dot"]))


if __name__ == "__main__":
    main()
