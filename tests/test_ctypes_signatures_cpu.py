"""Every ctypes call into the native libraries is checked against the C prototype it targets: argument count, and
per argument the class (pointer / 32-bit int / 64-bit int / float / stream).  The libraries are called without
declared ``argtypes``, so a call site that drifts from its prototype would corrupt the call silently."""
import ast
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
PROTO = re.compile(r"^(?:const\s+)?[A-Za-z_][\w ]*?[\s\*]+(afb_\w+)\s*\(([^)]*)\)\s*\{", re.M | re.S)


def c_prototypes():
    out = {}
    for path in list((ROOT / "csrc" / "kernels").glob("*.cu")) + list((ROOT / "csrc" / "host").glob("*.cpp")):
        text = re.sub(r"//[^\n]*", "", path.read_text())
        for m in PROTO.finditer(text):
            name, args = m.group(1), " ".join(m.group(2).split())
            kinds = []
            for a in [x.strip() for x in args.split(",") if x.strip() and x.strip() != "void"]:
                if "*" in a:
                    kinds.append("ptr")
                elif a.startswith("cudaStream_t"):
                    kinds.append("stream")
                elif re.match(r"(const )?(unsigned )?(long long|long|size_t|int64_t|uint64_t)\b", a):
                    kinds.append("i64")
                elif re.match(r"(const )?(float)\b", a):
                    kinds.append("f32")
                elif re.match(r"(const )?(double)\b", a):
                    kinds.append("f64")
                elif re.match(r"(const )?(unsigned |u)?(int|int32_t|uint32_t|bool|unsigned)\b", a):
                    kinds.append("i32")
                else:
                    kinds.append("?")
            out[name] = kinds
    return out


def classify(node) -> str:
    """Class of a call-site argument expression; '?' when it cannot be told from the source."""
    if isinstance(node, ast.Constant):
        return "ptr" if node.value is None else "?"
    if isinstance(node, ast.IfExp):
        a, b = classify(node.body), classify(node.orelse)
        return a if a == b or b == "?" else b if a == "?" else "mismatch"
    if isinstance(node, ast.Call):
        f = node.func
        name = f.attr if isinstance(f, ast.Attribute) else f.id if isinstance(f, ast.Name) else ""
        if name in ("_c_int", "c_int", "c_uint", "c_int32", "c_bool"):
            return "i32"
        if name in ("_c_long", "c_long", "c_int64", "c_longlong", "c_size_t", "c_uint64", "c_ulonglong"):
            return "i64"
        if name in ("_c_float", "c_float"):
            return "f32"
        if name in ("c_double",):
            return "f64"
        if name in ("ptr", "c_void_p", "data_as", "peers", "flag_ptr", "peer_flag_ptrs", "c_char_p", "byref",
                    "_ptr_array", "cast"):
            return "ptr"
        if name == "stream_ptr":
            return "stream"
    return "?"


def call_sites():
    for path in (ROOT / "antfly_b200").rglob("*.py"):
        tree = ast.parse(path.read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr.startswith("afb_"):
                if any(isinstance(a, ast.Starred) for a in node.args) or node.keywords:
                    continue
                yield path.relative_to(ROOT), node.lineno, node.func.attr, [classify(a) for a in node.args]


def test_call_sites_match_their_prototypes():
    protos = c_prototypes()
    assert len(protos) > 60, len(protos)
    problems, checked = [], 0
    for path, line, name, kinds in call_sites():
        if name not in protos:
            problems.append(f"{path}:{line}: {name} has no C definition")
            continue
        want = protos[name]
        if len(want) != len(kinds):
            problems.append(f"{path}:{line}: {name} takes {len(want)} arguments, call passes {len(kinds)}")
            continue
        checked += 1
        for i, (w, k) in enumerate(zip(want, kinds)):
            if k == "?" or w == "?":
                continue
            if k == "mismatch" or (w != k and not (w == "stream" and k == "ptr")):
                problems.append(f"{path}:{line}: {name} argument {i + 1} is {w} in C, {k} at the call")
    assert not problems, "\n".join(problems)
    assert checked > 80, checked
