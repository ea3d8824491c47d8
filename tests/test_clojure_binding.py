"""The Clojure side of the boundary (deep_diamond_b200/clj) cannot run where this library is built
(no JVM), so these tests read it as text and check what can be checked without running it:

* every exported function of include/dd_b200.h has exactly one `defdowncall` in impl.clj, with the
  same number of arguments and the same kind (int / 64-bit / double / pointer) for each argument and
  for the result, and the built library exports the symbol;
* every `(invoke dd-... )` in impl.clj passes as many arguments as that downcall takes;
* every call from core.clj to a `...*` function of impl.clj uses an arity that function defines;
* the numbers in constants.clj are the header's enum values;
* delimiters balance in every .clj file.

The reference's raw layer these files stand in for:
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/{impl,constants,core}.clj."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLJ = os.path.join(ROOT, "deep_diamond_b200", "clj", "uncomplicate", "diamond")
HEADER = os.path.join(ROOT, "include", "dd_b200.h")
POINTER_TYPES = {"ddHandle_t", "ddTensorDescriptor_t", "ddActivationDescriptor_t", "ddReduceTensorDescriptor_t",
                 "ddShardedHandle_t"}


def _read(*parts):
    with open(os.path.join(*parts)) as f:
        return f.read()


# ------------------------------------------------------------------ the header ----------------

def _kind(ctype):
    t = " ".join(ctype.replace("const", " ").split())
    if "*" in t or t in POINTER_TYPES:
        return "P"
    if t in ("int64_t", "size_t", "uint64_t"):
        return "L"
    if t == "double":
        return "D"
    if t == "float":
        return "F"
    return "I"          # int and every enum


def header_prototypes():
    src = re.sub(r"/\*.*?\*/", "", _read(HEADER), flags=re.S)
    out = {}
    for ret, name, args in re.findall(r"DD_API\s+([\w\s\*]+?)\s*\b(dd\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        args = " ".join(args.split())
        kinds = []
        if args != "void":
            for a in args.split(","):
                a = a.strip()
                ctype = a[:a.rindex("*") + 1] if "*" in a else a.rsplit(" ", 1)[0]
                kinds.append(_kind(ctype))
        out[name] = (_kind(ret), kinds)
    return out


def header_enums():
    src = re.sub(r"/\*.*?\*/", "", _read(HEADER), flags=re.S)
    return {k: int(v) for k, v in re.findall(r"\b(DD_[A-Z0-9_]+)\s*=\s*(-?\d+)", src)}


# ------------------------------------------------------------------ a small Clojure reader ----

def read_forms(src):
    """Nested lists of tokens for every top-level form; strings and comments are skipped over, the
    reader macros ' ` ~ ~@ ^ #' are treated as prefixes of the next form."""
    tokens = re.findall(r''';[^\n]*|"(?:\\.|[^"\\])*"|\\.|[()\[\]{}]|[^\s()\[\]{}";]+''', src)
    tokens = [t for t in tokens if not t.startswith(";")]
    close = {"(": ")", "[": "]", "{": "}"}
    pos = 0

    def form():
        nonlocal pos
        t = tokens[pos]
        pos += 1
        if t in close:
            items = [t]
            while tokens[pos] != close[t]:
                items.append(form())
            pos += 1
            return items
        if t in (")", "]", "}"):
            raise ValueError("unbalanced delimiter near token %d" % pos)
        return t
    out = []
    while pos < len(tokens):
        out.append(form())
    return out


def strip_meta(items):
    """Drops reader prefixes and ^meta forms so that argument counting sees real arguments only."""
    out, skip = [], False
    for it in items:
        if skip:
            skip = False
            continue
        if isinstance(it, str):
            if it == "^" or it == "#^":
                skip = True
                continue
            if it.startswith("^") and len(it) > 1:      # ^Type or ^:kw attached to the next form
                continue
            if it in ("'", "`", "~", "~@", "#'", "#"):
                continue
        out.append(it)
    return out


def walk(form):
    if isinstance(form, list):
        yield form
        for f in form[1:]:
            yield from walk(f)


def clj_files():
    found = []
    for d, _, files in os.walk(CLJ):
        found += [os.path.join(d, f) for f in files if f.endswith(".clj")]
    return sorted(found)


# ------------------------------------------------------------------ tests ---------------------

def downcalls():
    forms = read_forms(_read(CLJ, "internal", "b200", "impl.clj"))
    out = {}
    for f in forms:
        if isinstance(f, list) and f[0] == "(" and len(f) > 1 and f[1] == "defdowncall":
            _, _, clj_name, c_name, res, args = f
            assert args[0] == "["
            assert clj_name not in out, "two downcalls named %s" % clj_name
            out[clj_name] = (c_name.strip('"'), res, list(args[1:]))
    return out


def test_clj_files_are_there_and_balanced():
    files = clj_files()
    names = {os.path.relpath(f, CLJ) for f in files}
    for needed in ("b200.clj", "internal/b200/impl.clj", "internal/b200/constants.clj", "internal/b200/core.clj",
                   "internal/b200/protocols.clj"):
        assert needed in names
    for f in files:
        read_forms(_read(f))            # raises on an unbalanced or unclosed delimiter


def test_one_downcall_per_export_with_matching_signature():
    protos = header_prototypes()
    calls = downcalls()
    by_c = {}
    for clj_name, (c_name, res, args) in calls.items():
        assert c_name not in by_c, "%s is bound twice" % c_name
        by_c[c_name] = (res, args)
    assert sorted(by_c) == sorted(protos), (sorted(set(protos) - set(by_c)), sorted(set(by_c) - set(protos)))
    for name, (res, args) in protos.items():
        want_args = ["P" if a == "F" else a for a in args]     # no export takes a float by value
        assert by_c[name] == (res, want_args), (name, by_c[name], (res, want_args))


def test_library_exports_every_bound_symbol():
    from deep_diamond_b200 import _lib
    for c_name, _, _ in downcalls().values():
        assert hasattr(_lib.lib, c_name), c_name


def test_invoke_sites_pass_the_right_number_of_arguments():
    calls = downcalls()
    forms = read_forms(_read(CLJ, "internal", "b200", "impl.clj"))
    seen = set()
    for top in forms:
        for f in walk(top):
            items = strip_meta(f[1:])
            if f[0] == "(" and items and items[0] == "invoke" and isinstance(items[1], str) and items[1] in calls:
                handle = items[1]
                seen.add(handle)
                assert len(items) - 2 == len(calls[handle][2]), (handle, len(items) - 2, len(calls[handle][2]))
    assert seen == set(calls), sorted(set(calls) - seen)        # every downcall is used by some wrapper


def _defn_arities(forms):
    out = {}
    for f in forms:
        if not (isinstance(f, list) and f[0] == "(" and len(f) > 2 and f[1] in ("defn", "defn-")):
            continue
        items = strip_meta(f[1:])
        name = items[1]
        arities = set()
        for it in items[2:]:
            if isinstance(it, list) and it[0] == "[":                    # single arity
                arities.add(len(strip_meta(it[1:])))
                break
            if isinstance(it, list) and it[0] == "(" and len(it) > 1 and isinstance(it[1], list) and it[1][0] == "[":
                arities.add(len(strip_meta(it[1][1:])))                  # one of several arities
        out[name] = arities
    return out


def test_core_calls_impl_with_arities_that_exist():
    impl = _defn_arities(read_forms(_read(CLJ, "internal", "b200", "impl.clj")))
    star = {n: a for n, a in impl.items() if n.endswith("*")}
    assert len(star) >= 40
    used = set()
    for top in read_forms(_read(CLJ, "internal", "b200", "core.clj")):
        for f in walk(top):
            items = strip_meta(f[1:])
            if f[0] == "(" and items and isinstance(items[0], str) and items[0] in star:
                used.add(items[0])
                assert len(items) - 1 in star[items[0]], (items[0], len(items) - 1, sorted(star[items[0]]))
    assert len(used) >= 20


def _clj_map(name):
    src = _read(CLJ, "internal", "b200", "constants.clj")
    for top in read_forms(src):
        items = strip_meta(top[1:]) if isinstance(top, list) else []
        if items and items[0] == "def" and name in items:
            table = [it for it in items if isinstance(it, list) and it[0] == "{"][-1]
            body = table[1:]
            return {body[i]: int(body[i + 1]) for i in range(0, len(body), 2)
                    if re.fullmatch(r"-?\d+", str(body[i + 1]))} | \
                   {int(body[i]): body[i + 1] for i in range(0, len(body), 2) if re.fullmatch(r"-?\d+", str(body[i]))}
    raise AssertionError("no table %s" % name)


@pytest.mark.parametrize("table,prefix,names", [
    ("dd-data-type", "DD_DATA_", {"FLOAT": ":float", "DOUBLE": ":double", "HALF": ":half", "INT8": ":byte",
                                  "INT32": ":int", "UINT8": ":uint8", "BFLOAT16": ":bf16", "INT64": ":long"}),
    ("dd-activation-mode", "DD_ACTIVATION_", {"SIGMOID": ":sigmoid", "RELU": ":relu", "TANH": ":tanh",
                                              "CLIPPED_RELU": ":clipped-relu", "ELU": ":elu", "LINEAR": ":linear",
                                              "ABS": ":abs"}),
    ("dd-op-tensor-op", "DD_OP_TENSOR_", {"ADD": ":add", "MUL": ":mul", "MIN": ":min", "MAX": ":max", "SUB": ":sub",
                                          "DIV": ":div"}),
    ("dd-reduce-tensor-op", "DD_REDUCE_TENSOR_", {"ADD": ":add", "MUL": ":mul", "MIN": ":min", "MAX": ":max",
                                                  "AMAX": ":amax", "AVG": ":avg", "NORM1": ":norm1", "NORM2": ":norm2",
                                                  "MUL_NO_ZEROS": ":mul-no-zeros"}),
    ("dd-format", "DD_TENSOR_", {"NCHW": ":nchw", "NHWC": ":nhwc"}),
])
def test_constants_match_the_header(table, prefix, names):
    enums = header_enums()
    clj = _clj_map(table)
    for c_suffix, kw in names.items():
        assert clj[kw] == enums[prefix + c_suffix], (table, kw)


@pytest.mark.parametrize("table,prefix", [("dd-activation-mode", "DD_ACTIVATION_"), ("dd-reduce-tensor-op", "DD_REDUCE_TENSOR_"),
                                          ("dd-op-tensor-op", "DD_OP_TENSOR_")])
def test_every_header_enumerator_has_its_keyword(table, prefix):
    """Every enumerator of the header appears in the Clojure table under the keyword its C name spells
    (DD_ACTIVATION_GELU_TANH -> :gelu-tanh), apart from the ones the tables name after the reference."""
    aliases = {"DD_ACTIVATION_SIGMOID": ":sigmoid", "DD_DATA_INT8": ":byte"}
    clj = _clj_map(table)
    for name, code in header_enums().items():
        if name.startswith(prefix) and not name.endswith("_INDICES"):
            kw = aliases.get(name, ":" + name[len(prefix):].lower().replace("_", "-"))
            assert clj.get(kw) == code, (name, kw)


def test_reduce_indices_table():
    """cudnn/constants.clj:182-184 :no-indices / :flattened against the header and the Python table."""
    from deep_diamond_b200 import constants as K
    enums, clj = header_enums(), _clj_map("dd-reduce-tensor-indices")
    assert clj[":no-indices"] == enums["DD_REDUCE_TENSOR_NO_INDICES"] == K.REDUCE_INDICES["no-indices"]
    assert clj[":flattened"] == enums["DD_REDUCE_TENSOR_FLATTENED_INDICES"] == K.REDUCE_INDICES["flattened"]


def test_status_codes_match_the_header():
    enums = {k: v for k, v in header_enums().items() if k.startswith("DD_STATUS_")}
    clj = _clj_map("dd-status-codes")
    assert len(enums) == len(clj)
    for name, code in enums.items():
        assert clj[code] == ":" + name[len("DD_STATUS_"):].lower().replace("_", "-"), name


def test_python_and_clojure_tables_agree():
    """constants.py is the executed twin of constants.clj: same keywords, same numbers."""
    from deep_diamond_b200 import constants as K
    for table, py in (("dd-data-type", K.DATA_TYPE), ("dd-activation-mode", K.ACTIVATION_MODE),
                      ("dd-op-tensor-op", K.OP_TENSOR), ("dd-reduce-tensor-op", K.REDUCE_OP), ("dd-format", K.FORMAT)):
        clj = _clj_map(table)
        for kw, code in clj.items():
            if isinstance(kw, str) and kw.startswith(":"):
                assert py[kw[1:]] == code, (table, kw)
