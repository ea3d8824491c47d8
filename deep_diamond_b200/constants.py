"""Keyword -> enum tables, mirroring the reference's
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/constants.clj
(data types :64-89, widths :126-148, formats :43-55, activation modes :150-158, reduce ops
:171-180) with oneDNN's spellings (dnnl/constants.clj:277-308, 359-371, 393-402) accepted too.
Keywords are plain strings here: ``"float"`` for ``:float``.
"""
import numpy as np

from ._lib import DiamondError

DATA_TYPE = {
    "float": 0, "float32": 0, "f32": 0, float: 0, np.float32: 0,
    "double": 1, "float64": 1, "f64": 1, np.float64: 1,
    "half": 2, "float16": 2, "f16": 2, np.float16: 2,
    "byte": 3, "int8": 3, "s8": 3, np.int8: 3,
    "int": 4, "int32": 4, "s32": 4, int: 4, np.int32: 4,
    "uint8": 6, "u8": 6, np.uint8: 6,
    "bf16": 9, "bfloat16": 9,
    "long": 15, "int64": 15, "s64": 15, np.int64: 15,
}
DATA_TYPE_NAME = {0: "float", 1: "double", 2: "half", 3: "byte", 4: "int", 6: "uint8", 9: "bf16",
                  15: "long"}
DATA_TYPE_WIDTH = {0: 4, 1: 8, 2: 2, 3: 1, 4: 4, 6: 1, 9: 2, 15: 8}
NUMPY_TYPE = {0: np.float32, 1: np.float64, 2: np.float16, 3: np.int8, 4: np.int32, 6: np.uint8,
              9: np.uint16, 15: np.int64}

FORMAT = {"nchw": 0, "nhwc": 1, "abcd": 0, "acdb": 1, "oihw": 0, "ohwi": 1}

ACTIVATION_MODE = {"logistic": 0, "sigmoid": 0, "relu": 1, "tanh": 2, "clipped-relu": 3, "elu": 4,
                   "linear": 5, "identity": 5, "abs": 6,
                   # the rest of the DNNL backend's table (dnnl/constants.clj:277-308); the reference maps
                   # :square-dst-bwd onto oneDNN's sqrt_use_dst_for_bwd, and so does this table
                   "square": 7, "sqrt": 8, "exp": 9, "log": 10, "soft-relu": 11, "swish": 12, "gelu": 13,
                   "gelu-tanh": 13, "gelu-erf": 14, "hardswish": 15, "clip": 16, "clip-v2": 17, "pow": 18,
                   "mish": 19, "round": 20, "relu-dst-bwd": 21, "tanh-dst-bwd": 22, "elu-dst-bwd": 23,
                   "square-dst-bwd": 24, "sqrt-dst-bwd": 24, "logistic-dst-bwd": 25, "sigmoid-dst-bwd": 25,
                   "exp-dst-bwd": 26, "clip-v2-dst-bwd": 27}
ACTIVATION_NAME = {0: "logistic", 1: "relu", 2: "tanh", 3: "clipped-relu", 4: "elu", 5: "linear",
                   6: "abs", 7: "square", 8: "sqrt", 9: "exp", 10: "log", 11: "soft-relu", 12: "swish",
                   13: "gelu-tanh", 14: "gelu-erf", 15: "hardswish", 16: "clip", 17: "clip-v2", 18: "pow",
                   19: "mish", 20: "round", 21: "relu-dst-bwd", 22: "tanh-dst-bwd", 23: "elu-dst-bwd",
                   24: "sqrt-dst-bwd", 25: "logistic-dst-bwd", 26: "exp-dst-bwd", 27: "clip-v2-dst-bwd"}

OP_TENSOR = {"add": 0, "mul": 1, "min": 2, "max": 3, "sub": 4, "div": 5,
             "ge": 6, "gt": 7, "le": 8, "lt": 9, "eq": 10, "ne": 11}

REDUCE_OP = {"add": 0, "sum": 0, "mul": 1, "min": 2, "max": 3, "amax": 4, "avg": 5, "mean": 5,
             "norm1": 6, "norm2": 7, "mul-no-zeros": 8,
             # oneDNN's norm kinds, which take p and epsilon (dnnl/constants.clj:393-402)
             "norm-lp-max": 9, "norm-lp-sum": 10, "norm-lp-power-p-max": 11, "norm-lp-power-p-sum": 12}
REDUCE_NAME = {0: "add", 1: "mul", 2: "min", 3: "max", 4: "amax", 5: "avg", 6: "norm1", 7: "norm2",
               8: "mul-no-zeros", 9: "norm-lp-max", 10: "norm-lp-sum", 11: "norm-lp-power-p-max",
               12: "norm-lp-power-p-sum"}

# cudnn/constants.clj:182-184
REDUCE_INDICES = {"no-indices": 0, "flattened": 1}


def enc_keyword(table, kw, what="keyword"):
    """``enc-keyword``: unknown keywords raise like ``dragan-says-ex``."""
    try:
        return table[kw]
    except (KeyError, TypeError):
        raise DiamondError("This %s is not supported." % what,
                           {"requested": kw, "available": sorted(str(k) for k in table)})


def layout_strides(shape, layout):
    """Element strides of a named layout: any permutation keyword whose letters are the dims in
    physical order ("nchw", "nhwc", "nc", "tnc", "ntc", "x", ...).  The logical order of dims is
    the canonical one for the rank (n c [d] h w / t n c), as in oneDNN format tags."""
    nd = len(shape)
    if layout is None:
        return default_strides(shape)
    if not isinstance(layout, str):
        if len(layout) != nd:
            raise DiamondError("Shape and strides must have the same length.",
                               {"shape": list(shape), "strides": list(layout)})
        return [int(s) for s in layout]
    name = layout.lower()
    if len(name) != nd:
        raise DiamondError("Shape and layout must have the same length.",
                           {"shape": list(shape), "layout": layout})
    canon = _CANONICAL.get(frozenset(name))
    if canon is None or len(canon) != nd or len(set(name)) != nd:
        raise DiamondError("This format is not supported.", {"format": layout})
    # physical order = order of letters in `name`; logical dim index of a letter = its place in canon
    strides = [0] * nd
    run = 1
    for letter in reversed(name):
        i = canon.index(letter)
        strides[i] = run
        run *= max(int(shape[i]), 1)
    return strides


_CANONICAL = {
    frozenset("x"): "x", frozenset("a"): "a",
    frozenset("nc"): "nc", frozenset("ab"): "ab", frozenset("io"): "oi",
    frozenset("tnc"): "tnc", frozenset("ncw"): "ncw", frozenset("abc"): "abc",
    frozenset("nchw"): "nchw", frozenset("abcd"): "abcd", frozenset("oihw"): "oihw",
    frozenset("ncdhw"): "ncdhw", frozenset("abcde"): "abcde",
}


def default_strides(shape):
    """Row-major strides (deep-diamond-base/src/uncomplicate/diamond/internal/utils.clj:53-67)."""
    st, run = [], 1
    for d in reversed(list(shape)):
        st.append(run)
        run *= max(int(d), 1)
    return list(reversed(st))
