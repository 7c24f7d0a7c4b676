"""Accelerate's array language embedded in Python, compiled to functor snippets for the B200 skeletons.

The reference compiles every collective operation by pasting the user's scalar functions, translated to C
by its expression compiler, into a skeleton template (``codegenAcc``, Data/Array/Accelerate/CUDA/CodeGen.hs:91-136;
scalar expressions ``codegenOpenExp``, CodeGen.hs:338-821; arithmetic in CodeGen/Arithmetic.hs).  This module
does the same for the skeleton headers of this library: Python functions over ``Exp`` values are traced once,
printed as a functor struct (the contracts at the top of csrc/skeletons/*.cuh) and handed to the kernel cache.
Producers -- ``map``, ``zipWith``, ``zip``, ``generate``, ``backpermute`` -- are delayed and fused into their
consumer exactly as Accelerate's fusion hands them to the backend (``Delayed`` arrays, CodeGen.hs:134-136):
a ``fold`` over a ``zipWith`` is ONE kernel that reads both vectors with 128-bit loads.

    import importlib
    A = importlib.import_module("accelerate-cuda_b200.lang")
    dotp = A.run1(lambda xs, ys: A.fold(lambda a, b: a + b, 0.0, A.zipWith(lambda a, b: a * b, xs, ys)),
                  A.vector(np.float32), A.vector(np.float32))
    dotp(x, y)        # numpy in, numpy out

Semantics follow the reference's C forms: integer ``//`` and ``%`` round towards minus infinity
(Arithmetic.hs:103-134), ``quot``/``rem`` truncate (:89-101), ``round`` is C ``round`` (:281-282), ``min``/``max``
on floats are fminf/fmaxf (:322-336), integer arithmetic wraps, Bool is one byte.  The language is typed like
Accelerate: both operands of an operator have the same type (Python numbers take the type of the other operand);
``fromIntegral`` / ``toFloating`` / ``cast`` convert.

Shapes are known extent by extent as a constant plus, optionally, an extent of an argument or intermediate array
(``dim(arr, d)``, ``shape_of(arr)``): enough for ``replicate``, ``slice``, ``transpose``, ``reshape``, ``init``,
``tail``, ``take``, ``drop`` and for the exclusive scans along rows, whose rows grow by one; the host evaluates them
when the program runs, as the reference evaluates shape expressions (Execute.hs:194-199).  Scans along the
innermost dimension of matrices and the segmented ``scanl1Seg`` / ``scanr1Seg``, which the reference rejects
(PrefixSum.hs:39-46), are the scan skeleton over (value, restart flag) pairs.

Restrictions of this front end (not of the skeletons): ranks up to 3; the stencil skeletons serve arrays of one
component (tuple elements fall back to a gathering ``generate``); seeds and fill values are constants; a ``zipWith`` of arrays of different shape is an error at run time
instead of the intersection; no ``acond`` (branch in Python around compiled functions; ``awhile`` exists, see the
end of this file).
"""
from __future__ import annotations

import builtins
import hashlib
import importlib
import re
from typing import Callable, List, Sequence, Tuple

import numpy as np

_pkg = importlib.import_module(__name__.rsplit(".", 1)[0])
_zip = builtins.zip  # `zip` and `map` below are the array operations
KernelSpec = _pkg.KernelSpec
ArrayType = _pkg.ArrayType

# ------------------------------------------------------------------ program backends
_backends: List[object] = [_pkg]


def _be():
    """Where program nodes go: the package's op-list builder, or a recorder while only the kernels are wanted."""
    return _backends[-1]


class _DryNode:
    def __init__(self, prog, vid, atype):
        self.prog, self.id, self.type = prog, vid, atype
        self.shape_fn = lambda s: ()


class _DryProgram:
    """Stands in for a compiled program while tracing without a device: records the kernels."""

    def __init__(self, input_types):
        self.specs: List[KernelSpec] = []
        self.n = 0
        self.inputs = [self.new(t) for t in input_types]

    def new(self, atype) -> _DryNode:
        self.n += 1
        return _DryNode(self, self.n - 1, atype)


class _DryBackend:
    SCAN_PRIME = _pkg.SCAN_PRIME

    @staticmethod
    def _add(prog, spec, atype):
        prog.specs.append(spec)
        return prog.new(atype)

    def generate(self, prog, spec, env, shape, out_type, scalars=None):
        return self._add(prog, spec, out_type)

    def generate_dims(self, prog, spec, env, dims, out_type, scalars=None):
        return self._add(prog, spec, out_type)

    def map_transposed(self, spec, env, src, out_type, scalars=None):
        return self._add(src.prog, spec, out_type)

    def map_(self, spec, env, out_type, shape_like=None, scalars=None):
        return self._add(env[0].prog, spec, out_type)

    def fold(self, spec, env, out_dtypes, seed=None, all=False, shape_like=None):
        like = shape_like or env[0]
        return self._add(like.prog, spec, ArrayType(0 if (all or like.type.rank <= 1) else like.type.rank - 1, out_dtypes))

    def fold_seg(self, spec, env, offsets, out_dtypes, seed=None, shape_like=None):
        like = shape_like or env[0]
        return self._add(like.prog, spec, ArrayType(like.type.rank, out_dtypes))

    def scan(self, spec, env, out_dtypes, direction=0, kind=0, seed=None, shape_like=None):
        like = shape_like or env[0]
        prog = like.prog
        r = self._add(prog, spec, ArrayType(like.type.rank if kind == _pkg.SCAN_INCLUSIVE else 1, out_dtypes))
        return (r, prog.new(ArrayType(0, out_dtypes))) if kind == _pkg.SCAN_PRIME else r

    def permute(self, spec, env, defaults, shape_like=None):
        return self._add(defaults.prog, spec, defaults.type)

    def stencil(self, spec, src, out_dtype=None, boundary="clamp", constant=None, iters=1):
        return self._add(src.prog, spec, ArrayType(src.type.rank, out_dtype or src.type.dtypes))

    def stencil2(self, spec, a, b, out_dtype, boundary="clamp", constant=None):
        return self._add(a.prog, spec, ArrayType(a.type.rank, out_dtype))


# ------------------------------------------------------------------ scalar types
_CTYPE = {
    np.dtype(np.int8): "signed char", np.dtype(np.int16): "short", np.dtype(np.int32): "int",
    np.dtype(np.int64): "long long", np.dtype(np.uint8): "unsigned char", np.dtype(np.uint16): "unsigned short",
    np.dtype(np.uint32): "unsigned int", np.dtype(np.uint64): "unsigned long long",
    np.dtype(np.float32): "float", np.dtype(np.float64): "double", np.dtype(np.bool_): "unsigned char",
}
_UNSIGNED = {np.dtype(np.int8): "unsigned char", np.dtype(np.int16): "unsigned short", np.dtype(np.int32): "unsigned int",
             np.dtype(np.int64): "unsigned long long"}
BOOL = np.dtype(np.bool_)
I32 = np.dtype(np.int32)
I64 = np.dtype(np.int64)


def ctype(dt) -> str:
    return _CTYPE[np.dtype(dt)]


def _is_float(dt) -> bool:
    return np.dtype(dt).kind == "f"


def _is_int(dt) -> bool:
    return np.dtype(dt).kind in "iu"


def _literal(value, dt) -> str:
    dt = np.dtype(dt)
    if dt == BOOL:
        return "1" if value else "0"
    if _is_float(dt):
        v = float(value)
        if v != v:
            return "(%s)NAN" % ctype(dt)
        if v in (float("inf"), float("-inf")):
            return "(%s%s)INFINITY" % ("-" if v < 0 else "", ctype(dt))
        s = repr(float(np.float32(v))) if dt == np.float32 else repr(v)
        if "e" not in s and "." not in s:
            s += ".0"
        return s + ("f" if dt == np.float32 else "")
    v = int(value)
    info = np.iinfo(dt)
    if not info.min <= v <= info.max:
        raise OverflowError(f"{value} does not fit {dt}")
    if dt == np.int64:
        return f"({v}LL)" if v != info.min else "(-9223372036854775807LL - 1)"
    if dt == np.uint64:
        return f"{v}ULL"
    if dt == np.uint32:
        return f"{v}u"
    if dt == np.int32 and v == info.min:
        return "(-2147483647 - 1)"
    return f"(({ctype(dt)}){v})" if dt.itemsize < 4 else (f"({v})" if v < 0 else str(v))


# ------------------------------------------------------------------ code builders
class _Builder:
    """Statements of one functor method, in single-assignment form (shared sub-expressions are evaluated once,
    like the reference's let-bound scalar temporaries, CodeGen.hs:362-377)."""

    def __init__(self):
        self.lines: List[str] = []
        self.n = 0

    def emit(self, dt, expr: str) -> "Exp":
        name = f"t{self.n}"
        self.n += 1
        self.lines.append(f"const {ctype(dt)} {name} = {expr};")
        return Exp(dt, name)

    def raw(self, line: str):
        self.lines.append(line)


_builders: List[_Builder] = []


def _b() -> _Builder:
    if not _builders:
        raise RuntimeError("scalar expressions exist only inside the functions passed to array operations")
    return _builders[-1]


class Exp:
    """A scalar expression of one primitive type.  Tuples of expressions are Python tuples of Exp."""

    __slots__ = ("dt", "code")
    __array_priority__ = 1000

    def __init__(self, dt, code: str):
        self.dt = np.dtype(dt)
        self.code = code

    # -- helpers
    def _coerce(self, other) -> "Exp":
        if isinstance(other, Exp):
            if other.dt != self.dt:
                raise TypeError(f"operands have types {self.dt} and {other.dt}; convert one with fromIntegral / cast")
            return other
        if isinstance(other, (bool, np.bool_)) and self.dt != BOOL:
            raise TypeError("a Bool where a number is expected")
        if isinstance(other, (float, np.floating)) and not _is_float(self.dt):
            raise TypeError(f"a fractional literal where {self.dt} is expected")
        return Exp(self.dt, _literal(other, self.dt))

    def _bin(self, other, fmt: str, result_dt=None, swap=False) -> "Exp":
        o = self._coerce(other)
        a, b = (o, self) if swap else (self, o)
        return _b().emit(result_dt or self.dt, fmt.format(a=a.code, b=b.code, T=ctype(self.dt),
                                                         U=_UNSIGNED.get(self.dt, ctype(self.dt))))

    def _arith(self, other, op: str, swap=False) -> "Exp":
        if self.dt == BOOL:
            raise TypeError("arithmetic on Bool")
        if self.dt in _UNSIGNED:  # signed integers wrap like the unsigned ones
            return self._bin(other, "({T})(({U}){a} %s ({U}){b})" % op, swap=swap)
        return self._bin(other, "{a} %s {b}" % op, swap=swap)

    # -- arithmetic (CodeGen/Arithmetic.hs)
    def __add__(self, o): return self._arith(o, "+")
    def __radd__(self, o): return self._arith(o, "+", True)
    def __sub__(self, o): return self._arith(o, "-")
    def __rsub__(self, o): return self._arith(o, "-", True)
    def __mul__(self, o): return self._arith(o, "*")
    def __rmul__(self, o): return self._arith(o, "*", True)

    def __truediv__(self, o, swap=False):
        if not _is_float(self.dt):
            raise TypeError("(/) is defined on floating types; use // (div) or quot on integers")
        return self._bin(o, "{a} / {b}", swap=swap)

    def __rtruediv__(self, o): return self.__truediv__(o, True)

    def __floordiv__(self, o, swap=False):  # Haskell div: towards minus infinity
        if not _is_int(self.dt):
            raise TypeError("div is defined on integral types")
        return self._bin(o, "accb::idiv<{T}>({a}, {b})" if self.dt.kind == "i" else "{a} / {b}", swap=swap)

    def __rfloordiv__(self, o): return self.__floordiv__(o, True)

    def __mod__(self, o, swap=False):  # Haskell mod: sign of the divisor
        if not _is_int(self.dt):
            raise TypeError("mod is defined on integral types")
        return self._bin(o, "accb::imod<{T}>({a}, {b})" if self.dt.kind == "i" else "{a} % {b}", swap=swap)

    def __rmod__(self, o): return self.__mod__(o, True)

    def __pow__(self, o):
        if not _is_float(self.dt):
            raise TypeError("(**) is defined on floating types")
        return self._bin(o, "powf({a}, {b})" if self.dt == np.float32 else "pow({a}, {b})")

    def __neg__(self):
        if self.dt in _UNSIGNED:
            return _b().emit(self.dt, f"({ctype(self.dt)})(0 - ({_UNSIGNED[self.dt]}){self.code})")
        return _b().emit(self.dt, f"-{self.code}")

    def __abs__(self):
        if _is_float(self.dt):
            return _b().emit(self.dt, f"{'fabsf' if self.dt == np.float32 else 'fabs'}({self.code})")
        if self.dt.kind == "u":
            return self
        return _b().emit(self.dt, f"({self.code} < 0 ? ({ctype(self.dt)})(0 - ({_UNSIGNED[self.dt]}){self.code}) : {self.code})")

    # -- comparisons: Bool is one byte holding 0 or 1
    def _cmp(self, o, op):
        return self._bin(o, "(unsigned char)({a} %s {b})" % op, BOOL)

    def __lt__(self, o): return self._cmp(o, "<")
    def __le__(self, o): return self._cmp(o, "<=")
    def __gt__(self, o): return self._cmp(o, ">")
    def __ge__(self, o): return self._cmp(o, ">=")
    def __eq__(self, o): return self._cmp(o, "==")  # noqa: structural equality is not needed on Exp
    def __ne__(self, o): return self._cmp(o, "!=")
    __hash__ = None

    # -- logic and bits
    def __and__(self, o):
        return self._bin(o, "(unsigned char)({a} && {b})" if self.dt == BOOL else "{a} & {b}")

    def __or__(self, o):
        return self._bin(o, "(unsigned char)({a} || {b})" if self.dt == BOOL else "{a} | {b}")

    def __xor__(self, o):
        return self._bin(o, "(unsigned char)({a} != {b})" if self.dt == BOOL else "{a} ^ {b}")

    def __invert__(self):
        return _b().emit(self.dt, f"(unsigned char)(!{self.code})" if self.dt == BOOL else f"~{self.code}")

    def __lshift__(self, o):
        return _b().emit(self.dt, f"({ctype(self.dt)})({self.code} << {_index_code(o)})")

    def __rshift__(self, o):
        return _b().emit(self.dt, f"({ctype(self.dt)})({self.code} >> {_index_code(o)})")

    def __bool__(self):
        raise TypeError("an Exp has no truth value while the function is being traced: use cond(c, a, b)")


def _index_code(x) -> str:
    return x.code if isinstance(x, Exp) else str(int(x))


def constant(value, dtype) -> Exp:
    return Exp(dtype, _literal(value, dtype))


def _lift(x, like: Exp = None) -> Exp:
    if isinstance(x, Exp):
        return x
    if like is None:
        raise TypeError("a Python number needs a typed operand next to it, or constant(value, dtype)")
    return like._coerce(x)


def _flat(v) -> Tuple[Exp, ...]:
    """Flatten nested tuples of Exp (Accelerate's tuples are stored as flat SoA components)."""
    if isinstance(v, Exp):
        return (v,)
    out = []
    for e in v:
        out.extend(_flat(e))
    return tuple(out)


def _unflat1(vals: Sequence[Exp]):
    return vals[0] if len(vals) == 1 else tuple(vals)


# -- functions on expressions
def cond(c: Exp, t, e):
    """``c ? t : e`` (Cond, CodeGen.hs:379-386); works component-wise on tuples."""
    if isinstance(t, tuple) or isinstance(e, tuple):
        return tuple(cond(c, a, b) for a, b in _zip(t, e))
    t = _lift(t, e if isinstance(e, Exp) else None)
    e = t._coerce(e)
    if c.dt != BOOL:
        raise TypeError("the condition is not a Bool")
    return _b().emit(t.dt, f"{c.code} ? {t.code} : {e.code}")


def _fn1(names):
    def f(x: Exp) -> Exp:
        if not _is_float(x.dt):
            raise TypeError(f"{names[0]} is defined on floating types")
        return _b().emit(x.dt, f"{names[0] if x.dt == np.float32 else names[1]}({x.code})")
    return f


sqrt, exp, log = _fn1(("sqrtf", "sqrt")), _fn1(("expf", "exp")), _fn1(("logf", "log"))
sin, cos, tan = _fn1(("sinf", "sin")), _fn1(("cosf", "cos")), _fn1(("tanf", "tan"))
asin, acos, atan = _fn1(("asinf", "asin")), _fn1(("acosf", "acos")), _fn1(("atanf", "atan"))
sinh, cosh, tanh = _fn1(("sinhf", "sinh")), _fn1(("coshf", "cosh")), _fn1(("tanhf", "tanh"))
asinh, acosh, atanh = _fn1(("asinhf", "asinh")), _fn1(("acoshf", "acosh")), _fn1(("atanhf", "atanh"))
# not Accelerate primitives: reachable in the reference only as foreign CUDA functions (Foreign/Import.hs:107-111)
erf, erfc = _fn1(("erff", "erf")), _fn1(("erfcf", "erfc"))


def foreign(name: str, result_dtype, *args: Exp) -> Exp:
    """Call a CUDA device function by name (``foreignExp``, CUDAForeignExp, CodeGen.hs:793-805)."""
    return _b().emit(result_dtype, f"{name}({', '.join(a.code for a in args)})")


def atan2(y: Exp, x) -> Exp:
    return y._bin(x, "atan2f({a}, {b})" if y.dt == np.float32 else "atan2({a}, {b})")


def logBase(base: Exp, x) -> Exp:
    return log(_lift(x, base)) / log(base)


def minimum(a, b) -> Exp:
    a = _lift(a, b if isinstance(b, Exp) else None)
    if _is_float(a.dt):
        return a._bin(b, "fminf({a}, {b})" if a.dt == np.float32 else "fmin({a}, {b})")
    return a._bin(b, "({a} < {b} ? {a} : {b})")


def maximum(a, b) -> Exp:
    a = _lift(a, b if isinstance(b, Exp) else None)
    if _is_float(a.dt):
        return a._bin(b, "fmaxf({a}, {b})" if a.dt == np.float32 else "fmax({a}, {b})")
    return a._bin(b, "({a} > {b} ? {a} : {b})")


def quot(a: Exp, b) -> Exp:
    return a._bin(b, "{a} / {b}")


def rem(a: Exp, b) -> Exp:
    return a._bin(b, "{a} % {b}")


def signum(x: Exp) -> Exp:
    if _is_float(x.dt):
        return _b().emit(x.dt, f"({x.code} > 0 ? 1 : ({x.code} < 0 ? -1 : {x.code}))")
    return _b().emit(x.dt, f"({ctype(x.dt)})(({x.code} > 0) - ({x.code} < 0))")


def cast(x: Exp, dtype) -> Exp:
    dtype = np.dtype(dtype)
    if dtype == BOOL:
        return _b().emit(BOOL, f"(unsigned char)({x.code} != 0)")
    return _b().emit(dtype, f"({ctype(dtype)}){x.code}")


fromIntegral = toFloating = cast


def _round_with(fn32: str, fn64: str):
    def f(x: Exp, dtype=np.int32) -> Exp:
        if not _is_float(x.dt):
            raise TypeError("defined on floating types")
        call = f"{fn32 if x.dt == np.float32 else fn64}({x.code})" if fn32 else x.code
        return _b().emit(dtype, f"({ctype(dtype)}){call}")
    return f


floor, ceiling = _round_with("floorf", "floor"), _round_with("ceilf", "ceil")
round_ = _round_with("roundf", "round")  # C round: halves away from zero, as the reference (Arithmetic.hs:281-282)
truncate = _round_with("", "")


def isnan(x: Exp) -> Exp:
    return _b().emit(BOOL, f"(unsigned char)isnan({x.code})")


def isinf(x: Exp) -> Exp:
    return _b().emit(BOOL, f"(unsigned char)isinf({x.code})")


# ------------------------------------------------------------------ indices
class Index:
    """The index an element function is applied at: a linear position plus, on demand, its components
    (outermost first, as Accelerate writes ``Z :. y :. x``)."""

    def __init__(self, lin: Exp, dims: Sequence[Exp]):
        self.lin = lin              # long long
        self.dims = list(dims)      # extents, outermost first, int
        self._comps = None

    @property
    def rank(self):
        return len(self.dims)

    def comps(self) -> Tuple[Exp, ...]:
        if self._comps is None:
            b, r = _b(), self.rank
            if r == 0:
                self._comps = ()
            elif r == 1:
                self._comps = (b.emit(I32, f"(int){self.lin.code}"),)
            else:
                names = [f"ix{b.n}_{d}" for d in range(r)]
                b.n += 1
                b.raw("int " + ", ".join(names) + ";")
                if r == 2:
                    b.raw(f"accb::from_index2({self.dims[1].code}, {self.lin.code}, {names[0]}, {names[1]});")
                elif r == 3:
                    b.raw(f"accb::from_index3({self.dims[1].code}, {self.dims[2].code}, {self.lin.code}, "
                          f"{names[0]}, {names[1]}, {names[2]});")
                else:
                    raise NotImplementedError("ranks above 3")
                self._comps = tuple(Exp(I32, n) for n in names)
        return self._comps

    def __iter__(self):
        return iter(self.comps())

    def __getitem__(self, d):
        return self.comps()[d]

    def __len__(self):
        return self.rank


def _to_linear(idx, dims: Sequence[Exp]) -> Exp:
    """Row-major position of a multi-index (``toIndex``, CodeGen/Base.hs:195-205)."""
    if isinstance(idx, Index):
        return idx.lin
    comps = (idx,) if isinstance(idx, (Exp, int, np.integer)) else tuple(idx)
    if len(comps) != len(dims):
        raise TypeError(f"an index of rank {len(comps)} into an array of rank {len(dims)}")
    comps = [c if isinstance(c, Exp) else constant(c, I32) for c in comps]
    for c in comps:
        if not _is_int(c.dt):
            raise TypeError("index components are integers")
    if not comps:
        return Exp(I64, "0LL")
    code = f"(long long){comps[0].code}"
    for c, d in _zip(comps[1:], dims[1:]):
        code = f"({code} * {d.code} + {c.code})"
    return _b().emit(I64, code)


class _Ignore:
    """The index ``ignore``: a permute drops the element (IndexSpace.hs:200,229-233)."""


ignore = _Ignore()


# ------------------------------------------------------------------ kernel environment
class _KernelEnv:
    """Which manifest arrays a kernel reads and how: element-wise at the kernel's own index (they become the
    functor's ``In`` list and are read with vector loads) or gathered through ``env.in<T>(slot)``."""

    def __init__(self, prog, extent: "_Extent"):
        self.prog = prog
        self.extent = extent
        self.elem: List["Array"] = []
        self.gath: List["Array"] = []
        self.index: Index = None

    def _ordinal_token(self, arr: "Array") -> str:
        return f"@ORD{arr.node.id}@"

    def dims_of(self, arr: "Array") -> List[Exp]:
        """Extents of a manifest array, outermost first, read from the kernel's argument block."""
        if arr not in self.elem and arr not in self.gath:
            self.gath.append(arr)
        r = arr.rank
        return [Exp(I32, f"env.dim({self._ordinal_token(arr)}, {r - 1 - d})") for d in range(r)]

    def read(self, arr: "Array", idx) -> Tuple[Exp, ...]:
        ki = self.index
        if ki is not None and not isinstance(idx, Index) and ki._comps is not None:
            # the components of the kernel's own index, handed back one by one
            t = (idx,) if isinstance(idx, Exp) else (tuple(idx) if isinstance(idx, (tuple, list)) else None)
            if t is not None and len(t) == len(ki._comps) and all(a is b for a, b in _zip(t, ki._comps)):
                idx = ki
        if isinstance(idx, Index) and ki is not None and idx.lin is ki.lin and (
                (idx is ki and self.extent.same_as(arr.extent)) or getattr(idx, "same_position", False)):
            if not any(a is arr for a in self.elem):
                self.elem.append(arr)
            return tuple(Exp(dt, f"@IN{arr.node.id}_{c}@") for c, dt in enumerate(arr.dtypes))
        # anywhere else: a gather (an array read both ways appears twice in the environment)
        if not any(a is arr for a in self.gath):
            self.gath.append(arr)
        lin = _to_linear(idx, self.dims_of(arr))
        return tuple(_b().emit(dt, f"@G{arr.node.id}_{c}@[{lin.code}]") for c, dt in enumerate(arr.dtypes))

    def elementwise(self, arr: "Array") -> Tuple[Exp, ...]:
        """The components of arr as element-wise inputs, whatever the index (the skeleton pairs the positions)."""
        if not any(a is arr for a in self.elem):
            self.elem.append(arr)
        return tuple(Exp(dt, f"@IN{arr.node.id}_{c}@") for c, dt in enumerate(arr.dtypes))

    # -- final assembly
    def in_types(self) -> List[np.dtype]:
        return [dt for a in self.elem for dt in a.dtypes]

    def in_params(self) -> str:
        return "".join(f", {ctype(dt)} in{s}" for s, dt in enumerate(self.in_types()))

    def resolve(self, *codes: str) -> List[str]:
        """Fix the environment (arrays asked only for extents they never used are dropped) and replace the
        placeholders in the bodies of one functor's methods."""
        everything = "\n".join(codes)
        self.gath = [a for a in self.gath
                     if f"@G{a.node.id}_" in everything
                     or (self._ordinal_token(a) in everything and not any(e is a for e in self.elem))]
        out = []
        for code in codes:
            slot = 0
            pre = []
            for ordinal, (elementwise, a) in enumerate([(True, a) for a in self.elem] + [(False, a) for a in self.gath]):
                code = code.replace(self._ordinal_token(a), str(ordinal))  # the first place of an array read both ways
                for c, dt in enumerate(a.dtypes):
                    if elementwise:
                        code = code.replace(f"@IN{a.node.id}_{c}@", f"in{slot}")
                    else:
                        name = f"g{a.node.id}_{c}"
                        if f"@G{a.node.id}_{c}@" in code:
                            pre.append(f"const {ctype(dt)} *{name} = env.in<{ctype(dt)}>({slot});")
                        code = code.replace(f"@G{a.node.id}_{c}@", name)
                    slot += 1
            out.append("\n        ".join(pre + [code]) if pre else code)
        return out

    def nodes(self):
        return [a.node for a in self.elem + self.gath]


class _Dim:
    """One extent of a shape: a constant, plus -- when src is given -- extent `dim` (outermost first) of a
    manifest array.  What Accelerate writes as an Exp Int inside a shape."""

    def __init__(self, src: "Array" = None, dim: int = 0, add: int = 0, src2: "Array" = None, dim2: int = 0):
        # src2 / dim2: a second extent added to the first (the length of `xs ++ ys`)
        self.src, self.dim, self.add, self.src2, self.dim2 = src, dim, int(add), src2, dim2

    def key(self):
        if self.src is None:
            return ("lit", self.add)
        k = ("arr", self.src.prog_find(self.src.node.id), self.dim, self.add)
        return k if self.src2 is None else k + (self.src2.prog_find(self.src2.node.id), self.dim2)

    def code(self, kenv: "_KernelEnv") -> Exp:
        if self.src is None:
            return constant(self.add, I32)
        e = kenv.dims_of(self.src)[self.dim]
        if self.src2 is not None:
            e = Exp(I32, f"({e.code} + {kenv.dims_of(self.src2)[self.dim2].code})")
        return e if self.add == 0 else Exp(I32, f"({e.code} + {_literal(self.add, I32)})")

    def value(self, s) -> int:
        if self.src is None:
            return self.add
        second = self.src2.node.shape_fn(s)[self.dim2] if self.src2 is not None else 0
        return self.src.node.shape_fn(s)[self.dim] + second + self.add

    def __add__(self, n) -> "_Dim":
        if isinstance(n, _Dim):
            if n.src is None:
                return self + n.add
            if self.src is None:
                return n + self.add
            if self.src2 is not None or n.src2 is not None:
                raise NotImplementedError("an extent that adds up more than two array extents")
            return _Dim(self.src, self.dim, self.add + n.add, n.src, n.dim)
        return _Dim(self.src, self.dim, self.add + int(n), self.src2, self.dim2)

    def __sub__(self, n: int) -> "_Dim":
        return _Dim(self.src, self.dim, self.add - int(n), self.src2, self.dim2)


class _Extent:
    """The shape of an array as far as it is known while tracing: that of a manifest array (`like`), a tuple of
    constants (`literal`), or extent by extent (`parts`) from constants and the extents of manifest arrays."""

    def __init__(self, like: "Array" = None, literal: Tuple[int, ...] = None, parts: Sequence[_Dim] = None):
        if parts is not None:
            parts = list(parts)
            if all(p.src is None for p in parts):
                literal, parts = tuple(p.add for p in parts), None
            elif (parts[0].src is not None and len(parts) == parts[0].src.rank
                  and all(p.src is parts[0].src and p.dim == d and p.add == 0 and p.src2 is None
                          for d, p in enumerate(parts))):
                like, parts = parts[0].src, None
        self.like, self.literal, self.parts = like, literal, parts

    @property
    def rank(self):
        if self.parts is not None:
            return len(self.parts)
        return len(self.literal) if self.literal is not None else self.like.rank

    def part(self, d: int) -> _Dim:
        if self.parts is not None:
            return self.parts[d]
        return _Dim(None, 0, self.literal[d]) if self.literal is not None else _Dim(self.like, d, 0)

    def key(self):
        return tuple(self.part(d).key() for d in range(self.rank))

    def same_as(self, other: "_Extent") -> bool:
        return self.key() == other.key()

    def dims(self, kenv: _KernelEnv, own_out: bool) -> List[Exp]:
        """Extents as expressions inside a kernel whose iteration space this is."""
        r = self.rank
        if own_out and self.literal is None:  # a map writes an array of exactly this shape
            return [Exp(I32, f"env.out_dim({r - 1 - d})") for d in range(r)]
        return [self.part(d).code(kenv) for d in range(r)]

    def shape_fn(self):
        parts = [self.part(d) for d in range(self.rank)]
        return lambda s: tuple(p.value(s) for p in parts)


def _unify(prog, a: _Extent, b: _Extent) -> _Extent:
    """Both operands of a zipWith have the same shape: remember to check it at run time."""
    if a.same_as(b):
        return a
    if a.rank != b.rank:
        raise TypeError(f"arrays of rank {a.rank} and {b.rank} zipped")
    prog._shape_checks.append((a.shape_fn(), b.shape_fn()))
    if a.like is not None and b.like is not None:
        ra, rb = a.like.prog_find(a.like.node.id), b.like.prog_find(b.like.node.id)
        prog._same[rb] = ra
    return a if (a.like is not None or b.like is None) else b


# ------------------------------------------------------------------ arrays
class Array:
    """An array term: manifest (the value of a program node) or delayed (extent + element function)."""

    def __init__(self, prog, dtypes, extent: _Extent = None, node=None, fn: Callable = None):
        self.prog = prog
        self.dtypes = [np.dtype(d) for d in dtypes]
        self.node = node
        self.fn = fn
        self.extent = extent if extent is not None else _Extent(like=self)
        # (manifest sources, function of their elements): this array is a map over transposed matrices
        self.transposed = None

    @property
    def rank(self):
        return self.node.type.rank if self.node is not None else self.extent.rank

    @property
    def manifest(self):
        return self.node is not None

    def prog_find(self, nid: int) -> int:
        same = self.prog._same
        while same.get(nid, nid) != nid:
            nid = same[nid]
        return nid

    def at(self, kenv: _KernelEnv, idx) -> Tuple[Exp, ...]:
        """Components of the element at idx, inside the kernel being traced."""
        if self.manifest:
            return kenv.read(self, idx)
        if not isinstance(idx, Index):  # a delayed array indexed at a computed position
            dims = self.extent.dims(kenv, False)
            idx = Index(_to_linear(idx, dims), dims)
        return _flat(self.fn(kenv, idx))

    def __getitem__(self, idx):
        """``arr ! ix`` inside an element function."""
        return _unflat1(self.at(_kenvs[-1], idx))


_kenvs: List[_KernelEnv] = []


def vector(*dtypes) -> ArrayType:
    return ArrayType(1, list(dtypes))


def matrix(*dtypes) -> ArrayType:
    return ArrayType(2, list(dtypes))


def array(rank: int, *dtypes) -> ArrayType:
    return ArrayType(rank, list(dtypes))


def scalar(*dtypes) -> ArrayType:
    return ArrayType(0, list(dtypes))


def _as_array(x) -> Array:
    if not isinstance(x, Array):
        raise TypeError("an array term is expected")
    return x


# -- producers (delayed, fused into their consumer)
def map(f: Callable, arr: Array) -> Array:  # noqa: A001 (the Accelerate name)
    arr = _as_array(arr)
    with _probe(arr.prog) as pr:
        out = _flat(f(_unflat1(pr.symbols(arr.dtypes))))
    res = Array(arr.prog, [e.dt for e in out], arr.extent,
                fn=lambda kenv, ix: f(_unflat1(arr.at(kenv, ix))))
    if arr.transposed is not None:  # a map over a transpose is still a tiled transpose
        srcs, g = arr.transposed
        res.transposed = (srcs, lambda vs: f(g(vs)))
    return res


def zipWith(f: Callable, *arrs: Array) -> Array:
    arrs = [_as_array(a) for a in arrs]
    prog = arrs[0].prog
    ext = arrs[0].extent
    for a in arrs[1:]:
        ext = _unify(prog, ext, a.extent)
    with _probe(prog) as pr:
        out = _flat(f(*[_unflat1(pr.symbols(a.dtypes)) for a in arrs]))
    res = Array(prog, [e.dt for e in out], ext,
                fn=lambda kenv, ix: f(*[_unflat1(a.at(kenv, ix)) for a in arrs]))
    if all(a.transposed is not None for a in arrs):  # transposes zipped: their sources are read tile by tile
        groups = [a.transposed for a in arrs]
        counts = [len(srcs) for srcs, _ in groups]
        starts = [sum(counts[:k]) for k in range(len(groups))]
        res.transposed = ([s for srcs, _ in groups for s in srcs],
                          lambda vs: f(*[g(vs[st:st + n]) for (_, g), st, n in _zip(groups, starts, counts)]))
    return res


def zip(*arrs: Array) -> Array:  # noqa: A001
    return zipWith(lambda *xs: tuple(xs), *arrs)


def unzip(arr: Array) -> Tuple[Array, ...]:
    arr = _as_array(arr)
    return tuple(map(lambda t, c=c: _flat(t)[c], arr) for c in range(len(arr.dtypes)))


def generate(shape, f: Callable, prog=None) -> Array:
    """``generate sh f``: shape is a tuple of ints (outermost first) or ``shape_of(arr)``."""
    if isinstance(shape, _ShapeOf):
        ext, prog = shape.arr.extent, shape.arr.prog
    elif isinstance(shape, _Extent):
        ext = shape
        prog = prog or next((ext.part(d).src.prog for d in range(ext.rank) if ext.part(d).src is not None), None) or _tracing[-1]
    else:
        shape = (shape,) if isinstance(shape, (int, np.integer, _Dim)) else tuple(shape)
        parts = [e if isinstance(e, _Dim) else _Dim(None, 0, int(e)) for e in shape]
        ext = _Extent(parts=parts)
        prog = prog or next((p.src.prog for p in parts if p.src is not None), None) or _tracing[-1]
    with _probe(prog) as pr:
        out = _flat(f(pr.index(ext.rank)))
    return Array(prog, [e.dt for e in out], ext, fn=lambda kenv, ix: f(_user_index(ix)))


def fill(shape, value, dtype) -> Array:
    return generate(shape, lambda ix: constant(value, dtype))


def backpermute(shape, perm: Callable, arr: Array) -> Array:
    """``backpermute sh p arr``: element ix of the result is ``arr ! p ix`` (a gather)."""
    arr = _as_array(arr)
    return generate(shape, lambda ix: arr[perm(ix)], prog=arr.prog)


def _comps(u) -> Tuple[Exp, ...]:
    """The components of what an index function receives (one Exp for vectors, an Index otherwise)."""
    return (u,) if isinstance(u, Exp) else tuple(u)


def dim(arr: Array, d: int) -> _Dim:
    """Extent d (outermost first, negative from the end) of an array, for use in the shape of a ``generate``,
    ``backpermute``, ``replicate`` or ``reshape``; ``dim(a, 0) - 1`` and ``dim(a, 1) + 2`` are shapes too."""
    arr = _as_array(arr)
    return arr.extent.part(d % arr.rank)


def replicate(arr: Array, extent, axis: int = 0) -> Array:
    """``replicate``: a new dimension at position ``axis`` (outermost = 0) of the given extent (an int or a
    ``dim`` of another array) along which the array is repeated."""
    arr = _as_array(arr)
    parts = [arr.extent.part(d) for d in range(arr.rank)]
    parts.insert(axis, extent if isinstance(extent, _Dim) else _Dim(None, 0, int(extent)))

    def f(u):
        c = list(_comps(u))
        del c[axis]
        return arr[tuple(c) if len(c) != 1 else c[0]]
    return generate(_Extent(parts=parts), f, prog=arr.prog)


def slice(arr: Array, axis: int, index) -> Array:  # noqa: A001
    """``slice``: the sub-array at a fixed position of one dimension; index is an int or a function of no arguments
    that returns an Exp (e.g. ``lambda: the(k)``)."""
    arr = _as_array(arr)
    parts = [arr.extent.part(d) for d in range(arr.rank) if d != axis]

    def f(u):
        c = list(_comps(u)) if parts else []
        at = index() if callable(index) else constant(index, I32)
        c.insert(axis, at)
        return arr[tuple(c) if len(c) != 1 else c[0]]
    return generate(_Extent(parts=parts) if parts else (), f, prog=arr.prog)


def transpose(m: Array) -> Array:
    m = _as_array(m)
    if m.rank != 2:
        raise TypeError("transpose of a matrix")
    t = generate(_Extent(parts=[m.extent.part(1), m.extent.part(0)]), lambda u: m[(u[1], u[0])], prog=m.prog)
    if m.manifest:
        # When this array (or maps / zips over it) is made manifest, the source goes through shared-memory tiles
        # instead of being gathered; fused into any other consumer it stays the gather above.
        t.transposed = ([m], lambda vs: vs[0])
    return t


def reshape(shape, arr: Array) -> Array:
    """``reshape``: the same elements in row-major order under another shape of the same size."""
    arr = _as_array(arr)
    new = generate(shape, lambda u: constant(0, I32), prog=arr.prog).extent  # only its extent is wanted
    prog = arr.prog
    size = lambda fn: (lambda s: (int(np.prod(fn(s), dtype=np.int64)),))  # noqa: E731
    prog._shape_checks.append((size(new.shape_fn()), size(arr.extent.shape_fn())))

    def fn(kenv, ix):
        same = Index(ix.lin, arr.extent.dims(kenv, False))
        same.same_position = True  # the element with the same row-major position
        return _unflat1(arr.at(kenv, same))
    return Array(prog, arr.dtypes, new, fn=fn)


def reverse(v: Array) -> Array:
    v = _as_array(v)
    return generate(shape_of(v), lambda i: v[shape(v)[0] - 1 - i])


def init(v: Array) -> Array:
    v = _as_array(v)
    return generate((dim(v, 0) - 1,), lambda i: v[i])


def tail(v: Array) -> Array:
    v = _as_array(v)
    return generate((dim(v, 0) - 1,), lambda i: v[i + 1])


def take(n: int, v: Array) -> Array:
    """The first n elements (n a constant not larger than the length)."""
    v = _as_array(v)
    return generate((int(n),), lambda i: v[i], prog=v.prog)


def drop(n: int, v: Array) -> Array:
    v = _as_array(v)
    return generate((dim(v, 0) - int(n),), lambda i: v[i + int(n)])


def enumFromN(n, start, dtype=np.int32) -> Array:
    """The vector start, start + 1, ... of n elements (n an int or a ``dim``)."""
    return generate((n,), lambda i: cast(i, dtype) + start)


class _ShapeOf:
    def __init__(self, arr: Array):
        self.arr = arr


def shape_of(arr: Array) -> _ShapeOf:
    """The shape of an array, as the extent of a ``generate`` / ``backpermute``."""
    return _ShapeOf(_as_array(arr))


def shape(arr: Array) -> Tuple[Exp, ...]:
    """The extents of an array as expressions (outermost first), inside an element function."""
    arr = _as_array(arr)
    kenv = _kenvs[-1]
    if arr.manifest:
        return tuple(kenv.dims_of(arr))
    return tuple(arr.extent.dims(kenv, False))


def size(arr: Array) -> Exp:
    dims = shape(arr)
    code = "1"
    for d in dims:
        code = f"{code} * {d.code}"
    return _b().emit(I32, code)


def the(arr: Array) -> Exp:
    """The value of a rank-0 array inside an element function."""
    return _as_array(arr)[()]


def _user_index(ix: Index):
    """What a user's index function receives: the single component for vectors, the Index otherwise."""
    return ix.comps()[0] if ix.rank == 1 else ix


# -- probing a function for its result type: trace it on symbols, throw the code away
class _probe:
    def __init__(self, prog):
        self.prog = prog

    def __enter__(self):
        _builders.append(_Builder())
        _kenvs.append(_ProbeEnv(self.prog))
        return self

    def __exit__(self, *exc):
        _builders.pop()
        _kenvs.pop()
        return False

    def symbols(self, dtypes) -> Tuple[Exp, ...]:
        return tuple(Exp(dt, f"p{i}") for i, dt in enumerate(dtypes))

    def index(self, rank: int):
        ix = Index(Exp(I64, "i"), [Exp(I32, f"d{d}") for d in range(rank)])
        return _user_index(ix)


class _ProbeEnv(_KernelEnv):
    def __init__(self, prog):
        super().__init__(prog, _Extent(literal=()))

    def read(self, arr, idx):
        return tuple(Exp(dt, f"q{c}") for c, dt in enumerate(arr.dtypes))

    def dims_of(self, arr):
        return [Exp(I32, f"d{d}") for d in range(arr.rank)]


# ------------------------------------------------------------------ functor printing
_D = "static __device__ __forceinline__"


def _struct_for(name: str, dtypes) -> str:
    fields = " ".join(f"{ctype(dt)} c{c};" for c, dt in enumerate(dtypes))
    return f"struct {name} {{ {fields} }};"


def _trace(fn: Callable) -> Tuple[str, object]:
    """Run fn with a fresh statement list; returns (statements, fn's result)."""
    b = _Builder()
    _builders.append(b)
    try:
        res = fn()
    finally:
        _builders.pop()
    return "\n        ".join(b.lines), res


def _producer_body(arr: Array, kenv: _KernelEnv, own_out: bool):
    """Statements that compute the element of a (delayed or manifest) array at the kernel's index `i`."""
    def go():
        dims = arr.extent.dims(kenv, own_out)
        kenv.index = Index(Exp(I64, "i"), dims)
        _kenvs.append(kenv)
        try:
            return arr.at(kenv, kenv.index)
        finally:
            _kenvs.pop()
    return _trace(go)


def _combine_body(f: Callable, dtypes, a="a", b="b"):
    """Statements of the combination function on two element values held in structs / scalars a and b."""
    n = len(dtypes)

    def go():
        xs = tuple(Exp(dt, f"{a}.c{c}" if n > 1 else a) for c, dt in enumerate(dtypes))
        ys = tuple(Exp(dt, f"{b}.c{c}" if n > 1 else b) for c, dt in enumerate(dtypes))
        _kenvs.append(_NoEnv())
        try:
            out = _flat(f(_unflat1(xs), _unflat1(ys)))
        finally:
            _kenvs.pop()
        if [e.dt for e in out] != [np.dtype(d) for d in dtypes]:
            raise TypeError(f"the combination function returns {[str(e.dt) for e in out]}, expected {[str(d) for d in dtypes]}")
        return out
    return _trace(go)


class _NoEnv:
    def read(self, *a):
        raise NotImplementedError("array access inside a combination function")
    dims_of = read


def _is_plain(body: str, out, op: str, a="a", b="b") -> bool:
    """True when the traced function is exactly `a <op> b` on one component."""
    return len(out) == 1 and body.count("\n") == 0 and body.endswith(f"= {a} {op} {b};") and out[0].code == "t0"


def _name(kind: str, text: str) -> str:
    return kind + hashlib.sha1(text.encode()).hexdigest()[:12]


def _ret(dtypes, vals, sname: str) -> str:
    if len(dtypes) == 1:
        return f"return {vals[0].code};"
    sets = " ".join(f"r.c{c} = {v.code};" for c, v in enumerate(vals))
    return f"{sname} r; {sets} return r;"


def _elem_decl(dtypes, sname="E"):
    """(type name, struct declaration or '') of an element value."""
    if len(dtypes) == 1:
        return ctype(dtypes[0]), ""
    return sname, _struct_for(sname, dtypes)


def _put_take(dtypes, T: str) -> str:
    if len(dtypes) == 1:
        return ""
    refs = ", ".join(f"{ctype(dt)} &o{c}" for c, dt in enumerate(dtypes))
    crefs = ", ".join(f"const {ctype(dt)} &o{c}" for c, dt in enumerate(dtypes))
    puts = " ".join(f"o{c} = r.c{c};" for c in range(len(dtypes)))
    takes = " ".join(f"r.c{c} = o{c};" for c in range(len(dtypes)))
    return (f"    {_D} void put({T} r, {refs}) {{ {puts} }}\n"
            f"    {_D} {T} take({crefs}) {{ {T} r; {takes} return r; }}\n")


def _types_list(dtypes) -> str:
    return "accb::types<" + ", ".join(ctype(d) for d in dtypes) + ">"


# ------------------------------------------------------------------ consumers
def compute(arr: Array) -> Array:
    """Make an array manifest (the ``map`` skeleton over its producer); manifest arrays are returned as they are."""
    arr = _as_array(arr)
    if arr.manifest:
        return arr
    prog = arr.prog
    kenv = _KernelEnv(prog, arr.extent)
    if arr.transposed is not None:
        # map f (transpose m): the same functor as map f m, launched so that m goes through shared-memory tiles
        srcs, g = arr.transposed

        def go():
            kenv.index = Index(Exp(I64, "i"), arr.extent.dims(kenv, True))
            _kenvs.append(kenv)
            try:
                return _flat(g([_unflat1(kenv.elementwise(s)) for s in srcs]))
            finally:
                _kenvs.pop()
        body, vals = _trace(go)
    else:
        body, vals = _producer_body(arr, kenv, own_out=True)
    outs = "".join(f", {ctype(dt)} &out{c}" for c, dt in enumerate(arr.dtypes))
    sets = " ".join(f"out{c} = {v.code};" for c, v in enumerate(vals))
    text, = kenv.resolve(f"{body}\n        {sets}")
    name = _name("Map", text + str(kenv.in_types()))
    src = (f"struct {name} {{\n    using In = {_types_list(kenv.in_types())};\n    using Out = {_types_list(arr.dtypes)};\n"
           f"    {_D} void apply(const accb::Env &env, long long i{kenv.in_params()}{outs}) {{\n        {text}\n    }}\n}};\n")
    spec = KernelSpec("map", name, src)
    out_type = ArrayType(arr.rank, arr.dtypes)
    env_nodes = kenv.nodes()
    if arr.transposed is not None:
        node = _be().map_transposed(spec, env_nodes, arr.transposed[0][0].node, out_type)
        return Array(prog, arr.dtypes, node=node)
    if arr.extent.literal is not None:
        node = _be().generate(prog, spec, env_nodes, arr.extent.literal, out_type)
    elif arr.extent.like is not None:
        like = arr.extent.like.node
        node = _be().map_(spec, env_nodes or [like], out_type, shape_like=like)
    else:  # extents taken one by one from other arrays: the host computes the shape when the program runs
        parts = [arr.extent.part(d) for d in range(arr.rank)]
        node = _be().generate_dims(prog, spec, env_nodes,
                                   [(p.src.node if p.src is not None else None, p.dim, p.add,
                                     p.src2.node if p.src2 is not None else None, p.dim2) for p in parts], out_type)
    return _same_shape(Array(prog, arr.dtypes, node=node), arr)


def _fold_source(kind: str, f, seed, arr: Array, base: str):
    """Functor text shared by folds and scans: In list, get (the fused producer), combine."""
    prog = arr.prog
    kenv = _KernelEnv(prog, arr.extent)
    gbody, gvals = _producer_body(arr, kenv, own_out=False)
    T, decl = _elem_decl(arr.dtypes)
    cbody, cvals = _combine_body(f, arr.dtypes)
    wide = base == "Fold" and arr.dtypes == [np.dtype(np.float32)] and _is_plain(cbody, cvals, "+")
    get, = kenv.resolve(f"{gbody}\n        {_ret(arr.dtypes, gvals, T)}")
    if wide:  # a recognised (+) on Float accumulates in double and rounds once
        head = f"struct @N@ : accb::Fold<float, double> {{\n"
        comb = f"    {_D} double combine(double a, double b) {{ return a + b; }}\n"
    else:
        if len(arr.dtypes) == 1:
            head = f"struct @N@ : accb::{base}<{T}> {{\n"
        else:
            head = (f"{decl}\nstruct @N@ {{\n    typedef {T} elem; typedef {T} acc;\n    using Out = {_types_list(arr.dtypes)};\n"
                    + (f"    {_D} {T} lift({T} x) {{ return x; }}\n    {_D} {T} lower({T} x) {{ return x; }}\n" if base == "Fold" else ""))
        comb = f"    {_D} {T} combine({T} a, {T} b) {{\n        {cbody}\n        {_ret(arr.dtypes, cvals, T)}\n    }}\n"
    put = _put_take(arr.dtypes, T)
    if len(arr.dtypes) > 1:
        put = put.split("\n")[0] + "\n"  # folds and scans only write: put
    text = (head + f"    using In = {_types_list(kenv.in_types())};\n"
            f"    {_D} {T} get(const accb::Env &env, long long i{kenv.in_params()}) {{\n        {get}\n    }}\n" + comb + put + "};\n")
    name = _name(kind, text)
    return KernelSpec(kind_skeleton[kind], name, text.replace("@N@", name)), kenv


kind_skeleton = {"FoldAll": "fold_all", "FoldDim": "fold_dim", "FoldSeg": "fold_seg", "Scan": "scan"}


def _seed_value(seed, dtypes):
    if seed is None:
        return None
    vals = seed if isinstance(seed, (tuple, list)) else [seed]
    if len(vals) != len(dtypes):
        raise TypeError("the seed does not match the element type")
    return tuple(np.asarray(v, dtype=d)[()] for v, d in _zip(vals, dtypes))


def _env_or_like(kenv: _KernelEnv, arr: Array):
    """(env nodes, shape-like node) for a consumer of arr."""
    nodes = kenv.nodes()
    like = arr.extent.like.node  # consumers make arrays of literal extent manifest first
    return nodes or [like], like


def fold(f: Callable, seed, arr: Array) -> Array:
    """``fold f z``: reduce the innermost dimension (everything, for a vector)."""
    return _fold(f, seed, _as_array(arr), False)


def fold1(f: Callable, arr: Array) -> Array:
    return _fold(f, None, _as_array(arr), False)


def foldAll(f: Callable, seed, arr: Array) -> Array:
    return _fold(f, seed, _as_array(arr), True)


def fold1All(f: Callable, arr: Array) -> Array:
    return _fold(f, None, _as_array(arr), True)


def _fold(f, seed, arr: Array, all_: bool) -> Array:
    whole = all_ or arr.rank <= 1
    if arr.extent.like is None and not arr.manifest:
        arr = compute(arr)  # the row structure of a generated array comes from a manifest shape
    spec, kenv = _fold_source("FoldAll" if whole else "FoldDim", f, seed, arr, "Fold")
    nodes, like = _env_or_like(kenv, arr)
    node = _be().fold(spec, nodes, arr.dtypes, seed=_seed_value(seed, arr.dtypes), all=whole, shape_like=like)
    return Array(arr.prog, arr.dtypes, node=node)


def foldSeg(f: Callable, seed, arr: Array, segments: Array) -> Array:
    """``foldSeg f z arr segs``: segs holds the segment LENGTHS (Int32); the offsets are their exclusive scan, as in
    the reference (Execute.hs:320-324)."""
    arr, segments = _as_array(arr), _as_array(segments)
    if segments.dtypes != [I32]:
        raise TypeError("segment lengths are Int32")
    offsets = scanl(lambda a, b: a + b, 0, segments)
    if arr.extent.like is None and not arr.manifest:
        arr = compute(arr)
    spec, kenv = _fold_source("FoldSeg", f, seed, arr, "Fold")
    nodes, like = _env_or_like(kenv, arr)
    node = _be().fold_seg(spec, nodes, offsets.node, arr.dtypes, seed=_seed_value(seed, arr.dtypes), shape_like=like)
    return Array(arr.prog, arr.dtypes, node=node)


def fold1Seg(f: Callable, arr: Array, segments: Array) -> Array:
    return foldSeg(f, None, arr, segments)


def _same_shape(new: Array, old: Array) -> Array:
    """The manifest array `new` has the shape of `old` by construction: reads of it at the index of a kernel that
    iterates over `old` are element-wise."""
    if old.extent.like is not None and old.extent.like.node is not new.node:
        new.prog._same[new.node.id] = old.prog_find(old.extent.like.node.id)
    return new


def _segmented_scan(f: Callable, arr: Array, flag_of: Callable, direction) -> Array:
    """Inclusive scan of the row-major sequence of arr that restarts wherever flag_of(kenv, ix) holds: at the
    first element of a row or segment for a left scan, at the last one for a right scan.  The value type is
    widened to (value, flag) with the usual segmented operator, which is associative whenever f is; only the
    value components are written."""
    if arr.extent.like is None and not arr.manifest:
        arr = compute(arr)
    prog, right = arr.prog, direction == _pkg.SCAN_RIGHT
    kenv = _KernelEnv(prog, arr.extent)
    nv = len(arr.dtypes)

    def produce():
        kenv.index = Index(Exp(I64, "i"), arr.extent.dims(kenv, False))
        _kenvs.append(kenv)
        try:
            vals = arr.at(kenv, kenv.index)
            flag = flag_of(kenv, kenv.index)
            if flag.dt != BOOL:
                raise TypeError("segment flags are Bool")
            return vals + (flag,)
        finally:
            _kenvs.pop()
    gbody, gvals = _trace(produce)
    dtypes = arr.dtypes + [BOOL]
    decl = _struct_for("E", dtypes)

    def combine():
        # left scans: a precedes b and b's flag restarts; right scans call combine(later, earlier): the later
        # element is the first argument and its flag restarts (the new element is the left argument of f)
        first = tuple(Exp(dt, f"a.c{c}") for c, dt in enumerate(arr.dtypes))
        second = tuple(Exp(dt, f"b.c{c}") for c, dt in enumerate(arr.dtypes))
        fa, fb = Exp(BOOL, f"a.c{nv}"), Exp(BOOL, f"b.c{nv}")
        _kenvs.append(_NoEnv())
        try:
            both = _flat(f(_unflat1(first), _unflat1(second)))
        finally:
            _kenvs.pop()
        restart, kept = (fa, first) if right else (fb, second)
        return tuple(cond(restart, k, v) for k, v in _zip(kept, both)) + (fa | fb,)
    cbody, cvals = _trace(combine)
    get, = kenv.resolve(f"{gbody}\n        {_ret(dtypes, gvals, 'E')}")
    refs = ", ".join(f"{ctype(dt)} &o{c}" for c, dt in enumerate(arr.dtypes))
    puts = " ".join(f"o{c} = r.c{c};" for c in range(nv))
    text = (f"{decl}\nstruct @N@ {{\n    typedef E elem; typedef E acc;\n    using In = {_types_list(kenv.in_types())};\n"
            f"    using Out = {_types_list(arr.dtypes)};\n"
            f"    {_D} E get(const accb::Env &env, long long i{kenv.in_params()}) {{\n        {get}\n    }}\n"
            f"    {_D} E combine(E a, E b) {{\n        {cbody}\n        {_ret(dtypes, cvals, 'E')}\n    }}\n"
            f"    {_D} void put(E r, {refs}) {{ {puts} }}\n}};\n")
    name = _name("SegScan", text)
    spec = KernelSpec("scan", name, text.replace("@N@", name))
    nodes, like = _env_or_like(kenv, arr)
    node = _be().scan(spec, nodes, arr.dtypes, direction=direction, kind=_pkg.SCAN_INCLUSIVE, seed=None, shape_like=like)
    return _same_shape(Array(prog, arr.dtypes, node=node), arr)


def _segment_flags(arr: Array, seglens: Array, right: bool) -> Array:
    """A Bool array of arr's shape: True at the first (left scans) or last (right scans) element of every
    non-empty segment."""
    seglens = _as_array(seglens)
    if seglens.dtypes != [I32] or seglens.rank != 1 or arr.rank != 1:
        raise TypeError("segment lengths are a vector of Int32, the data a vector")
    offs = scanl(lambda a, b: a + b, 0, seglens)
    lens = seglens
    where = (lambda s: cond_index(lens[s] > 0, offs[s + 1] - 1)) if right else (lambda s: cond_index(lens[s] > 0, offs[s]))
    flags = permute(lambda x, y: x, fill(shape_of(arr), False, np.bool_), where, fill(shape_of(seglens), True, np.bool_))
    return _same_shape(flags, arr)


def scanl1Seg(f: Callable, arr: Array, seglens: Array) -> Array:
    """``scanl1Seg f arr segs``: an inclusive left scan inside every segment (segs = segment lengths)."""
    arr = _as_array(arr)
    if not arr.manifest:
        arr = compute(arr)
    flags = _segment_flags(arr, seglens, False)
    return _segmented_scan(f, arr, lambda kenv, ix: flags.at(kenv, ix)[0], _pkg.SCAN_LEFT)


def scanr1Seg(f: Callable, arr: Array, seglens: Array) -> Array:
    arr = _as_array(arr)
    if not arr.manifest:
        arr = compute(arr)
    flags = _segment_flags(arr, seglens, True)
    return _segmented_scan(f, arr, lambda kenv, ix: flags.at(kenv, ix)[0], _pkg.SCAN_RIGHT)


def _scan_prime_seg(f: Callable, seed, arr: Array, seglens: Array, right: bool):
    """scanl'Seg / scanr'Seg: inside every segment the exclusive scan (same length as the data), and one total per
    segment.  The exclusive scan is the inclusive segmented scan of the data shifted by one element, the seed
    entering at each segment's first (last, for right scans) position; the totals are a foldSeg."""
    arr = _as_array(arr)
    if not arr.manifest:
        arr = compute(arr)
    flags = _segment_flags(arr, seglens, right)
    zs = _seed_value(seed, arr.dtypes)
    src = arr

    def shifted(i):
        j = minimum(i + 1, shape(src)[0] - 1) if right else maximum(i - 1, 0)
        vals = _flat(src[j])
        return _unflat1(tuple(cond(flags[i], constant(z, dt), v) for z, dt, v in _zip(zs, src.dtypes, vals)))
    moved = generate(shape_of(src), shifted)
    body = _segmented_scan(f, moved, lambda kenv, ix: flags.at(kenv, ix)[0], _pkg.SCAN_RIGHT if right else _pkg.SCAN_LEFT)
    return body, foldSeg(f, seed, src, seglens)


def concat(xs: Array, ys: Array) -> Array:
    """``xs ++ ys`` on vectors: a generate over the sum of the two lengths."""
    xs, ys = _as_array(xs), _as_array(ys)
    if xs.rank != 1 or ys.rank != 1 or xs.dtypes != ys.dtypes:
        raise TypeError("(++) here joins two vectors of one element type")

    def pick(i):
        nx, ny = shape(xs)[0], shape(ys)[0]
        a = _flat(xs[maximum(minimum(i, nx - 1), 0)])
        b = _flat(ys[maximum(minimum(i - nx, ny - 1), 0)])
        return _unflat1(tuple(cond(i < nx, u, v) for u, v in _zip(a, b)))
    return generate(_Extent(parts=[xs.extent.part(0) + ys.extent.part(0)]), pick, prog=xs.prog)


def _scan_seg_exclusive(f: Callable, seed, arr: Array, seglens: Array, right: bool) -> Array:
    """scanlSeg / scanrSeg: every segment grows by one element, the seed in front (behind, for right scans), so the
    result has length(data) + length(segments) elements.  The seed positions are marked in the widened index
    space, a running count of the marks tells every other position which element of the data it holds, and the
    inclusive segmented scan of that widened vector, restarting at the marks, is the result."""
    arr, seglens = _as_array(arr), _as_array(seglens)
    if seglens.dtypes != [I32] or seglens.rank != 1 or arr.rank != 1:
        raise TypeError("segment lengths are a vector of Int32, the data a vector")
    if not arr.manifest:
        arr = compute(arr)
    if not seglens.manifest:
        seglens = compute(seglens)
    zs = _seed_value(seed, arr.dtypes)
    wide = _Extent(parts=[arr.extent.part(0) + seglens.extent.part(0)])
    offs = compute(scanl(lambda a, b: a + b, 0, seglens))
    marks = permute(lambda x, y: x, fill(wide, False, np.bool_), lambda s: (offs[s + 1] if right else offs[s]) + s,
                    fill(shape_of(seglens), True, np.bool_))
    counts = _same_shape(compute(scanl1(lambda a, b: a + b, map(lambda m: cond(m, constant(1, I32), constant(0, I32)), marks))), marks)
    src = arr

    def widened(j):
        at = maximum(minimum(j - counts[j], shape(src)[0] - 1), 0)  # marks up to here are not data
        vals = _flat(src[at])
        return _unflat1(tuple(cond(marks[j], constant(z, dt), v) for z, dt, v in _zip(zs, src.dtypes, vals)))
    moved = generate(shape_of(marks), widened)  # fused into the scan
    return _segmented_scan(f, moved, lambda kenv, ix: marks.at(kenv, ix)[0], _pkg.SCAN_RIGHT if right else _pkg.SCAN_LEFT)


def scanlSeg(f, seed, arr, seglens): return _scan_seg_exclusive(f, seed, arr, seglens, False)
def scanrSeg(f, seed, arr, seglens): return _scan_seg_exclusive(f, seed, arr, seglens, True)
def scanl_Seg(f, seed, arr, seglens): return _scan_prime_seg(f, seed, arr, seglens, False)   # scanl'Seg
def scanr_Seg(f, seed, arr, seglens): return _scan_prime_seg(f, seed, arr, seglens, True)    # scanr'Seg


def _scan(f, seed, arr: Array, direction, kind):
    arr = _as_array(arr)
    if arr.rank != 1:
        # Along the innermost dimension of a matrix or cube (the reference rejects these, PrefixSum.hs:39-46):
        # an inclusive scan of the whole array that restarts at the start (end, for right scans) of every row.
        right = direction == _pkg.SCAN_RIGHT
        if kind == _pkg.SCAN_PRIME:
            raise NotImplementedError("scanl' / scanr' along the innermost dimension: use scanl / scanr and slice the totals off")
        if kind == _pkg.SCAN_EXCLUSIVE:
            # every row grows by one element: the seed goes first (last, for scanr) and the inclusive scan of
            # the widened rows is the exclusive scan of the original ones
            zs = _seed_value(seed, arr.dtypes)
            src, r = arr, arr.rank
            parts = [src.extent.part(d) for d in range(r - 1)] + [src.extent.part(r - 1) + 1]

            def widened(u):
                c = list(_comps(u))
                x, cols = c[-1], shape(src)[-1]
                at_seed = (x == cols) if right else (x == 0)
                inside = minimum(x, cols - 1) if right else maximum(x - 1, 0)
                vals = _flat(src[tuple(c[:-1] + [inside])])
                return _unflat1(tuple(cond(at_seed, constant(z, dt), v) for z, dt, v in _zip(zs, src.dtypes, vals)))
            arr = generate(_Extent(parts=parts), widened, prog=src.prog)

        def row_edge(kenv, ix):
            x = ix.comps()[-1]
            return (x == ix.dims[-1] - 1) if right else (x == 0)
        return _segmented_scan(f, arr, row_edge, direction)
    if arr.extent.like is None and not arr.manifest:
        arr = compute(arr)
    spec, kenv = _fold_source("Scan", f, seed, arr, "Scan")
    nodes, like = _env_or_like(kenv, arr)
    res = _be().scan(spec, nodes, arr.dtypes, direction=direction, kind=kind, seed=_seed_value(seed, arr.dtypes),
                    shape_like=like)
    if kind == _pkg.SCAN_PRIME:
        return Array(arr.prog, arr.dtypes, node=res[0]), Array(arr.prog, arr.dtypes, node=res[1])
    return Array(arr.prog, arr.dtypes, node=res)


def scanl(f, seed, arr): return _scan(f, seed, arr, _pkg.SCAN_LEFT, _pkg.SCAN_EXCLUSIVE)
def scanr(f, seed, arr): return _scan(f, seed, arr, _pkg.SCAN_RIGHT, _pkg.SCAN_EXCLUSIVE)
def scanl1(f, arr): return _scan(f, None, arr, _pkg.SCAN_LEFT, _pkg.SCAN_INCLUSIVE)
def scanr1(f, arr): return _scan(f, None, arr, _pkg.SCAN_RIGHT, _pkg.SCAN_INCLUSIVE)
def scanl_(f, seed, arr): return _scan(f, seed, arr, _pkg.SCAN_LEFT, _pkg.SCAN_PRIME)    # scanl'
def scanr_(f, seed, arr): return _scan(f, seed, arr, _pkg.SCAN_RIGHT, _pkg.SCAN_PRIME)   # scanr'


def permute(f: Callable, defaults: Array, perm: Callable, arr: Array) -> Array:
    """``permute f defaults p arr``: out[p ix] = f (arr ! ix) (out ! p ix); ``p`` may return ``ignore``."""
    defaults, arr = compute(_as_array(defaults)), _as_array(arr)
    if defaults.dtypes != arr.dtypes:
        raise TypeError("defaults and source differ in element type")
    prog = arr.prog
    if arr.extent.like is None and not arr.manifest:
        arr = compute(arr)
    kenv = _KernelEnv(prog, arr.extent)
    gbody, gvals = _producer_body(arr, kenv, own_out=False)
    drank = defaults.rank
    ddims = [Exp(I32, f"env.out_dim({drank - 1 - d})") for d in range(drank)]

    def index_fn():
        _kenvs.append(kenv)
        try:
            ix = Index(Exp(I64, "i"), arr.extent.dims(kenv, False))
            kenv.index = ix
            dst = perm(_user_index(ix))
            if dst is ignore:
                return Exp(I64, "-1LL")
            if isinstance(dst, _CondIndex):
                lin = _to_linear(dst.ix, ddims)
                return _b().emit(I64, f"{dst.c.code} ? {lin.code} : -1LL")
            return _to_linear(dst, ddims)
        finally:
            _kenvs.pop()
    ibody, ival = _trace(index_fn)
    T, decl = _elem_decl(arr.dtypes)
    cbody, cvals = _combine_body(f, arr.dtypes, "x", "y")
    dt0 = arr.dtypes[0]
    # how the combiner can be made atomic: compare its text with that of the known operators
    atomic, ident = "Lock", None
    if len(arr.dtypes) == 1:
        def same_as(g):
            body, vals = _combine_body(g, arr.dtypes, "x", "y")
            return body == cbody and vals[0].code == cvals[0].code
        wide = dt0.itemsize >= 4
        if cbody == "" and cvals[0].code == "x":
            atomic = "None"                                     # the old value is ignored: a plain store
        elif wide and same_as(lambda x, y: x + y):
            atomic, ident = "Add", 0
        elif wide and _is_int(dt0) and same_as(minimum):
            atomic, ident = "Min", np.iinfo(dt0).max
        elif wide and _is_int(dt0) and same_as(maximum):
            atomic, ident = "Max", np.iinfo(dt0).min
        elif wide and _is_int(dt0) and same_as(lambda x, y: x & y):
            atomic, ident = "And", (np.iinfo(dt0).max if dt0.kind == "u" else -1)
        elif wide and _is_int(dt0) and same_as(lambda x, y: x | y):
            atomic, ident = "Or", 0
        elif wide and _is_int(dt0) and same_as(lambda x, y: x ^ y):
            atomic, ident = "Xor", 0
        elif wide:
            atomic = "Cas"                                      # any other function of one 4- or 8-byte value
    get, index = kenv.resolve(f"{gbody}\n        {_ret(arr.dtypes, gvals, T)}", f"{ibody}\n        return {ival.code};")
    if len(arr.dtypes) == 1:
        head = f"struct @N@ : accb::Permute<{T}, accb::Atomic::{atomic}> {{\n"
    else:
        head = (f"{decl}\nstruct @N@ {{\n    typedef {T} elem;\n    static constexpr accb::Atomic atomic = accb::Atomic::Lock;\n"
                f"    using Out = {_types_list(arr.dtypes)};\n")
    idn = f"    {_D} {T} identity() {{ return {_literal(ident, dt0)}; }}\n" if ident is not None else ""
    text = (head + f"    using In = {_types_list(kenv.in_types())};\n"
            f"    {_D} long long index(const accb::Env &env, long long i{kenv.in_params()}) {{\n        {index}\n    }}\n"
            f"    {_D} {T} get(const accb::Env &env, long long i{kenv.in_params()}) {{\n        {get}\n    }}\n"
            f"    {_D} {T} combine({T} x, {T} y) {{\n        {cbody}\n        {_ret(arr.dtypes, cvals, T)}\n    }}\n"
            + idn + _put_take(arr.dtypes, T) + "};\n")
    # native 4-byte reductions can be privatised in shared memory when the destination fits (the host decides)
    skeleton = "permute_smem" if ident is not None and dt0.itemsize == 4 and atomic in ("Add", "Min", "Max") else "permute"
    name = _name("Permute", text + skeleton)
    spec = KernelSpec(skeleton, name, text.replace("@N@", name))
    nodes, like = _env_or_like(kenv, arr)
    node = _be().permute(spec, nodes, defaults.node, shape_like=like)
    return Array(prog, arr.dtypes, node=node)


class _CondIndex:
    def __init__(self, c: Exp, ix):
        self.c, self.ix = c, ix


def compact(pred: Callable, arr: Array):
    """Stream compaction, the core of Accelerate's ``filter``: the elements of a vector that satisfy ``pred``, in
    order, at the front of a vector of the ORIGINAL length, and their number as a Scalar Int32.  (``filter`` itself
    returns a vector whose length is that number: a shape known only once the device has computed it, which a
    caller obtains by slicing with the count.)  An exclusive scan of the flags gives every kept element its
    position; a permute without atomics moves it there."""
    arr = _as_array(arr)
    if arr.rank != 1:
        raise TypeError("compact takes a vector")
    if not arr.manifest:
        arr = compute(arr)
    src = arr
    keep = compute(map(lambda e: pred(e), src))
    if keep.dtypes != [BOOL]:
        raise TypeError("the predicate yields a Bool")
    where, count = scanl_(lambda a, b: a + b, 0, map(lambda k: cond(k, constant(1, I32), constant(0, I32)), keep))
    where = _same_shape(compute(where), src)
    zeros = generate(shape_of(src), lambda i: _unflat1(tuple(constant(0, dt) for dt in src.dtypes)))
    moved = permute(lambda x, y: x, zeros, lambda i: cond_index(keep[i], where[i]), src)
    return moved, count


def cond_index(c: Exp, ix) -> _CondIndex:
    """A destination that is ``ix`` when c holds and ``ignore`` otherwise."""
    return _CondIndex(c, ix)


def _stencil_spec(f: Callable, narr: int, tin, tout_probe, pattern, kind: str):
    wy, wx = pattern
    ry, rx = wy // 2, wx // 2

    def go():
        wins = []
        for a in range(narr):
            name = "t" if narr == 1 else "ab"[a]
            w = [[Exp(tin[a], f"{name}[{y}][{x}]") for x in range(wx)] for y in range(wy)]
            wins.append(w[0] if wy == 1 and tout_probe == "rank1" else w)
        _kenvs.append(_NoEnv())
        try:
            return _flat(f(*wins))
        finally:
            _kenvs.pop()
    body, out = _trace(go)
    if len(out) != 1:
        raise NotImplementedError("stencils over tuples")
    args = ", ".join(f"const {ctype(tin[a])} (&{'t' if narr == 1 else 'ab'[a]})[{wy}][{wx}]" for a in range(narr))
    text = (f"struct @N@ : accb::Stencil<{ctype(tin[0])}, {ctype(out[0].dt)}, {ry}, {rx}> {{\n"
            f"    {_D} {ctype(out[0].dt)} apply(const accb::Env &, {args}) {{\n        {body}\n        return {out[0].code};\n    }}\n}};\n")
    name = _name(kind, text)
    return KernelSpec("stencil" if narr == 1 else "stencil2", name, text.replace("@N@", name)), out[0].dt


def _stencil3_spec(f: Callable, tin, pattern):
    """The functor of the rank-3 stencil skeleton (csrc/skeletons/stencil3.cuh): t[dz][dy][dx]."""
    wz, wy, wx = pattern

    def go():
        w = [[[Exp(tin[0], f"t[{z}][{y}][{x}]") for x in range(wx)] for y in range(wy)] for z in range(wz)]
        _kenvs.append(_NoEnv())
        try:
            return _flat(f(w))
        finally:
            _kenvs.pop()
    body, out = _trace(go)
    if len(out) != 1:
        raise NotImplementedError("stencils over tuples")
    # the taps the traced function reads: the skeleton neither loads nor shuffles the rest
    read = {tuple(int(g) for g in m.groups()) for m in re.finditer(r"\bt\[(\d+)\]\[(\d+)\]\[(\d+)\]", body + " " + out[0].code)}
    table = ", ".join("{" + ", ".join("{" + ", ".join("true" if (z, y, x) in read else "false" for x in range(wx)) + "}"
                                         for y in range(wy)) + "}" for z in range(wz))
    text = (f"struct @N@ : accb::Stencil3<{ctype(tin[0])}, {ctype(out[0].dt)}, {wz // 2}, {wy // 2}, {wx // 2}> {{\n"
            f"    static constexpr bool uses(int z, int y, int x) {{\n"
            f"        constexpr bool read[{wz}][{wy}][{wx}] = {{{table}}};\n        return read[z][y][x];\n    }}\n"
            f"    {_D} {ctype(out[0].dt)} apply(const accb::Env &, const {ctype(tin[0])} (&t)[{wz}][{wy}][{wx}]) {{\n"
            f"        {body}\n        return {out[0].code};\n    }}\n}};\n")
    name = _name("Stencil3", text)
    return KernelSpec("stencil3", name, text.replace("@N@", name)), out[0].dt


def _bound(i: Exp, n: Exp, mode: str) -> Exp:
    """One coordinate through the boundary function (Stencil/Extra.hs:200-226); Constant clamps, the caller
    replaces the value."""
    if mode in ("clamp", "constant"):
        return maximum(minimum(i, n - 1), 0)
    if mode == "mirror":
        return cond(i < 0, -i, cond(i >= n, n - (i - n + 2), i))
    if mode == "wrap":
        return cond(i < 0, n + i, cond(i >= n, i - n, i))
    raise ValueError(f"unknown boundary {mode!r}")


def _stencil_by_gather(f: Callable, boundary, arr: Array, pattern) -> Array:
    """A stencil of any rank and element type as a ``generate`` that gathers."""
    mode, cval = (boundary[0], boundary[1]) if isinstance(boundary, tuple) else (boundary, None)
    pattern = tuple(pattern)
    if len(pattern) != arr.rank or any(w % 2 == 0 for w in pattern):
        raise TypeError("the neighbourhood has one odd extent per dimension")
    radii = [w // 2 for w in pattern]

    def at(u):
        centre, dims = _comps(u), shape(arr)

        def tap(offs):
            moved = [c + o if o else c for c, o in _zip(centre, offs)]
            idx = tuple(_bound(m, n, mode) if o else m for m, n, o in _zip(moved, dims, offs))
            vals = _flat(arr[idx if len(idx) != 1 else idx[0]])
            if mode == "constant" and any(offs):
                inside = None
                for m, n, o in _zip(moved, dims, offs):
                    if o:
                        ok = (m >= 0) & (m < n)
                        inside = ok if inside is None else inside & ok
                consts = cval if isinstance(cval, (tuple, list)) else [cval]
                vals = tuple(cond(inside, v, constant(c, v.dt)) for v, c in _zip(vals, consts))
            return _unflat1(vals)

        def nest(d, offs):
            if d == arr.rank:
                return tap(offs)
            return [nest(d + 1, offs + [o]) for o in range(-radii[d], radii[d] + 1)]
        return f(nest(0, []))
    return generate(shape_of(arr), at)


def stencil(f: Callable, boundary, arr: Array, pattern=None, iterate: int = 1) -> Array:
    """``stencil f boundary arr``.  f receives the neighbourhood as nested lists, ``t[dy][dx]`` for a matrix
    (``t[dx]`` for a vector, ``t[dz][dy][dx]`` for a cube), centre in the middle; pattern = the extents of the
    neighbourhood, 3 per dimension by default.  boundary: "clamp", "mirror", "wrap" or ("constant", value).
    iterate > 1 applies it repeatedly.  Vectors, matrices and cubes of one component go through the stencil
    skeletons (tiles staged in shared memory); tuple elements gather, as every stencil of the reference does."""
    arr = compute(_as_array(arr))
    if arr.rank == 1 and isinstance(pattern, int):
        pattern = (1, pattern)
    cube = (arr.rank == 3 and len(arr.dtypes) == 1 and np.dtype(arr.dtypes[0]).itemsize == 4 and
            all(w % 2 == 1 and w <= 5 for w in (pattern or (3, 3, 3))))
    if cube:  # the rank-3 skeleton: a block marches along z with the planes it needs in shared memory
        spec, tout = _stencil3_spec(f, arr.dtypes, tuple(pattern or (3, 3, 3)))
        mode, const = (boundary[0], np.asarray(boundary[1], dtype=arr.dtypes[0])[()]) if isinstance(boundary, tuple) else (boundary, None)
        if np.dtype(tout).itemsize == 4 and (iterate <= 1 or tout == arr.dtypes[0]):
            node = _be().stencil(spec, arr.node, out_dtype=[tout], boundary=mode, constant=const, iters=iterate)
            return Array(arr.prog, [tout], node=node)
    if len(arr.dtypes) != 1 or arr.rank not in (1, 2) or (pattern is not None and pattern[-1] > 9):
        # tuple elements, 8-byte cubes, very wide neighbourhoods: the way the reference does every stencil -- each element
        # gathers its neighbourhood through the boundary function (CodeGen/Stencil.hs:55-114, Stencil/Extra.hs:191-226)
        out = arr
        for _ in range(max(1, iterate)):
            out = compute(_stencil_by_gather(f, boundary, out, pattern or (3,) * arr.rank))
        return out
    pattern = pattern or ((1, 3) if arr.rank == 1 else (3, 3))
    spec, tout = _stencil_spec(f, 1, arr.dtypes, "rank1" if arr.rank == 1 else "rank2", pattern, "Stencil")
    mode, const = (boundary[0], np.asarray(boundary[1], dtype=arr.dtypes[0])[()]) if isinstance(boundary, tuple) else (boundary, None)
    if iterate > 1 and tout != arr.dtypes[0]:
        raise TypeError("an iterated stencil maps its element type to itself")
    node = _be().stencil(spec, arr.node, out_dtype=[tout], boundary=mode, constant=const, iters=iterate)
    return Array(arr.prog, [tout], node=node)


def stencil2(f: Callable, boundary, a: Array, b: Array, pattern=None) -> Array:
    a, b = compute(_as_array(a)), compute(_as_array(b))
    if len(a.dtypes) != 1 or len(b.dtypes) != 1 or a.rank != b.rank or a.rank not in (1, 2):
        raise NotImplementedError("stencil2 over two vectors or two matrices of one component each")
    if a.dtypes != b.dtypes:
        raise NotImplementedError("stencil2 over sources of different element types")
    pattern = pattern or ((1, 3) if a.rank == 1 else (3, 3))
    spec, tout = _stencil_spec(f, 2, a.dtypes + b.dtypes, "rank1" if a.rank == 1 else "rank2", pattern, "Stencil2")
    mode, const = (boundary[0], np.asarray(boundary[1], dtype=a.dtypes[0])[()]) if isinstance(boundary, tuple) else (boundary, None)
    node = _be().stencil2(spec, a.node, b.node, [tout], boundary=mode, constant=const)
    return Array(a.prog, [tout], node=node)


# ------------------------------------------------------------------ running programs
_tracing: List[object] = []


def _trace_program(f: Callable, prog, inputs):
    """Apply the user's array function to the program's inputs; returns the (manifest) output nodes."""
    prog._same, prog._shape_checks = {}, []
    _tracing.append(prog)
    try:
        outs = f(*[Array(prog, a.type.dtypes, node=a) for a in inputs])
        outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
        return [compute(o).node for o in outs]
    finally:
        _tracing.pop()


def specs(f: Callable, *input_types: ArrayType) -> List[KernelSpec]:
    """The kernels an array function compiles to, in program order, without a device: what the reference's
    ``-ddump-cc`` shows (Compile.hs:560-562)."""
    prog = _DryProgram(input_types)
    _backends.append(_DryBackend())
    try:
        _trace_program(f, prog, prog.inputs)
    finally:
        _backends.pop()
    return prog.specs


def run1With(ctx, f: Callable, *input_types: ArrayType):
    """Compile an array function once (``run1With``, CUDA.hs:312-330); the result maps numpy arrays to numpy arrays."""
    if not input_types:
        raise NotImplementedError("a program without array arguments: pass the constants as arrays")
    prog = _pkg.run1With(ctx, lambda *accs: _trace_program(f, accs[0].prog, accs), *input_types)
    checks = prog._shape_checks
    if checks:
        first = prog._shape_fns[0]

        def checked(s):
            for fa, fb in checks:
                if tuple(fa(s)) != tuple(fb(s)):
                    raise ValueError(f"zipped arrays differ in shape: {tuple(fa(s))} and {tuple(fb(s))}")
            return first(s)
        prog._shape_fns[0] = checked
    return prog


def run1(f: Callable, *input_types: ArrayType):
    return run1With(_pkg.default_context(), f, *input_types)


def runWith(ctx, f: Callable, *arrays):
    """Compile and run once on numpy arrays (``runWith``, CUDA.hs:248-251)."""
    prog = run1With(ctx, f, *_pkg._types_of(arrays))
    try:
        return prog(*arrays)
    finally:
        prog.destroy()


def run(f: Callable, *arrays):
    return runWith(_pkg.default_context(), f, *arrays)


_awhile_keys = iter(range(0x7A000000, 0x7FFFFFFF))


def awhile(cond: Callable, body: Callable, *arrays, ctx=None, device: bool = True, max_iters: int = 1 << 20):
    """``awhile cond body init`` on numpy arrays: while ``cond(*state)`` (a Scalar Bool) holds, the state becomes
    ``body(*state)``, which must keep every array's type and shape.  The state stays on the device throughout;
    with ``device=True`` so does the flag (one CUDA graph with a conditional WHILE node), otherwise it is read
    back once per iteration as the reference does (Awhile, CUDA/Execute.hs:236-244).
    Returns ``(final_state, iterations)``."""
    import ctypes as C
    ctx = ctx or _pkg.default_context()
    types = _pkg._types_of(arrays)
    L, h = _pkg.lib(), ctx.handle
    progs, keys, state, hosts = [], [], [], []
    stream = C.c_void_p()
    _pkg._check(L.accb_stream_acquire(h, C.byref(stream)), h)
    try:
        progs.append(run1With(ctx, cond, *types))
        progs.append(run1With(ctx, body, *types))
        for x, t in builtins.zip(arrays, types):
            comps = [np.array(c, dtype=d, order="C", copy=True) for c, d in builtins.zip(_pkg._components(x), t.dtypes)]
            dev = []  # the copies receive the final state
            for c in comps:
                key, p = next(_awhile_keys), C.c_void_p()
                _pkg._check(L.accb_malloc(h, key, builtins.max(c.nbytes, 16), C.byref(p)), h)
                keys.append(key)
                _pkg._check(L.accb_poke(h, key, 0, c.ctypes.data, c.nbytes, stream), h)
                dev.append(_pkg.DeviceArray(p.value, c.shape, c.dtype))
            hosts.append(comps)
            state.append(tuple(dev) if len(dev) > 1 else dev[0])
        n = _pkg.awhile(progs[0], progs[1], state, device=device, max_iters=max_iters, stream=stream.value, count=True)
        k = iter(keys)
        for comps in hosts:
            for c in comps:
                _pkg._check(L.accb_peek(h, next(k), 0, c.ctypes.data, c.nbytes, stream), h)
        _pkg._check(L.accb_stream_sync(h, stream), h)
        res = [c[0] if len(c) == 1 else tuple(c) for c in hosts]
        return (res[0] if len(res) == 1 else tuple(res)), n
    finally:
        L.accb_stream_sync(h, stream)
        for p in progs:
            p.destroy()
        for key in keys:
            L.accb_free(h, key)
        L.accb_stream_release(h, stream)
