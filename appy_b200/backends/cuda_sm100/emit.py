"""Translation of loop-body Python (``ast``) into CUDA C text.

This is the part of the reference spread over
appy/backends/triton/passes/device_passes/{lower_subscripts,lower_constants,
rewrite_np_calls,rewrite_ternary}.py: subscripts become address arithmetic with
per-dimension strides (unit stride assumed in the last dimension unless the array says
otherwise), library calls are mapped to device math functions, ternaries to ``?:``.
Unknown functions raise ``ValueError("Unknown function: ...")`` as in
rewrite_np_calls.py:22-24.

The emitter is typed: every expression carries a ``Ty`` (see ``dtypes``) and casts are
inserted where NumPy would convert.  Lowerings customise memory accesses through
``load_override`` / ``store_override`` (expression text -> replacement), which is how
vector registers, reduction accumulators and lane guards are spliced in.
"""
from __future__ import annotations

import ast
import math
import re
from dataclasses import dataclass, field

from . import dtypes as T
from .dtypes import Ty


@dataclass
class ArraySym:
    name: str
    ty: Ty
    ndim: int
    unit_last: bool = True      # last-dimension stride is 1
    readonly: bool = True       # never stored by the kernel and does not overlap a stored array


@dataclass
class ScalarSym:
    name: str
    ty: Ty


@dataclass
class Env:
    arrays: dict = field(default_factory=dict)       # name -> ArraySym
    scalars: dict = field(default_factory=dict)      # name -> ScalarSym (kernel parameters)
    modules: set = field(default_factory=set)        # np, math, numpy
    locals: dict = field(default_factory=dict)       # name -> Ty
    indices: dict = field(default_factory=dict)      # loop index name -> Ty
    implicit: dict = field(default_factory=dict)     # X_shape_d / X_stride_d actually used -> (array, kind, dim)
    numerics: str = "numpy"     # "numpy": NEP-50 weak literals, IEEE division; "triton": the reference backend's rules


# python/numpy function name -> (double name, float name)
MATH1 = {
    "exp": ("exp", "expf"), "exp2": ("exp2", "exp2f"), "expm1": ("expm1", "expm1f"),
    "log": ("log", "logf"), "log2": ("log2", "log2f"), "log10": ("log10", "log10f"), "log1p": ("log1p", "log1pf"),
    "sqrt": ("sqrt", "sqrtf"), "cbrt": ("cbrt", "cbrtf"), "rsqrt": ("rsqrt", "rsqrtf"),
    "sin": ("sin", "sinf"), "cos": ("cos", "cosf"), "tan": ("tan", "tanf"),
    "sinh": ("sinh", "sinhf"), "cosh": ("cosh", "coshf"), "tanh": ("tanh", "tanhf"),
    "arcsin": ("asin", "asinf"), "asin": ("asin", "asinf"), "arccos": ("acos", "acosf"), "acos": ("acos", "acosf"),
    "arctan": ("atan", "atanf"), "atan": ("atan", "atanf"),
    "arcsinh": ("asinh", "asinhf"), "asinh": ("asinh", "asinhf"), "arccosh": ("acosh", "acoshf"),
    "acosh": ("acosh", "acoshf"), "arctanh": ("atanh", "atanhf"), "atanh": ("atanh", "atanhf"),
    "floor": ("floor", "floorf"), "ceil": ("ceil", "ceilf"), "trunc": ("trunc", "truncf"),
    "rint": ("rint", "rintf"), "round": ("rint", "rintf"), "nearbyint": ("nearbyint", "nearbyintf"),
    "erf": ("erf", "erff"), "erfc": ("erfc", "erfcf"), "erfinv": ("erfinv", "erfinvf"),
    "erfcinv": ("erfcinv", "erfcinvf"), "erfcx": ("erfcx", "erfcxf"),
    "lgamma": ("lgamma", "lgammaf"), "tgamma": ("tgamma", "tgammaf"), "gamma": ("tgamma", "tgammaf"),
    "fabs": ("fabs", "fabsf"), "exp10": ("exp10", "exp10f"), "sinpi": ("sinpi", "sinpif"),
    "cospi": ("cospi", "cospif"), "normcdf": ("normcdf", "normcdff"), "normcdfinv": ("normcdfinv", "normcdfinvf"),
    "j0": ("j0", "j0f"), "j1": ("j1", "j1f"), "y0": ("y0", "y0f"), "y1": ("y1", "y1f"),
    "logb": ("logb", "logbf"), "rcbrt": ("rcbrt", "rcbrtf"),
}
MATH2 = {
    "arctan2": ("atan2", "atan2f"), "atan2": ("atan2", "atan2f"), "hypot": ("hypot", "hypotf"),
    "power": ("pow", "powf"), "pow": ("pow", "powf"), "fmod": ("fmod", "fmodf"),
    "copysign": ("copysign", "copysignf"), "remainder": ("remainder", "remainderf"),
    "fdim": ("fdim", "fdimf"), "nextafter": ("nextafter", "nextafterf"), "rhypot": ("rhypot", "rhypotf"),
    "fmax": ("fmax", "fmaxf"), "fmin": ("fmin", "fminf"),
}
PREDICATES = {"isnan": "isnan", "isinf": "isinf", "isfinite": "isfinite", "signbit": "signbit",
              "finitef": "isfinite", "isfinited": "isfinite"}

# Names of the reference's device-function table (device_passes/tl_libdevice.py, 198 stubs bound to
# Triton's libdevice) that are not plain math-library calls: every one maps to the CUDA intrinsic or
# math function of the same meaning.  Entry: list of overloads (argument types, CUDA name, result type);
# the overload is chosen by the width of the promoted arguments, arguments are converted to its types.
_F, _D, _I, _U, _L, _UL = T.F32, T.F64, T.I32, Ty("u", 32), T.I64, Ty("u", 64)
DEVICE_FUNCS: dict = {}


def _dev(name, *overloads):
    DEVICE_FUNCS[name] = list(overloads)


for _m in ("rn", "rz", "rd", "ru"):
    for _op in ("add", "sub", "mul", "div"):
        _dev(f"{_op}_{_m}", ((_D, _D), f"__d{_op}_{_m}", _D), ((_F, _F), f"__f{_op}_{_m}", _F))
    _dev(f"fma_{_m}", ((_D, _D, _D), f"__fma_{_m}", _D), ((_F, _F, _F), f"__fmaf_{_m}", _F))
    _dev(f"rcp_{_m}", ((_D,), f"__drcp_{_m}", _D), ((_F,), f"__frcp_{_m}", _F))
    _dev(f"sqrt_{_m}", ((_D,), f"__dsqrt_{_m}", _D), ((_F,), f"__fsqrt_{_m}", _F))
    _dev(f"double2float_{_m}", ((_D,), f"__double2float_{_m}", _F))
    for _src, _sty in (("double", _D), ("float", _F)):
        _dev(f"{_src}2int_{_m}", ((_sty,), f"__{_src}2int_{_m}", _I))
        _dev(f"{_src}2uint_{_m}", ((_sty,), f"__{_src}2uint_{_m}", _U))
        _dev(f"{_src}2ll_{_m}", ((_sty,), f"__{_src}2ll_{_m}", _L))
        _dev(f"{_src}2ull_{_m}", ((_sty,), f"__{_src}2ull_{_m}", _UL))
    _dev(f"int2float_{_m}", ((_I,), f"__int2float_{_m}", _F))
    _dev(f"uint2float_{_m}", ((_U,), f"__uint2float_{_m}", _F))
    _dev(f"ll2float_{_m}", ((_L,), f"__ll2float_{_m}", _F))
    _dev(f"ull2float_{_m}", ((_UL,), f"__ull2float_{_m}", _F))
    _dev(f"ll2double_{_m}", ((_L,), f"__ll2double_{_m}", _D))
    _dev(f"ull2double_{_m}", ((_UL,), f"__ull2double_{_m}", _D))
_dev("int2double_rn", ((_I,), "__int2double_rn", _D))
_dev("uint2double_rn", ((_U,), "__uint2double_rn", _D))
_dev("rsqrt_rn", ((_F,), "__frsqrt_rn", _F))
_dev("hiloint2double", ((_I, _I), "__hiloint2double", _D))
_dev("double2loint", ((_D,), "__double2loint", _I))
_dev("double2hiint", ((_D,), "__double2hiint", _I))
_dev("int_as_float", ((_I,), "__int_as_float", _F))
_dev("float_as_int", ((_F,), "__float_as_int", _I))
_dev("uint_as_float", ((_U,), "__uint_as_float", _F))
_dev("float_as_uint", ((_F,), "__float_as_uint", _U))
_dev("longlong_as_double", ((_L,), "__longlong_as_double", _D))
_dev("double_as_longlong", ((_D,), "__double_as_longlong", _L))
for _n, _c in (("sinf", "__sinf"), ("cosf", "__cosf"), ("tanf", "__tanf"), ("log2f", "__log2f"), ("logf", "__logf"),
               ("expf", "__expf"), ("exp10f", "__exp10f"), ("log10f", "__log10f"), ("tanhf", "appy_tanh_approx")):
    _dev(f"fast_{_n}", ((_F,), _c, _F))
_dev("fast_powf", ((_F, _F), "__powf", _F))
_dev("fast_dividef", ((_F, _F), "__fdividef", _F))
_dev("saturatef", ((_F,), "__saturatef", _F))
_dev("clz", ((_I,), "__clz", _I), ((_L,), "__clzll", _I))
_dev("popc", ((_U,), "__popc", _I), ((_UL,), "__popcll", _I))
_dev("brev", ((_U,), "__brev", _U), ((_UL,), "__brevll", _UL))
_dev("ffs", ((_I,), "__ffs", _I), ((_L,), "__ffsll", _I))
_dev("mulhi", ((_I, _I), "__mulhi", _I), ((_L, _L), "__mul64hi", _L), ((_U, _U), "__umulhi", _U),
     ((_UL, _UL), "__umul64hi", _UL))
_dev("mul24", ((_I, _I), "__mul24", _I), ((_U, _U), "__umul24", _U))
_dev("hadd", ((_I, _I), "__hadd", _I), ((_U, _U), "__uhadd", _U))
_dev("rhadd", ((_I, _I), "__rhadd", _I), ((_U, _U), "__urhadd", _U))
_dev("sad", ((_I, _I, _U), "__sad", _U), ((_U, _U, _U), "__usad", _U))
_dev("byte_perm", ((_U, _U, _U), "__byte_perm", _U))
_dev("llrint", ((_D,), "llrint", _L), ((_F,), "llrintf", _L))
_dev("llround", ((_D,), "llround", _L), ((_F,), "llroundf", _L))
_dev("ilogb", ((_D,), "ilogb", _I), ((_F,), "ilogbf", _I))
_dev("ldexp", ((_D, _I), "ldexp", _D), ((_F, _I), "ldexpf", _F))
_dev("scalbn", ((_D, _I), "scalbn", _D), ((_F, _I), "scalbnf", _F))
_dev("yn", ((_I, _D), "yn", _D), ((_I, _F), "ynf", _F))
_dev("jn", ((_I, _D), "jn", _D), ((_I, _F), "jnf", _F))
_dev("cyl_bessel_i0", ((_D,), "cyl_bessel_i0", _D), ((_F,), "cyl_bessel_i0f", _F))
_dev("cyl_bessel_i1", ((_D,), "cyl_bessel_i1", _D), ((_F,), "cyl_bessel_i1f", _F))
_dev("norm3d", ((_D, _D, _D), "norm3d", _D), ((_F, _F, _F), "norm3df", _F))
_dev("rnorm3d", ((_D, _D, _D), "rnorm3d", _D), ((_F, _F, _F), "rnorm3df", _F))
_dev("norm4d", ((_D, _D, _D, _D), "norm4d", _D), ((_F, _F, _F, _F), "norm4df", _F))
_dev("rnorm4d", ((_D, _D, _D, _D), "rnorm4d", _D), ((_F, _F, _F, _F), "rnorm4df", _F))
# the one name of the reference's table without a CUDA C counterpart: rcp64h (upper half of a float64
# reciprocal estimate, an internal of libdevice's own division); it raises "Unknown function"
CASTS = {"float32": T.F32, "float64": T.F64, "double": T.F64, "single": T.F32, "int8": Ty("i", 8),
         "int16": Ty("i", 16), "int32": T.I32, "int64": T.I64, "uint8": Ty("u", 8), "uint16": Ty("u", 16),
         "uint32": Ty("u", 32), "uint64": Ty("u", 64), "bool_": T.BOOL, "intc": T.I32, "int_": T.I64}
CONSTANTS = {"pi": math.pi, "e": math.e, "inf": math.inf, "nan": math.nan, "tau": math.tau,
             "Inf": math.inf, "NaN": math.nan, "euler_gamma": 0.5772156649015329}


def float_literal(v: float) -> str:
    if math.isnan(v):
        return "__longlong_as_double(0x7ff8000000000000LL)"
    if math.isinf(v):
        return ("-" if v < 0 else "") + "__longlong_as_double(0x7ff0000000000000LL)"
    if v == 0.0:
        return "-0.0" if math.copysign(1.0, v) < 0 else "0.0"
    return float(v).hex()


def cast(code: str, src: Ty, dst: Ty) -> str:
    if src.kind == dst.kind and src.bits == dst.bits:
        return code
    if dst.is_bool:
        return f"(({code}) != 0)"
    return f"(({dst.c})({code}))"


class Emitter:
    def __init__(self, env: Env):
        self.env = env
        self.load_override: dict[str, tuple[str, Ty]] = {}     # text of a Subscript/Name -> (code, type)
        self.store_override: dict[str, object] = {}            # text of a target -> callable(code, ty) -> [lines]
        self.store_guard: str | None = None                    # e.g. "g.lane == 0" for scalar stores in group mode

    # ------------------------------------------------------------------ names
    def _implicit(self, name: str):
        m = re.fullmatch(r"(\w+?)_(shape|stride)_(\d+)", name)
        if m and m.group(1) in self.env.arrays:
            arr = self.env.arrays[m.group(1)]
            d = int(m.group(3))
            if d < arr.ndim:
                self.env.implicit[name] = (m.group(1), m.group(2), d)
                return (name, T.I64)
        return None

    def name(self, node: ast.Name):
        n = node.id
        if n in self.load_override:
            return self.load_override[n]
        e = self.env
        if n in e.indices:
            return (n, e.indices[n])
        if n in e.locals:
            return (n, e.locals[n])
        if n in e.scalars:
            return (n, e.scalars[n].ty)
        imp = self._implicit(n)
        if imp:
            return imp
        if n in e.arrays:
            raise RuntimeError(f"Array `{n}` is used as a scalar; only element accesses are supported")
        if n in ("True", "False"):
            return (n.lower(), T.BOOL)
        raise NameError(f"name `{n}` is not defined in the loop's scope")

    # ------------------------------------------------------------------ subscripts
    def offset(self, node: ast.Subscript) -> tuple[str, ArraySym]:
        if not isinstance(node.value, ast.Name) or node.value.id not in self.env.arrays:
            raise RuntimeError(f"Unsupported subscript base: {ast.unparse(node)}")
        arr: ArraySym = self.env.arrays[node.value.id]
        elts = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
        if len(elts) != arr.ndim:
            raise RuntimeError(f"`{ast.unparse(node)}`: array `{arr.name}` has {arr.ndim} dimension(s), "
                               f"{len(elts)} index(es) given (>1-D array expressions are not supported)")
        terms = []
        for d, e in enumerate(elts):
            if isinstance(e, ast.Slice):
                raise RuntimeError(f"Unsupported slice expression: {ast.unparse(node)}")
            if isinstance(e, ast.UnaryOp) and isinstance(e.op, ast.USub) and isinstance(e.operand, ast.Constant) \
                    and isinstance(e.operand.value, int):
                shape = f"{arr.name}_shape_{d}"
                self.env.implicit[shape] = (arr.name, "shape", d)
                code, ty = f"({shape} - {e.operand.value})", T.I64
            else:
                code, ty = self.expr(e)
            if not (ty.is_int or ty.is_bool):
                raise TypeError(f"Array index must be an integer: {ast.unparse(node)}")
            code = code if (ty.bits == 64 and ty.kind == "i") else f"(i64)({code})"
            if d < arr.ndim - 1 or not arr.unit_last:
                stride = f"{arr.name}_stride_{d}"
                self.env.implicit[stride] = (arr.name, "stride", d)
                terms.append(f"{code} * {stride}")
            else:
                terms.append(code)
        return " + ".join(terms), arr

    def load(self, node: ast.Subscript):
        key = ast.unparse(node)
        if key in self.load_override:
            return self.load_override[key]
        off, arr = self.offset(node)
        if arr.readonly:
            return (f"appy_ldg1({arr.name} + ({off}))", arr.ty)
        return (f"{arr.name}[{off}]", arr.ty)

    # ------------------------------------------------------------------ expressions
    def expr(self, node) -> tuple[str, Ty]:
        m = getattr(self, "e_" + type(node).__name__, None)
        if m is None:
            raise NotImplementedError(f"Unsupported expression: {ast.unparse(node)}")
        return m(node)

    def as_type(self, node, ty: Ty) -> str:
        code, t = self.expr(node)
        return cast(code, t, ty)

    def e_Constant(self, node):
        v = node.value
        if isinstance(v, bool):
            return ("true" if v else "false", T.BOOL)
        if isinstance(v, int):
            return (f"{v}LL" if abs(v) >= 2 ** 31 else str(v), T.WEAK_INT)
        if isinstance(v, float):
            if self.env.numerics == "triton":
                # the reference turns every float literal into a float64 scalar tensor
                # (device_passes/lower_constants.py:22-38): arithmetic that touches it runs in float64
                return (float_literal(v), T.F64)
            return (float_literal(v), T.WEAK_FLOAT)
        raise NotImplementedError(f"Unsupported constant: {v!r}")

    def e_Name(self, node):
        return self.name(node)

    def e_Subscript(self, node):
        # X.shape[d] that was not hoisted
        v = node.value
        if isinstance(v, ast.Attribute) and v.attr == "shape" and isinstance(v.value, ast.Name) \
                and isinstance(node.slice, ast.Constant):
            imp = self._implicit(f"{v.value.id}_shape_{node.slice.value}")
            if imp:
                return imp
        return self.load(node)

    def e_Attribute(self, node):
        if isinstance(node.value, ast.Name) and node.value.id in self.env.modules and node.attr in CONSTANTS:
            return (float_literal(CONSTANTS[node.attr]), T.WEAK_FLOAT)
        raise NotImplementedError(f"Unsupported attribute: {ast.unparse(node)}")

    def e_UnaryOp(self, node):
        code, ty = self.expr(node.operand)
        if isinstance(node.op, ast.USub):
            if ty.is_bool:
                code, ty = cast(code, ty, T.I64), T.WEAK_INT
            return (f"(-{code})", ty)
        if isinstance(node.op, ast.UAdd):
            return (code, ty)
        if isinstance(node.op, ast.Not):
            return (f"(!{cast(code, ty, T.BOOL)})", T.BOOL)
        if isinstance(node.op, ast.Invert):
            if ty.is_bool:
                return (f"(!{code})", T.BOOL)
            return (f"(~{code})", ty)
        raise NotImplementedError(ast.unparse(node))

    def e_BinOp(self, node):
        lc, lt = self.expr(node.left)
        rc, rt = self.expr(node.right)
        op = node.op
        if isinstance(op, (ast.BitAnd, ast.BitOr, ast.BitXor)):
            sym = {ast.BitAnd: "&", ast.BitOr: "|", ast.BitXor: "^"}[type(op)]
            if lt.is_bool and rt.is_bool:
                return (f"({lc} {sym} {rc})", T.BOOL)
            rty = T.promote(lt, rt)
            return (f"({cast(lc, lt, rty)} {sym} {cast(rc, rt, rty)})", rty)
        if isinstance(op, (ast.LShift, ast.RShift)):
            sym = "<<" if isinstance(op, ast.LShift) else ">>"
            rty = T.promote(lt, rt)
            return (f"({cast(lc, lt, rty)} {sym} {cast(rc, rt, rty)})", rty)
        rty = T.promote(lt, rt)
        if rty.is_bool:
            rty = T.WEAK_INT if (lt.weak and rt.weak) else T.I64
        if isinstance(op, ast.Div):
            rty = T.float_of(rty)
        a, b = cast(lc, lt, rty.strong()), cast(rc, rt, rty.strong())
        if isinstance(op, ast.Add):
            return (f"({a} + {b})", rty)
        if isinstance(op, ast.Sub):
            return (f"({a} - {b})", rty)
        if isinstance(op, ast.Mult):
            return (f"({a} * {b})", rty)
        if isinstance(op, ast.Div):
            if self.env.numerics == "triton" and rty.is_float and rty.bits == 32:
                return (f"appy_div_full({a}, {b})", rty)     # Triton's float32 `/` is div.full.f32 (2 ulp)
            return (f"({a} / {b})", rty)
        targ = "" if rty.is_float else f"<{rty.strong().c}>"    # integer literals are plain `int` in C
        if isinstance(op, ast.FloorDiv):
            return (f"appy_floordiv{targ}({a}, {b})", rty)
        if isinstance(op, ast.Mod):
            return (f"appy_pymod{targ}({a}, {b})", rty)
        if isinstance(op, ast.Pow):
            if isinstance(node.right, ast.Constant) and node.right.value in (2, 3) and not isinstance(
                    node.right.value, bool):
                base = cast(lc, lt, T.promote(lt, T.WEAK_INT).strong())
                bty = T.promote(lt, T.WEAK_INT)
                return ("(" + " * ".join([base] * node.right.value) + ")", bty)
            fty = T.float_of(rty)
            fn = "powf" if fty.bits == 32 else "pow"
            code = f"{fn}({cast(lc, lt, fty.strong())}, {cast(rc, rt, fty.strong())})"
            if rty.is_int:
                return (cast(code, fty, rty.strong()), rty)
            return (code, fty)
        raise NotImplementedError(f"Unsupported operator in: {ast.unparse(node)}")

    def e_Compare(self, node):
        parts = []
        left = node.left
        for op, right in zip(node.ops, node.comparators):
            lc, lt = self.expr(left)
            rc, rt = self.expr(right)
            sym = {ast.Lt: "<", ast.LtE: "<=", ast.Gt: ">", ast.GtE: ">=", ast.Eq: "==", ast.NotEq: "!="}.get(type(op))
            if sym is None:
                raise NotImplementedError(f"Unsupported comparison: {ast.unparse(node)}")
            ty = T.promote(lt, rt).strong()
            parts.append(f"({cast(lc, lt, ty)} {sym} {cast(rc, rt, ty)})")
            left = right
        return (parts[0] if len(parts) == 1 else "(" + " && ".join(parts) + ")", T.BOOL)

    def e_BoolOp(self, node):
        sym = " && " if isinstance(node.op, ast.And) else " || "
        parts = []
        for v in node.values:
            c, t = self.expr(v)
            parts.append(cast(c, t, T.BOOL))
        return ("(" + sym.join(parts) + ")", T.BOOL)

    def e_IfExp(self, node):
        cc, ct = self.expr(node.test)
        ac, at = self.expr(node.body)
        bc, bt = self.expr(node.orelse)
        ty = T.promote(at, bt)
        return (f"({cast(cc, ct, T.BOOL)} ? {cast(ac, at, ty.strong())} : {cast(bc, bt, ty.strong())})", ty)

    def _fname(self, func):
        if isinstance(func, ast.Name):
            return func.id, None
        if isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name):
            return func.attr, func.value.id
        return None, None

    def e_Call(self, node):
        code, ty = self._call(node)
        _name, mod = self._fname(node.func)
        if mod in ("np", "numpy") and ty.weak:
            # NumPy functions return NumPy scalars: np.sqrt(3.25) is a float64, no longer a weak Python
            # float, so `f32 * np.sqrt(3.25)` is computed in float64 (math.sqrt(3.25) stays weak)
            ty = ty.strong()
        return code, ty

    def _call(self, node):
        name, mod = self._fname(node.func)
        if name is None or node.keywords:
            raise ValueError(f"Unknown function: {ast.unparse(node.func)}")
        if mod is not None and mod not in self.env.modules and mod not in ("np", "numpy", "math", "appy", "tl",
                                                                           "libdevice"):
            raise ValueError(f"Unknown function: {ast.unparse(node.func)}")
        args = node.args
        if name == "float" and len(args) == 1 and isinstance(args[0], ast.Constant) and isinstance(args[0].value, str):
            s = args[0].value.strip().lower()
            table = {"inf": math.inf, "+inf": math.inf, "-inf": -math.inf, "infinity": math.inf,
                     "+infinity": math.inf, "-infinity": -math.inf, "nan": math.nan}
            if s not in table:
                raise ValueError(f"float() of a string supports only inf, -inf and nan: {ast.unparse(node)}")
            return (float_literal(table[s]), T.WEAK_FLOAT)
        if name in ("float", "int", "bool") and mod is None and len(args) == 1:
            c, t = self.expr(args[0])
            dst = {"float": T.WEAK_FLOAT, "int": T.WEAK_INT, "bool": T.BOOL}[name]
            return (cast(c, t, dst.strong()), dst)
        if name in CASTS and len(args) == 1:
            c, t = self.expr(args[0])
            return (cast(c, t, CASTS[name]), CASTS[name])
        if name in ("min", "max", "minimum", "maximum") and len(args) >= 2:
            vals = [self.expr(a) for a in args]
            ty = vals[0][1]
            for _, t in vals[1:]:
                ty = T.promote(ty, t)
            fn = "appy_tmax" if name in ("max", "maximum") else "appy_tmin"
            code = cast(vals[0][0], vals[0][1], ty.strong())
            for c, t in vals[1:]:
                code = f"{fn}<{ty.strong().c}>({code}, {cast(c, t, ty.strong())})"
            return (code, ty)
        if name in ("abs", "absolute", "fabs") and len(args) == 1:
            c, t = self.expr(args[0])
            if name == "fabs":
                t2 = T.float_of(t)
                return (f"{'fabsf' if t2.bits == 32 else 'fabs'}({cast(c, t, t2.strong())})", t2)
            if t.is_float:
                return (f"{'fabsf' if t.bits == 32 else 'fabs'}({c})", t)
            if t.is_bool or t.kind == "u":
                return (c, t)
            return (f"(({c}) < 0 ? -({c}) : ({c}))", t)
        if name == "where" and len(args) == 3:
            return self.e_IfExp(ast.IfExp(test=args[0], body=args[1], orelse=args[2]))
        if name == "sign" and len(args) == 1:
            c, t = self.expr(args[0])
            return (f"(({t.strong().c})((({c}) > 0) - (({c}) < 0)))", t)
        if name == "square" and len(args) == 1:
            c, t = self.expr(args[0])
            return (f"(({c}) * ({c}))", t)
        if name == "fma" and len(args) == 3:
            vals = [self.expr(a) for a in args]
            ty = T.float_of(T.promote(T.promote(vals[0][1], vals[1][1]), vals[2][1]))
            fn = "fmaf" if ty.bits == 32 else "fma"
            return (f"{fn}(" + ", ".join(cast(c, t, ty.strong()) for c, t in vals) + ")", ty)
        if name in MATH1 and len(args) == 1:
            c, t = self.expr(args[0])
            ft = T.float_of(t)
            fn = MATH1[name][1 if ft.bits == 32 else 0]
            return (f"{fn}({cast(c, t, ft.strong())})", ft)
        if name in MATH2 and len(args) == 2:
            (ac, at), (bc, bt) = self.expr(args[0]), self.expr(args[1])
            ft = T.float_of(T.promote(at, bt))
            fn = MATH2[name][1 if ft.bits == 32 else 0]
            return (f"{fn}({cast(ac, at, ft.strong())}, {cast(bc, bt, ft.strong())})", ft)
        if name in DEVICE_FUNCS:
            over = [o for o in DEVICE_FUNCS[name] if len(o[0]) == len(args)]
            if not over:
                raise ValueError(f"Unknown function: {ast.unparse(node.func)} with {len(args)} arguments")
            vals = [self.expr(a) for a in args]
            pick = over[0]
            if len(over) > 1:
                # width and kind of the arguments that the overloads disagree on
                vary = [i for i in range(len(args)) if len({o[0][i] for o in over}) > 1]
                ty = vals[vary[0]][1]
                for i in vary[1:]:
                    ty = T.promote(ty, vals[i][1])
                if over[0][0][vary[0]].is_float:
                    ty = T.float_of(ty)
                    pick = next((o for o in over if o[0][vary[0]].bits == ty.bits), over[0])
                else:
                    bits = 64 if (not ty.weak and ty.bits == 64) else 32
                    kind = "u" if ty.kind == "u" else "i"
                    pick = next((o for o in over if o[0][vary[0]].bits == bits and o[0][vary[0]].kind == kind),
                                next((o for o in over if o[0][vary[0]].bits == bits), over[0]))
            code = f"{pick[1]}(" + ", ".join(cast(c, t, want) for (c, t), want in zip(vals, pick[0])) + ")"
            return (code, pick[2])
        if name in PREDICATES and len(args) == 1:
            c, t = self.expr(args[0])
            ft = T.float_of(t)
            return (f"({PREDICATES[name]}({cast(c, t, ft.strong())}) != 0)", T.BOOL)
        raise ValueError(f"Unknown function: {ast.unparse(node.func)}")

    # ------------------------------------------------------------------ type inference for locals
    def infer_locals(self, stmts, skip: set[str] = frozenset()) -> None:
        """Fixpoint over assignments `name = expr`; results go to env.locals."""
        assigned: list[tuple[str, ast.AST]] = []
        loops: list[ast.For] = []

        def collect(block):
            for st in block:
                if isinstance(st, ast.Assign) and isinstance(st.targets[0], ast.Name):
                    assigned.append((st.targets[0].id, st.value))
                for fld in ("body", "orelse"):
                    b = getattr(st, fld, None)
                    if isinstance(b, list) and b and isinstance(b[0], ast.stmt):
                        collect(b)
                if isinstance(st, ast.For):
                    loops.append(st)

        collect(stmts)
        for lp in loops:
            self.env.indices.setdefault(lp.target.id, T.WEAK_INT)
        for _ in range(6):
            changed = False
            for name, value in assigned:
                if name in skip or name in self.env.indices:
                    continue
                try:
                    _, ty = self.expr(value)
                except NameError:
                    continue          # depends on a local whose type is not known yet
                new = T.join(self.env.locals.get(name), ty)
                if self.env.locals.get(name) != new:
                    self.env.locals[name] = new
                    changed = True
            if not changed:
                break
        for name, value in assigned:
            if name not in self.env.locals and name not in skip and name not in self.env.indices:
                self.expr(value)     # raises the real error

    def declare_locals(self, names=None) -> list[str]:
        out = []
        for n, ty in self.env.locals.items():
            if names is not None and n not in names:
                continue
            out.append(f"{ty.strong().c} {n} = 0;")
        return out

    # ------------------------------------------------------------------ statements
    def block(self, stmts, indent="  ") -> list[str]:
        out = []
        for st in stmts:
            out.extend(indent + line for line in self.stmt(st))
        return out

    def stmt(self, st) -> list[str]:
        m = getattr(self, "s_" + type(st).__name__, None)
        if m is None:
            raise NotImplementedError(f"Unsupported statement in a parallel loop: {ast.unparse(st)}")
        return m(st)

    def s_Pass(self, st):
        return []

    def s_Expr(self, st):
        if isinstance(st.value, ast.Constant):
            return []                      # docstring or pragma marker
        raise NotImplementedError(f"Unsupported statement in a parallel loop: {ast.unparse(st)}")

    def s_Break(self, st):
        return ["break;"]

    def s_Continue(self, st):
        return ["continue;"]

    def s_Assign(self, st):
        target = st.targets[0]
        key = ast.unparse(target)
        code, ty = self.expr(st.value)
        if key in self.store_override:
            return self.store_override[key](code, ty)
        if isinstance(target, ast.Name):
            n = target.id
            if n not in self.env.locals:
                raise NameError(f"assignment to `{n}`, which is not a loop-local variable")
            lt = self.env.locals[n].strong()
            return [f"{n} = {cast(code, ty, lt)};"]
        if isinstance(target, ast.Subscript):
            off, arr = self.offset(target)
            line = f"{arr.name}[{off}] = {cast(code, ty, arr.ty)};"
            if self.store_guard:
                return [f"if ({self.store_guard}) {line}"]
            return [line]
        raise NotImplementedError(f"Unsupported assignment target: {ast.unparse(st)}")

    def s_If(self, st):
        c, t = self.expr(st.test)
        out = [f"if ({cast(c, t, T.BOOL)}) {{"] + self.block(st.body) + ["}"]
        if st.orelse:
            out[-1] = "} else {"
            out += self.block(st.orelse) + ["}"]
        return out

    def s_While(self, st):
        c, t = self.expr(st.test)
        return [f"while ({cast(c, t, T.BOOL)}) {{"] + self.block(st.body) + ["}"]

    def range_bounds(self, loop: ast.For):
        it = loop.iter
        if not (isinstance(it, ast.Call) and isinstance(it.func, ast.Name) and it.func.id == "range"
                and len(it.args) == 3):
            raise NotImplementedError(f"Only `for v in range(...)` loops are supported: {ast.unparse(loop.iter)}")
        lo = self.as_type(it.args[0], T.I64)
        hi = self.as_type(it.args[1], T.I64)
        return lo, hi

    def s_For(self, st):
        """Sequential loop (lowerings intercept simd loops before they get here)."""
        lo, hi = self.range_bounds(st)
        v = st.target.id
        self.env.indices.setdefault(v, T.WEAK_INT)
        return [f"for (i64 {v} = {lo}; {v} < {hi}; ++{v}) {{"] + self.block(st.body) + ["}"]
