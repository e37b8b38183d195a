"""TEST INFRASTRUCTURE ONLY -- run the SOURCE of a Triton kernel on the CPU, one program at a time.

The reference's cache update is a Triton kernel (``_update_kv_cache``,
cascade/models/cascading_cache.py:145-774) that cannot run without a GPU, and the Triton interpreter
of the installed version rejects it.  Its source, however, is ordinary Python once ``tl`` means
something: this module provides a small stand-in for ``triton.language`` over torch CPU tensors and
executes the kernel functions' own source text with it, so that golden vectors for the score-driven
admission branch come from the reference's code and not from a restatement of it.

What the stand-in models (only what that kernel uses):

* values are 0-d or 1-d torch tensors (``V``) with ``.to(dtype)``; pointers are a flat view of a
  tensor's storage plus element offsets (``P``); ``tl.load`` / ``tl.store`` with ``mask`` / ``other``;
  ``tl.arange``, ``tl.full``, ``tl.sum``, ``tl.program_id``.
* integer ``%`` keeps the sign of the dividend (LLVM ``srem``, what Triton emits); **floating-point
  ``%`` is floor-mod**, ``a - floor(a / b) * b``: the meaning of triton 3.0.0, the version the
  reference pins (requirements.txt:378).  The kernel depends on it at :678-680, where
  ``(start - 1) % stored`` must give ``stored - 1`` for ``start == 0``.
* one source transformation, done on the AST before compiling: integer literals become stand-in
  scalars (``i = 0`` -> ``i = _c(0)``), because Triton's front end turns Python integers into tensor
  constants and the kernel calls ``.to()`` on variables initialised from literals; the ``@triton.jit``
  decorators are dropped.  Nothing else of the source is touched.
"""
from __future__ import annotations

import ast
import inspect
import textwrap

import torch


class DT:
    def __init__(self, name, tdtype):
        self.name, self.torch = name, tdtype

    def __repr__(self):
        return f"tl.{self.name}"


class V:
    """A scalar or a 1-d block of values."""

    __slots__ = ("t",)

    def __init__(self, t):
        self.t = t if isinstance(t, torch.Tensor) else torch.tensor(t)

    @property
    def dtype(self):
        return DT(str(self.t.dtype), self.t.dtype)

    def to(self, dt, **_):
        td = dt.torch if isinstance(dt, DT) else dt
        if td == torch.bool:
            return V(self.t != 0)
        return V(self.t.to(td))

    @staticmethod
    def _raw(x):
        return x.t if isinstance(x, V) else x

    def _bin(self, other, fn):
        return V(fn(self.t, V._raw(other)))

    def _rbin(self, other, fn):
        a = V._raw(other)
        a = a if isinstance(a, torch.Tensor) else torch.tensor(a)
        return V(fn(a, self.t))

    def __add__(self, o): return self._bin(o, torch.add)
    def __radd__(self, o): return self._rbin(o, torch.add)
    def __sub__(self, o): return self._bin(o, torch.sub)
    def __rsub__(self, o): return self._rbin(o, torch.sub)
    def __mul__(self, o): return self._bin(o, torch.mul)
    def __rmul__(self, o): return self._rbin(o, torch.mul)
    def __neg__(self): return V(-self.t)

    @staticmethod
    def _mod(a, b):
        b = b if isinstance(b, torch.Tensor) else torch.tensor(b)
        if a.is_floating_point() or b.is_floating_point():
            ft = a.dtype if a.is_floating_point() else b.dtype
            a, b = a.to(ft), b.to(ft)
            return a - torch.floor(a / b) * b          # triton 3.0.0: float % is floor-mod
        if bool((b == 0).any()):
            raise ZeroDivisionError("integer % by zero in the kernel source")
        return torch.fmod(a, b)                         # integers: sign of the dividend (srem)

    def __mod__(self, o): return self._bin(o, V._mod)
    def __rmod__(self, o): return self._rbin(o, V._mod)

    @staticmethod
    def _floordiv(a, b):
        b = b if isinstance(b, torch.Tensor) else torch.tensor(b)
        if a.is_floating_point() or b.is_floating_point():
            return torch.floor(a / b)
        return torch.div(a, b, rounding_mode="trunc")   # integers: sdiv truncates

    def __floordiv__(self, o): return self._bin(o, V._floordiv)

    def __lt__(self, o): return self._bin(o, torch.lt)
    def __le__(self, o): return self._bin(o, torch.le)
    def __gt__(self, o): return self._bin(o, torch.gt)
    def __ge__(self, o): return self._bin(o, torch.ge)
    def __eq__(self, o): return self._bin(o, torch.eq)
    def __ne__(self, o): return self._bin(o, torch.ne)
    __hash__ = None

    def __bool__(self):
        if self.t.numel() != 1:
            raise ValueError("a block of values has no truth value")
        return bool(self.t.item())

    def __int__(self): return int(self.t.item())
    def __index__(self): return int(self.t.item())

    def __repr__(self):
        return f"V({self.t!r})"


class P:
    """A pointer (or block of pointers): flat view of one tensor's storage + element offsets."""

    __slots__ = ("flat", "off")

    def __init__(self, flat, off=0):
        self.flat, self.off = flat, off

    @classmethod
    def of(cls, t: torch.Tensor):
        n = t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()
        flat = torch.empty(0, dtype=t.dtype).set_(t.untyped_storage(), t.storage_offset(), (n,), (1,))
        return cls(flat, 0)

    def __add__(self, o):
        return P(self.flat, self.off + o)

    __radd__ = __add__

    def index(self):
        off = V._raw(self.off)
        off = off if isinstance(off, torch.Tensor) else torch.tensor(off)
        return off.long()


class TL:
    """The stand-in for ``triton.language``."""

    int1 = DT("int1", torch.bool)
    int32 = DT("int32", torch.int32)
    int64 = DT("int64", torch.int64)
    float16 = DT("float16", torch.float16)
    bfloat16 = DT("bfloat16", torch.bfloat16)
    float32 = DT("float32", torch.float32)
    constexpr = object          # only ever used as an annotation

    def __init__(self):
        self.pid = (0, 0, 0)

    def program_id(self, axis):
        return V(torch.tensor(self.pid[int(axis)], dtype=torch.int32))

    @staticmethod
    def arange(a, b):
        return V(torch.arange(int(a), int(b), dtype=torch.int32))

    @staticmethod
    def full(shape, value, dtype):
        shape = tuple(int(s) for s in shape)
        return V(torch.full(shape, V._raw(value).item() if isinstance(value, V) else value, dtype=dtype.torch))

    @staticmethod
    def sum(x, axis=0):
        return V(x.t.sum(dim=int(axis)))

    @staticmethod
    def load(ptr, mask=None, other=0):
        idx = ptr.index()
        if mask is None:
            return V(ptr.flat[idx].clone())
        m = V._raw(mask).bool()
        safe = torch.where(m, idx, torch.zeros_like(idx))
        vals = ptr.flat[safe].clone()
        fill = torch.full_like(vals, V._raw(other).item() if isinstance(other, V) else other)
        return V(torch.where(m, vals, fill))

    @staticmethod
    def store(ptr, value, mask=None):
        idx = ptr.index()
        val = V._raw(value)
        val = val if isinstance(val, torch.Tensor) else torch.tensor(val)
        val = val.to(ptr.flat.dtype) if ptr.flat.dtype != torch.bool else (val != 0)
        if idx.dim() == 0:
            ptr.flat[idx] = val
            return
        val = val.expand(idx.shape) if val.dim() == 0 else val
        if mask is not None:
            m = V._raw(mask).bool()
            idx, val = idx[m], val[m]
        ptr.flat[idx] = val


class _IntLiterals(ast.NodeTransformer):
    """``0`` -> ``_c(0)`` for every integer literal outside annotations; decorators dropped."""

    def visit_FunctionDef(self, node):
        node.decorator_list = []
        for a in node.args.args + node.args.kwonlyargs:
            a.annotation = None
        node.returns = None
        self.generic_visit(node)
        return node

    def visit_Constant(self, node):
        if isinstance(node.value, int) and not isinstance(node.value, bool):
            return ast.copy_location(
                ast.Call(func=ast.Name(id="_c", ctx=ast.Load()), args=[node], keywords=[]), node)
        return node


def _shim_range(*args):
    for i in range(*(int(a) for a in args)):
        yield V(torch.tensor(i, dtype=torch.int32))


def compile_kernels(jit_functions: dict, extra_globals: dict):
    """Compile the source of each Triton ``JITFunction`` in ``jit_functions`` (name -> JITFunction) into
    plain Python functions that share one namespace with the stand-in ``tl``.  Returns ``(namespace, tl)``."""
    tl = TL()
    ns = {"tl": tl, "_c": lambda n: V(torch.tensor(n, dtype=torch.int32)), "range": _shim_range, "min": min,
          "max": max}
    ns.update(extra_globals)
    for name, jf in jit_functions.items():
        src = textwrap.dedent(inspect.getsource(jf.fn))
        tree = _IntLiterals().visit(ast.parse(src))
        ast.fix_missing_locations(tree)
        exec(compile(tree, f"<source of {name}>", "exec"), ns)
    return ns, tl


def as_kernel_arg(x):
    """What a Triton launch turns an argument into: tensors become pointers, Python integers scalars."""
    if isinstance(x, torch.Tensor):
        return P.of(x)
    if isinstance(x, bool):
        return x
    if isinstance(x, int):
        return V(torch.tensor(x, dtype=torch.int64))
    return x


def launch(fn, tl: TL, grid, *args):
    """Run ``fn`` once per program of ``grid`` (sequentially: the programs of this kernel are independent)."""
    kargs = [as_kernel_arg(a) for a in args]
    for n in range(grid[0]):
        for h in range(grid[1] if len(grid) > 1 else 1):
            tl.pid = (n, h, 0)
            fn(*kargs)
