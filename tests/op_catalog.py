"""A table of torch operations, each run on a ``torch.bool`` tensor and on its bit1 twin.

The checker is ``torch.bool`` itself: the same callable is applied to bool inputs and to the
bit1 tensors built from them, and the results are compared value for value. This is the method of
the reference's own op catalog (tests/ops_catalog.py:54-84 there: one spec per operation, consumed
by a parity driver, an edge-case driver and a fuzz driver); the table here is this repository's
own and is generated from compact rows, function form and method form side by side.

A row is ``(name, kind, arity, fn)`` or, where torch cannot run the op on bool, ``(..., oracle)``.
``kind`` picks the input shapes: "vector" (16,), "matrix" (4, 8), "diagvec" (6,), "matmul"
A (4, 64) with B (4, 64) stored as rows of output features.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch


@dataclass(frozen=True)
class Op:
    name: str
    kind: str                 # vector | matrix | diagvec | matmul
    arity: int
    fn: Callable
    oracle: Optional[Callable] = None     # run on the bool inputs instead of fn
    bit1_out: bool = True                 # a bool-valued result must come back as bit1
    edges: tuple = ("empty", "0-dim", "non-contig", "tail", "wide")


OPS: list = []


def _op(name, kind, arity, fn, oracle=None, bit1_out=True, edges=None):
    assert all(o.name != name for o in OPS), name
    if edges is None:
        edges = ("empty", "0-dim", "non-contig", "tail", "wide") + (("broadcast",) if arity == 2 else ())
    OPS.append(Op(name, kind, arity, fn, oracle, bit1_out, tuple(edges)))


def _both(name, kind, arity, torch_fn_name, *extra, method_name=None, **kw):
    """Function form ``torch.f(a, ...)`` and method form ``a.f(...)`` of one operation."""
    f = getattr(torch, torch_fn_name)
    m = method_name or torch_fn_name
    if arity == 1:
        _op(name + "_fn", kind, 1, lambda a, f=f: f(a, *extra), **kw)
        _op(name + "_method", kind, 1, lambda a, m=m: getattr(a, m)(*extra), **kw)
    else:
        _op(name + "_fn", kind, 2, lambda a, b, f=f: f(a, b, *extra), **kw)
        _op(name + "_method", kind, 2, lambda a, b, m=m: getattr(a, m)(b, *extra), **kw)


# ---- element-wise, two operands ---------------------------------------------------------------
for _n, _sym in (("and", lambda a, b: a & b), ("or", lambda a, b: a | b), ("xor", lambda a, b: a ^ b)):
    _op("operator_" + _n, "vector", 2, _sym)
    _both("bitwise_" + _n, "vector", 2, "bitwise_" + _n)
    _both("logical_" + _n, "vector", 2, "logical_" + _n)


def _inplace(which):
    def run(a, b):
        a = a.clone()
        if which == "and":
            a &= b
        elif which == "or":
            a |= b
        else:
            a ^= b
        return a
    return run


for _n in ("and", "or", "xor"):
    _op("inplace_" + _n, "vector", 2, _inplace(_n))

_op("operator_invert", "vector", 1, lambda a: ~a)
_both("bitwise_not", "vector", 1, "bitwise_not")
_both("logical_not", "vector", 1, "logical_not")

for _n, _sym in (("eq", lambda a, b: a == b), ("ne", lambda a, b: a != b), ("lt", lambda a, b: a < b),
                 ("le", lambda a, b: a <= b), ("gt", lambda a, b: a > b), ("ge", lambda a, b: a >= b)):
    _op("operator_" + _n, "vector", 2, _sym)
    _both(_n, "vector", 2, _n)
_both("equal", "vector", 2, "equal", bit1_out=False, edges=("empty", "tail", "wide"))

# ---- reductions --------------------------------------------------------------------------------
_FULL_EDGES = ("empty", "non-contig", "tail", "wide")
_NONEMPTY = ("non-contig", "tail", "wide")
_both("sum_full", "vector", 1, "sum", bit1_out=False, edges=_FULL_EDGES)
_both("count_nonzero_full", "vector", 1, "count_nonzero", bit1_out=False, edges=_FULL_EDGES)
_both("all_full", "vector", 1, "all", bit1_out=False, edges=_FULL_EDGES)
_both("any_full", "vector", 1, "any", bit1_out=False, edges=_FULL_EDGES)
_op("argmax_full_fn", "vector", 1, lambda a: torch.argmax(a), lambda b: torch.argmax(b.long()), False, _NONEMPTY)
_op("argmax_full_method", "vector", 1, lambda a: a.argmax(), lambda b: b.long().argmax(), False, _NONEMPTY)
_op("argmin_full_fn", "vector", 1, lambda a: torch.argmin(a), lambda b: torch.argmin(b.long()), False, _NONEMPTY)
_op("argmin_full_method", "vector", 1, lambda a: a.argmin(), lambda b: b.long().argmin(), False, _NONEMPTY)
_both("max_full", "vector", 1, "max", bit1_out=False, edges=_NONEMPTY)
_both("min_full", "vector", 1, "min", bit1_out=False, edges=_NONEMPTY)
_both("nonzero", "vector", 1, "nonzero", bit1_out=False, edges=_FULL_EDGES)
_both("argwhere", "vector", 1, "argwhere", bit1_out=False, edges=_FULL_EDGES)

_both("sum_dim0", "matrix", 1, "sum", 0, bit1_out=False, edges=_NONEMPTY)
_both("sum_dim1", "matrix", 1, "sum", 1, bit1_out=False, edges=_NONEMPTY)
_both("all_dim0", "matrix", 1, "all", 0, bit1_out=False, edges=_NONEMPTY)
_both("all_dim_last", "matrix", 1, "all", -1, bit1_out=False, edges=_NONEMPTY)
_both("any_dim0", "matrix", 1, "any", 0, bit1_out=False, edges=_NONEMPTY)
_both("any_dim_last", "matrix", 1, "any", -1, bit1_out=False, edges=_NONEMPTY)
_op("any_dim0_keepdim", "matrix", 1, lambda a: a.any(dim=0, keepdim=True), bit1_out=False, edges=_NONEMPTY)
_both("count_nonzero_dim0", "matrix", 1, "count_nonzero", 0, bit1_out=False, edges=_NONEMPTY)
_both("cumsum_dim_last", "matrix", 1, "cumsum", -1, bit1_out=False, edges=("non-contig", "wide"))

# ---- shape and view ----------------------------------------------------------------------------
_V = ("non-contig", "tail", "wide")
_op("view_flat", "matrix", 1, lambda a: a.contiguous().view(-1), edges=("tail", "wide"))
_op("view_split_rows", "matrix", 1, lambda a: a.contiguous().view(2, -1, a.shape[-1]), edges=("wide",))
_both("reshape_flat", "matrix", 1, "reshape", (-1,), edges=_V)
_both("flatten", "matrix", 1, "flatten", edges=_V)
_both("ravel", "matrix", 1, "ravel", edges=_V)
_op("squeeze_method", "matrix", 1, lambda a: a.unsqueeze(0).squeeze(0), edges=_V)
_op("squeeze_fn", "matrix", 1, lambda a: torch.squeeze(torch.unsqueeze(a, 0), 0), edges=_V)
_both("unsqueeze_0", "matrix", 1, "unsqueeze", 0, edges=_V)
_both("unsqueeze_last", "matrix", 1, "unsqueeze", -1, edges=_V)
_both("t", "matrix", 1, "t", edges=_V)
_both("transpose_01", "matrix", 1, "transpose", 0, 1, edges=_V)
_op("transpose_leading", "matrix", 1, lambda a: a.unsqueeze(0).transpose(0, 1), edges=_V)
_op("permute_method", "matrix", 1, lambda a: a.unsqueeze(0).permute(0, 2, 1), edges=_V)
_op("permute_fn", "matrix", 1, lambda a: torch.permute(a.unsqueeze(0), (1, 0, 2)), edges=_V)
_both("movedim", "matrix", 1, "movedim", 0, 1, edges=_V)
_both("moveaxis", "matrix", 1, "moveaxis", 0, -1, edges=_V)
_both("swapaxes", "matrix", 1, "swapaxes", 0, 1, edges=_V)
_both("swapdims", "matrix", 1, "swapdims", 0, 1, edges=_V)
_op("contiguous", "matrix", 1, lambda a: a.contiguous(), edges=_V)
_op("contiguous_of_t", "matrix", 1, lambda a: a.t().contiguous(), edges=_V)
_op("expand", "matrix", 1, lambda a: a.unsqueeze(0).expand(3, *a.shape), edges=_V)
_op("expand_as", "matrix", 1, lambda a: a.unsqueeze(0).expand_as(torch.empty(2, *a.shape)), edges=_V)
_op("broadcast_to_fn", "matrix", 1, lambda a: torch.broadcast_to(a, (2, *a.shape)), edges=_V)
_op("broadcast_to_method", "matrix", 1, lambda a: a.broadcast_to((2, *a.shape)), edges=_V)
_op("reshape_as", "matrix", 1, lambda a: a.reshape_as(torch.empty(a.shape[0], 1, a.shape[1])), edges=_V)
_op("view_as", "matrix", 1, lambda a: a.contiguous().view_as(torch.empty(1, *a.shape)), edges=("tail", "wide"))
_both("narrow", "matrix", 1, "narrow", 0, 1, 2, edges=_V)
_op("narrow_last", "matrix", 1, lambda a: a.narrow(-1, 1, 3), edges=_V)
_both("select_row", "matrix", 1, "select", 0, 1, edges=_V)
_op("select_col", "matrix", 1, lambda a: a.select(1, 2), edges=_V)
_op("atleast_2d", "vector", 1, lambda a: torch.atleast_2d(a), edges=("0-dim", "tail", "wide"))

# ---- combine / split ---------------------------------------------------------------------------
_op("cat_dim0", "matrix", 2, lambda a, b: torch.cat([a, b], dim=0), edges=_V)
_op("cat_dim_last", "matrix", 2, lambda a, b: torch.cat([a, b], dim=-1), edges=_V)
_op("stack_dim0", "matrix", 2, lambda a, b: torch.stack([a, b], dim=0), edges=_V)
_op("split_fn", "matrix", 1, lambda a: tuple(torch.split(a, 2, dim=0)), edges=_V)
_op("split_method", "matrix", 1, lambda a: tuple(a.split(3, dim=-1)), edges=_V)
_op("chunk_fn", "matrix", 1, lambda a: tuple(torch.chunk(a, 2, dim=0)), edges=_V)
_op("chunk_method", "matrix", 1, lambda a: tuple(a.chunk(2, dim=-1)), edges=_V)
_op("unbind_fn", "matrix", 1, lambda a: tuple(torch.unbind(a, dim=0)), edges=_V)
_op("unbind_method", "matrix", 1, lambda a: tuple(a.unbind(-1)), edges=_V)

# ---- indexing ----------------------------------------------------------------------------------
_op("getitem_row", "matrix", 1, lambda a: a[1], edges=_V)
_op("getitem_rows", "matrix", 1, lambda a: a[1:3], edges=_V)
_op("getitem_col", "matrix", 1, lambda a: a[:, 2], edges=_V)
_op("getitem_neg", "matrix", 1, lambda a: a[-1], edges=_V)
_op("getitem_ellipsis", "matrix", 1, lambda a: a[..., 1], edges=_V)
_op("getitem_col_slice", "matrix", 1, lambda a: a[:, 1:3], edges=_V)
_op("getitem_col_step", "matrix", 1, lambda a: a[..., ::2], edges=_V)
# tensor indices are reduced modulo the axis length: an out-of-range index held in a DEVICE tensor is
# not a Python exception on CUDA but a device-side assert, which no test here may cause
_op("getitem_row_list", "matrix", 1, lambda a: a[torch.tensor([2, 0, 2], device=a.device) % a.shape[0]], edges=_V)
_op("getitem_mask", "matrix", 1, lambda a: a[torch.arange(a.shape[0], device=a.device) % 2 == 0], edges=_V)


def _idx(a, dim, n, mod):
    return (torch.arange(n, device=a.device) * 7 + 1) % mod


_op("gather_fn", "matrix", 1,
    lambda a: torch.gather(a, 1, _idx(a, 1, a.shape[0] * 3, a.shape[1]).reshape(a.shape[0], 3)), edges=_V)
_op("gather_method", "matrix", 1,
    lambda a: a.gather(0, _idx(a, 0, 2 * a.shape[1], a.shape[0]).reshape(2, a.shape[1])), edges=_V)
_op("index_select_rows", "matrix", 1, lambda a: torch.index_select(a, 0, _idx(a, 0, 5, a.shape[0])), edges=_V)
_op("index_select_cols", "matrix", 1, lambda a: a.index_select(-1, _idx(a, 1, 6, a.shape[1])), edges=_V)
_op("take_fn", "matrix", 1, lambda a: torch.take(a, _idx(a, 0, 7, a.numel())), edges=_V)
_op("take_method", "matrix", 1, lambda a: a.take(_idx(a, 0, 7, a.numel())), edges=_V)


def _scatter(a, method):
    index = _idx(a, 1, a.shape[0] * 2, a.shape[1]).reshape(a.shape[0], 2)
    src = torch.ones(a.shape[0], 2, dtype=torch.bool, device=a.device)
    return a.clone().scatter(1, index, src) if method else torch.scatter(a.clone(), 1, index, src)


_op("scatter_fn", "matrix", 1, lambda a: _scatter(a, False), bit1_out=False, edges=_V)   # a plain bool src is mixed in
_op("scatter_method", "matrix", 1, lambda a: _scatter(a, True), bit1_out=False, edges=_V)


def _rows_mask(a):
    return (torch.arange(a.numel(), device=a.device).reshape(a.shape) % 3 == 0)


_op("masked_select_fn", "matrix", 1, lambda a: torch.masked_select(a, _rows_mask(a)), edges=_V)
_op("masked_select_method", "matrix", 1, lambda a: a.masked_select(_rows_mask(a)), edges=_V)
_op("masked_fill_fn", "matrix", 1, lambda a: torch.masked_fill(a, _rows_mask(a), True), edges=_V)
_op("masked_fill_method", "matrix", 1, lambda a: a.masked_fill(_rows_mask(a), False), edges=_V)
_op("where_fn", "matrix", 2, lambda a, b: torch.where(_rows_mask(a), a, b), edges=_V)
# Tensor.where is not in the reference's mask-taking set (brute/tensor.py:57-62): a plain bool mask demotes
_op("where_method", "matrix", 2, lambda a, b: a.where(_rows_mask(a), b), bit1_out=False, edges=_V)
_op("where_bit1_cond", "matrix", 2, lambda a, b: torch.where(a, a, b), edges=_V)


def _set(a, how):
    a = a.clone()
    if how == "row":
        a[1] = True
    elif how == "rows":
        a[0:2] = False
    elif how == "col":
        a[:, 2] = True
    elif how == "col_ellipsis":
        a[..., 1] = False
    elif how == "col_tensor":
        a[:, torch.tensor([0, 3], device=a.device) % a.shape[1]] = True
    elif how == "index_copy_last":
        cols = [a.shape[1] - 1, 0] if a.shape[1] >= 2 else [0]          # distinct, in range
        idx = torch.tensor(cols, device=a.device)
        src = torch.ones(a.shape[0], len(cols), dtype=torch.bool, device=a.device)
        src[::2, 0] = False
        a.index_copy_(-1, idx, src)
    elif how == "index_fill_last":
        a.index_fill_(-1, torch.tensor([1, 2], device=a.device) % a.shape[1], True)
    return a


for _how in ("row", "rows", "col", "col_ellipsis", "col_tensor", "index_copy_last", "index_fill_last"):
    _op("setitem_" + _how, "matrix", 1, lambda a, h=_how: _set(a, h), edges=_V)

# ---- copies and fills --------------------------------------------------------------------------
_both("clone", "matrix", 1, "clone", edges=_V)
_both("detach", "matrix", 1, "detach", edges=_V)
_op("fill_true", "matrix", 1, lambda a: a.clone().fill_(True), edges=_V + ("empty",))
_op("fill_false", "matrix", 1, lambda a: a.clone().fill_(False), edges=_V + ("empty",))
_op("zero_", "matrix", 1, lambda a: a.clone().zero_(), edges=_V + ("empty",))
_op("fill_after_op", "matrix", 2, lambda a, b: (a & b).fill_(True), edges=_V)
_op("zero_after_op", "matrix", 2, lambda a, b: (a | b).zero_(), edges=_V)
_op("copy_", "matrix", 2, lambda a, b: a.clone().copy_(b), edges=_V)

# ---- rearrangement -----------------------------------------------------------------------------
_both("roll_rows", "matrix", 1, "roll", 1, 0, edges=_V)
_both("roll_cols", "matrix", 1, "roll", 3, -1, edges=_V)
_op("roll_flat", "matrix", 1, lambda a: torch.roll(a, 5), edges=_V)
_both("flip_dim0", "matrix", 1, "flip", (0,), edges=_V)
_both("flip_dim1", "matrix", 1, "flip", (1,), edges=_V)
_op("flip_both", "matrix", 1, lambda a: a.flip(0, 1), edges=_V)
_both("fliplr", "matrix", 1, "fliplr", edges=_V)
_both("flipud", "matrix", 1, "flipud", edges=_V)
_both("rot90", "matrix", 1, "rot90", edges=_V)
_both("tile", "matrix", 1, "tile", (2, 1), edges=_V)
_op("tile_last", "matrix", 1, lambda a: a.tile((1, 3)), edges=_V)
_op("repeat", "matrix", 1, lambda a: a.repeat(2, 1), edges=_V)
_op("repeat_last", "matrix", 1, lambda a: a.repeat(1, 2), edges=_V)
_both("repeat_interleave", "matrix", 1, "repeat_interleave", 2, 0, edges=_V)
_op("repeat_interleave_last", "matrix", 1, lambda a: a.repeat_interleave(2, dim=-1), edges=_V)

# ---- diagonals and triangles -------------------------------------------------------------------
_both("diagonal", "matrix", 1, "diagonal", edges=_V)
_both("diag", "matrix", 1, "diag", edges=_V)
_both("diag_embed", "diagvec", 1, "diag_embed", edges=("tail",))
_both("diagflat", "diagvec", 1, "diagflat", edges=("tail",))
_both("tril", "matrix", 1, "tril", edges=_V)
_both("triu", "matrix", 1, "triu", edges=_V)

# ---- casts -------------------------------------------------------------------------------------
_C = ("empty", "0-dim", "non-contig", "tail", "wide")
for _n, _dt in (("float32", torch.float32), ("int32", torch.int32), ("int64", torch.int64), ("uint8", torch.uint8),
                ("bool", torch.bool), ("float16", torch.float16)):
    # an explicit torch dtype, torch.bool included, leaves the bit1 domain (brute/tensor.py:537-547)
    _op("to_" + _n, "vector", 1, lambda a, d=_dt: a.to(d), bit1_out=False, edges=_C)
    _op("to_" + _n + "_kw", "vector", 1, lambda a, d=_dt: a.to(dtype=d), bit1_out=False, edges=_C)
for _n in ("int", "short", "char", "half", "float", "long", "double"):
    _op("cast_" + _n, "vector", 1, lambda a, n=_n: getattr(a, n)(), bit1_out=False, edges=_C)
_op("type_as", "vector", 1, lambda a: a.type_as(torch.empty(1, dtype=torch.int16, device=a.device)), bit1_out=False,
    edges=_C)

# ---- matmul (bit1 semantics: +-1 dot product; the bool twin computes it in float) -------------
def _pm1(b):
    return b.float() * 2 - 1


def _mm_oracle(a, b):
    return (_pm1(a) @ _pm1(b).t()).to(torch.int32)


_MM = ("tail", "wide")
_op("matmul_operator", "matmul", 2, lambda a, b: a @ b.t(), _mm_oracle, False, _MM)
_op("matmul_fn", "matmul", 2, lambda a, b: torch.matmul(a, b.t()), _mm_oracle, False, _MM)
_op("matmul_method", "matmul", 2, lambda a, b: a.matmul(b.t()), _mm_oracle, False, _MM)
_op("mm_fn", "matmul", 2, lambda a, b: torch.mm(a, b.t()), _mm_oracle, False, _MM)
_op("mm_method", "matmul", 2, lambda a, b: a.mm(b.t()), _mm_oracle, False, _MM)
_op("matmul_transpose_fn", "matmul", 2, lambda a, b: a @ torch.transpose(b, 0, 1), _mm_oracle, False, _MM)
_op("matmul_rows_of_features", "matmul", 2, lambda a, b: a @ b if a.shape[-1] == b.shape[-1] != b.shape[0] else a @ b.t(),
    _mm_oracle, False, ("wide",))

# ---- bit1-only methods -------------------------------------------------------------------------
_op("popcount", "vector", 1, lambda a: a.popcount(), lambda b: b.long().sum(), False, _FULL_EDGES)
_op("hamming", "vector", 2, lambda a, b: a.hamming(b), lambda a, b: (a ^ b).long().sum(), False, _FULL_EDGES)
_op("unpack_pm1", "vector", 1, lambda a: a.unpack_pm1(), lambda b: _pm1(b), False, ("tail", "wide"))
_op("word_popcount_sum", "matrix", 1, lambda a: a.word_popcount().sum(-1), lambda b: b.long().sum(-1).to(torch.int64),
    False, ("tail", "wide"))


BY_NAME = {o.name: o for o in OPS}


# ================================================================================================
# inputs
# ================================================================================================
def rand_bool(shape, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if len(shape) and any(d == 0 for d in shape):
        return torch.zeros(shape, dtype=torch.bool, device=device)
    return torch.randint(0, 2, shape, generator=g, dtype=torch.uint8).bool().to(device)


def base_shapes(op: Op):
    if op.kind == "vector":
        return [(16,)] * op.arity
    if op.kind == "diagvec":
        return [(6,)] * op.arity
    if op.kind == "matrix":
        return [(4, 8)] * op.arity
    return [(4, 64), (4, 64)][:op.arity]


def edge_inputs(op: Op, edge: str, device):
    """bool inputs for one edge case, or None when the edge does not apply to the op."""
    n = op.arity
    vec = op.kind in ("vector", "diagvec")
    if edge == "base":
        return [rand_bool(s, device, 1 + i) for i, s in enumerate(base_shapes(op))]
    if edge == "empty":
        shape = (0,) if vec else ((4, 0) if op.kind == "matmul" else (0, 8))
        return [rand_bool(shape, device, 10 + i) for i in range(n)]
    if edge == "0-dim":
        return [rand_bool((), device, 20 + i) for i in range(n)] if vec else None
    if edge == "non-contig":
        if op.kind == "matmul":
            return None
        if vec:
            return [rand_bool((32,), device, 30 + i)[::2] for i in range(n)]
        return [rand_bool((8, 4), device, 30 + i).t() for i in range(n)]
    if edge == "broadcast":
        if n < 2 or vec or op.kind == "matmul":
            return None
        return [rand_bool((4, 8), device, 40), rand_bool((1, 8), device, 41)]
    if edge == "tail":          # last dimension not a multiple of 64
        if op.kind == "matmul":
            return [rand_bool((5, 13), device, 50), rand_bool((3, 13), device, 51)][:n]
        shape = (13,) if vec else (3, 13)
        return [rand_bool(shape, device, 50 + i) for i in range(n)]
    if edge == "wide":          # several packed words per row, ragged tail
        if op.kind == "matmul":
            return [rand_bool((9, 200), device, 60), rand_bool((7, 200), device, 61)][:n]
        shape = (200,) if vec else (6, 131)
        if op.kind == "diagvec":
            shape = (70,)
        return [rand_bool(shape, device, 60 + i) for i in range(n)]
    raise ValueError(edge)


# ================================================================================================
# comparison
# ================================================================================================
def to_plain(x):
    """Plain tensor with current values (a lazy bit1 tensor is materialised by ``.bool()``)."""
    if isinstance(x, torch.Tensor) and hasattr(x, "_ensure_bool_valid"):
        if x.__dict__.get("_is_bit1", False):
            return x.bool().as_subclass(torch.Tensor)
        return x.as_subclass(torch.Tensor)
    return x


def compare(got, want, note=""):
    if isinstance(got, (tuple, list)) or isinstance(want, (tuple, list)):
        assert isinstance(got, (tuple, list)) and isinstance(want, (tuple, list)) and len(got) == len(want), note
        for g, w in zip(got, want):
            compare(g, w, note)
        return
    if isinstance(got, torch.Tensor) or isinstance(want, torch.Tensor):
        g, w = to_plain(got), to_plain(want)
        assert isinstance(g, torch.Tensor) and isinstance(w, torch.Tensor), f"tensor vs scalar ({note})"
        assert tuple(g.shape) == tuple(w.shape), f"shape {tuple(g.shape)} vs {tuple(w.shape)} ({note})"
        if g.dtype != w.dtype:
            g, w = (g.double(), w.double()) if (g.is_floating_point() or w.is_floating_point()) else (g.long(), w.long())
        assert torch.equal(g.cpu(), w.cpu()), f"values differ ({note})"
        return
    assert got == want, f"{got!r} vs {want!r} ({note})"


def check_bit1_out(op: Op, got, want, brute, note=""):
    """Where torch returns bool, the bit1 twin must return a bit1 tensor (0-dim reductions stay plain)."""
    if not op.bit1_out:
        return
    gs = got if isinstance(got, (tuple, list)) else [got]
    ws = want if isinstance(want, (tuple, list)) else [want]
    for g, w in zip(gs, ws):
        if isinstance(w, torch.Tensor) and w.dtype == torch.bool:
            assert isinstance(g, brute.Tensor) and g.dtype == brute.bit1, f"expected a bit1 result ({note})"


def run_case(op: Op, bools, brute):
    """Run ``op`` on the bool inputs and on their bit1 twins; both raising counts as agreement."""
    bits = [brute.Tensor(b, dtype=brute.bit1) for b in bools]
    note = f"{op.name} on {[tuple(b.shape) for b in bools]}"
    try:
        want = (op.oracle or op.fn)(*bools)
    except Exception as e_ref:                                            # noqa: BLE001
        try:
            op.fn(*bits)
        except Exception:                                                 # noqa: BLE001
            return
        raise AssertionError(f"torch.bool raised {type(e_ref).__name__} but bit1 did not ({note})")
    got = op.fn(*bits)
    compare(got, want, note)
    if op.oracle is None:
        check_bit1_out(op, got, want, brute, note)
    # the inputs must be left as they were (ops are out-of-place or work on clones)
    for b, x in zip(bools, bits):
        compare(x, b, note + " [input changed]")
