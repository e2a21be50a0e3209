"""Python restatement of the reference's Matmul shape / dtype rules (TEST INFRASTRUCTURE).

Follows, in the reference project (FL33TW00D/ratchet):
  Shape::multi_broadcast      crates/ratchet-core/src/shape.rs:118-136
  Shape::is_vector            crates/ratchet-core/src/shape.rs:71-75
  Matmul::new                 crates/ratchet-core/src/ops/matmul.rs:258-282
  Matmul::compute_c_shape     crates/ratchet-core/src/ops/matmul.rs:284-361
  Matmul::check_dtypes        crates/ratchet-core/src/ops/matmul.rs:454-477
  GEMMSpec::new + accessors   crates/ratchet-core/src/ops/matmul.rs:53-245

It is used by the tests to check the library's C++ spec layer, and it is pinned itself
against torch.matmul's output shapes (the reference tests' ground truth).
"""
from __future__ import annotations

from dataclasses import dataclass
from math import prod


class ShapeError(Exception):
    """Where the reference returns an error (anyhow::bail!)."""


class InvariantError(Exception):
    """Where the reference panics."""


def multi_broadcast(shapes):
    if not shapes:
        return None
    max_rank = max(len(s) for s in shapes)
    out = []
    for i in range(max_rank):
        cur = 1
        for s in shapes:
            dim = s[len(s) - i - 1] if i < len(s) else 1
            if dim != 1:
                if cur != 1 and dim != cur:
                    return None
                cur = dim
        out.insert(0, cur)
    return out


def is_vector(shape) -> bool:
    return len([d for d in shape if d != 1]) <= 1


def compute_c_shape(a_shape, b_shape, trans_lhs, trans_rhs, trans_out):
    a, b = list(a_shape), list(b_shape)
    implicit_m = len(a) < 2
    implicit_n = len(b) < 2
    if implicit_m:
        a.insert(int(trans_lhs), 1)
    if implicit_n:
        b.insert(int(not trans_rhs), 1)
    while len(a) < len(b):
        a.insert(0, 1)
    while len(b) < len(a):
        b.insert(0, 1)
    prefix = multi_broadcast([a[:-2], b[:-2]]) if len(a) > 2 else []
    if prefix is None:
        raise ShapeError(f"Matmul broadcasting: a: {a} b: {b}")
    m, ka = a[-2], a[-1]
    kb, n = b[-2], b[-1]
    if trans_lhs:
        m, ka = ka, m
    if trans_rhs:
        kb, n = n, kb
    if ka != kb:
        raise ShapeError(f"Matmul broadcasting: ka != kb: {ka} != {kb}")
    c = list(prefix)
    if trans_out:
        if not implicit_n:
            c.append(n)
        if not implicit_m:
            c.append(m)
    else:
        if not implicit_m:
            c.append(m)
        if not implicit_n:
            c.append(n)
    return c


ALLOWED_PAIRS = {("F32", "F32"), ("F16", "F16"), ("Q8_0F", "F32"), ("Q8_0H", "F16")}


def check_dtypes(lhs_dt, rhs_dt, bias_dt=None):
    if (lhs_dt, rhs_dt) not in ALLOWED_PAIRS:
        raise InvariantError(f"Failed to validate DTypes: {lhs_dt}, {rhs_dt}")
    if bias_dt is not None and bias_dt != rhs_dt:
        raise InvariantError(f"Failed to validate DTypes: bias {bias_dt}, rhs {rhs_dt}")


@dataclass
class GEMMSpec:
    lhs_shape: list
    rhs_shape: list
    out_shape: list
    lhs_stack: int
    rhs_stack: int
    out_stack: int
    stacks: int
    trans_lhs: bool
    trans_rhs: bool
    trans_out: bool

    @property
    def dim_inner(self):
        return self.lhs_shape[0] if self.trans_lhs else self.lhs_shape[1]

    @property
    def dim_lhs_outer(self):
        return self.out_shape[0]

    @property
    def dim_rhs_outer(self):
        return self.out_shape[1]

    @property
    def is_gemv(self):
        return is_vector(self.rhs_shape) and not self.trans_lhs


def gemm_spec(lhs_shape, rhs_shape, out_shape, trans_lhs, trans_rhs, trans_out) -> GEMMSpec:
    lhs, rhs, c = list(lhs_shape), list(rhs_shape), list(out_shape)
    if len(lhs) < 2 or len(rhs) < 2:
        raise InvariantError("MatMul: inputs must be at least 2D")
    while len(lhs) < len(rhs):
        lhs.insert(0, 1)
    while len(rhs) < len(lhs):
        rhs.insert(0, 1)
    stack_dims = len(c) - 2
    stack_shape = c[:stack_dims]
    lhs_stack = prod(lhs[:stack_dims])
    rhs_stack = prod(rhs[:stack_dims])
    out_stack = prod(c[:stack_dims])
    lhs, rhs, c = lhs[stack_dims:], rhs[stack_dims:], c[stack_dims:]
    if lhs_stack != 1 and rhs_stack != 1:
        if not (lhs_stack == rhs_stack == out_stack):
            raise InvariantError("stacks must be equal or broadcast from 1")
    return GEMMSpec(lhs, rhs, c, lhs_stack, rhs_stack, out_stack, prod(stack_shape),
                    trans_lhs, trans_rhs, trans_out)


def matmul_new_guards(lhs_dt, bias_shape, trans_lhs):
    if bias_shape is not None and not is_vector(bias_shape):
        raise InvariantError("Bias must be a vector")
    if lhs_dt.startswith("Q") and trans_lhs:
        raise InvariantError("Transposed quantized inputs are not supported")
