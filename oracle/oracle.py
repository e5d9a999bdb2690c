"""ctypes front end of the CPU oracle (oracle/ts_oracle.c) plus an f64 numpy twin.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of the benchmark.  The product package never imports this module.

The C functions restate the reference's f32 arithmetic in the reference's operation
order (citations beside each function in ts_oracle.c).  The ``*_f64`` functions evaluate
the same definitions in float64; they are the "truth" against which both the f32
restatement and the device results are measured when summation order differs.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libts_oracle.so")
_f = C.POINTER(C.c_float)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, a second or two)."""
    newest = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("ts_oracle.c", "ts_oracle_unary.c", "ts_oracle_variants.c", "ts_oracle_reduce.c", "Makefile"))
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < newest:
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


def adam_update_amsgrad(p, g, m, v, vmax, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
    """In place on p, m, v, vmax (float32 arrays; vmax starts at zero); step is the global step after increment."""
    g = _c(g)
    for a in (p, m, v, vmax):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().ora_adam_update_amsgrad(_p(p), _p(g), _p(m), _p(v), _p(vmax), p.size, lr, beta1, beta2, eps, weight_decay, int(step))


def xorshift_u64(seed, n):
    out = np.empty(n, np.uint64)
    lib().ora_xorshift_u64(int(seed), out.ctypes.data_as(C.POINTER(C.c_uint64)), n)
    return out


def randn(shape, seed):
    out = np.empty(int(np.prod(shape, dtype=np.int64)), np.float32)
    lib().ora_randn(_p(out), out.size, int(seed))
    return out.reshape(shape)


class _MlpArgs(C.Structure):
    _fields_ = [
        ("layers", C.c_int), ("dims", C.POINTER(C.c_size_t)), ("batch", C.c_size_t),
        ("w", C.POINTER(_f)), ("b", C.POINTER(_f)), ("gw", C.POINTER(_f)), ("gb", C.POINTER(_f)),
        ("mw", C.POINTER(_f)), ("vw", C.POINTER(_f)), ("mb", C.POINTER(_f)), ("vb", C.POINTER(_f)),
        ("x", _f), ("target", _f), ("gx", _f), ("y_out", _f),
        ("loss_kind", C.c_int), ("relu_last", C.c_int), ("as_written", C.c_int), ("do_adam", C.c_int),
        ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
        ("weight_decay", C.c_float), ("step", C.c_uint64),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        sz = C.c_size_t
        for name in ("ora_add", "ora_sub", "ora_mul", "ora_div"):
            getattr(L, name).argtypes = [_f, _f, _f, sz]
        L.ora_matmul.argtypes = [_f, _f, _f, sz, sz, sz]
        L.ora_matmul_naive.argtypes = [_f, _f, _f, sz, sz, sz]
        L.ora_transpose.argtypes = [_f, _f, sz, sz]
        L.ora_add_row.argtypes = [_f, _f, _f, sz, sz]
        L.ora_relu.argtypes = [_f, _f, sz]
        L.ora_relu_bwd.argtypes = [_f, _f, _f, sz]
        L.ora_square.argtypes = [_f, _f, sz]
        L.ora_square_bwd.argtypes = [_f, _f, _f, sz]
        L.ora_mul_bwd.argtypes = [_f, _f, _f, _f, _f, sz]
        L.ora_div_bwd.argtypes = [_f, _f, _f, _f, _f, sz]
        L.ora_neg.argtypes = [_f, _f, sz]
        L.ora_fill.argtypes = [_f, C.c_float, sz]
        L.ora_sum.argtypes = [_f, sz]
        L.ora_sum.restype = C.c_float
        L.ora_mean.argtypes = [_f, sz]
        L.ora_mean.restype = C.c_float
        L.ora_colsum.argtypes = [_f, _f, sz, sz]
        L.ora_adam_update.argtypes = [_f, _f, _f, _f, sz, C.c_float, C.c_float, C.c_float,
                                      C.c_float, C.c_float, C.c_uint64]
        L.ora_mlp_step.argtypes = [C.POINTER(_MlpArgs)]
        L.ora_mlp_step.restype = C.c_float
        L.ora_unary.argtypes = [C.c_int, _f, _f, sz, C.c_float]
        L.ora_unary.restype = C.c_int
        L.ora_unary_backward.argtypes = [C.c_int, _f, _f, _f, sz, C.c_float]
        L.ora_unary_backward.restype = C.c_int
        L.ora_softmax.argtypes = [_f, _f, sz, sz, sz]
        L.ora_softmax_backward.argtypes = [_f, _f, _f, sz, sz, sz]
        L.ora_adam_update_amsgrad.argtypes = [_f, _f, _f, _f, _f, sz, C.c_float, C.c_float, C.c_float,
                                              C.c_float, C.c_float, C.c_uint64]
        L.ora_xorshift_u64.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), sz]
        L.ora_randn.argtypes = [_f, sz, C.c_uint64]
        szp, u8p = C.POINTER(C.c_size_t), C.POINTER(C.c_ubyte)
        L.ora_reduce_dims.argtypes = [C.c_int, _f, _f, _f, szp, C.c_int, u8p]
        L.ora_reduce_dims.restype = C.c_int
        L.ora_reduce_all.argtypes = [C.c_int, _f, sz, _f]
        L.ora_reduce_all.restype = C.c_float
        L.ora_reduce_dims_backward.argtypes = [C.c_int, _f, _f, _f, _f, _f, szp, C.c_int, u8p, C.c_int]
        L.ora_reduce_dims_backward.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f)


def _c(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------- f32 restatement

def matmul(a, b, naive=False):
    a, b = _c(a), _c(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    (lib().ora_matmul_naive if naive else lib().ora_matmul)(_p(a), _p(b), _p(c), m, n, k)
    return c


def _binary(name, a, b):
    a, b = _c(a), _c(b)
    assert a.shape == b.shape
    o = np.empty_like(a)
    getattr(lib(), name)(_p(a), _p(b), _p(o), a.size)
    return o


def add(a, b): return _binary("ora_add", a, b)
def sub(a, b): return _binary("ora_sub", a, b)
def mul(a, b): return _binary("ora_mul", a, b)
def div(a, b): return _binary("ora_div", a, b)


def add_row(z, b):
    z, b = _c(z), _c(b)
    o = np.empty_like(z)
    lib().ora_add_row(_p(z), _p(b), _p(o), z.shape[0], z.shape[1])
    return o


def relu(x):
    x = _c(x)
    o = np.empty_like(x)
    lib().ora_relu(_p(x), _p(o), x.size)
    return o


def relu_bwd(x, go):
    x, go = _c(x), _c(go)
    gi = np.empty_like(x)
    lib().ora_relu_bwd(_p(x), _p(go), _p(gi), x.size)
    return gi


def square(x):
    x = _c(x)
    o = np.empty_like(x)
    lib().ora_square(_p(x), _p(o), x.size)
    return o


def square_bwd(x, go):
    x, go = _c(x), _c(go)
    gi = np.empty_like(x)
    lib().ora_square_bwd(_p(x), _p(go), _p(gi), x.size)
    return gi


def mul_bwd(a, b, go):
    a, b, go = _c(a), _c(b), _c(go)
    ga, gb = np.empty_like(a), np.empty_like(a)
    lib().ora_mul_bwd(_p(a), _p(b), _p(go), _p(ga), _p(gb), a.size)
    return ga, gb


def div_bwd(a, b, go):
    a, b, go = _c(a), _c(b), _c(go)
    ga, gb = np.empty_like(a), np.empty_like(a)
    lib().ora_div_bwd(_p(a), _p(b), _p(go), _p(ga), _p(gb), a.size)
    return ga, gb


def neg(x):
    x = _c(x)
    o = np.empty_like(x)
    lib().ora_neg(_p(x), _p(o), x.size)
    return o


# operation codes of ora_unary / ora_unary_backward (ts_oracle_unary.c); the device library uses the same numbers
UNARY = {"exp": 0, "log": 1, "sqrt": 2, "tanh": 3, "sigmoid": 4, "leaky_relu": 5, "add_scalar": 6, "sub_scalar": 7,
         "mul_scalar": 8, "div_scalar": 9, "pow_scalar": 10}
# what the reference's GradFn saves for each op: "out", "in" or None
UNARY_SAVES = {"exp": "out", "log": "in", "sqrt": "out", "tanh": "out", "sigmoid": "out", "leaky_relu": "in",
               "add_scalar": None, "sub_scalar": None, "mul_scalar": None, "div_scalar": None, "pow_scalar": "in"}


class DomainError(ArithmeticError):
    """Where the reference panics: log of x <= 0, division by a zero scalar."""


def unary(name, x, param=0.0, check=True):
    x = _c(x)
    o = np.empty_like(x)
    st = lib().ora_unary(UNARY[name], _p(x), _p(o), x.size, float(param))
    if st == -2:
        raise ValueError(name)
    if st == -1 and check:
        raise DomainError(name)
    return o


def unary_backward(name, saved, go, param=0.0):
    go = _c(go)
    gi = np.empty_like(go)
    sp = _p(_c(saved)) if saved is not None else None
    st = lib().ora_unary_backward(UNARY[name], sp, _p(go), _p(gi), go.size, float(param))
    if st != 0:
        raise ValueError(name)
    return gi


def _softmax_axes(shape, dim):
    outer = int(np.prod(shape[:dim], dtype=np.int64))
    inner = int(np.prod(shape[dim + 1:], dtype=np.int64))
    return outer, int(shape[dim]), inner


def softmax(x, dim):
    x = _c(x)
    y = np.empty_like(x)
    o, r, i = _softmax_axes(x.shape, dim)
    lib().ora_softmax(_p(x), _p(y), o, r, i)
    return y


def softmax_backward(y, go, dim):
    y, go = _c(y), _c(go)
    gi = np.empty_like(y)
    o, r, i = _softmax_axes(y.shape, dim)
    lib().ora_softmax_backward(_p(y), _p(go), _p(gi), o, r, i)
    return gi


REDUCE = {"sum": 0, "mean": 1, "max": 2, "min": 3, "norm": 4, "var": 5, "std": 6}


def _red_args(shape, dims):
    rank = len(shape)
    d = (C.c_size_t * rank)(*[int(s) for s in shape])
    flags = [0] * rank
    for a in dims:
        if not 0 <= int(a) < rank:
            raise IndexError(f"dim {a} out of bounds for rank {rank}")
        flags[int(a)] = 1
    return d, (C.c_ubyte * rank)(*flags), flags


def reduce_out_shape(shape, dims, keepdim):
    """sum.rs:236-249: a reduced axis becomes 1 (keepdim) or disappears; nothing left means [1]."""
    flags = [i in set(int(a) for a in dims) for i in range(len(shape))]
    out = [1 if f else s for s, f in zip(shape, flags)] if keepdim else [s for s, f in zip(shape, flags) if not f]
    return out or [1]


def reduce_dims(kind, x, dims, keepdim=False, want_mean=False):
    """sum_dims / mean_dims / max_dims / min_dims / norm_dims / var_dims / std_dims of the reference."""
    x = _c(x)
    if len(dims) == 0:
        raise ValueError(f"{kind}_dims requires at least one dimension")
    d, flags, _ = _red_args(x.shape, dims)
    oshape = reduce_out_shape(x.shape, dims, keepdim)
    out = np.empty(oshape, np.float32)
    mean = np.empty(oshape, np.float32)
    st = lib().ora_reduce_dims(REDUCE[kind], _p(x), _p(out), _p(mean), d, x.ndim, flags)
    assert st == 0
    return (out, mean) if want_mean else out


def reduce_all(kind, x, want_mean=False):
    """max() / min() / norm() / var() / std() of the reference: one value, shape [1]."""
    x = _c(x)
    m = np.zeros(1, np.float32)
    v = lib().ora_reduce_all(REDUCE[kind], _p(x.reshape(-1)), x.size, _p(m))
    out = np.array([v], np.float32)
    return (out, m) if want_mean else out


def reduce_dims_backward(kind, x, y, mean, go, dims):
    """dims=None means the whole-tensor form (every axis reduced)."""
    x, go = _c(x), _c(go)
    axes = list(range(x.ndim)) if dims is None else dims
    d, flags, _ = _red_args(x.shape, axes)
    gi = np.empty_like(x)
    yp = _p(_c(y).reshape(-1)) if y is not None else None
    mp = _p(_c(mean).reshape(-1)) if mean is not None else None
    st = lib().ora_reduce_dims_backward(REDUCE[kind], _p(x), yp, mp, _p(go.reshape(-1)), _p(gi), d, x.ndim, flags, 1 if go.size == 1 else 0)
    assert st == 0
    return gi


def permute(x, dims):
    """The contiguous result of tensor/transform/permute.rs:147-190 (a strided view: output axis i walks input axis
    dims[i]) read out in order, as contiguous.rs:205-345 does.  Pure data movement: exact."""
    return np.ascontiguousarray(np.transpose(_c(x), tuple(int(d) for d in dims)))


def _batch_broadcast(a_batch, b_batch):
    """tensor/ops/matmul/mod.rs:661-690: batch axes pair up from the right; 1 stretches; anything else must agree."""
    n = max(len(a_batch), len(b_batch))
    out = []
    for i in range(n):
        da = a_batch[len(a_batch) - 1 - i] if i < len(a_batch) else 1
        db = b_batch[len(b_batch) - 1 - i] if i < len(b_batch) else 1
        if da == 1:
            out.append(db)
        elif db == 1 or da == db:
            out.append(da)
        else:
            raise ValueError(f"Cannot broadcast dimensions {da} and {db}")
    return out[::-1]


def _batch_offset(idx, batch, own, mat):
    """mod.rs:764-835: the element offset of batch entry idx in an operand whose own batch dims are `own`."""
    off, stride = 0, mat
    for i in range(len(batch)):
        bd = batch[len(batch) - 1 - i]
        coord, idx = idx % bd, idx // bd
        if i < len(own):
            od = own[len(own) - 1 - i]
            if od != 1:
                off += coord * stride
            stride *= od
    return off


def batched_matmul(a, b):
    """mod.rs:634-740: one matrix product per entry of the broadcast batch, each the same blocked kernel as the 2-D
    case, then the leading axis of extent 1 squeezed away when one operand was 2-D (mod.rs:752-756)."""
    a, b = _c(a), _c(b)
    if a.ndim < 2 or b.ndim < 2:
        raise ValueError("Batched matmul requires at least 2D tensors")
    m, k, k2, n = a.shape[-2], a.shape[-1], b.shape[-2], b.shape[-1]
    if k != k2:
        raise ValueError(f"Inner dimensions must match for batched matmul: {k} vs {k2}")
    ab, bb = list(a.shape[:-2]), list(b.shape[:-2])
    batch = _batch_broadcast(ab, bb)
    count = int(np.prod(batch, dtype=np.int64)) if batch else 1
    out = np.empty((count, m, n), np.float32)
    af, bf = a.reshape(-1), b.reshape(-1)
    for i in range(count):
        ao, bo = _batch_offset(i, batch, ab, m * k), _batch_offset(i, batch, bb, k * n)
        out[i] = matmul(af[ao:ao + m * k].reshape(m, k), bf[bo:bo + k * n].reshape(k, n))
    dims = batch + [m, n]
    if (a.ndim == 2 or b.ndim == 2) and len(dims) > 2 and dims[0] == 1:
        dims = dims[1:]
    return out.reshape(dims)


def _reduce_to_shape(g, want, last_first=True):
    """grad_fn/ops/matmul.rs:276-331 reduce_gradient_to_original_shape (last_first) and grad_fn/utils.rs:23-60
    reduce_gradient_to_shape (not last_first): extra leading axes are summed away one at a time with sum_dims(&[0]),
    then each axis the operand held at extent 1 is summed with keepdim, from the last such axis backwards in the
    first function and from the first forwards in the second."""
    want = list(want)
    g = _c(g)
    if list(g.shape) == want:
        return g
    while g.ndim > len(want):
        rest = g.shape[1:]
        g = reduce_dims("sum", g, [0], keepdim=False).reshape(rest if rest else (1,))
        if not rest:
            break
    dims = [i for i in range(min(g.ndim, len(want))) if want[i] == 1 and g.shape[i] > 1]
    for i in (reversed(dims) if last_first else dims):
        g = reduce_dims("sum", g, [i], keepdim=True)
    return np.ascontiguousarray(g).reshape(want)


def broadcast_shape(sa, sb):
    """tensor/ops/broadcasting.rs:100-135 and the panic text of add.rs:114-122."""
    sa, sb = [int(x) for x in sa], [int(x) for x in sb]
    n = max(len(sa), len(sb))
    out = []
    for i in range(n):
        da = sa[len(sa) - 1 - i] if i < len(sa) else 1
        db = sb[len(sb) - 1 - i] if i < len(sb) else 1
        if da == db or db == 1:
            out.append(da)
        elif da == 1:
            out.append(db)
        else:
            raise ValueError(f"Cannot broadcast tensor shapes {sa} and {sb}: Cannot broadcast shapes {sa} and {sb}: "
                             f"incompatible dimensions at axis {n - 1 - i}")
    return out[::-1]


_BINARY = {"add": add, "sub": sub, "mul": mul, "div": div}


def binary_broadcast(name, a, b):
    """add/sub/mul/div_tensor with broadcasting (add.rs:107-146): both operands are stretched to the common shape
    (the reference materialises them, broadcasting.rs:299-333) and the same-shape loop runs over the copies."""
    a, b = _c(a), _c(b)
    shape = broadcast_shape(a.shape, b.shape)
    return _BINARY[name](np.broadcast_to(a, shape).copy(), np.broadcast_to(b, shape).copy())


def binary_broadcast_backward(name, a, b, go):
    """grad_fn/ops/{add,sub,mul,div}.rs with original_shapes: the full-size gradients over the broadcast shape, each
    reduced to its operand's shape by grad_fn/utils.rs:23-60."""
    a, b, go = _c(a), _c(b), _c(go)
    shape = broadcast_shape(a.shape, b.shape)
    fa, fb = np.broadcast_to(a, shape).copy(), np.broadcast_to(b, shape).copy()
    go = go.reshape(shape)
    if name == "add":
        ga, gb = go, go
    elif name == "sub":
        ga, gb = go, neg(go)
    elif name == "mul":
        ga, gb = mul_bwd(fa, fb, go)
    else:
        ga, gb = div_bwd(fa, fb, go)
    return _reduce_to_shape(ga, a.shape, last_first=False), _reduce_to_shape(gb, b.shape, last_first=False)


def batched_matmul_backward(a, b, go):
    """grad_fn/ops/matmul.rs, the batched branches: dA = go . B^T and dB = A^T . go per batch entry, then reduced to
    the operand's own shape.  go may carry the squeezed shape of the forward's result."""
    a, b = _c(a), _c(b)
    batch = _batch_broadcast(list(a.shape[:-2]), list(b.shape[:-2]))
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    go = _c(go).reshape(batch + [m, n])
    bt = np.ascontiguousarray(np.swapaxes(b, -1, -2))
    at = np.ascontiguousarray(np.swapaxes(a, -1, -2))
    ga = batched_matmul(go, bt).reshape(batch + [m, k])
    gb = batched_matmul(at, go).reshape(batch + [k, n])
    return _reduce_to_shape(ga, a.shape), _reduce_to_shape(gb, b.shape)


def reshape_dims(size, new_shape):
    """transform/reshape.rs:185-215: one -1 is inferred; other entries must be positive; sizes must agree."""
    dims, infer, known = [], None, 1
    for i, d in enumerate(new_shape):
        d = int(d)
        if d == -1:
            if infer is not None:
                raise ValueError("Only one dimension can be -1 for automatic inference")
            infer = i
            dims.append(0)
        elif d <= 0:
            raise ValueError(f"Dimension sizes must be positive, got {d}")
        else:
            dims.append(d)
            known *= d
    if infer is not None:
        if known == 0 or size % known != 0:
            raise ValueError("Cannot infer dimension size")
        dims[infer] = size // known
    if int(np.prod(dims, dtype=np.int64)) != size:
        raise ValueError("Cannot reshape tensor")
    return dims


def total(x) -> np.float32:
    x = _c(x)
    return np.float32(lib().ora_sum(_p(x), x.size))


def mean(x) -> np.float32:
    x = _c(x)
    return np.float32(lib().ora_mean(_p(x), x.size))


def colsum(g):
    g = _c(g)
    o = np.empty(g.shape[1], np.float32)
    lib().ora_colsum(_p(g), _p(o), g.shape[0], g.shape[1])
    return o


def adam_update(p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
    """In place on p, m, v (float32 arrays); step is the global step after increment."""
    g = _c(g)
    for a in (p, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().ora_adam_update(_p(p), _p(g), _p(m), _p(v), p.size, lr, beta1, beta2, eps, weight_decay,
                          int(step))


LOSS_SUM, LOSS_MEAN, LOSS_MSE = 0, 1, 2


class MlpState:
    """Parameters, gradients and Adam moments of an MLP held as float32 numpy arrays."""

    def __init__(self, weights, biases):
        self.w = [_c(w).copy() for w in weights]
        self.b = [_c(b).copy() for b in biases]
        self.gw = [np.zeros_like(w) for w in self.w]
        self.gb = [np.zeros_like(b) for b in self.b]
        self.mw = [np.zeros_like(w) for w in self.w]
        self.vw = [np.zeros_like(w) for w in self.w]
        self.mb = [np.zeros_like(b) for b in self.b]
        self.vb = [np.zeros_like(b) for b in self.b]
        self.step = 0


def mlp_step(st: MlpState, x, target=None, loss_kind=LOSS_MSE, relu_last=False, do_adam=True,
             as_written=False, want_gx=False, want_y=False, lr=1e-3, beta1=0.9, beta2=0.999,
             eps=1e-8, weight_decay=0.0):
    """One fwd + bwd (+ Adam) step of the reference's canonical loop. Returns a dict."""
    x = _c(x)
    L = len(st.w)
    dims = (C.c_size_t * (L + 1))(*([st.w[0].shape[0]] + [w.shape[1] for w in st.w]))
    arr = lambda lst: (_f * L)(*[_p(a) for a in lst])
    gx = np.empty_like(x) if want_gx else None
    nout = st.w[-1].shape[1]
    y = np.empty((x.shape[0], nout), np.float32) if want_y else None
    tgt = _c(target) if target is not None else None
    if do_adam:
        st.step += 1
    keep = [arr(st.w), arr(st.b), arr(st.gw), arr(st.gb), arr(st.mw), arr(st.vw), arr(st.mb),
            arr(st.vb)]
    a = _MlpArgs(L, dims, x.shape[0], *keep, _p(x), _p(tgt) if tgt is not None else None,
                 _p(gx) if gx is not None else None, _p(y) if y is not None else None,
                 loss_kind, int(relu_last), int(as_written), int(do_adam), lr, beta1, beta2, eps,
                 weight_decay, st.step)
    loss = lib().ora_mlp_step(C.byref(a))
    return {"loss": np.float32(loss), "gx": gx, "y": y}


# ----------------------------------------------------------------------- f64 twin

def matmul_f64(a, b):
    return np.asarray(a, np.float64) @ np.asarray(b, np.float64)


def mlp_step_f64(weights, biases, x, target=None, loss_kind=LOSS_MSE, relu_last=False):
    """Forward and gradients of the same graph in float64 (no Adam). Returns a dict."""
    w = [np.asarray(a, np.float64) for a in weights]
    b = [np.asarray(a, np.float64) for a in biases]
    h = [np.asarray(x, np.float64)]
    z = []
    L = len(w)
    for l in range(L):
        zl = h[l] @ w[l] + b[l]
        z.append(zl)
        h.append(np.maximum(zl, 0.0) if (l + 1 < L or relu_last) else zl)
    y = h[-1]
    if loss_kind == LOSS_SUM:
        loss, g = y.sum(), np.ones_like(y)
    elif loss_kind == LOSS_MEAN:
        loss, g = y.mean(), np.full_like(y, 1.0 / y.size)
    else:
        d = y - np.asarray(target, np.float64)
        loss, g = (d * d).mean(), 2.0 * d / y.size
    gw, gb = [None] * L, [None] * L
    for l in reversed(range(L)):
        if l + 1 < L or relu_last:
            g = g * (z[l] > 0)
        gb[l] = g.sum(axis=0)
        gw[l] = h[l].T @ g
        g = g @ w[l].T
    return {"loss": loss, "y": y, "z": z, "gw": gw, "gb": gb, "gx": g}


def reduced_precision_step_check(weights, biases, x, target, device_masks, got_gw, got_gb, loss_kind=LOSS_MSE,
                                 relu_last=False, band_rel=2e-3):
    """The checkable form of "gradients within rel 2e-3" for a GEMM mode that does not reproduce FP32 bits.

    A pre-activation z within the GEMM's rounding error of zero can take the other ReLU branch than in exact
    arithmetic, and a flipped mask element changes that element's gradient outright whatever the GEMM's accuracy.
    So: (1) the masks the device forward produced (`device_masks`, one boolean array per activated layer) must agree
    with the float64 ones wherever |z| lies outside the band `band_rel * sum_k |a||w|`; (2) the gradients are
    compared, as Frobenius-norm relative errors, with a float64 evaluation that uses the device's own masks, so that
    what is left is GEMM arithmetic.  Returns {"outside_mismatch": [...], "flips": [...], "in_band": [...],
    "elements": [...], "rel_gw": [...], "rel_gb": [...]}, one entry per layer (mask lists: per activated layer)."""
    w = [np.asarray(a, np.float64) for a in weights]
    b = [np.asarray(a, np.float64) for a in biases]
    L = len(w)
    exact = mlp_step_f64(weights, biases, x, target, loss_kind=loss_kind, relu_last=relu_last)
    out = {"outside_mismatch": [], "flips": [], "in_band": [], "elements": [], "rel_gw": [None] * L, "rel_gb": [None] * L}
    act = np.asarray(x, np.float64)
    n_act = L if relu_last else L - 1
    for l in range(n_act):
        band = band_rel * (np.abs(act) @ np.abs(w[l]))
        z = exact["z"][l]
        outside = np.abs(z) > band
        dm = np.asarray(device_masks[l], bool)
        out["outside_mismatch"].append(int((dm[outside] != (z > 0)[outside]).sum()))
        out["flips"].append(int((dm != (z > 0)).sum()))
        out["in_band"].append(int((~outside).sum()))
        out["elements"].append(int(z.size))
        act = np.maximum(z, 0.0)
    # float64 forward and backward with the device's masks
    hs = [np.asarray(x, np.float64)]
    for l in range(L):
        zl = hs[l] @ w[l] + b[l]
        hs.append(zl * np.asarray(device_masks[l], bool) if l < n_act else zl)
    y = hs[L]
    if loss_kind == LOSS_SUM:
        g = np.ones_like(y)
    elif loss_kind == LOSS_MEAN:
        g = np.full_like(y, 1.0 / y.size)
    else:
        g = 2.0 * (y - np.asarray(target, np.float64)) / y.size
    rel = lambda a, r: float(np.linalg.norm(np.asarray(a, np.float64) - r) / max(np.linalg.norm(r), 1e-300))
    for l in reversed(range(L)):
        if l < n_act:
            g = g * np.asarray(device_masks[l], bool)
        out["rel_gw"][l] = rel(got_gw[l], hs[l].T @ g)
        out["rel_gb"][l] = rel(got_gb[l], g.sum(axis=0))
        g = g @ w[l].T
    return out


def adam_update_f64(p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
    """Textbook Adam in float64 using the f32-rounded hyper-parameters, out of place."""
    b1, b2 = float(np.float32(beta1)), float(np.float32(beta2))
    lr, eps = float(np.float32(lr)), float(np.float32(eps))
    p, g, m, v = (np.asarray(a, np.float64) for a in (p, g, m, v))
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh = m / (1 - b1 ** step)
    vh = v / (1 - b2 ** step)
    return p - lr * mh / (np.sqrt(vh) + eps), m, v
