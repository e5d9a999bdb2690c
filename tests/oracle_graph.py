"""A minimal tape over the CPU oracle's primitives, used by tests to evaluate the small
programs of tests/golden/reference_known_answers.json (and the same programs on the device).
It mirrors the reference's GradFns (gradtrack/grad_fn/ops/*.rs, grad_fn/reductions/*.rs)
for the hot-path ops only.  Test infrastructure, not product code."""
import numpy as np


class OVal:
    _next = 1

    def __init__(self, data, rg=False):
        self.data = np.array(data, dtype=np.float32, order="C")  # keeps 0-d results 0-d
        self.rg = rg
        self.node = None
        self.id = OVal._next
        OVal._next += 1


class OracleGraph:
    def __init__(self, ora):
        self.o = ora
        self.grads = {}

    def leaf(self, data, dims, rg=False):
        return OVal(np.asarray(data, np.float32).reshape(dims), rg)

    def _mk(self, data, inputs, bw):
        out = OVal(data, any(i.rg for i in inputs))
        if out.rg:
            out.node = (inputs, bw)
        return out

    @staticmethod
    def _unbroadcast(o, g, shape):
        if g.shape == tuple(shape):
            return g
        if int(np.prod(shape)) == g.size:
            return g.reshape(shape)
        cols = int(np.prod(shape))
        g2 = g.reshape(-1, cols)
        # sum_dims over the leading dimension, rows in ascending order (reductions/sum.rs:255-290)
        return (o.colsum(g2) if cols > 1 else np.array([o.total(g2)], np.float32)).reshape(shape)

    def op(self, name, *args):
        o = self.o
        if name == "matmul" and (args[0].data.ndim > 2 or args[1].data.ndim > 2):
            a, b = args

            def bw(g):
                ga, gb = o.batched_matmul_backward(a.data, b.data, g)
                return [ga if a.rg else None, gb if b.rg else None]
            return self._mk(o.batched_matmul(a.data, b.data), [a, b], bw)
        if name == "matmul":
            a, b = args
            a2 = a.data.reshape(1, -1) if a.data.ndim == 1 else a.data
            b2 = b.data.reshape(-1, 1) if b.data.ndim == 1 else b.data
            out_shape = ([a.data.shape[0]] if a.data.ndim == 2 else []) + ([b.data.shape[1]] if b.data.ndim == 2 else [])
            r = o.matmul(a2, b2).reshape(out_shape)

            def bw(g):
                g2 = g.reshape(a2.shape[0], b2.shape[1])
                ga = o.matmul(g2, np.ascontiguousarray(b2.T)).reshape(a.data.shape) if a.rg else None
                gb = o.matmul(np.ascontiguousarray(a2.T), g2).reshape(b.data.shape) if b.rg else None
                return [ga, gb]
            return self._mk(r, [a, b], bw)
        if name == "add_tensor":
            a, b = args
            if a.data.shape == b.data.shape:
                r = o.add(a.data, b.data)
            else:
                big, small = (a, b) if a.data.size >= b.data.size else (b, a)
                cols = small.data.size
                r = (o.add_row(big.data.reshape(-1, cols), small.data.reshape(-1)) if cols > 1
                     else o.add(big.data, np.full_like(big.data, small.data.reshape(-1)[0]))).reshape(big.data.shape)
            return self._mk(r, [a, b], lambda g: [self._unbroadcast(o, g, a.data.shape) if a.rg else None,
                                                  self._unbroadcast(o, g, b.data.shape) if b.rg else None])
        if name in ("sub_tensor", "mul_tensor", "div_tensor") and args[0].data.shape != args[1].data.shape:
            a, b = args                      # NumPy-style broadcasting: the stretched operands, then the same-shape op
            kind = name[:3]

            def bw(g):
                ga, gb = o.binary_broadcast_backward(kind, a.data, b.data, g)
                return [ga if a.rg else None, gb if b.rg else None]
            return self._mk(o.binary_broadcast(kind, a.data, b.data), [a, b], bw)
        if name == "sub_tensor":
            a, b = args
            return self._mk(o.sub(a.data, b.data), [a, b], lambda g: [g if a.rg else None, o.neg(g) if b.rg else None])
        if name == "mul_tensor":
            a, b = args

            def bw(g):
                ga, gb = o.mul_bwd(a.data, b.data, g)
                return [ga if a.rg else None, gb if b.rg else None]
            return self._mk(o.mul(a.data, b.data), [a, b], bw)
        if name == "div_tensor":
            a, b = args

            def bw(g):
                ga, gb = o.div_bwd(a.data, b.data, g)
                return [ga if a.rg else None, gb if b.rg else None]
            return self._mk(o.div(a.data, b.data), [a, b], bw)
        if name == "relu":
            (x,) = args
            return self._mk(o.relu(x.data), [x], lambda g: [o.relu_bwd(x.data, g)])
        if name == "pow2":
            (x,) = args
            return self._mk(o.square(x.data), [x], lambda g: [o.square_bwd(x.data, g)])
        if name == "sum":
            (x,) = args
            return self._mk(np.array([o.total(x.data)], np.float32), [x],
                            lambda g: [np.full(x.data.shape, g.reshape(-1)[0], np.float32)])
        if name == "mean":
            (x,) = args
            n = x.data.size
            return self._mk(np.array([o.mean(x.data)], np.float32), [x],
                            lambda g: [np.full(x.data.shape, np.float32(1.0) / np.float32(n) * g.reshape(-1)[0], np.float32)])
        if name in o.UNARY:   # exp, log, sqrt, tanh, sigmoid, leaky_relu, *_scalar, pow_scalar: [x, param?]
            x, *params = args
            p = float(params[0]) if params else 0.0
            y = o.unary(name, x.data, p)
            saved = {"out": y, "in": x.data, None: None}[o.UNARY_SAVES[name]]
            return self._mk(y, [x], lambda g: [o.unary_backward(name, saved, g, p)])
        if name in ("permute", "transpose", "t", "reshape", "flatten", "contiguous"):
            x, *params = args
            shape = x.data.shape
            if name == "reshape" or name == "flatten":
                new = o.reshape_dims(x.data.size, params[0] if name == "reshape" else [-1])
                return self._mk(x.data.reshape(new), [x], lambda g: [g.reshape(shape)])       # grad_fn/transforms/reshape.rs
            if name == "contiguous":
                return self._mk(x.data.copy(), [x], lambda g: [g])
            if name == "permute":
                perm = [int(d) for d in params[0]]
            else:
                d0, d1 = (len(shape) - 2, len(shape) - 1) if name == "t" else (int(params[0]), int(params[1]))
                if d0 == d1:   # transpose.rs:169-171: a detached clone
                    return OVal(x.data.copy(), False)
                perm = list(range(len(shape)))
                perm[d0], perm[d1] = perm[d1], perm[d0]
            inv = [perm.index(i) for i in range(len(perm))]
            return self._mk(o.permute(x.data, perm), [x], lambda g: [o.permute(g, inv)])      # grad_fn/transforms/permute.rs
        if name.endswith("_dims") and name[:-5] in o.REDUCE:       # sum_dims, mean_dims, max_dims, ...: [x, dims, keepdim]
            kind = name[:-5]
            x, dims, keepdim = args
            y, mu = o.reduce_dims(kind, x.data, dims, bool(keepdim), want_mean=True)
            return self._mk(y, [x], lambda g: [o.reduce_dims_backward(kind, x.data, y, mu, g, dims)])
        if name in ("max", "min", "norm", "var", "std"):           # whole-tensor forms, result [1]
            (x,) = args
            y, mu = o.reduce_all(name, x.data, want_mean=True)
            return self._mk(y, [x], lambda g: [o.reduce_dims_backward(name, x.data, y, mu, g, None)])
        if name == "softmax":
            x, dim = args
            y = o.softmax(x.data, int(dim))
            return self._mk(y, [x], lambda g: [o.softmax_backward(y, g, int(dim))])
        raise KeyError(name)

    def backward(self, root, grad_output=None):
        g0 = np.ones(root.data.shape, np.float32) if grad_output is None else grad_output.data
        pend = {root.id: (root, g0)}
        while pend:
            vid = max(pend)
            v, g = pend.pop(vid)
            if v.node is None:
                self.grads[v.id] = self.o.add(self.grads[v.id], g) if v.id in self.grads else g
                continue
            inputs, bw = v.node
            for inp, gi in zip(inputs, bw(g)):
                if gi is None or not inp.rg:
                    continue
                gi = np.ascontiguousarray(gi, np.float32)
                if inp.id in pend:
                    pend[inp.id] = (inp, self.o.add(pend[inp.id][1], gi))
                else:
                    pend[inp.id] = (inp, gi)

    def grad(self, v):
        return self.grads.get(v.id)


def run_case_oracle(ora, case):
    G = OracleGraph(ora)
    env = {k: G.leaf(v["data"], v["dims"], v.get("rg", False)) for k, v in case["inputs"].items()}
    for out, opname, *args in case["program"]:
        # string arguments name tensors; numbers are the op's own parameter (slope, scalar, exponent, axis)
        env[out] = G.op("pow2" if opname == "pow_scalar2" else opname, *[env[a] if isinstance(a, str) else a for a in args])
    if "backward" in case:
        go = case["backward"]["grad_output"]
        G.backward(env[case["backward"]["of"]], env[go] if go else None)
    values = {k: v.data for k, v in env.items()}
    grads = {k: G.grad(v) for k, v in env.items()}
    return values, grads


def run_case_device(ts, case):
    env = {}
    for k, v in case["inputs"].items():
        t = ts.Tensor.from_slice(v["data"], v["dims"])
        env[k] = t.with_requires_grad() if v.get("rg", False) else t
    for out, opname, *args in case["program"]:
        a = [env[x] if isinstance(x, str) else x for x in args]
        env[out] = a[0].pow_scalar(2.0) if opname == "pow_scalar2" else getattr(a[0], opname)(*a[1:])
    if "backward" in case:
        go = case["backward"]["grad_output"]
        env[case["backward"]["of"]].backward(env[go] if go else None)
    values = {k: (v.data(), v.shape().dims) for k, v in env.items()}
    grads = {}
    for k, v in env.items():
        g = v.grad_by_value()
        grads[k] = None if g is None else (g.data(), g.shape().dims)
    return values, grads
