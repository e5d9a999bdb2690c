"""Host-side mirror of the reference's ``Tensor`` API for the training-step hot path.

Method names, argument meaning and error behaviour follow the Rust API
(src/tensor/core/utils.rs, src/tensor/ops/*.rs, src/tensor/reductions/*.rs) so that tests
read like the reference's own: ``x.matmul(w).add_tensor(b).relu().sum().backward(None)``.
All data lives on the GPU; every method forwards to the C ABI.  Where the reference
panics (shape mismatch), these raise ``TrainStationError``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from ._ffi import TrainStationError, check, u64, vp


def _dims(shape: Sequence[int]):
    shape = [int(s) for s in shape]
    return (u64 * max(len(shape), 1))(*shape), len(shape)


class Shape:
    """Subset of the reference's ``Shape`` (src/tensor/core/shape.rs:96-143): ``dims`` and ``size``."""

    def __init__(self, dims):
        self.dims = list(dims)
        self.size = int(np.prod(dims)) if len(dims) else 1

    def rank(self) -> int:
        return len(self.dims)

    def __eq__(self, other):
        return isinstance(other, Shape) and self.dims == other.dims

    def __repr__(self):
        return f"Shape(dims={self.dims})"


class Tensor:
    __slots__ = ("_h", "_keep")

    def __init__(self, handle, keep=None):
        if not handle:
            raise TrainStationError(_ffi.last_error())
        self._h = vp(handle)
        self._keep = keep  # host buffers that must outlive an asynchronous upload

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _ffi.lib().ts_tensor_free(h)
            except Exception:
                pass

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def new(shape_dims: Sequence[int]) -> "Tensor":
        """Uninitialised tensor (core/utils.rs:121-171)."""
        d, r = _dims(shape_dims)
        return Tensor(_ffi.lib().ts_tensor_new(d, r))

    @staticmethod
    def zeros(shape_dims: Sequence[int]) -> "Tensor":
        d, r = _dims(shape_dims)
        return Tensor(_ffi.lib().ts_tensor_zeros(d, r))

    @staticmethod
    def ones(shape_dims: Sequence[int]) -> "Tensor":
        d, r = _dims(shape_dims)
        return Tensor(_ffi.lib().ts_tensor_ones(d, r))

    @staticmethod
    def from_slice(data, shape_dims: Sequence[int]) -> "Tensor":
        """init/data.rs:227-247: errors when the data length does not match the shape."""
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        n = int(np.prod([int(s) for s in shape_dims])) if len(shape_dims) else 1
        if a.size != n:
            raise TrainStationError(f"from_slice: data has {a.size} elements, shape {list(shape_dims)} needs {n}")
        d, r = _dims(shape_dims)
        return Tensor(_ffi.lib().ts_tensor_from_slice(a.ctypes.data_as(vp), d, r))

    @staticmethod
    def randn(shape_dims: Sequence[int], seed: Optional[int] = None) -> "Tensor":
        """init/random.rs:231-236: with a seed, the reference's own stream value for value (xorshift64 and
        Box-Muller, generated on the host); without one, a clock-derived seed."""
        d, r = _dims(shape_dims)
        if seed is None:
            return Tensor(_ffi.lib().ts_tensor_randn(d, r, 0, 0))
        return Tensor(_ffi.lib().ts_tensor_randn(d, r, int(seed) & 0xFFFFFFFFFFFFFFFF, 1))

    @staticmethod
    def from_pinned_async(pinned: "PinnedBuffer", shape_dims: Sequence[int]) -> "Tensor":
        """Upload from page-locked memory on the copy stream; overlaps kernels already queued."""
        d, r = _dims(shape_dims)
        n = int(np.prod([int(s) for s in shape_dims]))
        if n > pinned.size:
            raise TrainStationError("from_pinned_async: shape larger than the pinned buffer")
        return Tensor(_ffi.lib().ts_tensor_from_pinned_async(pinned.ptr, d, r), keep=pinned)

    # ------------------------------------------------------------------ properties
    def id(self) -> int:
        return int(_ffi.lib().ts_tensor_id(self._h))

    def size(self) -> int:
        return int(_ffi.lib().ts_tensor_size(self._h))

    def shape(self) -> Shape:
        r = _ffi.lib().ts_tensor_rank(self._h)
        buf = (u64 * max(r, 1))()
        check(_ffi.lib().ts_tensor_dims(self._h, buf), "shape")
        return Shape([int(buf[i]) for i in range(r)])

    def requires_grad(self) -> bool:
        return bool(_ffi.lib().ts_tensor_requires_grad(self._h))

    def with_requires_grad(self) -> "Tensor":
        check(_ffi.lib().ts_tensor_set_requires_grad(self._h, True), "with_requires_grad")
        return self

    def set_requires_grad(self, flag: bool) -> None:
        check(_ffi.lib().ts_tensor_set_requires_grad(self._h, bool(flag)), "set_requires_grad")

    def data_ptr(self) -> int:
        p = _ffi.lib().ts_tensor_data_ptr(self._h)
        check(p, "data_ptr")
        return int(p)

    def data(self) -> np.ndarray:
        """Tensor::data(): a host copy, shaped like the tensor."""
        sh = self.shape().dims
        out = np.empty(self.size(), np.float32)
        check(_ffi.lib().ts_tensor_to_host(self._h, out.ctypes.data_as(vp)), "data")
        return out.reshape(sh)

    def value(self) -> float:
        """Tensor::value(): the single element of a one-element tensor."""
        if self.size() != 1:
            raise TrainStationError("value() can only be called on tensors with exactly one element")
        return float(self.data().reshape(-1)[0])

    def get(self, idx: Sequence[int]) -> float:
        return float(self.data()[tuple(idx)])

    def copy_from_host(self, data) -> None:
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        if a.size != self.size():
            raise TrainStationError("copy_from_host: size mismatch")
        check(_ffi.lib().ts_tensor_copy_from_host(self._h, a.ctypes.data_as(vp)), "copy_from_host")

    def fill(self, value: float) -> None:
        check(_ffi.lib().ts_tensor_fill(self._h, float(value)), "fill")

    # ------------------------------------------------------------------ ops
    def _bin(self, other: "Tensor", fn) -> "Tensor":
        if not isinstance(other, Tensor):
            raise TypeError("operand must be a Tensor")
        return Tensor(fn(self._h, other._h))

    def matmul(self, other: "Tensor") -> "Tensor":
        return self._bin(other, _ffi.lib().ts_tensor_matmul)

    def add_tensor(self, other: "Tensor") -> "Tensor":
        return self._bin(other, _ffi.lib().ts_tensor_add_tensor)

    def sub_tensor(self, other: "Tensor") -> "Tensor":
        return self._bin(other, _ffi.lib().ts_tensor_sub_tensor)

    def mul_tensor(self, other: "Tensor") -> "Tensor":
        return self._bin(other, _ffi.lib().ts_tensor_mul_tensor)

    def div_tensor(self, other: "Tensor") -> "Tensor":
        return self._bin(other, _ffi.lib().ts_tensor_div_tensor)

    def relu(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_relu(self._h))

    def pow_scalar(self, exponent: float) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_pow_scalar(self._h, float(exponent)))

    def sum(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_sum(self._h))

    def mean(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_mean(self._h))

    # unary and scalar ops (tensor/ops/{exp,log,sqrt,tanh,sigmoid,leaky_relu,softmax}.rs, *_scalar of add/sub/mul/div.rs)
    def exp(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_exp(self._h))

    def log(self) -> "Tensor":
        """Raises where the reference panics: an element <= 0 (log.rs:68-107)."""
        return Tensor(_ffi.lib().ts_tensor_log(self._h))

    def sqrt(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_sqrt(self._h))

    def tanh(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_tanh(self._h))

    def sigmoid(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_sigmoid(self._h))

    def leaky_relu(self, negative_slope: float) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_leaky_relu(self._h, float(negative_slope)))

    def softmax(self, dim: int) -> "Tensor":
        if dim < 0:
            raise ValueError("softmax dim is an unsigned axis index (softmax.rs:110)")
        return Tensor(_ffi.lib().ts_tensor_softmax(self._h, int(dim)))

    def add_scalar(self, scalar: float) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_add_scalar(self._h, float(scalar)))

    def sub_scalar(self, scalar: float) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_sub_scalar(self._h, float(scalar)))

    def mul_scalar(self, scalar: float) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_mul_scalar(self._h, float(scalar)))

    def div_scalar(self, scalar: float) -> "Tensor":
        """Raises where the reference panics: a zero scalar (div.rs:511-514)."""
        return Tensor(_ffi.lib().ts_tensor_div_scalar(self._h, float(scalar)))

    # reductions over axes (tensor/reductions/*.rs); kinds as enum ts_reduce_kind
    def _reduce_dims(self, kind: int, dims: Sequence[int], keepdim: bool) -> "Tensor":
        if any(int(d) < 0 for d in dims):
            raise TrainStationError("reduction axes are unsigned")
        arr = (C.c_ulonglong * max(len(dims), 1))(*[int(d) for d in dims])
        return Tensor(_ffi.lib().ts_tensor_reduce_dims(self._h, kind, arr, len(dims), 1 if keepdim else 0))

    def sum_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":     # sum.rs:225-306
        return self._reduce_dims(0, dims, keepdim)

    def mean_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":    # mean.rs:186-215
        return self._reduce_dims(1, dims, keepdim)

    def max_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":     # max.rs:65-145
        return self._reduce_dims(2, dims, keepdim)

    def min_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":
        return self._reduce_dims(3, dims, keepdim)

    def norm_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":
        return self._reduce_dims(4, dims, keepdim)

    def var_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":
        return self._reduce_dims(5, dims, keepdim)

    def std_dims(self, dims: Sequence[int], keepdim: bool) -> "Tensor":
        return self._reduce_dims(6, dims, keepdim)

    def max(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_reduce_all(self._h, 2))

    def min(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_reduce_all(self._h, 3))

    def norm(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_reduce_all(self._h, 4))

    def var(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_reduce_all(self._h, 5))

    def std(self) -> "Tensor":
        return Tensor(_ffi.lib().ts_tensor_reduce_all(self._h, 6))

    # shape and layout (tensor/transform/{reshape,flatten,squeeze,unsqueeze,transpose,permute,contiguous}.rs)
    def reshape(self, new_shape: Sequence[int]) -> "Tensor":
        """reshape.rs:139-215: shares the storage; one dimension may be -1."""
        arr = (C.c_longlong * max(len(new_shape), 1))(*[int(d) for d in new_shape])
        return Tensor(_ffi.lib().ts_tensor_reshape(self._h, arr, len(new_shape)))

    def flatten(self) -> "Tensor":                       # flatten.rs:124-126
        return self.reshape([-1])

    def squeeze(self, dim: Optional[int] = None) -> "Tensor":
        """squeeze.rs:184-214, including its checks."""
        dims = self.shape().dims
        if dim is not None:
            if not 0 <= dim < len(dims):
                raise TrainStationError(f"Dimension {dim} out of bounds")
            if dims[dim] != 1:
                raise TrainStationError(f"Cannot squeeze dimension {dim} with size {dims[dim]}")
            new = [s for i, s in enumerate(dims) if i != dim]
        else:
            new = [s for s in dims if s != 1]
        return self.reshape(new or [1])

    def unsqueeze(self, dim: int) -> "Tensor":           # unsqueeze.rs:218-224
        dims = list(self.shape().dims)
        if not 0 <= dim <= len(dims):
            raise TrainStationError(f"Dimension {dim} out of bounds")
        dims.insert(dim, 1)
        return self.reshape(dims)

    def is_contiguous(self) -> bool:
        """False for a transposed / permuted view, which shares its source's storage."""
        return bool(_ffi.lib().ts_tensor_is_contiguous(self._h))

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        """transpose.rs:156-200: a view that shares the storage; contiguous() makes the copy."""
        if dim0 < 0 or dim1 < 0:
            raise TrainStationError("transpose axes are unsigned")
        return Tensor(_ffi.lib().ts_tensor_transpose(self._h, int(dim0), int(dim1)))

    def t(self) -> "Tensor":                             # transpose.rs:283-291
        rank = self.shape().rank()
        if rank < 2:
            raise TrainStationError(f"Matrix transpose requires at least 2 dimensions, got {rank}")
        return self.transpose(rank - 2, rank - 1)

    def permute(self, dims: Sequence[int]) -> "Tensor":  # permute.rs:147-190
        if any(d < 0 for d in dims):
            raise TrainStationError("permute axes are unsigned")
        arr = (C.c_ulonglong * max(len(dims), 1))(*[int(d) for d in dims])
        return Tensor(_ffi.lib().ts_tensor_permute(self._h, arr, len(dims)))

    def contiguous(self) -> "Tensor":                    # contiguous.rs:123-137
        return Tensor(_ffi.lib().ts_tensor_contiguous(self._h))

    def view(self, new_shape: Sequence[int]) -> "Tensor":
        """core/utils.rs:1285-1289: a view with a new shape over the same storage (the reshape of a contiguous tensor)."""
        return self.reshape(new_shape)

    def clone(self) -> "Tensor":
        """Clone (tensor/core/mod.rs:344-378): a copy of the values with no gradient history."""
        return Tensor(_ffi.lib().ts_tensor_clone(self._h))

    # joining and splitting (tensor/transform/{cat,stack,split}.rs)
    @staticmethod
    def cat(tensors: Sequence["Tensor"], dim: int) -> "Tensor":
        if len(tensors) == 0:
            raise TrainStationError("cat requires at least one tensor")
        if dim < 0:
            raise TrainStationError("cat axis is unsigned")
        arr = (vp * len(tensors))(*[t._h for t in tensors])
        return Tensor(_ffi.lib().ts_tensor_cat(arr, len(tensors), int(dim)), keep=list(tensors))

    @staticmethod
    def stack(tensors: Sequence["Tensor"], dim: int) -> "Tensor":
        """stack.rs:165-230: a new axis of length len(tensors) at `dim`; here the concatenation of the unsqueezed inputs."""
        if len(tensors) == 0:
            raise TrainStationError("stack requires at least one tensor")
        base = tensors[0].shape().dims
        for t in tensors:
            if t.shape().dims != base:
                raise TrainStationError("All tensors must have identical shapes for stack")
        if not 0 <= dim <= len(base):
            raise TrainStationError(f"stack dim {dim} out of bounds for rank {len(base)}")
        return Tensor.cat([t.unsqueeze(dim) for t in tensors], dim)

    def split(self, split_size: int, dim: int) -> list:
        """split.rs:159-180: pieces of `split_size` along `dim`, the last one shorter."""
        dims = self.shape().dims
        if len(dims) == 0:
            raise TrainStationError("split requires non-zero rank")
        if not 0 <= dim < len(dims):
            raise TrainStationError(f"split dim {dim} out of bounds for rank {len(dims)}")
        if split_size <= 0:
            raise TrainStationError("split_size must be > 0")
        sizes, remaining = [], dims[dim]
        while remaining > 0:
            sizes.append(min(remaining, split_size))
            remaining -= sizes[-1]
        return self.split_with_sizes(sizes, dim) if sizes else []

    def split_with_sizes(self, split_sizes: Sequence[int], dim: int) -> list:
        """split.rs:284-330.  Each piece is a contiguous copy (the reference returns a view for the first one)."""
        dims = self.shape().dims
        if len(dims) == 0:
            raise TrainStationError("split requires non-zero rank")
        if not 0 <= dim < len(dims):
            raise TrainStationError(f"split dim {dim} out of bounds for rank {len(dims)}")
        if sum(split_sizes) != dims[dim]:
            raise TrainStationError(f"sum of split sizes {sum(split_sizes)} must equal size {dims[dim]} of dim {dim}")
        out, start = [], 0
        for n in split_sizes:
            out.append(Tensor(_ffi.lib().ts_tensor_split_piece(self._h, int(dim), int(start), int(n))))
            start += n
        return out

    # operator sugar: tensor/core/operators.rs forwards Tensor (op) Tensor to the *_tensor methods (:120-410),
    # Tensor (op) f32 to the *_scalar methods (:418-660) and -Tensor to mul_scalar(-1.0) (:690-705)
    @staticmethod
    def _is_scalar(v) -> bool:
        return isinstance(v, (int, float, np.floating, np.integer))

    def __add__(self, other):
        return self.add_scalar(other) if Tensor._is_scalar(other) else self.add_tensor(other)

    def __sub__(self, other):
        return self.sub_scalar(other) if Tensor._is_scalar(other) else self.sub_tensor(other)

    def __mul__(self, other):
        return self.mul_scalar(other) if Tensor._is_scalar(other) else self.mul_tensor(other)

    def __truediv__(self, other):
        return self.div_scalar(other) if Tensor._is_scalar(other) else self.div_tensor(other)

    def __radd__(self, scalar):      # f32 + &Tensor -> add_scalar (operators.rs:448-472)
        return self.add_scalar(scalar)

    def __rmul__(self, scalar):      # f32 * &Tensor -> mul_scalar (operators.rs:595-620)
        return self.mul_scalar(scalar)

    def __rsub__(self, scalar):
        """f32 - &Tensor (operators.rs:535-547): the reference negates a detached clone and adds the scalar,
        so the result carries no gradient history; the same holds here."""
        lib = _ffi.lib()
        lib.ts_no_grad_push()
        try:
            return self.mul_scalar(-1.0).add_scalar(scalar)
        finally:
            lib.ts_no_grad_pop()

    def __rtruediv__(self, scalar):  # f32 / &Tensor -> pow_scalar(-1.0).mul_scalar(s) (operators.rs:665-685)
        return self.pow_scalar(-1.0).mul_scalar(scalar)

    def __neg__(self):
        return self.mul_scalar(-1.0)

    __matmul__ = matmul

    # ------------------------------------------------------------------ checkpoints (serialization/mod.rs:271-460)
    # The reference's JSON and TS_B binary formats (see serialization.py).  `device` is what the file records: "Cpu" by
    # default, so that a reference build without CUDA can load it; loading ignores the recorded device and puts the
    # tensor on this thread's current device.
    def _fields(self, device: str):
        from . import serialization as S
        return S.tensor_fields(self.data(), self.shape().dims, self.requires_grad(), device=device, index=0)

    def to_json(self, device: str = "Cpu") -> str:
        from . import serialization as S
        return S.fields_to_json(self._fields(device))

    def to_binary(self, device: str = "Cpu") -> bytes:
        from . import serialization as S
        return S.fields_to_binary(self._fields(device))

    @staticmethod
    def _from_fields(f) -> "Tensor":
        from . import serialization as S
        arr, rg, _dev, _idx = S.tensor_from_fields(f)
        t = Tensor.from_slice(arr, list(arr.shape))
        return t.with_requires_grad() if rg else t

    @staticmethod
    def from_json(text: str) -> "Tensor":
        from . import serialization as S
        return Tensor._from_fields(S.json_to_fields(text))

    @staticmethod
    def from_binary(data: bytes) -> "Tensor":
        from . import serialization as S
        return Tensor._from_fields(S.binary_to_fields(data))

    def save(self, path: str, format: str) -> None:
        """format: "json" or "binary" (serialization/mod.rs Format)."""
        _save(path, format, self.to_json, self.to_binary)

    @staticmethod
    def load(path: str, format: str) -> "Tensor":
        return _load(path, format, Tensor.from_json, Tensor.from_binary)

    # StructSerializable's shorthands (serialization/core/traits.rs:265-340)
    def save_json(self, path: str) -> None:
        self.save(path, "json")

    def save_binary(self, path: str) -> None:
        self.save(path, "binary")

    @staticmethod
    def load_json(path: str) -> "Tensor":
        return Tensor.load(path, "json")

    @staticmethod
    def load_binary(path: str) -> "Tensor":
        return Tensor.load(path, "binary")

    # ------------------------------------------------------------------ gradtrack
    def backward(self, grad_output: Optional["Tensor"] = None) -> None:
        """core/utils.rs:634-636 -> gradtrack/engine.rs:962-1047."""
        g = grad_output._h if grad_output is not None else None
        check(_ffi.lib().ts_tensor_backward(self._h, g), "backward")

    def grad_by_value(self) -> Optional["Tensor"]:
        """core/utils.rs:525-534: the accumulated gradient, or None."""
        h = _ffi.lib().ts_tensor_grad_by_value(self._h)
        return Tensor(h) if h else None

    def __repr__(self):
        return f"Tensor(id={self.id()}, dims={self.shape().dims}, requires_grad={self.requires_grad()})"


def _save(path: str, format: str, to_json, to_binary) -> None:
    fmt = str(format).lower()
    if fmt == "json":
        with open(path, "w", encoding="utf-8") as fh:
            fh.write(to_json())
    elif fmt in ("binary", "bin"):
        with open(path, "wb") as fh:
            fh.write(to_binary())
    else:
        raise TrainStationError(f"unknown format {format!r} (json or binary)")


def _load(path: str, format: str, from_json, from_binary):
    fmt = str(format).lower()
    if fmt == "json":
        with open(path, "r", encoding="utf-8") as fh:
            return from_json(fh.read())
    if fmt in ("binary", "bin"):
        with open(path, "rb") as fh:
            return from_binary(fh.read())
    raise TrainStationError(f"unknown format {format!r} (json or binary)")


class PinnedBuffer:
    """Page-locked host memory viewed as a float32 numpy array (for overlapped uploads)."""

    def __init__(self, n_elements: int):
        self.size = int(n_elements)
        p = _ffi.lib().ts_host_alloc_pinned(self.size)
        check(p, "ts_host_alloc_pinned")
        self.ptr = vp(p)
        self.array = np.ctypeslib.as_array(C.cast(self.ptr, C.POINTER(C.c_float)), shape=(self.size,))

    def __del__(self):
        p, self.ptr = getattr(self, "ptr", None), None
        if p:
            try:
                _ffi.lib().ts_host_free_pinned(p)
            except Exception:
                pass
