"""Mirror of the reference's ``optimizers`` module for Adam (src/optimizers/mod.rs:260-306,
src/optimizers/adam/mod.rs:91-117, 287-320, 1036-1068).  The update runs as one fused
multi-tensor kernel on the GPU."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

from . import _ffi
from ._ffi import TrainStationError, check, vp
from .tensor import Tensor


@dataclass
class AdamConfig:
    """Defaults as in adam/mod.rs:91-117."""
    learning_rate: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    amsgrad: bool = False


class Optimizer:
    """The ``Optimizer`` trait: step, zero_grad, learning_rate, set_learning_rate."""

    def step(self, parameters: Sequence[Tensor]) -> None: raise NotImplementedError
    def zero_grad(self, parameters: Sequence[Tensor]) -> None: raise NotImplementedError
    def learning_rate(self) -> float: raise NotImplementedError
    def set_learning_rate(self, lr: float) -> None: raise NotImplementedError


class Adam(Optimizer):
    def __init__(self, config: AdamConfig | None = None):
        self.config = config or AdamConfig()
        c = self.config
        h = _ffi.lib().ts_adam_new_amsgrad(c.learning_rate, c.beta1, c.beta2, c.eps, c.weight_decay, 1 if c.amsgrad else 0)
        check(h, "Adam::new")
        self._h = vp(h)
        self.grad_scale = 1.0      # 1/world after a data-parallel gradient all-reduce
        self.last_message = ""     # what the reference would eprintln! (skipped parameters)
        self._linked: List[Tensor] = []   # in insertion order (adam/mod.rs:201-206), for checkpoints
        self._saved = None                # (states by saved id, insertion order) of a loaded checkpoint awaiting relink_parameters

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _ffi.lib().ts_adam_free(h)
            except Exception:
                pass

    # constructors named as in the reference
    @staticmethod
    def new() -> "Adam":
        return Adam()

    @staticmethod
    def with_config(config: AdamConfig) -> "Adam":
        return Adam(config)

    @staticmethod
    def with_learning_rate(lr: float) -> "Adam":
        return Adam(AdamConfig(learning_rate=lr))

    def add_parameter(self, p: Tensor) -> None:
        check(_ffi.lib().ts_adam_add_parameter(self._h, p._h), "add_parameter")
        if all(q.id() != p.id() for q in self._linked):
            self._linked.append(p)

    def add_parameters(self, params: Sequence[Tensor]) -> None:
        for p in params:
            self.add_parameter(p)

    @staticmethod
    def _table(params: Sequence[Tensor]):
        arr = (vp * max(len(params), 1))(*[p._h for p in params])
        return arr, len(params)

    def step(self, parameters: Sequence[Tensor]) -> None:
        arr, n = self._table(parameters)
        check(_ffi.lib().ts_adam_step(self._h, arr, n, float(self.grad_scale)), "Adam::step")
        self.last_message = _ffi.last_error()

    def zero_grad(self, parameters: Sequence[Tensor]) -> None:
        arr, n = self._table(parameters)
        _ffi.lib().ts_adam_zero_grad(self._h, arr, n)

    def learning_rate(self) -> float:
        return float(_ffi.lib().ts_adam_learning_rate(self._h))

    def set_learning_rate(self, lr: float) -> None:
        _ffi.lib().ts_adam_set_learning_rate(self._h, float(lr))

    def step_count(self) -> int:
        return int(_ffi.lib().ts_adam_step_count(self._h))

    def state(self, p: Tensor) -> List[Tensor]:
        """[m, v] of a linked parameter (views of the optimizer's device state)."""
        m = _ffi.lib().ts_adam_state_m(self._h, p._h)
        v = _ffi.lib().ts_adam_state_v(self._h, p._h)
        if not m or not v:
            raise TrainStationError("parameter is not linked to this optimizer")
        out = [Tensor(m), Tensor(v)]
        if self.config.amsgrad:   # v_hat_max (adam/mod.rs:130-150 ParameterState)
            out.append(Tensor(_ffi.lib().ts_adam_state_v_hat_max(self._h, p._h)))
        return out

    # ------------------------------------------------------------------ checkpoints
    # optimizers/adam/serialization.rs:692-752: config, per-parameter states keyed by tensor id, the global step count
    # and the insertion order.  A loaded optimizer holds its states on the host until relink_parameters (mod.rs:396-458)
    # attaches them, by position, to the tensors of the new process.
    def _fields(self):
        from . import serialization as S
        lib = _ffi.lib()
        cfg = {"learning_rate": self.learning_rate(), "beta1": self.config.beta1, "beta2": self.config.beta2, "eps": self.config.eps,
               "weight_decay": self.config.weight_decay, "amsgrad": self.config.amsgrad}
        if self._saved is not None:
            states, order = self._saved
            return S.adam_fields(cfg, states, self.step_count(), order)
        states = {}
        for p in self._linked:
            st = self.state(p)
            states[p.id()] = {"m": st[0].data(), "v": st[1].data(), "v_hat_max": st[2].data() if self.config.amsgrad else None,
                              "step": int(lib.ts_adam_param_step(self._h, p._h)), "dims": p.shape().dims}
        return S.adam_fields(cfg, states, self.step_count(), [p.id() for p in self._linked])

    def to_json(self) -> str:
        from . import serialization as S
        return S.fields_to_json(self._fields())

    def to_binary(self) -> bytes:
        from . import serialization as S
        return S.fields_to_binary(self._fields())

    @staticmethod
    def _from_fields(f) -> "Adam":
        from . import serialization as S
        config, states, step_count, order = S.adam_from_fields(f)
        opt = Adam(AdamConfig(**config))
        _ffi.lib().ts_adam_set_step_count(opt._h, int(step_count))
        opt._saved = (states, order)
        return opt

    @staticmethod
    def from_json(text: str) -> "Adam":
        from . import serialization as S
        return Adam._from_fields(S.json_to_fields(text))

    @staticmethod
    def from_binary(data: bytes) -> "Adam":
        from . import serialization as S
        return Adam._from_fields(S.binary_to_fields(data))

    def save(self, path: str, format: str) -> None:
        from .tensor import _save
        _save(path, format, self.to_json, self.to_binary)

    @staticmethod
    def load(path: str, format: str) -> "Adam":
        from .tensor import _load
        return _load(path, format, Adam.from_json, Adam.from_binary)

    def save_json(self, path: str) -> None:
        self.save(path, "json")

    def save_binary(self, path: str) -> None:
        self.save(path, "binary")

    @staticmethod
    def load_json(path: str) -> "Adam":
        return Adam.load(path, "json")

    @staticmethod
    def load_binary(path: str) -> "Adam":
        return Adam.load(path, "binary")

    def saved_parameter_count(self) -> int:
        """Parameters in a loaded checkpoint that relink_parameters still has to attach (0 once linked)."""
        return len(self._saved[1]) if self._saved is not None else 0

    def relink_parameters(self, parameters: Sequence[Tensor]) -> None:
        """adam/mod.rs:396-458: attach the loaded states to `parameters` in the order the checkpoint recorded them."""
        if self._saved is None:
            raise TrainStationError("relink_parameters: this optimizer was not loaded from a checkpoint")
        states, order = self._saved
        for i, p in enumerate(parameters):
            if not p.requires_grad():
                raise TrainStationError(f"Parameter at index {i} must require gradients")
        if len(parameters) != len(order):
            raise TrainStationError(f"Parameter count mismatch: expected {len(order)} parameters, got {len(parameters)}")
        for i, p in enumerate(parameters):
            if order[i] not in states:
                raise TrainStationError(f"No saved state found for parameter at position {i}")
            if list(states[order[i]]["dims"]) != p.shape().dims:
                raise TrainStationError(f"Shape mismatch for parameter at position {i}: expected {list(states[order[i]]['dims'])}, "
                                        f"got {p.shape().dims}")
        lib = _ffi.lib()
        for i, p in enumerate(parameters):
            s = states[order[i]]
            self.add_parameter(p)
            views = self.state(p)
            views[0].copy_from_host(s["m"])
            views[1].copy_from_host(s["v"])
            if self.config.amsgrad and s["v_hat_max"] is not None:
                views[2].copy_from_host(s["v_hat_max"])
            check(lib.ts_adam_set_param_step(self._h, p._h, int(s["step"])), "relink_parameters")
        self._saved = None
