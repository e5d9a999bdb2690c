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
