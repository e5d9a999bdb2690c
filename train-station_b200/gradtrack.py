"""Grad-mode control and tape utilities (src/gradtrack/no_grad_track.rs:96-260,
src/gradtrack/engine.rs:812-816).  State is per host thread, as in the reference."""
from __future__ import annotations

from . import _ffi


class NoGradTrack:
    """RAII guard of the reference, usable as ``with NoGradTrack():`` or new()/drop()."""

    def __init__(self):
        _ffi.lib().ts_no_grad_push()
        self._active = True

    @staticmethod
    def new() -> "NoGradTrack":
        return NoGradTrack()

    def drop(self) -> None:
        if self._active:
            self._active = False
            _ffi.lib().ts_no_grad_pop()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.drop()
        return False

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass


def with_no_grad(f):
    g = NoGradTrack()
    try:
        return f()
    finally:
        g.drop()


def is_grad_enabled() -> bool:
    return bool(_ffi.lib().ts_is_grad_enabled())


_forced_off = []


def set_grad_enabled(enabled: bool) -> None:
    """no_grad_track.rs:155-200: switches tracking for the current thread."""
    if enabled:
        while _forced_off:
            _forced_off.pop().drop()
    elif is_grad_enabled():
        _forced_off.append(NoGradTrack())


def clear_gradients() -> None:
    _ffi.lib().ts_clear_gradients()


def tape_len() -> int:
    return int(_ffi.lib().ts_tape_len())
