"""Raw device buffers through the reference's own FFI calls (cuda_malloc / cuda_memcpy / cuda_free),
for tests that drive the kernel launchers directly."""
import ctypes as C

import numpy as np


class DevBuf:
    def __init__(self, ts, data=None, n=None, offset=0):
        """offset (in elements) yields a deliberately misaligned pointer for alignment tests."""
        self.lib = ts._ffi.lib()
        self.check = ts._ffi.check
        if data is not None:
            data = np.ascontiguousarray(data, dtype=np.float32)
            n = data.size
        self.n = int(n)
        self.offset = int(offset)
        base = self.lib.cuda_malloc(self.n + self.offset + 4)
        self.check(base, "cuda_malloc")
        self.base = base
        self.ptr = base + 4 * self.offset
        self.shape = data.shape if data is not None else (self.n,)
        if data is not None and self.n:
            self.check(self.lib.cuda_memcpy(self.ptr, data.ctypes.data, self.n, 0), "cuda_memcpy h2d")

    def get(self):
        out = np.empty(self.n, np.float32)
        if self.n:
            self.check(self.lib.cuda_memcpy(out.ctypes.data, self.ptr, self.n, 1), "cuda_memcpy d2h")
        return out.reshape(self.shape)

    def free(self):
        if self.base:
            self.lib.cuda_free(self.base)
            self.base = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
