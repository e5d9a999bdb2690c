"""Host logic, no GPU: which kernel a product is sent to.  The routing is plain arithmetic on the shape, the operand
layout, the epilogue and the SM count (`ts_debug_gemm_route`), so the products of the five benchmark configurations can be
pinned here; a threshold that moves shows up as a failing line instead of as a slower step somewhere."""
import ctypes as C

import pytest

FP32, FP32_SPLIT_K, THIN_NN, THIN_TN, THIN_NT, TC128, TC256, TC_PAIRS, TC_SPLIT_K128, TC_SPLIT_K256 = range(10)
BIAS, RELU, MASK, ROUND, COLSUM = 1, 2, 4, 8, 16
SMS = 148
F32, TF32, TF32X3 = 0, 1, 2


@pytest.fixture(scope="module")
def route(ts):
    lib = ts._ffi.lib()

    def ask(m, n, k, ta=0, tb=0, precision=TF32, epilogue=0, sms=SMS):
        splits = C.c_ulonglong(0)
        kind = lib.ts_debug_gemm_route(m, n, k, ta, tb, precision, epilogue, sms, C.byref(splits))
        return kind, splits.value
    return ask


def test_c5_and_c3_products_run_on_cta_pairs(route):
    for batch in (65536, 32768, 16384, 8192):                     # one GPU, and the per-rank shards of 2, 4 and 8
        assert route(batch, 8192, 4096, epilogue=BIAS | RELU | ROUND) == (TC_PAIRS, 1)          # x.W1 + b1, ReLU
        assert route(batch, 4096, 8192, epilogue=BIAS) == (TC_PAIRS, 1)                         # h2.W3 + b3
        assert route(4096, 8192, batch, ta=1) == (TC_PAIRS, 1)                                  # dW1 = x^T.dh1
        assert route(batch, 8192, 8192, tb=1, epilogue=MASK | ROUND | COLSUM) == (TC_PAIRS, 1)  # dh1 = dh2.W2^T
    for ta, tb in ((0, 0), (0, 1), (1, 0)):
        assert route(8192, 8192, 8192, ta, tb) == (TC_PAIRS, 1)


def test_c4_products(route):
    assert route(4096, 1024, 784, epilogue=BIAS | RELU | ROUND) == (TC256, 1)       # one wave of 128 x 256 tiles
    assert route(4096, 1024, 1024, epilogue=BIAS | RELU | ROUND) == (TC256, 1)
    assert route(4096, 10, 1024, epilogue=BIAS) == (THIN_NN, 1)                     # the 10-class layer
    assert route(1024, 10, 4096, ta=1) == (THIN_TN, 1)                              # its weight gradient
    assert route(4096, 1024, 10, tb=1, epilogue=MASK | ROUND | COLSUM) == (THIN_NT, 1)   # its input gradient
    assert route(1024, 1024, 4096, ta=1) == (TC_SPLIT_K256, 4)                      # dW2: wide tiles, four splits of K
    assert route(784, 1024, 4096, ta=1) == (TC_SPLIT_K256, 4)                       # dW1
    assert route(4096, 1024, 1024, tb=1, epilogue=MASK | ROUND | COLSUM) == (TC256, 1)   # an epilogue keeps K whole
    for shape in ((4096, 1024, 784), (4096, 10, 1024), (1024, 10, 4096), (1024, 1024, 4096)):
        assert route(*shape, ta=int(shape[2] == 4096), precision=F32) == (FP32, 1), "FP32 mode: one chain per element, never split"
    assert route(4096, 10, 1024, precision=TF32X3)[0] == THIN_NN


def test_small_and_odd_products(route):
    assert route(32, 128, 784, epilogue=BIAS | RELU) == (TC128, 1)                  # the README step
    assert route(784, 128, 32, ta=1) == (TC128, 1)
    assert route(100, 30, 50) == (FP32, 1)                                          # row pitch not a multiple of 16 bytes
    assert route(1000, 30, 4096, ta=1) == (FP32_SPLIT_K, 32)                        # ... with a long reduction: split on the FP32 kernel
    assert route(128, 128, 16384) == (TC_SPLIT_K128, 16)                            # one narrow tile over a very long K
    assert route(200, 10, 100) == (FP32, 1)                                         # too short for the thin layout to pay
    assert route(2048, 1024, 1024)[0] == TC128                                      # 64 wide tiles: narrow ones fill one wave
    assert route(2048 + 512, 1024, 1024)[0] == TC256                                # 80 wide tiles: one wave of those
    assert route(4096, 4096, 96)[0] == TC_PAIRS                                     # 256 tiles of 256 x 256


def test_routing_follows_the_sm_count(route):
    assert route(4096, 1024, 1024, sms=64)[0] == TC_PAIRS                           # 64 tiles of 256 x 256 are enough for 32 pairs
    assert route(1024, 1024, 4096, ta=1, sms=64) == (TC128, 1)                      # 64 narrow tiles already fill 64 SMs: no split
    assert route(512, 512, 4096, ta=1, sms=64) == (TC_SPLIT_K128, 4)
