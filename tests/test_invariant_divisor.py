"""The host side of integer division by a scalar (no GPU): the multiplier and shifts the library derives from a divisor
reproduce floor division for every magnitude a signed element can have."""
import ctypes
import random

import pytest

from cumo_b200 import _lib


@pytest.mark.parametrize("bits", [32, 64])
def test_multiplier_and_shifts_reproduce_floor_division(bits):
    lib = _lib.load()
    fn = lib.cb200_invariant_divisor_u32 if bits == 32 else lib.cb200_invariant_divisor_u64
    word = ctypes.c_uint32 if bits == 32 else ctypes.c_uint64
    fn.restype = None
    fn.argtypes = [word, ctypes.POINTER(word), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    rng = random.Random(bits)
    top = 1 << (bits - 1)                                   # |minimum| of the signed type: the largest magnitude
    divisors = [1, 2, 3, 5, 7, 10, 641, 4096, 6700417, top, top - 1, (top >> 1) + 1]
    divisors += [rng.randrange(1, top + 1) for _ in range(200)] + [rng.randrange(1, 1000) for _ in range(100)]
    for d in divisors:
        m, s1, s2 = word(), ctypes.c_int(), ctypes.c_int()
        fn(d, ctypes.byref(m), ctypes.byref(s1), ctypes.byref(s2))
        assert 0 <= s1.value <= 1 and 0 <= s2.value < bits
        ns = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, top, top - 1] + [rng.randrange(0, top + 1) for _ in range(200)]
        for n in ns:
            if not 0 <= n <= top:
                continue
            t = (m.value * n) >> bits
            q = (t + ((n - t) >> s1.value)) >> s2.value
            assert q == n // d, (bits, n, d)
