"""GPU: the issue-rate diagnostic (bqq_instruction_rate) answers for every kind and refuses bad arguments."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def test_instruction_rates_are_positive_and_ordered():
    from bqq_b200 import _cabi
    lib = _cabi.lib
    rates = []
    for kind in range(10):
        v = ctypes.c_double()
        assert lib.bqq_instruction_rate(kind, 512, ctypes.byref(v), None) == 0
        assert 0.0 < v.value < 8.0, (kind, v.value)          # at most 4 schedulers x 1 warp-instruction per clock
        rates.append(v.value)
    # the byte-operand MMA the decode kernel uses is far faster than the 1-bit shape it decided against
    assert rates[0] > 4 * rates[4]
    v = ctypes.c_double()
    assert lib.bqq_instruction_rate(10, 512, ctypes.byref(v), None) == -2
    assert lib.bqq_instruction_rate(0, 0, ctypes.byref(v), None) == -2
    assert lib.bqq_instruction_rate(0, 512, None, None) == -1
