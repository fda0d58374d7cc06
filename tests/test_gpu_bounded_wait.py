"""A device-side wait that runs out of its budget: the kernel gives up and returns, the host learns of it at the
next synchronisation as TOPS_ERR_DEVICE_TIMEOUT, and the library keeps working afterwards.  The wait is on a barrier
nothing arms, with a budget of one millisecond: nothing faults, traps or spins without a limit."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_an_expired_device_wait_is_reported_and_the_library_stays_usable():
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    lib.tops_clear_error()
    assert lib.tops_selftest_wait_timeout(1000) == 1          # the wait gave up
    assert lib.tops_sync() == 6                               # TOPS_ERR_DEVICE_TIMEOUT
    assert lib.tops_last_error() == 6 and b"wait expired" in lib.tops_last_error_message()
    lib.tops_clear_error()
    assert lib.tops_last_error() == 0
    # the next operator runs as usual
    a = DeviceArray.from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4), "float32")
    o = DeviceArray.empty((3, 4), "float32")
    lib.add_forward(a.handle, a.handle, o.handle)
    assert np.array_equal(o.numpy(), 2 * np.arange(12, dtype=np.float32).reshape(3, 4))
    assert lib.tops_sync() == 0
    capi.check(lib)
    assert lib.tops_selftest_wait_timeout(0) == -1            # budgets outside 1 us .. 100 ms are refused
    lib.tops_clear_error()
