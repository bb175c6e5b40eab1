"""A wait that cannot complete gives up, the kernel exits normally, the host sees the status."""
import time

import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports(cuda_device):
    import torch

    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi

    lib = pkg.load_library()
    pkg.device_status()  # clean slate
    with torch.cuda.device(cuda_device):
        t0 = time.perf_counter()
        rc = lib.pa_selftest_wait_timeout(2000)  # a barrier nothing sets, 2 ms limit
        dt = time.perf_counter() - t0
    assert rc == _cabi.PA_OK, lib.pa_last_error().decode()
    assert dt < 1.0  # the limit bounds the wait; the context stays usable
    with pytest.raises(RuntimeError, match="bounded wait"):
        pkg.device_status()  # the time-out was recorded ...
    pkg.device_status()  # ... and is reported once
    x = torch.ones(4, device=cuda_device)
    assert float(x.sum()) == 4.0  # the device still answers
