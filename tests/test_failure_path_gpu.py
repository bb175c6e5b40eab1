"""A wait that cannot complete gives up, the kernel exits normally, the host sees the status."""
import time

import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports(cuda_device):
    import torch

    import flash_attention_factory_b200 as pkg
    from flash_attention_factory_b200 import _cabi, _test_aids

    pkg.device_status()  # clean slate
    with torch.cuda.device(cuda_device):
        t0 = time.perf_counter()
        word = _test_aids.selftest_wait_timeout(2000)  # a barrier nothing sets, 2 ms limit
        dt = time.perf_counter() - t0
    assert dt < 1.0  # the limit bounds the wait; the context stays usable
    # the kernel left through its normal exit and recorded the time-out in the status word,
    # which the status reader (the code pa_device_status applies to each product unit) cleared
    assert word == _cabi.PA_ERR_TIMEOUT
    with torch.cuda.device(cuda_device):
        assert _test_aids.selftest_wait_timeout(500) == _cabi.PA_ERR_TIMEOUT  # reported once per time-out
    pkg.device_status()  # the product's own kernels never timed out
    x = torch.ones(4, device=cuda_device)
    assert float(x.sum()) == 4.0  # the device still answers
