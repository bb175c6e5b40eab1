"""The read-only streaming probe: reads, writes nothing, returns a plausible rate, rejects bad input."""
import pytest

pytestmark = pytest.mark.gpu


def test_read_probe_reports_a_rate_and_leaves_the_buffer_alone(cuda_device):
    import torch

    from flash_attention_factory_b200 import _test_aids as _cabi

    with torch.cuda.device(cuda_device):
        buf = torch.randint(0, 255, (512 * 2**20 + 48,), dtype=torch.uint8, device=cuda_device)
        before = int(buf[:: 4099].to(torch.int64).sum())
        rate = _cabi.measure_read_bandwidth(buf.data_ptr(), buf.numel(), iters=5)
        assert 500.0 < rate < 20000.0  # GB/s: an HBM-sized figure, not zero and not a cache artefact
        half = 256 * 2**20
        both = _cabi.measure_read_bandwidth(buf.data_ptr(), half, 5, 0, buf.data_ptr() + half, half)
        assert 500.0 < both < 20000.0  # two buffers in one launch
        bulk = _cabi.measure_read_bandwidth(buf.data_ptr(), half, 5, 0, buf.data_ptr() + half, half, method=1)
        assert 500.0 < bulk < 20000.0  # bulk copies into shared memory
        assert int(buf[:: 4099].to(torch.int64).sum()) == before
        with pytest.raises(RuntimeError, match="16-byte aligned"):
            _cabi.measure_read_bandwidth(buf.data_ptr() + 8, 65536)
        with pytest.raises(RuntimeError, match="iters"):
            _cabi.measure_read_bandwidth(buf.data_ptr(), 65536, iters=0)
