"""Failure detection without faulting the GPU: a bounded wait that can never be satisfied gives
up, reports through the device status word, and leaves the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_and_context_survives():
    import b200_hpu_ops
    from b200_hpu_ops import abi
    assert b200_hpu_ops.device_status() == 0
    assert abi.lib.b200q_selftest_wait_timeout(4242, abi.stream_ptr()) == 0
    assert b200_hpu_ops.device_status() == 4242          # reported ...
    assert b200_hpu_ops.device_status() == 0             # ... and cleared by the read
    # the context is intact: a real kernel runs and is correct afterwards
    x = torch.arange(64, dtype=torch.float32, device="cuda")
    out, amax = torch.ops.hpu.cast_to_fp8_v2(x, None, False, True, torch.float8_e4m3fn)
    assert amax.item() == 63.0 and torch.equal(out.float().cpu(), torch.arange(64, dtype=torch.float32).to(torch.float8_e4m3fn).float())
    assert abi.lib.b200q_selftest_wait_timeout(0, None) == -1


def test_status_codes_have_text():
    from b200_hpu_ops import abi
    assert b"bounded wait" in abi.lib.b200q_strerror(-5)
