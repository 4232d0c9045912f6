"""Host-side behaviour of the c10d backend "dicl" that needs no GPU: the blocking wait's time-out (the reference's
WorkDICL::synchronize polls isCompleted() and throws "Operation timed out!" after opTimeout_,
dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:154-167) and the backend's registration."""
import importlib

import pytest


@pytest.fixture(scope="module")
def c10d(pkg):
    adapter = importlib.import_module(pkg.__name__ + ".torch_adapter")
    if adapter._c10d is None:
        pytest.skip("the c10d extension module is not built")
    return adapter._c10d


def test_blocking_wait_returns_when_the_work_completes(c10d):
    waited = c10d.blocking_wait_selftest(2000, 30)
    assert 25.0 <= waited < 1000.0


def test_blocking_wait_gives_up_after_the_time_out(c10d):
    with pytest.raises(RuntimeError, match="Operation timed out!"):
        c10d.blocking_wait_selftest(50, -1)       # never completes
    with pytest.raises(RuntimeError, match="Operation timed out!"):
        c10d.blocking_wait_selftest(20, 500)      # completes too late


def test_blocking_wait_without_a_limit_waits(c10d):
    assert c10d.blocking_wait_selftest(0, 40) >= 35.0   # 0 = no limit, as c10d's kNoTimeout


def test_backend_is_registered_for_the_dipu_device(c10d):
    import torch.distributed as dist
    assert "dicl" in dist.Backend.backend_list
    assert dist.Backend.default_device_backend_map.get("dipu") == "dicl" or "dipu" in str(dist.Backend.backend_capability.get("dicl", ""))
