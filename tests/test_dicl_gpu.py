"""DICL communicator over NCCL on 2+ GPUs: every collective of the interface with closed-form expectations, and a
tensor-parallel decoder layer against the unsharded CPU oracle. One process per GPU, as ProcessGroupDICL requires."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip("needs at least %d GPUs" % world)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_and_tp_layer(world):
    _need(world)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as rdv:
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dicl_worker.py"), str(r), str(world), rdv], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                p.kill()  # the exact child started above
                out, _ = p.communicate()
                out += "\n[timed out]"
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and "rank %d ok" % r in out, "rank %d failed:\n%s" % (r, out[-3000:])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_c10d_backend(world):
    """torch.distributed with backend "dicl" on dipu tensors (the reference's ProcessGroupDICL, here over the adapter)."""
    _need(world)
    port = 29741 + world
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "c10d_worker.py"), str(r), str(world), str(port)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()  # the exact child started above
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % r in out, "rank %d failed:\n%s" % (r, out[-3000:])
