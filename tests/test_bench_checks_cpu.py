"""The parity helpers bench.py and the multi-GPU tests share (bench_checks.py): error figures and bounds, on the CPU."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench_checks  # noqa: E402


def test_bf16_ulp():
    assert bench_checks.bf16_ulp(1.0) == 2.0 ** -7 and bench_checks.bf16_ulp(1.99) == 2.0 ** -7
    assert bench_checks.bf16_ulp(44.25) == 0.25 and bench_checks.bf16_ulp(0.75) == 2.0 ** -8
    assert bench_checks.bf16_ulp(0.0) == 0.0 and bench_checks.bf16_ulp(float("inf")) == 0.0
    # agrees with the spacing torch's bfloat16 has at that magnitude: value + one ulp is the next representable value
    for x in (0.3, 1.5, 12.7, 44.25, 300.0):
        lo = torch.tensor([x], dtype=torch.float32).to(torch.bfloat16).float().item()
        ulp = bench_checks.bf16_ulp(lo)
        hi = torch.tensor([lo + ulp], dtype=torch.float32).to(torch.bfloat16).float().item()
        mid = torch.tensor([lo + 0.25 * ulp], dtype=torch.float32).to(torch.bfloat16).float().item()
        assert hi - lo == ulp and mid == lo

def test_parity_entry_bounds():
    g = torch.Generator().manual_seed(0)
    want = torch.randn(4096, generator=g) * 10.0
    scale = want.abs().max().item()
    ok = bench_checks.parity_entry(want + 1e-3, {"x": (want, 1e-2)})
    assert ok["ok"] and ok["x"]["max_abs_bound"] == round(max(2e-2 * scale, 4 * bench_checks.bf16_ulp(scale)), 6)
    off = want.clone()
    off[7] += 1.5 * ok["x"]["max_abs_bound"]          # one element beyond the max-abs bound
    assert not bench_checks.parity_entry(off, {"x": (want, 1e-2)})["ok"]
    assert not bench_checks.parity_entry(want * 1.02, {"x": (want, 1e-2)})["ok"]   # relative L2 2e-2 > 1e-2
    nan = want.clone()
    nan[0] = float("nan")
    assert not bench_checks.parity_entry(nan, {"x": (want, 1e-2)})["ok"]           # NaN never passes
    # against fp32: the bound follows the CPU bf16 path's own distance where that is larger than 1e-2
    bf = (want * 1.03)
    rel, floor = bench_checks.fp32_bound(bf, want)
    assert abs(rel - 1.25 * 0.03) < 1e-4 and floor > 0
    assert bench_checks.parity_entry(want * 1.035, {"fp32": (want, (rel, floor))})["ok"]
