"""Host-side helpers of the measurement programs: no GPU needed."""
import importlib
import sys
import types
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture()
def bench(monkeypatch):
    monkeypatch.syspath_prepend(str(ROOT))
    sys.modules.pop("bench", None)
    return importlib.import_module("bench")


def _sampler(bench, lines):
    sampler = object.__new__(bench.ClockSampler)      # no nvidia-smi, no NVML: only the record and its summary
    sampler.lines, sampler.proc, sampler.nvml = list(lines), None, None
    return sampler


def test_clock_summary_takes_the_median_and_names_the_active_reasons(bench):
    lines = ["1965, 1965, 612.10, Not Active, Not Active, Not Active, Not Active",
             "1800, 1965, 980.55, Not Active, Not Active, Not Active, Active",
             "garbage",
             "1905, 1965, 955.00, Not Active, Not Active, Not Active, Active"]
    got = _sampler(bench, lines).summary()
    assert got == {"sm_mhz": 1905.0, "sm_max_mhz": 1965.0, "power_w_max": 980.55, "samples": 3, "reasons": ["sw_power_cap"]}
    assert _sampler(bench, lines).summary(0, 1)["reasons"] == []
    hot = _sampler(bench, ["1200, 1965, 700.0, Active, Active, Not Active, Not Active"]).summary()
    assert hot["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]
    assert _sampler(bench, []).summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}


def test_a_snapshot_through_nvml_has_the_format_of_the_periodic_samples(bench):
    nv = types.SimpleNamespace(
        NVML_CLOCK_SM=1, nvmlClocksEventReasonHwSlowdown=8, nvmlClocksEventReasonHwThermalSlowdown=64,
        nvmlClocksEventReasonSwThermalSlowdown=32, nvmlClocksEventReasonSwPowerCap=4,
        nvmlDeviceGetClockInfo=lambda handle, kind: 1830, nvmlDeviceGetMaxClockInfo=lambda handle, kind: 1965,
        nvmlDeviceGetPowerUsage=lambda handle: 987654, nvmlDeviceGetCurrentClocksEventReasons=lambda handle: 4 | 32)
    sampler = _sampler(bench, [])
    sampler.snap()                                    # without NVML nothing is recorded
    assert sampler.lines == []
    sampler.nvml = (nv, object())
    mark = sampler.mark()
    sampler.snap()
    assert sampler.lines == ["1830, 1965, 987.65, Not Active, Not Active, Active, Active"]
    assert sampler.summary(mark, sampler.mark()) == {"sm_mhz": 1830.0, "sm_max_mhz": 1965.0, "power_w_max": 987.65,
                                                     "samples": 1, "reasons": ["sw_thermal_slowdown", "sw_power_cap"]}
    broken = types.SimpleNamespace(**{**vars(nv), "nvmlDeviceGetClockInfo": lambda handle, kind: 1 / 0})
    sampler.nvml = (broken, object())
    sampler.snap()                                    # a failing query is skipped, not raised
    assert len(sampler.lines) == 1


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2(bench, capsys):
    assert bench.main(["--gpus", "2"]) == 2
    out = capsys.readouterr().out.strip().splitlines()
    assert len(out) == 1 and '"n_gpus": 2' in out[0] and "unsupported" in out[0]


def test_parts_provided_for_split_decode_attention():
    """The grid of the decode attention kernel: about 256 blocks in all, at most 16 parts a request, 32 where
    contexts may be long, one when the batch fills the GPU by itself."""
    from torchinferno_b200.kernels.ops import decode_num_splits
    parts = {b: decode_num_splits(b, 32, 8) for b in (1, 2, 4, 8, 16, 32, 64, 200)}
    assert parts == {1: 16, 2: 16, 4: 8, 8: 4, 16: 2, 32: 1, 64: 1, 200: 1}
    assert decode_num_splits(1, 32, 8, max_kv_len=8192) == 16 and decode_num_splits(1, 32, 8, max_kv_len=8193) == 32
    assert decode_num_splits(2, 32, 8, max_kv_len=100000) == 16          # 16 blocks of kv heads x 16 parts are 256
    assert decode_num_splits(1, 64, 2) == 16 and decode_num_splits(3, 40, 40) == 2   # groups above 16 take more row tiles
    # a batch a little over one round of blocks (296 at once) is cut so that its last round is not nearly empty
    assert {b: decode_num_splits(b, 32, 8) for b in (37, 38, 44, 45, 53, 54, 74, 80)} == {37: 1, 38: 3, 44: 3, 45: 2, 53: 2, 54: 1, 74: 1, 80: 1}
