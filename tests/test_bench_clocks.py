"""CPU: the clock record of a bench line is built from `nvidia-smi -lms` lines by time stamp."""
import datetime
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("flexsae_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _line(t, mhz, bits):
    stamp = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{stamp}, {mhz}, 1965, 0x{bits:016x}"


def test_samples_are_selected_by_time_stamp_and_reasons_decoded():
    bench = _bench()
    t0 = 1_800_000_000.0
    text = "\n".join([_line(t0 - 1.0, 1200, 0x8),            # long before the region: ignored, its hw_slowdown too
                      _line(t0 - 0.010, 1900, 0x0),          # just outside
                      _line(t0 + 0.005, 1965, 0x4), _line(t0 + 0.015, 1950, 0x0), _line(t0 + 0.025, 1965, 0x0),
                      "garbage line", _line(t0 + 5.0, 1000, 0x40)])
    got = bench.ClockSampler.parse(text, t0, t0 + 0.030)
    assert got["samples"] == 3 and got["samples_within_20ms"] == 1
    assert got["sm_mhz"] == 1965 and got["sm_min_mhz"] == 1950 and got["sm_max_mhz"] == 1965
    assert got["reasons"] == ["sw_power_cap"]
    # a region shorter than the sampling period: the nearest samples around it are used, and said to be
    near = bench.ClockSampler.parse(text, t0 - 0.004, t0)
    assert near["samples"] == 0 and near["samples_within_20ms"] == 3 and near["sm_mhz"] == 1950
    assert bench.ClockSampler.parse("", t0, t0 + 1)["reasons"] == ["unavailable"]
