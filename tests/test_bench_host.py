"""CPU-only checks of bench.py's host logic: the clock record built from nvidia-smi samples."""
import datetime
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _line(t, index, sm, cap):
    stamp = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{stamp}, {index}, {sm}, 1965, 700.00, 0x0000000000000004, Not Active, Not Active, Not Active, {'Active' if cap else 'Not Active'}\n"


def test_clock_samples_split_at_the_end_of_the_timed_region():
    bench = _bench()
    t0 = 1_800_000_000.0
    lines = [_line(t0 + 0.0, 0, 1965, False), _line(t0 + 0.1, 0, 1950, False),      # timed region
             _line(t0 + 0.1, 1, 300, True),                                          # another GPU: ignored
             _line(t0 + 0.3, 0, 1700, True), _line(t0 + 0.4, 0, 1690, True),        # untimed repeats reach the power cap
             "garbage\n"]
    c = bench.summarise_clock_samples(lines, {0}, t_mark=t0 + 0.2)
    assert c["samples"] == 4 and c["samples_in_timed_region"] == 2
    assert c["reasons"] == ["sw_power_cap"] and c["reasons_in_timed_region"] == []
    assert c["sm_max_mhz"] == 1965.0 and c["sm_mhz"] == 1957.5   # median of the upper half
    c = bench.summarise_clock_samples(lines, {0}, t_mark=t0 + 1.0)
    assert c["reasons_in_timed_region"] == ["sw_power_cap"]
    assert bench.summarise_clock_samples([], {0})["sm_mhz"] is None
