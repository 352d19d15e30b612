"""CPU-only checks of bench.py's host logic: the clock record built from NVML samples."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_samples_are_attributed_to_the_timed_regions():
    bench = _bench()
    t0 = 1_800_000_000.0
    cap = 0x4
    samples = [(t0 + 0.00, 0, 1965.0, 1965.0, 600.0, 0), (t0 + 0.01, 0, 1950.0, 1965.0, 700.0, 0),     # headline timed region
               (t0 + 0.01, 1, 1900.0, 1965.0, 650.0, 0),
               (t0 + 0.30, 0, 1700.0, 1965.0, 990.0, cap), (t0 + 0.40, 0, 1690.0, 1965.0, 995.0, cap),   # untimed repeats reach the power cap
               (t0 + 0.50, 0, 1800.0, 1965.0, 800.0, 0x20)]                                              # a sub-record's region
    c = bench.summarise_clock_samples(samples, {"headline": (t0, t0 + 0.05), "cfg2": (t0 + 0.45, t0 + 0.55)})
    assert c["samples"] == 6 and c["samples_in_timed_region"] == 3
    assert c["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"] and c["reasons_in_timed_region"] == []
    assert c["sm_max_mhz"] == 1965.0 and c["sm_mhz_in_timed_region"] == 1950.0
    assert c["sm_mhz"] == 1950.0      # "under load" = the headline timed region, not the idle samples around it
    no_window = bench.summarise_clock_samples(samples, {"headline": (t0 + 9.0, t0 + 9.5)})
    assert no_window["samples_in_timed_region"] == 0 and no_window["sm_mhz"] is not None   # falls back to what was seen
    assert c["windows"]["cfg2"]["samples"] == 1 and c["windows"]["cfg2"]["reasons"] == ["sw_thermal_slowdown"]
    assert c["power_w_max"] == 995.0
    empty = bench.summarise_clock_samples([], {"headline": (t0, t0 + 1)})
    assert empty["sm_mhz"] is None and empty["samples_in_timed_region"] == 0


def test_default_workload_is_the_sharded_large_contraction():
    bench = _bench()
    w = bench.WORKLOADS["cfg5"]
    assert w["strong"] == "a" and w["ext"] == dict(a=128, b=128, c=128, d=128, e=128, f=128)
    assert bench.WORKLOADS["cfg3"]["strong"] == "a"
    assert {s[0] for s in bench.SUB_RECORDS} == {"cfg2", "cfg3", "cfg4"}
