"""Host-side pieces of bench.py that need no GPU: the clock sampler's summary and the byte counts."""

import datetime
import time

import bench


class _DoneProcess:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        pass


def _line(t, clock, watts, power_cap):
    stamp = datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    return f"{stamp}, {clock}, 1965, {watts}, Not Active, Not Active, Not Active, {power_cap}"


def test_clock_summary_counts_only_samples_inside_the_timed_region():
    sampler = bench.ClockSampler(0)
    sampler.proc = _DoneProcess()
    now = time.time()
    sampler.samples = [
        _line(now - 1.0, 1965, 200.0, "Not Active"),   # before the region: idle at full clock
        _line(now + 0.05, 1965, 400.0, "Not Active"),  # inside, but within the settle time
        _line(now + 0.3, 1700, 990.0, "Active"),
        _line(now + 0.5, 1650, 995.0, "Active"),
        _line(now + 2.0, 1965, 150.0, "Not Active"),   # after
        "garbage",
    ]
    sampler.window(now, now + 1.0)
    out = sampler.stop()
    assert out["samples"] == 2 and out["samples_outside_timed_regions"] == 3
    assert out["sm_mhz"] == 1675.0 and out["sm_min_mhz"] == 1650.0 and out["sm_max_mhz"] == 1965.0
    assert out["power_w"] == 992.5
    assert out["reasons"] == ["sw_power_cap"]


def test_clock_summary_without_samples():
    sampler = bench.ClockSampler(0)
    sampler.proc = _DoneProcess()
    sampler.window(0.0, 1.0)
    out = sampler.stop()
    assert out["samples"] == 0 and out["sm_mhz"] is None


def test_algorithmic_bytes():
    # m*k/2 packed weights + 4m scales + 64 codebook + 2nk activations + 2nm outputs
    assert bench.alg_bytes(28672, 16, 4096) == 59883584
    assert bench.alg_bytes(4096, 16, 14336) == 29966400
