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


def test_neighbouring_copies_are_merged():
    """HostSequence issues runs of tensors that are adjacent on both sides as one copy of the same bytes."""
    import torch

    from tuna_b200.ops import _merge_copies

    dst, src = torch.zeros(100, dtype=torch.float16), torch.arange(100, dtype=torch.float16)
    copies = [(dst[0:10], src[0:10]), (dst[10:30], src[10:30]),   # adjacent on both sides: one run
              (dst[40:50], src[40:50]),                            # a gap on both sides: its own copy
              (dst[50:60], src[60:70])]                            # adjacent destinations, sources are not
    merged = _merge_copies(copies)
    assert [d.numel() * d.element_size() for d, _ in merged] == [60, 20, 20]
    for d, s in merged:
        d.copy_(s)
    want = torch.zeros(100, dtype=torch.float16)
    want[0:30], want[40:50], want[50:60] = src[0:30], src[40:50], src[60:70]
    assert torch.equal(dst, want)
    other = torch.zeros(10, dtype=torch.float16)
    assert len(_merge_copies([(dst[0:10], src[0:10]), (other, src[10:20])])) == 2  # different allocations never merge
