"""Energy bookkeeping on CPU with a scripted power source: the integration rule of the
reference's monitor (energy_utils.py:126-164), the energy-counter shortcut, the report rows
and the module hooks."""
import pytest
import torch

from sparser_faster_llms_b200 import energy


class ScriptedReader:
    """Power follows ``watts(t)`` of a fake clock; optional cumulative counter."""

    def __init__(self, clock, watts, counter=None, backend="scripted"):
        self.clock, self.watts, self.counter, self.backend = clock, watts, counter, backend

    def read_power_w(self):
        return self.watts(self.clock())

    def read_energy_j(self):
        return None if self.counter is None else self.counter(self.clock())


class Clock:
    def __init__(self):
        self.t = 10.0

    def __call__(self):
        return self.t


def test_trapezoid_integration_matches_the_reference_rule():
    samples = [(0.0, 100.0), (1.0, 300.0), (1.5, 300.0)]
    # 0..1: 200 J; 1..1.5: 150 J; tail held at 300 W for 0.5 s: 150 J
    assert energy.integrate_power(samples, 0.0, 2.0) == pytest.approx(500.0)
    assert energy.integrate_power([], 0.0, 1.0) == 0.0
    assert energy.integrate_power([(0.0, 50.0)], 0.0, 2.0) == pytest.approx(100.0)


def test_monitor_integrates_polled_power_without_a_counter():
    clk = Clock()
    mon = energy.GPUEnergyMonitor(reader=ScriptedReader(clk, lambda t: 100.0 * (t - 10.0)), clock=clk)
    assert mon.enabled and mon.results() is None
    assert mon.start(background=False)
    for _ in range(4):
        clk.t += 0.5
        mon.sample()
    mon.stop()
    st = mon.results()
    # power ramps 0 -> 200 W over 2 s: 200 J; trapezoids are exact on a ramp
    assert st.energy_joules == pytest.approx(200.0) and st.duration_s == pytest.approx(2.0)
    assert st.avg_power_w == pytest.approx(100.0) and st.num_samples == 6
    assert st.backend == "scripted"


def test_monitor_prefers_the_energy_counter():
    clk = Clock()
    reader = ScriptedReader(clk, lambda t: 123.0, counter=lambda t: 5000.0 + 400.0 * (t - 10.0))
    mon = energy.GPUEnergyMonitor(reader=reader, clock=clk)
    mon.start(background=False)
    clk.t += 3.0
    mon.stop()
    st = mon.results()
    assert st.energy_joules == pytest.approx(1200.0) and st.avg_power_w == pytest.approx(400.0)
    assert st.backend == "scripted+energy_counter"
    # a counter that did not advance (too short a window) falls back to the samples
    mon2 = energy.GPUEnergyMonitor(reader=ScriptedReader(clk, lambda t: 50.0, counter=lambda t: 7.0),
                                   clock=clk)
    mon2.start(background=False)
    clk.t += 2.0
    mon2.stop()
    assert mon2.results().energy_joules == pytest.approx(100.0)
    assert mon2.results().backend == "scripted"


def test_background_polling_collects_samples():
    reader = ScriptedReader(lambda: 0.0, lambda t: 80.0)
    mon = energy.GPUEnergyMonitor(poll_interval_s=0.005, reader=reader)
    assert mon.start() and not mon.start()            # second start refused while running
    import time
    time.sleep(0.08)
    mon.stop()
    st = mon.results()
    assert st.num_samples >= 4 and st.avg_power_w == pytest.approx(80.0, rel=1e-6)


def test_disabled_monitor_and_report_rows():
    off = energy.GPUEnergyMonitor(reader=ScriptedReader(lambda: 0.0, lambda t: 1.0, backend=None))
    assert not off.enabled and not off.start() and off.results() is None
    off.stop()
    assert energy.summarize_energy(None, 10) == {}
    st = energy.EnergyStats(250.0, 500.0, 2.0, 40, "x")
    assert energy.summarize_energy(st, 0) == {}
    row = energy.summarize_energy(st, 100, prefix="mlp_")
    assert row == {"mlp_avg_power_w": 250.0, "mlp_total_energy_j": 500.0,
                   "mlp_energy_per_forward_j": 5.0, "mlp_energy_duration_s": 2.0,
                   "mlp_energy_samples": 40, "mlp_energy_backend": "x"}
    merged = energy.merge_energy_stats([st, energy.EnergyStats(100.0, 100.0, 1.0, 10, "x")])
    assert merged.energy_joules == 600.0 and merged.duration_s == 3.0
    assert merged.avg_power_w == pytest.approx(200.0) and merged.num_samples == 50
    assert energy.merge_energy_stats([]) is None


def test_hooks_scope_the_monitor_to_the_ffn_blocks():
    clk = Clock()
    mon = energy.GPUEnergyMonitor(reader=ScriptedReader(clk, lambda t: 10.0), clock=clk)
    events = []

    class Block(torch.nn.Module):
        def forward(self, x):
            events.append(mon._t0 is not None and mon._t1 is None)   # inside the window?
            clk.t += 1.0
            return x

    blocks = [Block(), Block(), Block()]
    orig_start = mon.start
    mon.start = lambda: orig_start(background=False)
    hooks = energy.MlpEnergyHooks(mon, blocks, sync_on_stop=False)
    x = torch.zeros(1)
    for b in blocks:
        x = b(x)
    assert events == [True, True, True] and not hooks.started
    assert mon.results().energy_joules == pytest.approx(30.0)
    hooks.remove()
    assert hooks.handles == []
    empty = energy.MlpEnergyHooks(mon, [])
    assert empty.handles == []


def test_power_reader_without_a_gpu_reports_no_backend_or_none_readings():
    r = energy.GPUPowerReader(0)
    assert r.backend in (None, "pynvml", "nvidia-smi")
    if r.backend is None:
        assert r.read_power_w() is None and r.read_energy_j() is None
    assert energy.device_pci_bus_id(torch.device("cuda:0")) is None or torch.cuda.is_available()
