"""GPU energy per forward, read-only.

Counterpart of the reference's ``energy_utils.py`` (``GPUPowerReader`` :22-74,
``GPUEnergyMonitor`` :77-164, ``summarize_energy`` :167-180, ``merge_energy_stats``
:183-199, ``MlpEnergyHooks`` :202-240) behind the same names, which its benchmark uses as
``monitor.start(); <reps forwards>; monitor.stop(); monitor.results()``
(``benchmark_inference.py:280-343``).

Two differences.  Where NVML exposes the board's cumulative energy counter
(``nvmlDeviceGetTotalEnergyConsumption``, millijoules since the driver loaded - present on
B200) the monitor reads it at start and stop and reports the difference: no sampling error,
and the polling thread only collects power samples for the average / sample count.  Without
the counter it integrates polled power by the trapezoid rule, as the reference does.  And
the power source is injectable (``reader=``), so the arithmetic is tested on CPU with a
scripted reader.  Nothing here changes a GPU setting; every call is a query.
"""
from __future__ import annotations

import shutil
import subprocess
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class EnergyStats:
    avg_power_w: float
    energy_joules: float
    duration_s: float
    num_samples: int
    backend: str


class GPUPowerReader:
    """Instantaneous board power (W) and, where available, the cumulative energy counter (J).

    ``backend`` is ``"pynvml"``, ``"nvidia-smi"`` or ``None`` (nothing to read from)."""

    def __init__(self, gpu_index: int = 0, pci_bus_id: Optional[str] = None):
        self.gpu_index = int(gpu_index)
        self._nvml = None
        self._handle = None
        self.backend: Optional[str] = None
        try:
            import pynvml
            pynvml.nvmlInit()
            if pci_bus_id is not None:    # NVML numbers all boards; CUDA only the visible ones
                self._handle = pynvml.nvmlDeviceGetHandleByPciBusId(pci_bus_id.encode())
            else:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._nvml = pynvml
            self.backend = "pynvml"
        except Exception:
            if shutil.which("nvidia-smi") is not None:
                self.backend = "nvidia-smi"

    def read_power_w(self) -> Optional[float]:
        try:
            if self.backend == "pynvml":
                return self._nvml.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
            if self.backend == "nvidia-smi":
                out = subprocess.check_output(
                    ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=power.draw",
                     "--format=csv,noheader,nounits"],
                    encoding="utf-8", stderr=subprocess.DEVNULL, timeout=1.0)
                return float(out.strip().splitlines()[0])
        except Exception:
            return None
        return None

    def read_energy_j(self) -> Optional[float]:
        """Cumulative energy counter in joules, or None where the driver has none."""
        if self.backend != "pynvml":
            return None
        try:
            return self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._handle) / 1000.0
        except Exception:
            return None


def device_pci_bus_id(device: torch.device) -> Optional[str]:
    """``domain:bus:device.0`` of a CUDA device, for an NVML lookup that does not depend on
    CUDA_VISIBLE_DEVICES; None where torch does not expose it."""
    try:
        p = torch.cuda.get_device_properties(device)
        return f"{p.pci_domain_id:08X}:{p.pci_bus_id:02X}:{p.pci_device_id:02X}.0"
    except Exception:
        return None


def integrate_power(samples: Sequence[Tuple[float, float]], start_t: float,
                    end_t: float) -> float:
    """Trapezoid integral of ``(time, watts)`` samples, the last sample held up to
    ``end_t`` (the reference's rule, ``energy_utils.py:139-150``)."""
    energy = 0.0
    for (t0, p0), (t1, p1) in zip(samples, samples[1:]):
        if t1 > t0:
            energy += 0.5 * (p0 + p1) * (t1 - t0)
    if samples and end_t > samples[-1][0]:
        energy += samples[-1][1] * (end_t - samples[-1][0])
    return energy


class GPUEnergyMonitor:
    """Energy of whatever runs between :meth:`start` and :meth:`stop`.

    ``reader`` needs ``backend``, ``read_power_w()`` and optionally ``read_energy_j()``;
    ``clock`` is the time source (both injectable for tests)."""

    def __init__(self, gpu_index: int = 0, poll_interval_s: float = 0.05, reader=None,
                 clock: Callable[[], float] = time.perf_counter):
        self.gpu_index = int(gpu_index)
        self.poll_interval_s = float(poll_interval_s)
        self.reader = reader if reader is not None else GPUPowerReader(self.gpu_index)
        self.enabled = self.reader.backend is not None
        self._clock = clock
        self._halt = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._samples: List[Tuple[float, float]] = []
        self._t0: Optional[float] = None
        self._t1: Optional[float] = None
        self._e0: Optional[float] = None
        self._e1: Optional[float] = None

    def _counter(self) -> Optional[float]:
        read = getattr(self.reader, "read_energy_j", None)
        return read() if read is not None else None

    def _sample(self, ts: Optional[float] = None) -> None:
        ts = self._clock() if ts is None else ts
        watts = self.reader.read_power_w()
        if watts is not None:
            self._samples.append((ts, float(watts)))

    def _poll(self) -> None:
        while not self._halt.is_set():
            self._sample()
            self._halt.wait(self.poll_interval_s)

    def start(self, background: bool = True) -> bool:
        """Begin a measurement; ``background=False`` skips the polling thread (the caller
        calls :meth:`sample` itself, or relies on the energy counter alone)."""
        if not self.enabled or self._thread is not None:
            return False
        self._samples.clear()
        self._halt.clear()
        self._t1 = self._e1 = None
        self._t0 = self._clock()
        self._e0 = self._counter()
        self._sample(self._t0)
        if background:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return True

    def sample(self) -> None:
        self._sample()

    def stop(self) -> None:
        if not self.enabled or self._t0 is None:
            return
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=1.5)
        self._thread = None
        self._t1 = self._clock()
        self._e1 = self._counter()
        self._sample(self._t1)

    def results(self) -> Optional[EnergyStats]:
        if not self.enabled or self._t0 is None or not self._samples:
            return None
        end_t = self._t1 if self._t1 is not None else self._samples[-1][0]
        duration = end_t - self._t0
        if duration <= 0.0:
            return None
        backend = self.reader.backend or "unknown"
        if self._e0 is not None and self._e1 is not None and self._e1 > self._e0:
            energy = self._e1 - self._e0
            backend += "+energy_counter"
        else:
            energy = integrate_power(self._samples, self._t0, end_t)
        return EnergyStats(avg_power_w=energy / duration, energy_joules=energy,
                           duration_s=duration, num_samples=len(self._samples),
                           backend=backend)


def summarize_energy(stats: Optional[EnergyStats], reps: int, prefix: str = "") -> Dict[str, float]:
    """Flat report row; empty when nothing was measured (``energy_utils.py:167-180``)."""
    if stats is None or reps <= 0:
        return {}
    return {
        f"{prefix}avg_power_w": float(stats.avg_power_w),
        f"{prefix}total_energy_j": float(stats.energy_joules),
        f"{prefix}energy_per_forward_j": float(stats.energy_joules / reps),
        f"{prefix}energy_duration_s": float(stats.duration_s),
        f"{prefix}energy_samples": int(stats.num_samples),
        f"{prefix}energy_backend": str(stats.backend),
    }


def merge_energy_stats(stats: List[EnergyStats]) -> Optional[EnergyStats]:
    """Sum of several measurement windows (``energy_utils.py:183-199``)."""
    if not stats:
        return None
    energy = sum(s.energy_joules for s in stats)
    duration = sum(s.duration_s for s in stats)
    return EnergyStats(avg_power_w=energy / duration if duration > 0 else float("nan"),
                       energy_joules=energy, duration_s=duration,
                       num_samples=sum(s.num_samples for s in stats), backend=stats[0].backend)


class MlpEnergyHooks:
    """Scope the monitor to the FFN blocks of a model: start before the first module's
    forward, stop (after a device synchronise) behind the last one's
    (``energy_utils.py:202-240``)."""

    def __init__(self, monitor: GPUEnergyMonitor, mlp_modules: List[torch.nn.Module],
                 sync_on_stop: bool = True):
        self.monitor = monitor
        self.sync_on_stop = sync_on_stop
        self.started = False
        self.handles = []
        if not mlp_modules or not monitor.enabled:
            return
        self.handles.append(mlp_modules[0].register_forward_pre_hook(self._before))
        self.handles.append(mlp_modules[-1].register_forward_hook(self._after))

    def _before(self, module, _inputs):
        if not self.started and self.monitor.enabled:
            self.started = self.monitor.start()

    def _after(self, module, _inputs, _output):
        if not self.started:
            return
        if self.sync_on_stop and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.monitor.stop()
        self.started = False

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


def measure_replays(run: Callable[[], None], device: torch.device, min_seconds: float = 1.5,
                    chunk: int = 50, gpu_index: Optional[int] = None,
                    monitor: Optional[GPUEnergyMonitor] = None) -> Optional[Dict[str, float]]:
    """Energy per call of ``run`` (a CUDA-graph replay or any launch sequence): calls it in
    chunks until ``min_seconds`` have passed, synchronising per chunk, and divides.  Returns
    ``summarize_energy`` keys plus ``reps``, or None where no power source exists."""
    if monitor is None:
        if gpu_index is None:
            gpu_index = device.index if device.index is not None else torch.cuda.current_device()
        reader = GPUPowerReader(gpu_index, pci_bus_id=device_pci_bus_id(device))
        if reader.backend != "pynvml":           # bus-id lookup refused: fall back to the index
            reader = GPUPowerReader(gpu_index)
        monitor = GPUEnergyMonitor(gpu_index=gpu_index, poll_interval_s=0.02, reader=reader)
    if not monitor.enabled:
        return None
    for _ in range(chunk):                       # settle clocks and power before the window
        run()
    torch.cuda.synchronize(device)
    reps = 0
    monitor.start()
    t_end = time.perf_counter() + min_seconds
    while time.perf_counter() < t_end:
        for _ in range(chunk):
            run()
        torch.cuda.synchronize(device)
        reps += chunk
    monitor.stop()
    row = summarize_energy(monitor.results(), reps)
    if not row:
        return None
    row["reps"] = reps
    return row
