"""Named timers.

``TimerItLogger`` keeps the reference's wall-clock interface (start/end by key,
printing ``tm:: key : seconds`` when ``do_print`` is set; necklace/utils/tmrit.py:5-27).
``DeviceTimer`` adds what a device-timed metric needs: CUDA-event spans on the
current stream, optional NVTX ranges, and per-key accumulation that is only read
back (synchronised) when asked for.
"""
from __future__ import annotations

import time


class TimerItLogger:
    def __init__(self, cfg=None, *args, **kwargs):
        self.cfg = cfg or {}
        self.do_print = self.cfg.get("do_print", False) or kwargs.get("do_print", False)
        self.tms_d = {}
        self.totals = {}

    def start(self, key):
        tm = time.time()
        self.tms_d[key] = [tm, tm]

    def end(self, key):
        if key not in self.tms_d:
            return 0.0
        tm = time.time()
        self.tms_d[key][1] = tm
        dt = tm - self.tms_d[key][0]
        self.totals[key] = self.totals.get(key, 0.0) + dt
        if self.do_print:
            print("tm::", key, ":", dt)
        return dt


class DeviceTimer:
    """CUDA-event timer with named spans; falls back to wall clock without CUDA."""

    def __init__(self, enabled: bool = True, nvtx: bool = False):
        import torch
        self.torch = torch
        self.cuda = torch.cuda.is_available()
        self.enabled, self.nvtx = enabled, nvtx and self.cuda
        self._open, self._spans = {}, {}

    def start(self, key):
        if not self.enabled:
            return
        if self.nvtx:
            self.torch.cuda.nvtx.range_push(key)
        if self.cuda:
            ev = self.torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[key] = ev
        else:
            self._open[key] = time.perf_counter()

    def end(self, key):
        if not self.enabled or key not in self._open:
            return
        if self.cuda:
            ev = self.torch.cuda.Event(enable_timing=True)
            ev.record()
            self._spans.setdefault(key, []).append((self._open.pop(key), ev))
        else:
            self._spans.setdefault(key, []).append((self._open.pop(key), time.perf_counter()))
        if self.nvtx:
            self.torch.cuda.nvtx.range_pop()

    def totals_ms(self, reset: bool = True) -> dict:
        """Synchronises once and returns accumulated milliseconds per key."""
        if self.cuda:
            self.torch.cuda.synchronize()
        out = {}
        for k, spans in self._spans.items():
            if self.cuda:
                out[k] = sum(a.elapsed_time(b) for a, b in spans)
            else:
                out[k] = sum((b - a) * 1e3 for a, b in spans)
        if reset:
            self._spans = {}
        return out
