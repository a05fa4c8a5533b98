"""Layer profiler: named ranges timed with CUDA events on the current stream (wall clock on
CPU), mirrored as NVTX ranges so that the same names show up in a system trace.

Same surface as the reference's profiler (include/cg_profiler.h: init, enable, begin_layer,
end_layer, step_end, report, reset; src/utils/profiler.c keeps a fixed table of 64 names and
uses clock()): unlimited names here, device time instead of host CPU time, plus the count of
kernels this library launched inside each range.
"""
from __future__ import annotations

import contextlib
import time
from collections import OrderedDict

import torch

from ..ops import _lib


class Profiler:
    def __init__(self, enabled: bool = True, nvtx: bool = True):
        self.enabled, self.nvtx = enabled, nvtx
        self.reset()

    # -- cg_profiler_* surface
    def init(self):
        self.reset()
        self.enabled = True

    def enable(self, on: bool):
        self.enabled = on

    def reset(self):
        self.stats = OrderedDict()          # name -> [calls, total_ms, launches]
        self._open = {}
        self._pending = []                  # (name, start_event, end_event)
        self.steps = 0

    def begin_layer(self, name: str):
        if not self.enabled:
            return
        cuda = torch.cuda.is_available()
        if cuda:
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[name] = (ev, _lib.launches())
        else:
            self._open[name] = (time.perf_counter(), _lib.launches())

    def end_layer(self, name: str):
        if not self.enabled or name not in self._open:
            return
        start, l0 = self._open.pop(name)
        rec = self.stats.setdefault(name, [0, 0.0, 0])
        rec[0] += 1
        rec[2] += _lib.launches() - l0
        if isinstance(start, float):
            rec[1] += (time.perf_counter() - start) * 1e3
        else:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pending.append((name, start, end))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    @contextlib.contextmanager
    def range(self, name: str):
        self.begin_layer(name)
        try:
            yield
        finally:
            self.end_layer(name)

    def step_end(self):
        """Resolve the device timings recorded since the last call (one synchronisation)."""
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.stats[name][1] += a.elapsed_time(b)
            self._pending = []
        if self.enabled:
            self.steps += 1

    def total_ms(self, name: str) -> float:
        self.step_end() if self._pending else None
        return self.stats.get(name, [0, 0.0, 0])[1]

    def count(self, name: str) -> int:
        return self.stats.get(name, [0, 0.0, 0])[0]

    def report(self, file=None) -> str:
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.stats[name][1] += a.elapsed_time(b)
            self._pending = []
        total = sum(v[1] for v in self.stats.values()) or 1.0
        lines = [f"{'layer':<32}{'calls':>8}{'total ms':>12}{'mean ms':>12}{'share':>8}{'launches':>10}"]
        for name, (calls, ms, launches) in self.stats.items():
            lines.append(f"{name:<32}{calls:>8}{ms:>12.3f}{ms / max(calls, 1):>12.4f}{100 * ms / total:>7.1f}%{launches:>10}")
        lines.append(f"steps: {self.steps}")
        text = "\n".join(lines)
        print(text, file=file)
        return text


def instrument(model: torch.nn.Module, profiler: Profiler, depth: int = 2):
    """Wrap the forward of every sub-module down to `depth` in a named range."""
    handles = []
    for name, mod in model.named_modules():
        if not name or name.count(".") >= depth:
            continue
        handles.append(mod.register_forward_pre_hook(lambda m, a, n=name: profiler.begin_layer(n)))
        handles.append(mod.register_forward_hook(lambda m, a, o, n=name: profiler.end_layer(n)))
    return handles
