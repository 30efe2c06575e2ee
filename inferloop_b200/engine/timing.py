"""Device time of a step, whole or kernel by kernel.

The reference has the same switch, `--device-timing off|graph|node`
(crates/foundation/ir/src/device_timing.rs:11-24): `graph` brackets a whole replayed graph
with two events, `node` gives every kernel node its own pair
(crates/backend/cuda/src/device/device_timer.rs:1-37).  Here:

  off    nothing is recorded;
  graph  two CUDA events around every step the runner launches (recorded graphs stay on);
  node   a pair of events around every kernel launch, attributed to the op class the
         launching part names with `ops.scope(...)`; steps run kernel by kernel (no recorded
         graphs), because a replayed graph is one launch to the stream.  The events between
         the kernels also end the overlap of a kernel's prologue with its predecessor's tail
         that dependent launches give, so the sum over a step is a little above the time of
         the same step in `graph` mode: read the shares, and the step time from `graph`.

Events are created per launch and read in `summary()`, which synchronises.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

MODES = ("off", "graph", "node")


class DeviceTimer:
    def __init__(self, device: torch.device, mode: str = "off") -> None:
        if mode not in MODES:
            raise ValueError(f"device timing mode {mode!r}: use one of {MODES}")
        self.device = device
        self.mode = mode
        self._steps: List[Tuple[int, torch.cuda.Event, torch.cuda.Event]] = []
        self._nodes: List[Tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self._open: Optional[torch.cuda.Event] = None

    # ---------------------------------------------------------------- recording
    def step_begin(self) -> None:
        if self.mode == "off":
            return
        self._open = torch.cuda.Event(enable_timing=True)
        self._open.record(torch.cuda.current_stream(self.device))

    def step_end(self, n_tokens: int) -> None:
        if self.mode == "off" or self._open is None:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record(torch.cuda.current_stream(self.device))
        self._steps.append((int(n_tokens), self._open, end))
        self._open = None

    def node_begin(self) -> Optional[torch.cuda.Event]:
        if self.mode != "node":
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def node_end(self, scope: str, kernel: str, begin: Optional[torch.cuda.Event]) -> None:
        if begin is None:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record(torch.cuda.current_stream(self.device))
        self._nodes.append((scope, kernel, begin, end))

    def reset(self) -> None:
        self._steps.clear()
        self._nodes.clear()
        self._open = None

    # ---------------------------------------------------------------- reading
    def summary(self) -> dict:
        """{"mode", "steps": {"count", "ms_total", "ms_mean", "tokens"}, "ops": {scope:
        {"launches", "ms", "share", "kernels": {entry point: {"launches", "ms"}}}}};
        synchronises the device."""
        torch.cuda.synchronize(self.device)
        out: dict = {"mode": self.mode}
        if self._steps:
            ms = [a.elapsed_time(b) for _, a, b in self._steps]
            out["steps"] = {"count": len(ms), "ms_total": round(sum(ms), 4), "ms_mean": round(sum(ms) / len(ms), 4),
                            "tokens": sum(n for n, _, _ in self._steps)}
        if self._nodes:
            ops: "OrderedDict[str, dict]" = OrderedDict()
            for scope, kernel, a, b in self._nodes:
                rec = ops.setdefault(scope, {"launches": 0, "ms": 0.0, "kernels": {}})
                ms = a.elapsed_time(b)
                rec["launches"] += 1
                rec["ms"] += ms
                per = rec["kernels"].setdefault(kernel, {"launches": 0, "ms": 0.0})
                per["launches"] += 1
                per["ms"] += ms
            total = sum(r["ms"] for r in ops.values()) or 1.0
            for r in ops.values():
                r["share"] = round(r["ms"] / total, 4)
                r["ms"] = round(r["ms"], 4)
                for per in r["kernels"].values():
                    per["ms"] = round(per["ms"], 4)
            out["ops"] = dict(ops)
            out["ops_ms_total"] = round(total, 4)
        return out
