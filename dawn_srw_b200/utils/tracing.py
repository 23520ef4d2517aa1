"""Named ranges around the model's building blocks: NVTX ranges for external
profilers and device-timed per-range totals for the trainer's own report.

Both are off by default and cost one dictionary lookup per range when off.

* ``DAWN_NVTX=1`` (or ``enable(nvtx=True)``): every range pushes / pops an NVTX
  range on CUDA, so Nsight tools show ``attn/srw_qkv``, ``know/srw`` ... on the
  timeline.
* ``enable(timers=True)``: every range is bracketed by CUDA events on the
  current stream (``perf_counter`` on CPU); ``report()`` synchronises once and
  returns ``{name: (calls, total_ms)}``, backward work is attributed to the
  forward range that created it only through autograd's own kernels, i.e. the
  table covers the forward pass and whatever runs inside explicit ranges
  (``backward``, ``optimizer``) that the trainer opens.

The reference has no tracing at all apart from a start-up micro-profiler
(scripts/train_jax.py:2413-2746); that table is ``train/startup.py``.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, List, Tuple

import torch

_STATE = {"nvtx": os.environ.get("DAWN_NVTX", "0") == "1", "timers": False}
_EVENTS: Dict[str, List[Tuple[object, object]]] = {}
_CPU_MS: Dict[str, List[float]] = {}


def enable(nvtx: bool = None, timers: bool = None) -> None:
    if nvtx is not None:
        _STATE["nvtx"] = bool(nvtx)
    if timers is not None:
        _STATE["timers"] = bool(timers)


def active() -> bool:
    return _STATE["nvtx"] or _STATE["timers"]


@contextlib.contextmanager
def trace(name: str):
    """``with trace("attn/srw_qkv"): ...``"""
    if not (_STATE["nvtx"] or _STATE["timers"]):
        yield
        return
    cuda = torch.cuda.is_available() and torch.cuda.is_initialized()
    if _STATE["nvtx"] and cuda:
        torch.cuda.nvtx.range_push(name)
    ev = None
    t0 = 0.0
    if _STATE["timers"]:
        if cuda:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        else:
            t0 = time.perf_counter()
    try:
        yield
    finally:
        if _STATE["timers"]:
            if ev is not None:
                ev[1].record()
                _EVENTS.setdefault(name, []).append(ev)
            else:
                _CPU_MS.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)
        if _STATE["nvtx"] and cuda:
            torch.cuda.nvtx.range_pop()


def report(reset: bool = True) -> Dict[str, Tuple[int, float]]:
    """{range name: (calls, total milliseconds)}; synchronises the device once."""
    out: Dict[str, Tuple[int, float]] = {}
    if _EVENTS:
        torch.cuda.synchronize()
    for name, evs in _EVENTS.items():
        out[name] = (len(evs), sum(a.elapsed_time(b) for a, b in evs))
    for name, ms in _CPU_MS.items():
        n, tot = out.get(name, (0, 0.0))
        out[name] = (n + len(ms), tot + sum(ms))
    if reset:
        _EVENTS.clear()
        _CPU_MS.clear()
    return out


def format_report(rep: Dict[str, Tuple[int, float]]) -> str:
    total = sum(v[1] for k, v in rep.items() if "/" not in k) or sum(v[1] for v in rep.values()) or 1.0
    lines = ["range                          calls     total ms    share"]
    for name, (n, ms) in sorted(rep.items(), key=lambda kv: -kv[1][1]):
        lines.append("%-30s %5d %12.3f %7.1f %%" % (name, n, ms, 100.0 * ms / total))
    return "\n".join(lines)
