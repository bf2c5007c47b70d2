"""What the host sees of the device through a stream: the floor of every host-clocked "stream is idle" figure.

    python -m reef_b200.stream_latency [--iters 2000] [--device 0]

Prints the median cost of the preempt-flag write call (reef_write32_async), of that write plus its completion as seen
from the host (a completion-only event behind it, polled), and of a bare event's round trip on an idle stream, without and
with a timestamp.  The scheduler's
preemption drain (flag write -> best-effort streams idle) cannot be shorter than the second figure plus the time the
best-effort blocks need to leave.
"""
from __future__ import annotations

import argparse
import ctypes as C


def main():
    from . import capi
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=2000)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    w, wc, ev, evt = capi.probe_stream_latency(a.iters, a.device)
    print(f"write call {w:.2f} us | write + completion seen by the host {wc:.2f} us | completion-only event round trip "
          f"{ev:.2f} us | timed event round trip {evt:.2f} us (medians of {a.iters})")


if __name__ == "__main__":
    main()
