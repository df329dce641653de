"""Counts of the bytes that cross between host and device on the serving path.

Every host-to-device and device-to-host copy a step makes goes through three places: the step's one packed
upload (``engine.batch.StepContext.upload``), the sampler's parameter rows (``sampling.device.sample``) and the
read-back of the sampled ids with the error word (``engine.engine.Engine``).  Each adds what it copied here, so a
benchmark can report the bytes a step really moved instead of a formula.
"""
from __future__ import annotations

h2d_bytes = 0
d2h_bytes = 0


def add_h2d(n: int) -> None:
    global h2d_bytes
    h2d_bytes += int(n)


def add_d2h(n: int) -> None:
    global d2h_bytes
    d2h_bytes += int(n)


def snapshot():
    return h2d_bytes, d2h_bytes
