"""Device sampler: one kernel launch for all rows of a step."""
from __future__ import annotations

import struct
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops, transfers
from .params import SamplingParams

_ROW = struct.Struct("<fiffQQ")   # temperature, top_k, top_p, min_p, seed, counter: 32 bytes


def pack_params(params: Sequence[SamplingParams], counters: Sequence[int]) -> np.ndarray:
    buf = bytearray(_ROW.size * len(params))
    for i, (p, c) in enumerate(zip(params, counters)):
        _ROW.pack_into(buf, i * _ROW.size, float(p.temperature), int(p.top_k), float(p.top_p), float(p.min_p),
                       int(p.seed) & ((1 << 64) - 1), int(c) & ((1 << 64) - 1))
    return np.frombuffer(buf, dtype=np.uint8)          # a view of the bytearray: writable


_scratch = {}


def _argmax_scratch(device, rows: int):
    got = _scratch.get(device)
    if got is None or got[0].numel() < rows * 32:
        n = max(rows, 64) * 32
        got = (torch.empty(n, dtype=torch.float32, device=device), torch.empty(n, dtype=torch.int32, device=device))
        _scratch[device] = got
    return got


_staging = {}


def _param_staging(device, nbytes: int):
    """Pinned and device buffers for the parameter rows, from a ring of four (pinning memory per call costs more
    than the kernel); a slot is taken again only after the copy out of it has run."""
    ring = _staging.setdefault(device, {"at": 0, "slots": []})
    if len(ring["slots"]) < 4:
        n = max(nbytes, 64 * _ROW.size)
        ring["slots"].append([torch.empty(n, dtype=torch.uint8, pin_memory=True),
                              torch.empty(n, dtype=torch.uint8, device=device), torch.cuda.Event()])
        return ring["slots"][-1]
    ring["at"] = (ring["at"] + 1) % 4
    slot = ring["slots"][ring["at"]]
    slot[2].synchronize()
    if slot[0].numel() < nbytes:
        slot[0] = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
        slot[1] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return slot


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per row of ``logits`` [rows, vocab] (fp32, device); returns int32 [rows] on the device."""
    rows, vocab = logits.shape
    if len(params) != rows or len(counters) != rows:
        raise ops.KernelError(f"sample: {len(params)} parameter sets for {rows} rows")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if all(p.greedy for p in params):
        # argmax needs no parameters on the device and is spread over many blocks per row
        part_v, part_i = _argmax_scratch(logits.device, rows)
        ops.argmax(logits, out, rows, part_v, part_i)
        return out
    host, dev, event = _param_staging(logits.device, rows * _ROW.size)
    host[:rows * _ROW.size].copy_(torch.from_numpy(pack_params(params, counters)))
    dev[:rows * _ROW.size].copy_(host[:rows * _ROW.size], non_blocking=True)
    event.record()
    transfers.add_h2d(rows * _ROW.size)
    ops.sample(logits, dev, out, rows)
    return out
