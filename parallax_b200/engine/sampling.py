"""Host side of the sampling penalties: which tokens each row has seen, packed for the penalty kernel.

The reference hands repetition / presence / frequency penalties to its GPU backend's batch info
(``src/parallax/sglang/batch_info.py:43-59``); here the last stage applies them to the logits with
``ops.apply_penalties`` right before arg-max / sampling.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from parallax_b200 import ops


def build_penalties(reqs) -> Optional[dict]:
    """CSR arrays for the rows of ``reqs`` (in logit-row order), or None when no row has a penalty."""
    if not any(r.sampling_params.has_penalties for r in reqs):
        return None
    row_off = [0]
    toks: list[int] = []
    cnts: list[int] = []
    for r in reqs:
        if r.sampling_params.has_penalties:
            t, c = r.penalty_entries()
            toks += t
            cnts += c
        row_off.append(len(toks))
    sps = [r.sampling_params for r in reqs]
    return {"row_off": np.asarray(row_off, dtype=np.int32), "tok_ids": np.asarray(toks, dtype=np.int32),
            "out_cnt": np.asarray(cnts, dtype=np.int32),
            "rep": np.asarray([sp.repetition_penalty for sp in sps], dtype=np.float32),
            "pres": np.asarray([sp.presence_penalty for sp in sps], dtype=np.float32),
            "freq": np.asarray([sp.frequency_penalty for sp in sps], dtype=np.float32)}


def apply_penalties(logits: torch.Tensor, pen: Optional[dict]) -> torch.Tensor:
    """Apply packed penalties (see :func:`build_penalties`) in place; a no-op for None."""
    if pen is None or pen["tok_ids"].size == 0:
        return logits
    dev = logits.device
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in pen.items()}
    return ops.apply_penalties(logits, t["row_off"], t["tok_ids"], t["out_cnt"], t["rep"], t["pres"], t["freq"])
