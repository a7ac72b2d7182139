"""What a part sees of the step it runs in."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .batch import BatchLayout
from .model import Runtime


@dataclass
class StepContext:
    rt: Runtime
    ops: Any                 # kernel backend (csrc.ops.CudaBackend)
    layout: BatchLayout
    position: Any            # the model's position-encoding part
    cache: Any               # SequenceCache
    # storage of the schedule entry that is running (set by the model before each layer)
    kv: Any = None           # LayerKV or None
    state: Any = None        # fp32 [n_slots, n_elements] or None
    writes_cache: bool = True
