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
