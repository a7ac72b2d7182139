"""Position encodings."""
from __future__ import annotations

from .base import TABLE, ParamSpec, Position, register_part


@register_part("position", "learned_absolute")
class LearnedAbsolute(Position):
    """A learned row per absolute position, added to the token embedding
    (src/model.rs:288-293).  Sequences cannot be longer than the table."""
    graph_safe = True

    def __init__(self, max_positions: int, width: int):
        self.max_positions = int(max_positions)
        self.width = int(width)
        self.table = None

    def param_specs(self):
        return {"table": ParamSpec((self.max_positions, self.width), TABLE)}


@register_part("position", "none")
class NoPosition(Position):
    """No position information is added anywhere."""
    graph_safe = True

    def __init__(self, max_positions: int | None = None):
        self.max_positions = max_positions
        self.table = None
