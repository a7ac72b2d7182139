"""Load a model's parameters from a weight file by tensor name.

An architecture supplies a :class:`WeightPlan`: for every parameter path of the model, which
tensors of the file it is made from (with the shape each must have) and how they are
combined (transpose, concatenate).  The loader checks the whole file against the plan first
and raises ONE :class:`WeightError` that lists every missing tensor, every unexpected tensor
and every wrong shape; only then does it read, combine, convert and upload.

Element types: vectors (biases, norm weights) are held in fp32 and integer tables in int32.
Matrices and embedding tables are held in fp32 when the run is ``float32``.  In a
``bfloat16`` run a matrix stored in bf16 stays bf16, and a tensor stored in 32-bit stays so
(16-bit IEEE halves are widened to fp32, which loses nothing) and runs on the fp32 kernels:
whoever wrote a file with bf16 matrices and kept one tensor in 32-bit meant it.  A file that
holds *no* bf16 matrix at all is a full-precision checkpoint (published GPT-2 files are);
asking for a ``bfloat16`` run of it means rounding its matrices to bf16, and that is what
happens unless ``cast_weights=False`` keeps the stored types.  ``cast_weights=True`` rounds
every matrix to bf16.

The reference finds ``weights.safetensors`` or ``model.safetensors`` in the model folder and
reads tensors by name (src/engine.rs:74-79,110-225).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Sequence

import torch

from ..parts.base import INDEX, MATRIX, TABLE, VECTOR, ParamSpec
from .safetensors_io import SafeTensorsFile

WEIGHT_FILE_NAMES = ("weights.safetensors", "model.safetensors")


class WeightError(ValueError):
    def __init__(self, path, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"weights in {path} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class Source:
    name: str
    shapes: tuple[tuple[int, ...], ...]   # accepted shapes in the file (usually one)
    optional: bool = False


@dataclass
class Recipe:
    """``combine`` gets one CPU tensor per source (``None`` for an absent optional one) and
    returns the parameter, or ``None`` if the (optional) parameter is absent."""
    sources: Sequence[Source]
    combine: Callable[[list], torch.Tensor | None]


@dataclass
class WeightPlan:
    recipes: dict[str, Recipe]
    ignored: set[str] = field(default_factory=set)   # names in the file that are no weights


class TensorDict:
    """In-memory tensors with the reading interface of :class:`SafeTensorsFile`."""

    def __init__(self, tensors: dict, path: str = "<memory>"):
        self._t = dict(tensors)
        self.path = path

    def names(self):
        return sorted(self._t)

    def __contains__(self, name):
        return name in self._t

    def info(self, name):
        return self._t[name]          # a tensor has .shape, which is all the loader asks for

    def tensor(self, name):
        return self._t[name]


def find_weight_file(model_dir: str | Path) -> Path:
    d = Path(model_dir)
    for n in WEIGHT_FILE_NAMES:
        if (d / n).exists():
            return d / n
    raise FileNotFoundError(f"no weights.safetensors or model.safetensors in {d}")


def stored_dtype(info) -> torch.dtype:
    """Element type of a tensor as the source holds it (a file's header entry or a tensor)."""
    dt = getattr(info, "torch_dtype", None)
    return dt if dt is not None else info.dtype


def target_dtype(role: str, stored: torch.dtype, precision: str, cast_weights: bool) -> torch.dtype:
    if role == VECTOR:
        return torch.float32
    if role == INDEX:
        return torch.int32
    if precision == "float32":
        return torch.float32
    if stored == torch.bfloat16 or cast_weights:
        return torch.bfloat16
    return torch.float32


def load_params(param_specs: dict[str, ParamSpec], plan: WeightPlan, file: SafeTensorsFile,
                *, precision: str, device, cast_weights: bool | None = None) -> dict:
    """``cast_weights``: in a ``bfloat16`` run, round matrices stored in 32-bit to bf16
    (``True``), keep them as stored (``False``), or (``None``) round them only when the file
    holds no bf16 matrix at all, i.e. is a full-precision checkpoint."""
    names = set(file.names())
    missing: list[str] = []
    wrong: list[str] = []
    other: list[str] = []
    used: set[str] = set()
    todo: list[tuple[str, ParamSpec, Recipe]] = []

    for path, spec in param_specs.items():
        recipe = plan.recipes.get(path)
        if recipe is None:
            if not spec.optional:
                other.append(f"parameter {path}: the architecture names no source tensor")
            continue
        present = [s for s in recipe.sources if s.name in names]
        required_absent = [s for s in recipe.sources if not s.optional and s.name not in names]
        if required_absent:
            if spec.optional and not present:
                continue  # the whole optional parameter is absent
            missing.extend(s.name for s in required_absent)
            used.update(s.name for s in present)
            continue
        ok = True
        for s in present:
            used.add(s.name)
            got = tuple(file.info(s.name).shape)
            if got not in s.shapes:
                want = " or ".join(str(list(x)) for x in s.shapes)
                wrong.append(f"{s.name} is {list(got)}, expected {want}")
                ok = False
        if ok and present:
            todo.append((path, spec, recipe))

    unexpected = sorted(names - used - plan.ignored)
    if missing or wrong or unexpected or other:
        raise WeightError(file.path, sorted(set(missing)), unexpected, wrong, other)

    if cast_weights is None:
        kinds = {stored_dtype(file.info(s.name)) for _, spec, recipe in todo
                 if spec.role in (MATRIX, TABLE) for s in recipe.sources if s.name in names}
        cast_weights = torch.bfloat16 not in kinds
    out: dict[str, torch.Tensor | None] = {p: None for p in param_specs}
    for path, spec, recipe in todo:
        tensors = [file.tensor(s.name) if s.name in names else None for s in recipe.sources]
        t = recipe.combine(tensors)
        if t is None:
            continue
        if tuple(t.shape) != tuple(spec.shape):
            raise WeightError(file.path, wrong_shape=[
                f"{path} came out as {list(t.shape)}, expected {list(spec.shape)}"])
        dt = target_dtype(spec.role, t.dtype, precision, cast_weights)
        out[path] = t.to(dt).contiguous().to(device)
    return out


# ---- helpers for plans --------------------------------------------------------------------
def take(name: str, shape, optional: bool = False) -> Recipe:
    """The tensor as stored."""
    return Recipe([Source(name, (tuple(shape),), optional)], lambda ts: ts[0])


def take_transposed(name: str, stored_shape, optional: bool = False) -> Recipe:
    """A linear weight stored ``(in, out)`` and held ``(out, in)`` (src/engine.rs:93-101)."""
    return Recipe([Source(name, (tuple(stored_shape),), optional)],
                  lambda ts: None if ts[0] is None else ts[0].t().contiguous())


def _common(ts):
    dts = {t.dtype for t in ts}
    if len(dts) == 1:
        return ts
    return [t.to(torch.float32) for t in ts]


def concat_transposed(names_shapes) -> Recipe:
    """Several ``(in, out_i)`` matrices → one ``(sum out_i, in)`` matrix."""
    srcs = [Source(n, (tuple(s),)) for n, s in names_shapes]
    return Recipe(srcs, lambda ts: torch.cat([t.t() for t in _common(ts)], dim=0).contiguous())


def concat_optional_vectors(names_lengths) -> Recipe:
    """Several optional vectors → their concatenation, absent ones as zeros; ``None`` if all
    are absent."""
    srcs = [Source(n, ((int(l),),), optional=True) for n, l in names_lengths]
    lengths = [int(l) for _, l in names_lengths]

    def combine(ts):
        if all(t is None for t in ts):
            return None
        return torch.cat([torch.zeros(l, dtype=torch.float32) if t is None else t.to(torch.float32)
                          for t, l in zip(ts, lengths)])

    return Recipe(srcs, combine)
