from .batch import BatchLayout, build_layout
from .context import StepContext
from .engine import Engine
from .generate import SequenceProgress, plan_batches, token_budget
from .model import Layer, Model, Runtime
from .spec import LayerSpec, ModelSpec
