from .params import DEFAULT_SEED, SamplingParams
from .rng import Xoshiro256pp, sequence_seed
from .device import BatchSampler, SequenceSampler
