from kairyu_b200.weights.loading import WeightError, load_into, read_config
from kairyu_b200.weights.random_init import init_random, random_tensors, write_random_model
from kairyu_b200.weights.reader import CheckpointReader

__all__ = [
    "CheckpointReader", "WeightError", "init_random", "load_into", "random_tensors", "read_config", "write_random_model",
]
