"""A B200-native generation library for the Qwen2 dense decoder.

From a model folder (config.json, model.safetensors) to generated tokens on one
GPU: a typed configuration and an architecture registry (`config`), weights by
tensor name (`weights`), layers put together from parts (`parts`), a cache with
a slot for each live sequence (`cache`), one step function over batches of
unequal lengths with a generation loop above it (`engine`), greedy and
temperature sampling (`sampling`), all on hand-written CUDA kernels for sm_100a
(`csrc`, `ops`).

    from semantic_aware_adaptive_kv_cache_precision_b200 import Engine
    engine = Engine("model_dir").load_weights()
    new_ids = engine.generate([1, 2, 3], max_new_tokens=16)
"""

from .config import ConfigError, Qwen2Config, config_from_dict, config_from_folder, \
    known_architectures, register_architecture
from .weights import WeightError, write_random_model
from .cache import CacheFull
from .errors import OutOfDeviceMemory
from .engine import COMPLETE, DECODING, EXHAUSTED, PREFILLING, Ending, Engine

__version__ = "0.1.0"

__all__ = ["ConfigError", "Qwen2Config", "config_from_dict", "config_from_folder",
           "known_architectures", "register_architecture", "WeightError", "write_random_model",
           "CacheFull", "OutOfDeviceMemory", "COMPLETE", "DECODING", "EXHAUSTED", "PREFILLING", "Ending", "Engine"]
