"""janis_b200: a small Gemma2 generation library for one NVIDIA B200.

    import janis_b200
    eng = janis_b200.open("/path/to/model")            # config.json + model.safetensors
    replies = eng.generate([[2, 651, 6037]], temp=0.0, max_tokens=32)
    eng.close()

`open` (alias `load`) reads the folder; `from_config` builds random weights on the
device; `write_random_model` writes a folder of random weights.  `Engine.step` is
the step function, `Engine.generate` the loop above it.  Architectures and kinds
of parts are registered by name (`register_architecture`, `parts.registry`).
"""
from .config.base import ConfigError
from .config.gemma2 import Gemma2Config
from .registry import architectures, register_architecture, resolve, unregister_architecture
from .models import gemma2 as _gemma2            # registers Gemma2ForCausalLM
from .engine.engine import Engine, build_model, from_config, load, open, write_random_model
from .engine.step import StepEntry, StepError
from .engine.generate import Reply
from .sampling.sampler import SamplingParams
from .weights.loader import WeightsError

__version__ = "0.1.0"

__all__ = ["open", "load", "from_config", "write_random_model", "build_model", "Engine", "StepEntry", "StepError",
           "Reply", "SamplingParams", "Gemma2Config", "ConfigError", "WeightsError", "register_architecture",
           "unregister_architecture", "architectures", "resolve", "__version__"]
