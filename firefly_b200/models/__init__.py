from . import kefisun, kolorax, papusun, pepolorn, qwen3  # noqa: F401  (register the designs)
from .decoder import DecoderModel, expected_weights
from .registry import (architecture_of, config_from_dict, known_architectures, load_config,
                       register_architecture, spec_for)

__all__ = ["DecoderModel", "expected_weights", "architecture_of", "config_from_dict",
           "known_architectures", "load_config", "register_architecture", "spec_for"]
