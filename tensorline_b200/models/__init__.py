"""Models as data (`ModelSpec`), the built `Model`, and the registry of architectures."""
from .spec import LayerSpec, RunEntry, ModelSpec, Model
from .registry import (register_architecture, architecture, registered_architectures, load_config, build_model,
                       load_model, expected_tensors)
