"""The one registry from an architecture's name to its configuration class.

`architectures[0]` of config.json selects the entry, as in the reference
(v3/crates/rvllm-core/src/config/model.rs:20-29,70-79); an unknown name is an error that
lists the known ones.  A registered class needs `from_dict(obj, where)` and `to_spec()`.
"""
from __future__ import annotations

from typing import Any, Dict, Type

from ..errors import ConfigError
from .model_config import LlamaConfig, Qwen2Config, read_config_json

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_class: Type) -> None:
    """Add (or replace) an architecture.  `config_class.from_dict` reads its config.json keys
    and `to_spec()` returns the `ModelSpec` the generic model is built from."""
    for attr in ("from_dict", "to_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"{config_class.__name__} needs `{attr}` to be registered")
    _ARCHITECTURES[name] = config_class


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(obj: Dict[str, Any], where: str = "config.json"):
    archs = obj.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("missing key `architectures` (a list whose first entry names the model)", where)
    cls = _ARCHITECTURES.get(archs[0])
    if cls is None:
        raise ConfigError(f"unsupported architecture {archs[0]!r}; known: {', '.join(known_architectures())}", where)
    return cls.from_dict(obj, where)


def load_config(model_dir: str):
    """Read `model_dir/config.json` into the typed configuration of its architecture."""
    import os
    return config_from_dict(read_config_json(model_dir), os.path.join(model_dir, "config.json"))


register_architecture("LlamaForCausalLM", LlamaConfig)
register_architecture("Qwen2ForCausalLM", Qwen2Config)
