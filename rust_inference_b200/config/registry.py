"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

The reference has a single code path and uses the architecture string only to pick
defaults and the metadata prefix (model.rs:65-71, :89-95).  Here a name maps to an
`Architecture`: how to read its config.json into a typed config, and how to turn that
config into a `ModelSpec` (the list of layers, each assembled from named parts).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed config
    build_spec: Callable[[Any], Any]                    # typed config -> parts.spec.ModelSpec
    # True: parse_config also takes `shapes` (tensor name -> shape of the folder's weight file), for a size that
    # config.json leaves to a tensor's shape
    reads_shapes: bool = False


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec, *, replace: bool = False,
                          reads_shapes: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, parse_config, build_spec, reads_shapes)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}"
        ) from None


def architecture_name(d: Mapping[str, Any]) -> str:
    """The name config.json gives its model: the first entry of `architectures`, or `architecture`."""
    archs = d.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    if isinstance(d.get("architecture"), str) and d["architecture"]:
        return d["architecture"]
    raise ConfigError("config.json: 'architectures' must be a non-empty list (or 'architecture' a name)")


def config_from_dict(d: Mapping[str, Any]):
    """Pick the architecture named by the dict and parse it into that architecture's config."""
    return get_architecture(architecture_name(d)).parse_config(d)


def _folder_shapes(model_dir: str) -> dict:
    """Tensor name -> shape from the folder's weight file (its header only); empty without one."""
    from ..weights.safetensors_io import ModelFiles
    try:
        files = ModelFiles(model_dir)
    except (OSError, ValueError):
        return {}
    try:
        return {name: tuple(files.shape(name)) for name in files.names()}
    finally:
        files.close()


def _parse(arch: Architecture, d: Mapping[str, Any], model_dir: str):
    if arch.reads_shapes:
        return arch.parse_config(d, shapes=_folder_shapes(model_dir))
    return arch.parse_config(d)


def load_config(model_dir: str):
    d = read_config_json(model_dir)
    return _parse(get_architecture(architecture_name(d)), d, model_dir)


def load_spec(model_dir: str):
    """(config, ModelSpec) of a model folder: config.json's architecture name picks the
    architecture, which parses the config and builds the spec."""
    d = read_config_json(model_dir)
    arch = get_architecture(architecture_name(d))
    config = _parse(arch, d, model_dir)
    return config, arch.build_spec(config)


def _ensure_builtin() -> None:
    # The built-in models register themselves on import.
    from ..models import dense_decoder, lulisun, vadodra, redodra, belizen  # noqa: F401
