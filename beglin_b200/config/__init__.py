from .reader import ConfigError, ConfigFields
from .registry import ARCHITECTURES, Architecture, register_architecture, resolve_architecture

__all__ = ["ConfigError", "ConfigFields", "ARCHITECTURES", "Architecture", "register_architecture",
           "resolve_architecture", "load_config"]


def load_config(source, tensor_names=None):
    """(architecture, typed configuration) of a model folder, a config.json path or a dict."""
    import beglin_b200.models  # noqa: F401  (registers the architectures)
    fields = ConfigFields(source) if isinstance(source, dict) else ConfigFields.from_file(source)
    arch = resolve_architecture(fields)
    return arch, arch.config_class.from_fields(fields, tensor_names=tensor_names)
