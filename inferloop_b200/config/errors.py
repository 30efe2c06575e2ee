"""Error kinds of the configuration layer.

The reference separates malformed input (`Error::invalid`) from valid input that names
something the engine does not model (`Error::unsupported`); see
crates/model/package/src/providers/qwen/mod.rs:176-180 and :414-424.
"""


class ConfigError(ValueError):
    """config.json is malformed or inconsistent."""


class UnsupportedConfig(ConfigError):
    """config.json is well formed but asks for semantics that are not modelled."""
