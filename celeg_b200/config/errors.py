"""Error types raised while a model folder is read."""


class ConfigError(ValueError):
    """config.json is unreadable, incomplete or inconsistent; the message names the key."""


class UnknownArchitectureError(ConfigError):
    """config.json names a model_type that no architecture is registered for."""
