"""Errors raised while reading a model's configuration."""


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model.

    The message names the key and the value that was refused.
    """


class UnknownArchitectureError(ConfigError):
    """config.json names an architecture that no registered builder handles."""
