"""Errors raised while reading a configuration."""


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or contradicts another."""
