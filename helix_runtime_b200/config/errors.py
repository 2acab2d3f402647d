"""Errors a user can cause with a bad model folder."""


class ConfigError(ValueError):
    """``config.json`` is malformed, or asks for something this engine does not run."""
