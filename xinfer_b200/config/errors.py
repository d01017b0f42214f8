"""The error every configuration reader raises; it belongs to no architecture."""
from __future__ import annotations


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong type or asks for something this engine lacks."""
