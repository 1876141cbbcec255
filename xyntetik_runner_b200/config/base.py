"""What every architecture's configuration shares: the error type and the reader of config.json."""
from __future__ import annotations

import json
import os


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine refuses."""


def read_config_json(path: str) -> dict:
    """Read `path` (a model folder or the json file itself) into a dict."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
