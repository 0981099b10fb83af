"""What every architecture's configuration shares: the error type and the reader of config.json.

The reference reads ``DIR/config.json`` once and reports a file it cannot open or parse as
one error (cleanroom-transformer/src/model.c:109-127); each architecture's own file then
interprets the keys.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict


class ConfigError(ValueError):
    """Raised for a config.json that cannot be read or that its architecture cannot run."""


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except OSError as e:
        raise ConfigError(f"config: cannot open {path}: {e.strerror}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config: {path} is not valid JSON: {e}") from None
