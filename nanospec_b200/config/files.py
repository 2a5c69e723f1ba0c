"""What every architecture's configuration shares: the error type and the reading of a model
folder's config.json and generation_config.json (model/loader.py:33-38 in the reference)."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that this framework cannot run, with the reason."""


def read_config_files(folder: str | Path) -> tuple[dict[str, Any], dict[str, Any] | None]:
    """config.json and, when present, generation_config.json of a model folder."""
    folder = Path(folder)
    path = folder / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    cfg = json.loads(path.read_text())
    gen_path = folder / "generation_config.json"
    gen = json.loads(gen_path.read_text()) if gen_path.is_file() else None
    return cfg, gen
