"""Reading a model folder's config.json, whatever architecture it names.

The limits and error classes are the reference's (src/models/llama/config.rs:
9-10, 82-109, 203-206): at most 1 MiB, a read failure is `ConfigRead`, a file
that is no JSON object is `ConfigJson`. Which keys the document must hold is
the business of the architecture that the document names.
"""
from __future__ import annotations

import json
import os
from typing import Mapping

from . import errors

CONFIG_FILE = "config.json"
MAX_CONFIG_BYTES = 1024 * 1024  # src/models/llama/config.rs:10


def read_config_json(directory: str) -> dict:
    path = os.path.join(directory, CONFIG_FILE)
    try:
        size = os.stat(path).st_size
    except OSError as exc:
        raise errors.ConfigRead(f"cannot read {path}: {exc}") from exc
    if size > MAX_CONFIG_BYTES:
        raise errors.ConfigTooLarge(f"{path} holds {size} bytes, the limit is {MAX_CONFIG_BYTES}")
    try:
        with open(path, "rb") as handle:
            raw = handle.read()
    except OSError as exc:
        raise errors.ConfigRead(f"cannot read {path}: {exc}") from exc
    return decode_json(raw)


def decode_json(source) -> dict:
    if isinstance(source, Mapping):
        return dict(source)
    try:
        doc = json.loads(source)
    except (ValueError, TypeError) as exc:
        raise errors.ConfigJson(f"config is not valid JSON: {exc}") from exc
    if not isinstance(doc, dict):
        raise errors.ConfigJson("config.json does not hold a JSON object")
    return doc
