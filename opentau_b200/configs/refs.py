"""``{"$ref": "file.json", ...overrides}`` includes inside JSON configs.

A dict containing ``$ref`` is replaced by the referenced file's content (path relative to the including
file), deep-merged with the dict's other keys (the overrides win).  Cycles are rejected.  Behaviour
follows OpenTau ``src/opentau/configs/refs.py:66-142``.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

REF_KEY = "$ref"


def deep_merge(base: Any, over: Any) -> Any:
    if isinstance(base, dict) and isinstance(over, dict):
        out = dict(base)
        for k, v in over.items():
            out[k] = deep_merge(base[k], v) if k in base else v
        return out
    return over


def resolve_refs(node: Any, base_dir: Path, _stack: tuple[Path, ...] = ()) -> Any:
    if isinstance(node, list):
        return [resolve_refs(x, base_dir, _stack) for x in node]
    if not isinstance(node, dict):
        return node
    if REF_KEY in node:
        ref = node[REF_KEY]
        if not isinstance(ref, str):
            raise ValueError(f"{REF_KEY} must be a string path, got {ref!r}")
        path = (base_dir / ref).resolve()
        if path in _stack:
            raise ValueError(f"circular {REF_KEY}: {' -> '.join(map(str, _stack + (path,)))}")
        if not path.is_file():
            raise FileNotFoundError(f"{REF_KEY} target not found: {path}")
        with open(path) as f:
            loaded = json.load(f)
        loaded = resolve_refs(loaded, path.parent, _stack + (path,))
        overrides = {k: resolve_refs(v, base_dir, _stack) for k, v in node.items() if k != REF_KEY}
        return deep_merge(loaded, overrides) if overrides else loaded
    return {k: resolve_refs(v, base_dir, _stack) for k, v in node.items()}


def load_json_with_refs(path: str | Path) -> Any:
    path = Path(path)
    with open(path) as f:
        raw = json.load(f)
    return resolve_refs(raw, path.parent.resolve(), (path.resolve(),))
