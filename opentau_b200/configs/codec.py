"""Dataclass <-> JSON codec with choice registries and dotted command-line overrides.

A small, dependency-free stand-in for the ``draccus`` behaviour the reference relies on
(OpenTau ``src/opentau/configs/parser.py:286-400``, ``configs/policies.py:291,524-531``):

* a class deriving from :class:`ChoiceRegistry` registers subclasses under a ``type`` name;
  the JSON form of such a field is ``{"type": "<name>", ...fields}``;
* ``decode(cls, dict)`` builds nested dataclasses, tuples, lists, dicts, enums, optionals;
* ``apply_overrides(dict, ["--a.b=c", ...])`` edits the raw dict before decoding, with values
  parsed as JSON when possible (``true``, ``1e-4``, ``[1,2]``) and kept as strings otherwise.
"""

from __future__ import annotations

import dataclasses
import enum
import json
import types
import typing
from pathlib import Path
from typing import Any, Union, get_args, get_origin, get_type_hints


class ChoiceRegistry:
    """Base for config families selected by a ``type`` string."""

    _choice_registry: dict[str, type]

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        if ChoiceRegistry in cls.__bases__:
            cls._choice_registry = {}

    @classmethod
    def register_subclass(cls, name: str):
        def deco(sub):
            cls._choice_registry[name] = sub
            sub._choice_name = name
            return sub
        return deco

    @classmethod
    def get_choice_class(cls, name: str) -> type:
        if name not in cls._choice_registry:
            raise KeyError(f"unknown {cls.__name__} type {name!r}; known: {sorted(cls._choice_registry)}")
        return cls._choice_registry[name]

    @classmethod
    def get_known_choices(cls) -> dict[str, type]:
        return dict(cls._choice_registry)

    def get_choice_name(self) -> str:
        return getattr(type(self), "_choice_name", type(self).__name__)


def _is_registry_base(tp) -> bool:
    return isinstance(tp, type) and issubclass(tp, ChoiceRegistry) and "_choice_registry" in tp.__dict__


def encode(obj: Any) -> Any:
    """Dataclass tree -> JSON-able structure."""
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        out: dict[str, Any] = {}
        if isinstance(obj, ChoiceRegistry) and hasattr(type(obj), "_choice_name"):
            out["type"] = obj.get_choice_name()
        for f in dataclasses.fields(obj):
            if f.metadata.get("skip_encode"):
                continue
            out[f.name] = encode(getattr(obj, f.name))
        return out
    if isinstance(obj, enum.Enum):
        return obj.value
    if isinstance(obj, Path):
        return str(obj)
    if isinstance(obj, (list, tuple)):
        return [encode(x) for x in obj]
    if isinstance(obj, dict):
        return {(k.value if isinstance(k, enum.Enum) else str(k) if not isinstance(k, (str, int)) else k): encode(v)
                for k, v in obj.items()}
    return obj


def decode(tp: Any, value: Any, path: str = "") -> Any:
    """JSON-able structure -> instance of ``tp`` (dataclass, container or scalar)."""
    if tp is Any or tp is None:
        return value
    origin = get_origin(tp)
    if origin in (Union, types.UnionType):
        args = get_args(tp)
        if value is None and type(None) in args:
            return None
        members = [a for a in args if a is not type(None)]
        if len(members) == 1:
            return decode(members[0], value, path)
        last: Exception | None = None
        for a in args:
            if a is type(None):
                continue
            try:
                return decode(a, value, path)
            except (TypeError, ValueError, KeyError) as e:  # try the next member
                last = e
        raise TypeError(f"{path}: cannot decode {value!r} as {tp}: {last}")
    if origin in (list, typing.List):
        (a,) = get_args(tp) or (Any,)
        return [decode(a, v, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (tuple, typing.Tuple):
        args = get_args(tp)
        if len(args) == 2 and args[1] is Ellipsis:
            return tuple(decode(args[0], v, path) for v in value)
        if args:
            return tuple(decode(a, v, path) for a, v in zip(args, value))
        return tuple(value)
    if origin in (dict, typing.Dict):
        ka, va = get_args(tp) or (Any, Any)
        return {decode(ka, k, path): decode(va, v, f"{path}.{k}") for k, v in value.items()}
    if isinstance(tp, type) and issubclass(tp, enum.Enum):
        if isinstance(value, tp):
            return value
        try:
            return tp(value)
        except ValueError:
            return tp[value]
    if isinstance(tp, type) and dataclasses.is_dataclass(tp):
        if isinstance(value, tp):
            return value
        if not isinstance(value, dict):
            raise TypeError(f"{path}: expected an object for {tp.__name__}, got {type(value).__name__}")
        value = dict(value)
        cls = tp
        if isinstance(tp, type) and issubclass(tp, ChoiceRegistry):
            base = next((b for b in tp.__mro__ if _is_registry_base(b)), None)
            name = value.pop("type", None)
            if name is not None and base is not None:
                cls = base.get_choice_class(name)
            elif _is_registry_base(tp):
                raise KeyError(f"{path}: a 'type' key is required to choose a {tp.__name__}")
        hints = get_type_hints(cls)
        kwargs, post = {}, {}
        names = {f.name: f for f in dataclasses.fields(cls)}
        deprecated = getattr(cls, "_deprecated_fields", ())
        for k, v in value.items():
            if k in deprecated:
                continue
            if k not in names:
                raise KeyError(f"{path}: {cls.__name__} has no field {k!r}")
            dv = decode(hints.get(k, Any), v, f"{path}.{k}" if path else k)
            (kwargs if names[k].init else post)[k] = dv
        obj = cls(**kwargs)
        for k, v in post.items():
            setattr(obj, k, v)
        return obj
    if tp is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if tp is int and isinstance(value, float) and value.is_integer():
        return int(value)
    if tp is Path:
        return Path(value)
    if tp is tuple and isinstance(value, (list, tuple)):
        return tuple(value)
    if tp is list and isinstance(value, (list, tuple)):
        return list(value)
    if tp is bool and isinstance(value, str):
        if value.lower() in ("true", "1", "yes"):
            return True
        if value.lower() in ("false", "0", "no"):
            return False
        raise ValueError(f"{path}: not a bool: {value!r}")
    if isinstance(tp, type) and tp in (int, float, str, bool):
        if isinstance(value, tp) and not (tp is int and isinstance(value, bool)):
            return value
        if tp is str:
            return str(value)
        if isinstance(value, str):
            return tp(value)
        raise TypeError(f"{path}: expected {tp.__name__}, got {value!r}")
    return value


def parse_cli_value(text: str) -> Any:
    try:
        return json.loads(text)
    except (json.JSONDecodeError, ValueError):
        return text


def apply_overrides(raw: dict, args: list[str]) -> dict:
    """Applies ``--a.b.c=value`` (or ``--a.b.c value``) edits to a nested dict; list indices allowed."""
    i = 0
    while i < len(args):
        a = args[i]
        if not a.startswith("--"):
            raise ValueError(f"unexpected argument {a!r}")
        if "=" in a:
            key, val = a[2:].split("=", 1)
        else:
            key = a[2:]
            if i + 1 < len(args) and not args[i + 1].startswith("--"):
                val = args[i + 1]
                i += 1
            else:
                val = "true"
        i += 1
        node: Any = raw
        parts = key.split(".")
        for j, p in enumerate(parts[:-1]):
            nxt = parts[j + 1]
            if isinstance(node, list):
                node = node[int(p)]
                continue
            if p not in node or node[p] is None:
                node[p] = [] if nxt.isdigit() else {}
            node = node[p]
        last = parts[-1]
        v = parse_cli_value(val)
        if isinstance(node, list):
            idx = int(last)
            while len(node) <= idx:
                node.append(None)
            node[idx] = v
        else:
            node[last] = v
    return raw


def load_json(path: str | Path) -> dict:
    with open(path) as f:
        return json.load(f)


def save_json(obj: Any, path: str | Path) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        json.dump(encode(obj), f, indent=4)
