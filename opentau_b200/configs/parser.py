"""Command-line front end: ``@parser.wrap()`` turns ``main(cfg: TrainPipelineConfig)`` into a CLI.

``--config_path=<json | dir | repo@rev>`` selects the base file, every other ``--a.b.c=value`` is a dotted
override.  Arguments injected by distributed launchers (``--local_rank`` …) are dropped, and
``--accelerate-config <yaml>`` is accepted and mapped onto ``distributed.*`` for compatibility with the
reference's launcher (OpenTau ``src/opentau/configs/parser.py:286-400``, ``scripts/launch.py:30-99``).
"""

from __future__ import annotations

import functools
import importlib
import inspect
import sys
from typing import Any, Callable

LAUNCHER_ARGS = ("--local_rank", "--local-rank", "--node_rank", "--nproc_per_node", "--master_addr", "--master_port")


def filter_distributed_args(argv: list[str]) -> list[str]:
    out, skip = [], False
    for a in argv:
        if skip:
            skip = False
            continue
        key = a.split("=", 1)[0]
        if key in LAUNCHER_ARGS:
            skip = "=" not in a
            continue
        out.append(a)
    return out


def get_cli_value(argv: list[str], name: str) -> str | None:
    for i, a in enumerate(argv):
        if a.startswith(f"--{name}="):
            return a.split("=", 1)[1]
        if a == f"--{name}" and i + 1 < len(argv):
            return argv[i + 1]
    return None


def strip_arg(argv: list[str], name: str) -> list[str]:
    out, skip = [], False
    for a in argv:
        if skip:
            skip = False
            continue
        if a.startswith(f"--{name}="):
            continue
        if a == f"--{name}":
            skip = True
            continue
        out.append(a)
    return out


def load_plugin(path: str) -> None:
    """Imports a user plugin package so that it can register policies / envs / optimizers."""
    try:
        importlib.import_module(path)
    except ModuleNotFoundError as e:
        raise ModuleNotFoundError(f"plugin {path!r} could not be imported: {e}") from e


def describe_fields(config_cls, prefix: str = "", depth: int = 0, max_depth: int = 2) -> list[str]:
    """``--a.b=<type> (default)`` lines for the help text: the dataclass's fields, nested dataclasses two levels deep."""
    import dataclasses
    import typing
    lines: list[str] = []
    if not dataclasses.is_dataclass(config_cls):
        return lines
    try:
        hints = typing.get_type_hints(config_cls)
    except Exception:  # noqa: BLE001 - forward references that cannot be resolved here
        hints = {}
    for f in dataclasses.fields(config_cls):
        tp = hints.get(f.name, f.type)
        inner = next((a for a in typing.get_args(tp) if dataclasses.is_dataclass(a)), None)
        nested = tp if dataclasses.is_dataclass(tp) else inner
        name = f"{prefix}{f.name}"
        if nested is not None and depth < max_depth:
            lines.append(f"  --{name}.*")
            lines += describe_fields(nested, f"{name}.", depth + 1, max_depth)
            continue
        if f.default is not dataclasses.MISSING:
            default = repr(f.default)
        elif f.default_factory is not dataclasses.MISSING:      # type: ignore[misc]
            default = "<factory>"
        else:
            default = "<required>"
        tname = getattr(tp, "__name__", None) or str(tp).replace("typing.", "")
        lines.append(f"  --{name}=<{tname}>  (default {default})")
    return lines


def print_help(config_cls, doc: str | None = None) -> None:
    prog = sys.argv[0].rsplit("/", 1)[-1]
    print(f"usage: {prog} [--config_path=<json | dir | repo@rev>] [--<field>=<value> ...]\n")
    if doc:
        print(doc.strip() + "\n")
    print(f"fields of {config_cls.__name__} (dotted overrides; nested blocks as --a.b=value):")
    print("\n".join(describe_fields(config_cls)))
    print("\nalso accepted: --plugin=<package>, --accelerate-config=<yaml>; launcher arguments (--local_rank ...) are ignored")


def _build(config_cls, raw: dict[str, Any]):
    """``config_cls.from_dict`` where the class has one (pipeline configs), the generic decoder otherwise."""
    if hasattr(config_cls, "from_dict"):
        return config_cls.from_dict(raw)
    from .codec import decode
    return decode(config_cls, raw, config_cls.__name__)


def parse_config(config_cls, argv: list[str] | None = None, doc: str | None = None):
    argv = filter_distributed_args(list(sys.argv[1:] if argv is None else argv))
    if any(a in ("-h", "--help") for a in argv):
        print_help(config_cls, doc)
        raise SystemExit(0)
    plugin = get_cli_value(argv, "plugin")
    if plugin:
        load_plugin(plugin)
        argv = strip_arg(argv, "plugin")
    accel = get_cli_value(argv, "accelerate-config") or get_cli_value(argv, "accelerate_config")
    argv = strip_arg(strip_arg(argv, "accelerate-config"), "accelerate_config")
    config_path = get_cli_value(argv, "config_path")
    argv = strip_arg(argv, "config_path")
    if config_path is not None:
        if hasattr(config_cls, "from_pretrained"):
            cfg = config_cls.from_pretrained(config_path, cli_overrides=argv)
        else:
            from .codec import apply_overrides
            from .refs import load_json_with_refs
            cfg = _build(config_cls, apply_overrides(load_json_with_refs(config_path), argv))
    else:
        from .codec import apply_overrides, encode
        policy_path = get_cli_value(argv, "policy.path")
        raw: dict[str, Any] = apply_overrides({}, strip_arg(argv, "policy.path"))
        if policy_path is not None:
            # the policy block starts from the checkpoint's own configuration; dotted --policy.* overrides win
            from ..policies.factory import _import_all_configs
            from .policies import PreTrainedConfig
            _import_all_configs()                       # the registry of policy types fills on import
            merged = encode(PreTrainedConfig.from_pretrained(policy_path))
            merged.update({k: v for k, v in (raw.get("policy") or {}).items() if k != "type"})
            merged["pretrained_path"] = policy_path
            raw["policy"] = merged
        cfg = _build(config_cls, raw)
    if accel is not None and hasattr(cfg, "distributed"):
        from .default import DistributedConfig
        d = DistributedConfig.from_accelerate_yaml(accel)
        d.comm, d.tp, d.cp = cfg.distributed.comm, cfg.distributed.tp, cfg.distributed.cp
        cfg.distributed = d
    return cfg


def wrap(config_path: str | None = None) -> Callable:
    """Decorator: the wrapped function's first parameter annotation names the config class."""

    def deco(fn: Callable) -> Callable:
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if args or kwargs:
                return fn(*args, **kwargs)
            hints = inspect.get_annotations(fn, eval_str=True)
            first = next(iter(inspect.signature(fn).parameters))
            cfg = parse_config(hints[first], doc=sys.modules[fn.__module__].__doc__ or fn.__doc__)
            return fn(cfg)
        return inner
    return deco
