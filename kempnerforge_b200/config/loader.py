"""TOML preset + ``--section.key=value`` overrides -> ``JobConfig``.

Layering is defaults < TOML file < command line.  The merge happens on plain
nested dictionaries; a single recursive ``_convert`` then turns the merged tree
into typed dataclasses using each field's annotation, so every ``__post_init__``
sees final values exactly once.  Unknown keys are errors at every depth.

Parity: kempnerforge/config/loader.py:26-328 (type coercion for
Optional/Literal/Enum/tuple/list-of-dataclass/dict, ``arch``-dispatched ``[vlm]``
subclass, CLI grammar: ``--a.b=v``, bare ``--a.b`` means true, values parsed as
Python literals with a fallback to the raw string).
"""

from __future__ import annotations

import ast
import dataclasses
import enum
import tomllib
import types
import typing
from pathlib import Path
from typing import Any

from kempnerforge_b200.config.job import JobConfig
from kempnerforge_b200.config.vlm import VLMConfig


class ConfigError(ValueError):
    """A key or value in a preset / override could not be applied."""


# --------------------------------------------------------------------------- typed conversion
def _hints(cls: type) -> dict[str, Any]:
    return typing.get_type_hints(cls)


def _convert(value: Any, annot: Any, where: str) -> Any:
    """Coerce ``value`` (TOML / literal data) to the annotated type ``annot``."""
    origin = typing.get_origin(annot)

    if annot is Any:
        return value
    if origin in (typing.Union, types.UnionType):
        options = typing.get_args(annot)
        if value is None or (isinstance(value, str) and value.lower() in ("none", "null")):
            if type(None) in options:
                return None
        errors = []
        for opt in options:
            if opt is type(None):
                continue
            try:
                return _convert(value, opt, where)
            except (ConfigError, ValueError, TypeError) as exc:  # try the next member
                errors.append(str(exc))
        raise ConfigError(f"{where}: cannot convert {value!r} to {annot}: {errors}")
    if origin is typing.Literal:
        allowed = typing.get_args(annot)
        if value not in allowed:
            raise ConfigError(f"{where}: {value!r} is not one of {allowed}")
        return value
    if origin in (list, typing.List):
        (item_t,) = typing.get_args(annot) or (Any,)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{where}: expected a list, got {type(value).__name__}")
        return [_convert(v, item_t, f"{where}[{i}]") for i, v in enumerate(value)]
    if origin in (tuple, typing.Tuple):
        args = typing.get_args(annot)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{where}: expected a sequence, got {type(value).__name__}")
        if len(args) == 2 and args[1] is Ellipsis:
            return tuple(_convert(v, args[0], f"{where}[{i}]") for i, v in enumerate(value))
        if args and len(args) != len(value):
            raise ConfigError(f"{where}: expected {len(args)} items, got {len(value)}")
        return tuple(
            _convert(v, args[i] if args else Any, f"{where}[{i}]") for i, v in enumerate(value)
        )
    if origin in (dict, typing.Dict):
        k_t, v_t = typing.get_args(annot) or (Any, Any)
        if not isinstance(value, dict):
            raise ConfigError(f"{where}: expected a table, got {type(value).__name__}")
        return {
            _convert(k, k_t, where): _convert(v, v_t, f"{where}.{k}") for k, v in value.items()
        }
    if isinstance(annot, type):
        if dataclasses.is_dataclass(annot):
            if isinstance(value, annot):
                return value
            if not isinstance(value, dict):
                raise ConfigError(f"{where}: expected a table for {annot.__name__}")
            return _build_dataclass(annot, value, where)
        if issubclass(annot, enum.Enum):
            if isinstance(value, annot):
                return value
            if value is None:  # "--scheduler.name=none" reaches here as None: an enum may have a member of that name
                for member in annot:
                    if str(member.value).lower() in ("none", "null"):
                        return member
            try:
                return annot(value)
            except ValueError:
                names = [m.value for m in annot]
                raise ConfigError(f"{where}: {value!r} is not one of {names}") from None
        if annot is bool:
            if isinstance(value, bool):
                return value
            if isinstance(value, str) and value.lower() in ("true", "false"):
                return value.lower() == "true"
            raise ConfigError(f"{where}: expected a boolean, got {value!r}")
        if annot is int:
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise ConfigError(f"{where}: expected an integer, got {value!r}")
            if isinstance(value, float) and not value.is_integer():
                raise ConfigError(f"{where}: expected an integer, got {value!r}")
            return int(value)
        if annot is float:
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                if isinstance(value, str):
                    try:
                        return float(value)
                    except ValueError:
                        pass
                raise ConfigError(f"{where}: expected a number, got {value!r}")
            return float(value)
        if annot is str:
            if not isinstance(value, str):
                return str(value)
            return value
    return value


def _build_dataclass(cls: type, table: dict[str, Any], where: str) -> Any:
    # ``[vlm]`` is a discriminated union: pick the registered subclass for ``arch``
    if cls is VLMConfig or (isinstance(cls, type) and issubclass(cls, VLMConfig)):
        arch = table.get("arch", "joint_decoder")
        from kempnerforge_b200.config.registry import registry

        if not registry.has("vlm_config", arch):
            raise ConfigError(
                f"Unknown vlm.arch: {arch!r}. Registered: {sorted(registry.list('vlm_config'))}."
            )
        cls = registry.get("vlm_config", arch)
    hints = _hints(cls)
    known = {f.name for f in dataclasses.fields(cls) if f.init}
    unknown = sorted(set(table) - known)
    if unknown:
        raise ConfigError(
            f"Unknown config keys {unknown} in [{where}] (valid keys: {sorted(known)})"
        )
    kwargs = {k: _convert(v, hints[k], f"{where}.{k}") for k, v in table.items()}
    return cls(**kwargs)


# --------------------------------------------------------------------------- CLI overrides
def _literal(text: str) -> Any:
    low = text.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        return text


def parse_cli_overrides(args: list[str]) -> dict[str, Any]:
    """``["--train.seq_len=128", "--optimizer.fused"]`` -> nested dict."""
    tree: dict[str, Any] = {}
    for raw in args:
        if not raw.startswith("--"):
            if "=" in raw:   # looks like an override that lost its dashes: say so instead of dropping it
                raise ConfigError(f"override {raw!r} must look like --section.key=value")
            continue         # positional arguments (the preset path of a command line) are not overrides
        body = raw[2:]
        dotted, has_eq, text = body.partition("=")
        value = _literal(text) if has_eq else True
        parts = dotted.split(".")
        if len(parts) < 2 or not all(parts):
            raise ConfigError(f"override {raw!r} needs a section and a key (--section.key=value)")
        node = tree
        for part in parts[:-1]:
            nxt = node.setdefault(part, {})
            if not isinstance(nxt, dict):
                raise ConfigError(f"override {raw!r} descends into a non-table value")
            node = nxt
        node[parts[-1]] = value
    return tree


_parse_cli_overrides = parse_cli_overrides  # alias kept for scripts that used the private name


def _deep_merge(base: dict[str, Any], top: dict[str, Any]) -> dict[str, Any]:
    out = dict(base)
    for key, val in top.items():
        if isinstance(val, dict) and isinstance(out.get(key), dict):
            out[key] = _deep_merge(out[key], val)
        else:
            out[key] = val
    return out


# --------------------------------------------------------------------------- public surface
def config_from_dict(tree: dict[str, Any]) -> JobConfig:
    """Build a validated ``JobConfig`` from a nested dictionary of sections."""
    for section, table in tree.items():
        if not isinstance(table, dict):
            raise ConfigError(f"top-level key {section!r} must be a table")
    return _build_dataclass(JobConfig, tree, "job")


def load_toml(path: str | Path) -> dict[str, Any]:
    p = Path(path)
    if not p.is_file():
        raise FileNotFoundError(f"Config file not found: {p}")
    with p.open("rb") as fh:
        return tomllib.load(fh)


def load_config(path: str | Path | None = None, cli_args: list[str] | None = None, *,
                config_path: str | Path | None = None) -> JobConfig:
    """Defaults, overlaid by the TOML preset at ``path`` (also ``config_path=``), overlaid by ``cli_args``."""
    path = path if path is not None else config_path
    tree: dict[str, Any] = load_toml(path) if path is not None else {}
    if cli_args:
        tree = _deep_merge(tree, parse_cli_overrides(list(cli_args)))
    return config_from_dict(tree)


def config_to_dict(cfg: Any) -> Any:
    """Plain-data view of a config (enums -> values); inverse of ``config_from_dict``."""
    if dataclasses.is_dataclass(cfg) and not isinstance(cfg, type):
        return {
            f.name: config_to_dict(getattr(cfg, f.name))
            for f in dataclasses.fields(cfg)
            if getattr(cfg, f.name) is not None
        }
    if isinstance(cfg, enum.Enum):
        return cfg.value
    if isinstance(cfg, (list, tuple)):
        return [config_to_dict(v) for v in cfg]
    if isinstance(cfg, dict):
        return {k: config_to_dict(v) for k, v in cfg.items()}
    return cfg
