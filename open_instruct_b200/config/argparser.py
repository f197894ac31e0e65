"""Dataclass-driven command line / YAML parser with the calling convention of the reference's
``ArgumentParserPlus`` (``open_instruct/utils.py:681-757``):

    parser = ArgumentParserPlus((FlatArguments, TokenizerConfig))
    args, tc = parser.parse()            # `script.py cfg.yaml --k v ...`  or plain CLI

Written from scratch on ``argparse`` (no HfArgumentParser dependency):
* every dataclass field becomes ``--name``; ``bool`` fields accept ``--flag``, ``--flag true|false``
  and ``--no_flag``; ``list[...]`` fields take one or more values; ``Literal`` becomes ``choices``;
  ``dict`` fields (and ``dict | str``) accept a JSON string; ``X | None`` accepts the string ``none``;
* ``parse()``: if the first positional argument ends in ``.yaml``/``.yml``/``.json`` it is loaded first
  and the remaining ``--k v`` / ``--k=v`` options override it;
* ``set_defaults(**kw)`` changes per-entry-point defaults before parsing;
* unknown keys in a config file are an error (typos must not pass silently).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import sys
import types
import typing
from enum import Enum
from typing import Any, Literal, Union, get_args, get_origin


def _str2bool(v):
    if isinstance(v, bool):
        return v
    s = str(v).lower()
    if s in ("1", "true", "t", "yes", "y", "on"):
        return True
    if s in ("0", "false", "f", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def _unwrap_optional(tp):
    """(inner type, is_optional) for ``X | None`` / ``Optional[X]``; unions of several non-None types stay."""
    origin = get_origin(tp)
    if origin is Union or origin is types.UnionType:
        args = [a for a in get_args(tp) if a is not type(None)]
        optional = len(args) != len(get_args(tp))
        if len(args) == 1:
            return args[0], optional
        return tuple(args), optional
    return tp, False


def _make_converter(tp):
    """String -> value converter for a (non-list) annotation."""
    inner, optional = _unwrap_optional(tp)

    def conv(s):
        if optional and isinstance(s, str) and s.lower() in ("none", "null"):
            return None
        cands = inner if isinstance(inner, tuple) else (inner,)
        last = None
        # try the most specific types first (dict before str, int before float before str)
        order = sorted(cands, key=lambda t: {dict: 0, bool: 1, int: 2, float: 3}.get(t, 9 if t is str else 5))
        for t in order:
            try:
                if t is dict or get_origin(t) is dict:
                    if isinstance(s, dict):
                        return s
                    val = json.loads(s)
                    if not isinstance(val, dict):
                        raise ValueError("not a JSON object")
                    return val
                if t is bool:
                    return _str2bool(s)
                if get_origin(t) is Literal:
                    for lit in get_args(t):
                        if str(lit) == str(s):
                            return lit
                    raise ValueError(f"{s!r} not in {get_args(t)}")
                if isinstance(t, type) and issubclass(t, Enum):
                    return t(s) if not isinstance(s, t) else s
                if t is Any:
                    return s
                return t(s)
            except (ValueError, TypeError, json.JSONDecodeError, argparse.ArgumentTypeError) as e:
                last = e
        raise argparse.ArgumentTypeError(str(last))

    return conv


class ArgumentParserPlus(argparse.ArgumentParser):
    def __init__(self, dataclass_types, **kwargs):
        kwargs.setdefault("formatter_class", argparse.ArgumentDefaultsHelpFormatter)
        kwargs.setdefault("allow_abbrev", False)
        super().__init__(**kwargs)
        if dataclasses.is_dataclass(dataclass_types):
            dataclass_types = (dataclass_types,)
        self.dataclass_types = tuple(dataclass_types)
        self._field_owner: dict[str, type] = {}
        self._fields: dict[str, dataclasses.Field] = {}
        self._hints: dict[str, Any] = {}
        for dt in self.dataclass_types:
            hints = typing.get_type_hints(dt)
            for f in dataclasses.fields(dt):
                if not f.init:
                    continue
                if f.name in self._fields:
                    raise ValueError(f"field {f.name} is defined by two config dataclasses")
                self._field_owner[f.name] = dt
                self._fields[f.name] = f
                self._hints[f.name] = hints[f.name]
                self._add_field(f, hints[f.name])

    # ------------------------------------------------------------------ argparse wiring
    def _add_field(self, f: dataclasses.Field, tp) -> None:
        name = f"--{f.name}"
        helptext = (f.metadata or {}).get("help")
        kw: dict[str, Any] = {"dest": f.name, "help": helptext}
        default = dataclasses.MISSING
        if f.default is not dataclasses.MISSING:
            default = f.default
        elif f.default_factory is not dataclasses.MISSING:  # type: ignore[misc]
            default = f.default_factory()  # type: ignore[misc]
        required = default is dataclasses.MISSING
        inner, _ = _unwrap_optional(tp)
        origin = get_origin(inner) if not isinstance(inner, tuple) else None
        if inner is bool:
            kw.update(type=_str2bool, nargs="?", const=True)
            if not required:
                kw["default"] = default
            self.add_argument(name, required=required, **kw)
            self.add_argument(f"--no_{f.name}", dest=f.name, action="store_false", help=argparse.SUPPRESS,
                              default=argparse.SUPPRESS)
            return
        if origin in (list, tuple) or inner in (list, tuple):
            elem = (get_args(inner) or (str,))[0]
            kw.update(nargs="*", type=_make_converter(elem))
        elif origin is Literal:
            kw.update(type=_make_converter(inner), choices=list(get_args(inner)))
        else:
            kw.update(type=_make_converter(tp))
        if not required:
            kw["default"] = default
        self.add_argument(name, required=required, **kw)

    def set_defaults(self, **kwargs):  # noqa: D401 - same name as argparse on purpose
        for k in kwargs:
            if k not in self._fields:
                raise KeyError(f"set_defaults: unknown field {k}")
        for action in self._actions:
            if action.dest in kwargs and action.option_strings and not action.option_strings[0].startswith("--no_"):
                action.default = kwargs[action.dest]
                action.required = False
        super().set_defaults(**kwargs)

    # ------------------------------------------------------------------ parsing
    def _build(self, namespace: argparse.Namespace):
        outs = []
        for dt in self.dataclass_types:
            kw = {f.name: getattr(namespace, f.name) for f in dataclasses.fields(dt) if f.init}
            outs.append(dt(**kw))
        return tuple(outs)

    def parse_args_into_dataclasses(self, args=None):
        ns = self.parse_args(args)
        return self._build(ns)

    def parse_dict(self, cfg: dict, overrides=None, allow_extra_keys: bool = False):
        """Build the dataclasses from a mapping (config file) plus CLI-style overrides."""
        unknown = [k for k in cfg if k not in self._fields]
        if unknown and not allow_extra_keys:
            raise ValueError(f"unknown config keys: {sorted(unknown)}")
        cfg = {k: v for k, v in cfg.items() if k in self._fields}
        argv = []
        for k, v in cfg.items():
            tp = self._hints[k]
            inner, _ = _unwrap_optional(tp)
            if v is None:
                argv += [f"--{k}", "none"]
            elif isinstance(v, bool):
                argv += [f"--{k}", str(v).lower()]
            elif isinstance(v, (list, tuple)):
                argv += [f"--{k}", *[json.dumps(x) if isinstance(x, dict) else str(x) for x in v]]
            elif isinstance(v, dict):
                argv += [f"--{k}", json.dumps(v)]
            else:
                argv += [f"--{k}", str(v)]
        return self.parse_args_into_dataclasses(argv + list(overrides or []))

    def parse_yaml_and_args(self, path: str, overrides=None, allow_extra_keys: bool = False):
        import yaml

        with open(path) as fh:
            cfg = json.load(fh) if path.endswith(".json") else (yaml.safe_load(fh) or {})
        return self.parse_dict(cfg, overrides, allow_extra_keys)

    def parse(self, argv=None, allow_extra_keys: bool = False):
        """`script.py config.yaml [--k v ...]` or plain CLI.  Returns one dataclass or a tuple."""
        argv = list(sys.argv[1:] if argv is None else argv)
        if argv and not argv[0].startswith("-") and argv[0].rsplit(".", 1)[-1] in ("yaml", "yml", "json"):
            out = self.parse_yaml_and_args(argv[0], argv[1:], allow_extra_keys)
        else:
            out = self.parse_args_into_dataclasses(argv)
        return out[0] if len(out) == 1 else out
