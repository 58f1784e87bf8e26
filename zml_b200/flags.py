"""Strict command-line flags driven by a dataclass.

Contract of the reference's `stdx.flags` (stdx/flags.zig:1-140): long options only,
``--key=value`` syntax (never ``--key value``), booleans are bare ``--flag``, optional
fields default to None, enums are given by name, a nested dataclass field called
``positional`` collects positional arguments in order, a ``help`` class attribute
answers ``-h`` / ``--help``, subcommands are a mapping name -> dataclass, and unknown,
malformed or repeated options are fatal.  Field names use ``_`` in Python and ``-`` on
the command line (both spellings are accepted).
"""
from __future__ import annotations

import dataclasses
import enum
import sys
import typing
from typing import Any, Mapping, Optional, Sequence, Type, Union


class FlagsError(SystemExit):
    def __init__(self, message: str):
        super().__init__(1)
        self.message = message

    def __str__(self) -> str:
        return self.message


def fatal(message: str):
    """Prints `error: ...` to stderr and ends the process with exit code 1."""
    print(f"error: {message}", file=sys.stderr)
    raise FlagsError(message)


def _unwrap_optional(tp):
    origin = typing.get_origin(tp)
    if origin is Union or (hasattr(__import__("types"), "UnionType") and isinstance(tp, __import__("types").UnionType)):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0], True
    return tp, False


def _parse_value(name: str, tp, raw: str):
    tp, _ = _unwrap_optional(tp)
    if isinstance(tp, type) and issubclass(tp, enum.Enum):
        try:
            return tp[raw]
        except KeyError:
            fatal(f"{name}: expected one of {', '.join(m.name for m in tp)}, got '{raw}'")
    if tp is int:
        try:
            s = raw.replace("_", "")
            mult = 1
            for suf, m in (("KiB", 1 << 10), ("MiB", 1 << 20), ("GiB", 1 << 30), ("TiB", 1 << 40)):
                if s.endswith(suf):
                    s, mult = s[: -len(suf)], m
            return int(s, 0) * mult
        except ValueError:
            fatal(f"{name}: expected an integer value, but found '{raw}'")
    if tp is float:
        try:
            return float(raw)
        except ValueError:
            fatal(f"{name}: expected a number, but found '{raw}'")
    if tp is str or tp is Any:
        if raw == "":
            fatal(f"{name}: argument is empty")
        return raw
    fatal(f"{name}: unsupported flag type {tp}")


def _hints(cls) -> dict:
    return typing.get_type_hints(cls)


def parse_flags(argv: Sequence[str], cls: Type):
    """Parses `argv` (without the program name) into dataclass `cls`."""
    if cls is None:
        if argv:
            fatal(f"unexpected argument: '{argv[0]}'")
        return None
    hints = _hints(cls)
    fields = {f.name: f for f in dataclasses.fields(cls)}
    pos_cls = None
    if "positional" in fields:
        pos_cls = hints["positional"]
        if not dataclasses.is_dataclass(pos_cls):
            raise TypeError("`positional` must be a dataclass")
    values: dict[str, Any] = {}
    pos_values: list[str] = []
    parsing_flags = True
    for arg in argv:
        if parsing_flags and arg in ("-h", "--help") and hasattr(cls, "help"):
            print(cls.help)
            raise SystemExit(0)
        if parsing_flags and arg == "--":
            parsing_flags = False
            continue
        if parsing_flags and arg.startswith("--"):
            body = arg[2:]
            key, eq, raw = body.partition("=")
            name = key.replace("-", "_")
            if name == "positional" or name not in fields:
                fatal(f"unexpected argument: '{arg}'")
            if name in values:
                fatal(f"--{key}: duplicate argument")
            tp, _ = _unwrap_optional(hints[name])
            if tp is bool:
                if eq:
                    if raw not in ("true", "false"):
                        fatal(f"--{key}: expected true or false, got '{raw}'")
                    values[name] = raw == "true"
                else:
                    values[name] = True
            else:
                if not eq:
                    fatal(f"--{key}: expected value separator '='")
                values[name] = _parse_value(f"--{key}", hints[name], raw)
            continue
        if parsing_flags and arg.startswith("-") and arg != "-":
            fatal(f"unexpected argument: '{arg}' (only long --options are accepted)")
        if pos_cls is None:
            fatal(f"unexpected argument: '{arg}'")
        pos_values.append(arg)
    for name, f in fields.items():
        if name == "positional" or name in values:
            continue
        _, optional = _unwrap_optional(hints[name])
        if f.default is not dataclasses.MISSING:
            values[name] = f.default
        elif f.default_factory is not dataclasses.MISSING:  # type: ignore[misc]
            values[name] = f.default_factory()               # type: ignore[misc]
        elif optional:
            values[name] = None
        elif _unwrap_optional(hints[name])[0] is bool:
            values[name] = False
        else:
            fatal(f"--{name.replace('_', '-')}: argument is required")
    if pos_cls is not None:
        pf = dataclasses.fields(pos_cls)
        ph = _hints(pos_cls)
        if len(pos_values) > len(pf):
            fatal(f"unexpected argument: '{pos_values[len(pf)]}'")
        kw = {}
        for i, f in enumerate(pf):
            if i < len(pos_values):
                kw[f.name] = _parse_value(f"<{f.name}>", ph[f.name], pos_values[i])
            elif f.default is not dataclasses.MISSING:
                kw[f.name] = f.default
            elif _unwrap_optional(ph[f.name])[1]:
                kw[f.name] = None
            else:
                fatal(f"<{f.name}>: argument is required")
        values["positional"] = pos_cls(**kw)
    return cls(**values)


def parse_commands(argv: Sequence[str], commands: Mapping[str, Optional[Type]], help_text: Optional[str] = None):
    """Subcommand dispatch: returns (name, parsed flags)."""
    if not argv:
        fatal(f"subcommand required, expected {' or '.join(commands)}")
    first = argv[0]
    if first in ("-h", "--help") and help_text is not None:
        print(help_text)
        raise SystemExit(0)
    if first not in commands:
        fatal(f"unknown subcommand: '{first}'")
    return first, parse_flags(argv[1:], commands[first])


def parse(argv: Optional[Sequence[str]], spec, help_text: Optional[str] = None):
    """`spec` is a dataclass (flags) or a mapping of subcommands.  argv=None uses sys.argv[1:]."""
    argv = list(sys.argv[1:] if argv is None else argv)
    if isinstance(spec, Mapping):
        return parse_commands(argv, spec, help_text)
    return parse_flags(argv, spec)
