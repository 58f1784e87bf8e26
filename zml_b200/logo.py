"""Start-up banner of the command-line tools: block letters with a colour gradient, written with ANSI escapes when
the terminal takes them (the reference prints its own art the same way, zml/logo.zig; examples/llm/main.zig:201-206).

`detect_color_support` follows the usual conventions: `NO_COLOR` switches colour off, `CLICOLOR_FORCE` forces it on
for a pipe, `COLORTERM=truecolor|24bit` selects 24-bit colour, a `TERM` with `256color` the 256-colour palette.
"""
from __future__ import annotations

import os
import sys
from typing import Mapping, Optional, TextIO

NO_COLOR, ANSI_256, TRUE_COLOR = "no_color", "256", "true_color"

# name -> (24-bit r, g, b; xterm-256 index)
PALETTE = {"cyan": ((0, 255, 255), 51), "sky": ((0, 221, 255), 45), "blue": ((135, 143, 255), 105),
           "violet": ((215, 90, 219), 170), "pink": ((255, 95, 175), 205), "shine": ((255, 255, 255), 231)}

# Six rows per letter; every block shares the row count.  "zb200" in box-drawing block letters.
_BLOCKS = [
    ("cyan", ["███████╗", "╚══███╔╝", "  ███╔╝ ", " ███╔╝  ", "███████╗", "╚══════╝"]),
    ("sky", ["██████╗ ", "██╔══██╗", "██████╔╝", "██╔══██╗", "██████╔╝", "╚═════╝ "]),
    ("blue", ["██████╗ ", "╚════██╗", " █████╔╝", "██╔═══╝ ", "███████╗", "╚══════╝"]),
    ("violet", [" ██████╗ ", "██╔═████╗", "██║██╔██║", "████╔╝██║", "╚██████╔╝", " ╚═════╝ "]),
    ("pink", [" ██████╗ ", "██╔═████╗", "██║██╔██║", "████╔╝██║", "╚██████╔╝", " ╚═════╝ "]),
]
_SHINE = set("╔╗╚╝═║")


def detect_color_support(stream: Optional[TextIO] = None, env: Optional[Mapping[str, str]] = None) -> str:
    env = os.environ if env is None else env
    stream = sys.stdout if stream is None else stream
    if env.get("NO_COLOR"):
        return NO_COLOR
    is_tty = bool(getattr(stream, "isatty", lambda: False)())
    if not is_tty and not env.get("CLICOLOR_FORCE"):
        return NO_COLOR
    if env.get("TERM", "") == "dumb":
        return NO_COLOR
    if env.get("COLORTERM", "").lower() in ("truecolor", "24bit"):
        return TRUE_COLOR
    return ANSI_256 if "256color" in env.get("TERM", "") or env.get("CLICOLOR_FORCE") else NO_COLOR


def escape(color: str, support: str) -> str:
    if support == NO_COLOR:
        return ""
    if color == "reset":
        return "\x1b[0m"
    (r, g, b), idx = PALETTE[color]
    return f"\x1b[38;2;{r};{g};{b}m" if support == TRUE_COLOR else f"\x1b[38;5;{idx}m"


def write_row(out: TextIO, text: str, color: str, support: str, rtrim: bool = False) -> None:
    """One row of one block: the fill in `color`, the box-drawing edges in the shine colour."""
    if rtrim:
        text = text.rstrip()
    if not text:
        return
    shiny = None
    for ch in text:
        want = ch in _SHINE
        if want != shiny:
            out.write(escape("shine" if want else color, support))
            shiny = want
        out.write(ch)
    out.write(escape("reset", support))


def write(out: Optional[TextIO] = None, support: Optional[str] = None, blocks=_BLOCKS) -> None:
    out = sys.stdout if out is None else out
    support = detect_color_support(out) if support is None else support
    rows = len(blocks[0][1])
    if any(len(b[1]) != rows for b in blocks):
        raise ValueError("logo blocks differ in their number of rows")
    for r in range(rows):
        visible = [i for i, (_, text) in enumerate(blocks) if text[r].strip()]
        if visible:
            for i, (color, text) in enumerate(blocks[:visible[-1] + 1]):
                write_row(out, text[r], color, support, rtrim=(i == visible[-1]))
        out.write("\n")


write_art = write
