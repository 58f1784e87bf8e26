import enum
from dataclasses import dataclass
from typing import Optional

import pytest

from zml_b200 import flags


class Backend(enum.Enum):
    auto = 0
    cuda_fa2 = 1


@dataclass
class Positional:
    path: str
    count: int = 1


@dataclass
class Args:
    model: str
    positional: Positional
    prompt: Optional[str] = None
    seqlen: int = 2048
    topk: int = 1
    backend: Backend = Backend.auto
    profile: bool = False
    help = "usage: llm --model=<path> [--prompt=..] <path>"


def test_parses_key_value_bools_enums_positional():
    a = flags.parse(["--model=/m", "--seqlen=4096", "--backend=cuda_fa2", "--profile", "in.bin", "3"], Args)
    assert a.model == "/m" and a.seqlen == 4096 and a.backend is Backend.cuda_fa2 and a.profile
    assert a.prompt is None and a.positional.path == "in.bin" and a.positional.count == 3
    b = flags.parse(["--model=/m", "x", "--topk=4"], Args)
    assert b.topk == 4 and b.positional.count == 1 and not b.profile
    assert flags.parse(["--model=x", "p", "--seqlen=2KiB"], Args).seqlen == 2048


@pytest.mark.parametrize("argv,msg", [
    (["--model", "/m", "p"], "expected value separator"),
    (["--model=/m", "--model=/n", "p"], "duplicate"),
    (["--model=/m", "--nope=1", "p"], "unexpected argument"),
    (["p"], "required"),
    (["--model=/m"], "required"),
    (["--model=/m", "p", "1", "extra"], "unexpected argument"),
    (["--model=/m", "--seqlen=abc", "p"], "integer"),
    (["--model=/m", "--backend=zzz", "p"], "expected one of"),
    (["--model=/m", "-x", "p"], "only long"),
    (["--model=", "p"], "empty"),
])
def test_fatal_errors(argv, msg):
    with pytest.raises(flags.FlagsError) as e:
        flags.parse(argv, Args)
    assert msg in str(e.value)


def test_help_and_subcommands(capsys):
    with pytest.raises(SystemExit) as e:
        flags.parse(["--help"], Args)
    assert e.value.code == 0 and "usage: llm" in capsys.readouterr().out

    @dataclass
    class Cat:
        positional: Positional

    name, parsed = flags.parse(["cat", "file"], {"cat": Cat, "tree": None})
    assert name == "cat" and parsed.positional.path == "file"
    assert flags.parse(["tree"], {"cat": Cat, "tree": None}) == ("tree", None)
    with pytest.raises(flags.FlagsError):
        flags.parse(["rm"], {"cat": Cat, "tree": None})
    with pytest.raises(flags.FlagsError):
        flags.parse([], {"cat": Cat, "tree": None})
