"""Command lines for the external profilers (tools/nsys.sh of the reference, and its Nsight
Compute counterpart used for the kernels of this package).

`python -m zml_b200.profiling.wrappers nsys -- <program> [args...]` execs the profiler around a
program; the argument lists are also importable for tests and notebooks.  `ZML_NSYS_ARGS` /
`ZB_NCU_ARGS` replace the default arguments, as `ZML_NSYS_ARGS` does in the reference.  Every
`ncu` line carries `--clock-control none`: the profiler must not lock the clocks of a GPU that
other jobs share.
"""
from __future__ import annotations

import os
import shlex
import shutil
import sys
from typing import Optional, Sequence

NSYS_DEFAULT = ["profile", "-t", "cuda,nvtx,cublas,cudnn,osrt", "--inherit-environment=true", "--cuda-memory-usage", "true",
                "--cuda-event-trace=false", "--cuda-graph-trace=node"]
NCU_DEFAULT = ["--set", "full", "--clock-control", "none"]


def nsys_command(program: Sequence[str], output: Optional[str] = None) -> list[str]:
    args = shlex.split(os.environ["ZML_NSYS_ARGS"]) if os.environ.get("ZML_NSYS_ARGS") else list(NSYS_DEFAULT)
    if output:
        args += ["-o", output]
    return ["nsys", *args, *program]


def ncu_command(program: Sequence[str], kernel_regex: Optional[str] = None, launch_count: int = 3, skip: int = 0,
                output: Optional[str] = None, metrics: Optional[Sequence[str]] = None) -> list[str]:
    """One kernel, a few launches, a small case - the capture must end by itself."""
    if os.environ.get("ZB_NCU_ARGS"):
        args = shlex.split(os.environ["ZB_NCU_ARGS"])
        if "--clock-control" not in args:
            args += ["--clock-control", "none"]
    elif metrics:
        args = ["--metrics", ",".join(metrics), "--clock-control", "none"]
    else:
        args = list(NCU_DEFAULT)
    if kernel_regex:
        args += ["-k", f"regex:{kernel_regex}"]
    if skip:
        args += ["-s", str(skip)]
    args += ["-c", str(launch_count)]
    if output:
        args += ["-o", output]
    return ["ncu", *args, *program]


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 3 or argv[0] not in ("nsys", "ncu") or "--" not in argv:
        print("usage: python -m zml_b200.profiling.wrappers {nsys|ncu} [-k REGEX] [-o OUT] -- <program> [args...]", file=sys.stderr)
        return 1
    tool, rest = argv[0], argv[1:]
    sep = rest.index("--")
    opts, program = rest[:sep], rest[sep + 1:]
    out = opts[opts.index("-o") + 1] if "-o" in opts else None
    if tool == "nsys":
        cmd = nsys_command(program, out)
    else:
        cmd = ncu_command(program, opts[opts.index("-k") + 1] if "-k" in opts else None, output=out)
    if shutil.which(cmd[0]) is None:
        print(f"{cmd[0]} is not installed; the command would be:\n  {shlex.join(cmd)}", file=sys.stderr)
        return 127
    env = dict(os.environ, ZB_SKIP_BUILTIN_PROFILER="true")
    os.execvpe(cmd[0], cmd, env)
    return 0


if __name__ == "__main__":
    sys.exit(main())
