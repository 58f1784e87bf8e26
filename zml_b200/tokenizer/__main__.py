"""Round-trip checker (zml/tokenizer/main.zig):
    python -m zml_b200.tokenizer --tokenizer=<path> --prompt=<text> [--expected=1,2,3] [--backend=homemade]
"""
import sys
from dataclasses import dataclass
from typing import Optional

from .. import flags
from . import Tokenizer


@dataclass
class Args:
    tokenizer: str
    prompt: str
    expected: Optional[str] = None
    backend: Optional[str] = None
    help = __doc__


def main(argv=None) -> int:
    a = flags.parse(argv, Args)
    tok = Tokenizer.from_file(a.tokenizer, a.backend)
    ids = tok.encode(a.prompt)
    print("tokens:", ids)
    print("decoded:", repr(tok.decode(ids)))
    if a.expected is not None:
        want = [int(x) for x in a.expected.split(",") if x.strip()]
        if want != ids:
            print(f"MISMATCH: expected {want}", file=sys.stderr)
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
