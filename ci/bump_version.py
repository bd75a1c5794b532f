#!/usr/bin/env python3
"""Set the release version in the two places that carry it:
``awex_b200/version.py`` (``__version__``) and ``pyproject.toml`` (``version``).

    python ci/bump_version.py 0.2.0
"""

import argparse
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SEMVER = re.compile(r"\d+\.\d+\.\d+")


def rewrite(path: Path, pattern: str, replacement: str) -> None:
    text = path.read_text()
    new, count = re.subn(pattern, replacement, text, count=1, flags=re.MULTILINE)
    if count != 1:
        raise SystemExit(f"no version line found in {path}")
    path.write_text(new)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("version", help="x.y.z")
    ap.add_argument("--root", type=Path, default=ROOT)
    args = ap.parse_args(argv)
    if not SEMVER.fullmatch(args.version):
        raise SystemExit(f"version must look like x.y.z, got {args.version!r}")
    rewrite(args.root / "awex_b200" / "version.py", r'^__version__ = "[^"]+"$', f'__version__ = "{args.version}"')
    rewrite(args.root / "pyproject.toml", r'^version = "[^"]+"$', f'version = "{args.version}"')
    print(args.version)
    return 0


if __name__ == "__main__":
    sys.exit(main())
