"""Starts a command of longbow_quarrel_b200 from this checkout, whatever the working
directory is: the checkout's root goes to the front of the import path (in place of
this folder), so a package of the same name elsewhere is never picked up."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path[0] = str(ROOT)

if __name__ == "__main__":
    command, sys.argv = sys.argv[1], [sys.argv[1]] + sys.argv[2:]
    if command == "trace_run":
        from longbow_quarrel_b200.trace import main
    elif command == "quarrel":
        from longbow_quarrel_b200.cli import main
    else:
        raise SystemExit(f"unknown command {command!r}")
    sys.exit(main(sys.argv[1:]))
