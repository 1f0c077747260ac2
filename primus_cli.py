"""Console-script locator of the bash launcher: finds ``runner/primus-cli`` next to this file (source tree) or inside
an installed package layout and replaces the process with ``bash runner/primus-cli <args>``.  Standard library only.
``PRIMUS_BASH`` overrides the shell.  (Role of the reference's primus_cli.py:27-109.)"""
import os
import shutil
import sys


def find_launcher() -> str:
    here = os.path.dirname(os.path.abspath(__file__))
    for root in (here, os.path.join(here, "primus_b200"), os.path.dirname(here)):
        cand = os.path.join(root, "runner", "primus-cli")
        if os.path.isfile(cand):
            return cand
    raise FileNotFoundError("runner/primus-cli not found next to primus_cli.py")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    bash = os.environ.get("PRIMUS_BASH") or shutil.which("bash")
    if not bash:
        print("primus-cli: bash not found (set PRIMUS_BASH)", file=sys.stderr)
        return 127
    launcher = find_launcher()
    os.execv(bash, [bash, launcher, *argv])
    return 0  # not reached


if __name__ == "__main__":
    sys.exit(main())
