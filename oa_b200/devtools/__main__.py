"""`python -m oa_b200.devtools gate` runs every source gate (architecture, generated-table drift, kernel audit); the other
sub-commands forward to their modules: archcheck, autogen, evidence, determinism."""
import sys

from . import archcheck, autogen, determinism, evidence


def main(argv) -> int:
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "gate":
        rc = archcheck.main([])
        rc |= autogen.main(["--check"])
        rc |= autogen.main(["--audit"])
        return rc
    mods = {"archcheck": archcheck, "autogen": autogen, "evidence": evidence, "determinism": determinism}
    if cmd not in mods:
        print(f"unknown sub-command {cmd!r}: gate, " + ", ".join(mods))
        return 2
    return mods[cmd].main(rest)


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
