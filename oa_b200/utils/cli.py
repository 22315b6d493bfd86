"""OaCli: command-line front end of a configuration record with three-way precedence
(Source/Public/Oa/Core/Cli.h:1-140 of the reference: struct defaults < YAML file < arguments the user explicitly typed).

    @dataclass
    class TrainConfig:
        Lr: float = 3e-4
        Data: str = ""

    class TrainCli(OaCli):
        def __init__(self):
            super().__init__("train", "Train a model", TrainConfig())
            self.AddOption("--lr", "Lr", "learning rate")
            self.AddOption("--data,-d", "Data", "data file")
        def LoadYaml(self, node):                # node: the parsed YAML mapping
            self.Cfg.Lr = float(node.get("lr", self.Cfg.Lr))

    cli = TrainCli()
    if cli.Parse(sys.argv): run(cli.Cfg)

Flow, as in the reference: the record starts with its defaults; `--config / -c` is taken from the arguments before anything
else is parsed and the YAML file overwrites what it names; then only the options that appear on the command line overwrite
the record (an option's default never does).  `-v / --verbose` and `--help-all` are always there.
"""
from __future__ import annotations

import argparse
import dataclasses
import sys
from typing import Any, List, Optional, Sequence


class OaCli:
    def __init__(self, name: str, description: str, config: Any):
        self.Cfg = config
        self.ConfigPath = ""
        self.Verbose = 0
        self.Error = ""
        self._parser = argparse.ArgumentParser(prog=name, description=description, argument_default=argparse.SUPPRESS, add_help=True)
        self._parser.add_argument("-c", "--config", dest="_config", help="YAML config file")
        self._parser.add_argument("-v", "--verbose", dest="_verbose", type=int, help="verbose level (0-3)")
        self._parser.add_argument("--help-all", action="help", help="show all options")
        self._fields: List[str] = []

    # ---- options
    def AddOption(self, flags: str, field: str, help_text: str = "", choices: Optional[Sequence] = None) -> None:
        """`flags` is a comma-separated list ("--data,-d"); the option's type is that of the record's field."""
        if not hasattr(self.Cfg, field):
            raise AttributeError(f"configuration has no field {field!r}")
        cur = getattr(self.Cfg, field)
        names = [f.strip() for f in flags.split(",") if f.strip()]
        kw = {"dest": field, "help": f"{help_text} (default: {cur!r})"}
        if choices is not None:
            kw["choices"] = list(choices)
        if isinstance(cur, bool):
            self._parser.add_argument(*names, action=argparse.BooleanOptionalAction, **kw)
        elif isinstance(cur, (list, tuple)):
            elem = type(cur[0]) if len(cur) else str
            self._parser.add_argument(*names, nargs="*", type=elem, **kw)
        else:
            self._parser.add_argument(*names, type=type(cur) if cur is not None else str, **kw)
        self._fields.append(field)

    def AddFlag(self, flags: str, field: str, help_text: str = "") -> None:
        names = [f.strip() for f in flags.split(",") if f.strip()]
        self._parser.add_argument(*names, dest=field, action="store_true", help=help_text)
        self._fields.append(field)

    # ---- hooks
    def LoadYaml(self, node: dict) -> None:
        """Default: every top-level key that names a field of the record (case-insensitive, '_' ignored) overwrites it."""
        names = {f.name.lower().replace("_", ""): f.name for f in dataclasses.fields(self.Cfg)} if dataclasses.is_dataclass(self.Cfg) else \
            {k.lower().replace("_", ""): k for k in vars(self.Cfg)}
        for k, v in (node or {}).items():
            f = names.get(str(k).lower().replace("_", ""))
            if f is not None:
                cur = getattr(self.Cfg, f)
                setattr(self.Cfg, f, type(cur)(v) if cur is not None and not isinstance(v, (dict, list)) else v)

    def Validate(self) -> Optional[str]:
        """Override: return a message to refuse the parsed configuration."""
        return None

    # ---- parsing
    @staticmethod
    def _find_config(argv: Sequence[str]) -> str:
        for i, a in enumerate(argv):
            if a in ("--config", "-c") and i + 1 < len(argv):
                return argv[i + 1]
            if a.startswith("--config="):
                return a[9:]
            if a.startswith("-c="):
                return a[3:]
        return ""

    def Parse(self, argv: Optional[Sequence[str]] = None) -> bool:
        """`argv` includes the program name (as sys.argv).  False (with `Error` set) on a bad file, option or validation."""
        argv = list(sys.argv if argv is None else argv)[1:]
        self.ConfigPath = self._find_config(argv)
        if self.ConfigPath:
            try:
                import yaml
                with open(self.ConfigPath) as f:
                    self.LoadYaml(yaml.safe_load(f) or {})
            except Exception as e:                    # the reference warns and goes on with the defaults
                self.Error = f"[OA CONFIG] YAML load failed: {e} (using defaults)"
                print(self.Error, file=sys.stderr)
        try:
            ns = self._parser.parse_args(argv)
        except SystemExit as e:                       # argparse exits on --help and on errors
            self.Error = self.Error or ("" if e.code in (0, None) else "invalid command line")
            return False
        for k, v in vars(ns).items():                 # only what the user typed is present (defaults are suppressed)
            if k == "_verbose":
                self.Verbose = int(v)
            elif k != "_config":
                setattr(self.Cfg, k, v)
        msg = self.Validate()
        if msg:
            self.Error = msg
            print(f"{self._parser.prog}: {msg}", file=sys.stderr)
            return False
        return True

    def Usage(self) -> str:
        return self._parser.format_help()
