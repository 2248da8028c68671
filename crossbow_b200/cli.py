"""Command-line handling: ``--flag value`` pairs only, booleans included (cli/CommandLine.java:14-53, cli/Options.java,
cli/Option.java).  Every application gets the system, model and solver options for free and may add its own."""
from __future__ import annotations

import sys
from typing import Any, Callable, Dict, List, Optional

from .conf import ModelConf, SolverConf, SystemConf


class Option:
    def __init__(self, name: str, type_: Callable[[str], Any] = str, default=None, required=False, help_: str = ""):
        if not name.startswith("--"):
            raise ValueError("error: option names start with --")
        self.name, self.type, self.default, self.required, self.help = name, type_, default, required, help_
        self.value = default
        self.is_set = False

    def setType(self, t):
        self.type = (lambda s: str(s).lower() == "true") if t is bool else t
        return self

    def set(self, raw: str):
        self.value = self.type(raw)
        self.is_set = True

    def get(self):
        return self.value


class Options:
    def __init__(self, app: str = "app"):
        self.app = app
        self.own: Dict[str, Option] = {}

    def add(self, opt: Option):
        self.own[opt.name] = opt
        return self

    addOption = add

    def get(self, name: str) -> Option:
        return self.own[name]

    def names(self) -> List[str]:
        return sorted(list(self.own) + list(SystemConf.OPTIONS) + list(ModelConf.OPTIONS) + list(SolverConf.OPTIONS))

    def usage(self) -> str:
        lines = [f"usage: {self.app} [--flag value]..."]
        for n in self.names():
            o = self.own.get(n)
            lines.append(f"  {n}" + (f"  ({o.help})" if o is not None and o.help else ""))
        return "\n".join(lines)


class CommandLine:
    def __init__(self, options: Options):
        self.options = options

    def parse(self, argv: Optional[List[str]] = None, system: Optional[SystemConf] = None, model: Optional[ModelConf] = None):
        argv = list(sys.argv[1:] if argv is None else argv)
        system = system or SystemConf.getInstance()
        model = model or ModelConf.getInstance()
        if len(argv) % 2:
            raise SystemExit(f"error: every flag takes a value\n{self.options.usage()}")
        for flag, value in zip(argv[0::2], argv[1::2]):
            if not flag.startswith("--"):
                raise SystemExit(f"error: invalid flag {flag}\n{self.options.usage()}")
            if flag in self.options.own:
                self.options.own[flag].set(value)
            elif system.parse(flag, value) or model.parse(flag, value):
                pass
            else:
                raise SystemExit(f"error: unknown flag {flag}\n{self.options.usage()}")
        missing = [o.name for o in self.options.own.values() if o.required and not o.is_set]
        if missing:
            raise SystemExit(f"error: missing required flags {missing}\n{self.options.usage()}")
        return self
