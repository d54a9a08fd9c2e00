"""``bergson <command> --flags`` or ``bergson <config.yaml>`` (a ``steps:`` list run in
order); every run writes a ``config.yaml`` that replays it
(reference ``bergson/__main__.py:81-115``)."""

from __future__ import annotations

import os
import sys


class Main:
    """A parsed command line: ``Main(command).execute()`` runs it
    (reference ``bergson/__main__.py:30-53``)."""

    def __init__(self, command):
        self.command = command

    def execute(self):
        self.command.execute()


def run_config(config_path: str, registry: dict[str, type]) -> None:
    from .config.config_io import parse_steps, read_config, save_pipeline_config

    config = read_config(config_path)
    steps = parse_steps(config["steps"], registry)
    if len(steps) > 1:
        save_pipeline_config(steps, config.get("run_path"))
    for i, (name, cmd) in enumerate(steps, start=1):
        if len(steps) > 1:
            print(f"\n[Pipeline] Step {i}/{len(steps)}: {name.title()}")
        cmd.execute()


def main(argv: list[str] | None = None):
    from .cli.commands import COMMANDS
    from .config.parsing import parse_command

    args = list(sys.argv[1:] if argv is None else argv)
    config_path = None
    if len(args) == 1 and os.path.isfile(args[0]):
        config_path = args[0]
    elif len(args) == 2 and os.path.isfile(args[1]):
        config_path = args[1]
    if config_path is not None:
        run_config(config_path, COMMANDS)
        return
    Main(parse_command(COMMANDS, args, prog="bergson")).execute()


if __name__ == "__main__":
    main()
