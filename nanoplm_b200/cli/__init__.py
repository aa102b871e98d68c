"""`nanoplm` command line: `data`, `pretrain` and `distill` groups with the reference's sub-commands
(src/nanoplm/cli/__init__.py:8-22)."""
from __future__ import annotations

import click

from nanoplm_b200 import __version__


@click.group(context_settings={"help_option_names": ["-h", "--help"]})
@click.version_option(__version__, prog_name="nanoplm")
def cli() -> None:
    """nanoplm: protein language model pretraining and distillation (B200-native build)."""


def _attach() -> None:
    from .data import data
    from .distill import distill
    from .pretrain import pretrain
    cli.add_command(data)
    cli.add_command(distill)
    cli.add_command(pretrain)


_attach()


def main() -> None:
    cli()


def main_data() -> None:
    from .data import data
    data()


def main_pretrain() -> None:
    from .pretrain import pretrain
    pretrain()


def main_distill() -> None:
    from .distill import distill
    distill()
