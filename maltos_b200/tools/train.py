"""Training entry point: ``python -m maltos_b200.tools.train --config recipe.yaml [flags]`` (or under ``torchrun``)."""
from maltos_b200.train import cli as _cli
from maltos_b200.train.cli import *  # noqa: F401,F403  (the builders are importable from here, as in the reference tool)
from maltos_b200.train.cli import main


if __name__ == "__main__":
    main()
