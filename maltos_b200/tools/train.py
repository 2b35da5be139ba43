"""Training entry point: ``python -m maltos_b200.tools.train --config recipe.yaml [flags]`` (or under ``torchrun``)."""
from maltos_b200.train import cli as _cli
from maltos_b200.train.cli import *  # noqa: F401,F403  (the builders are importable from here, as in the reference tool)
from maltos_b200.train.flags import (_load_config_defaults, build_arg_parser, build_runtime_spec, parse_args, parse_args_from,  # noqa: F401
                                     parse_runtime_spec_args)
from maltos_b200.train.cli import (_build_dataloader, _build_hdp_config, _build_logging, _build_model, _build_optimizer_factory,  # noqa: F401
                                   _build_runtime, _build_scheduler_factory, _global_batch_tokens, main)


if __name__ == "__main__":
    main()
