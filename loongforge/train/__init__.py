"""``from loongforge.train import parse_train_args, build_model_trainer`` (reference: loongforge/train/__init__.py)
and the console-script target ``loongforge.train:main``."""
from loongforge_b200.config.arguments import parse_args as _parse_args
from loongforge_b200.runtime.trainer_builder import build_model_trainer  # noqa: F401


def parse_train_args(argv=None):
    """Flags (reference spelling) -> namespace; leftovers are YAML overrides and stay on ``args.yaml_overrides``."""
    args, overrides = _parse_args(argv)
    args.yaml_overrides = overrides
    return args


def main():
    from loongforge_b200.train import main as _main

    return _main()
