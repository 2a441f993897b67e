"""Entry point of the embodied stack: ``python -m loongforge_b200.embodied.train --model-name pi05 key=value ...``
(under torchrun for several GPUs). Reference: loongforge/embodied/train.py."""
from __future__ import annotations

import os
import sys

from .config import parse_args
from .trainer import build_trainer


def main(argv=None):
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    args = parse_args(argv, repo_root=root)
    return build_trainer(args).train()


if __name__ == "__main__":
    main(sys.argv[1:])
