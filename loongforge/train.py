"""``torchrun ... $LOONGFORGE_PATH/loongforge/train.py <flags>``: the launch line of the reference's example scripts
(reference: loongforge/train.py:17-27). Forwards to ``loongforge_b200.train``."""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
os.environ.setdefault("LOONGFORGE_PATH", _ROOT)


def main():
    from loongforge_b200.train import main as _main

    return _main()


if __name__ == "__main__":
    sys.exit(main())
