"""Entry-point compatibility package: launchers written for the reference framework call
``$LOONGFORGE_PATH/loongforge/train.py`` (or the ``LoongForge`` console script, ``loongforge.train:main``) with its
flag spelling. Everything here forwards to ``loongforge_b200``."""
