#!/usr/bin/env python
"""Worker entry point: decode the configuration handed over by launch.py and run pre-training
(reference: train.py:13-29)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from savanna_b200.config import GlobalConfig  # noqa: E402
from savanna_b200.train.trainer import pretrain  # noqa: E402


def main(argv=None):
    cfg = GlobalConfig.consume_global_config(argv)
    cfg.build_tokenizer()
    cfg.initialize_tensorboard_writer()
    if (cfg.rank or 0) == 0:
        cfg.print()
    pretrain(cfg)


if __name__ == "__main__":
    main()
