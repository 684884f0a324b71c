#!/usr/bin/env python
"""Trainer entry point:  torchrun ... zorse.py --config_file training_config.json [flags]

Same command line as the reference trainer (README.md:45, zorse.py:212-283).
"""
import sys

from zorse_b200.cli.train import main

if __name__ == "__main__":
    sys.exit(main())
