"""Launcher shim: ``python run.py --config-path examples/llama3 --config-name train_1b_adamw action=dryrun``."""
import sys

from sga_b200.launcher.run import main

if __name__ == "__main__":
    sys.exit(main())
