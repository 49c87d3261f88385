"""``torchrun --nproc_per_node=N -m scripts.train --config=<config.py> -- experiment=<name> ...`` (thin alias of
``cosmos_predict25_b200.cli.train`` kept at the path the reference documents)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from cosmos_predict25_b200.cli.train import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
