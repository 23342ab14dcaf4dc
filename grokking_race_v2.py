#!/usr/bin/env python
"""Command-line entry of the grokking race (same file name and flags as the reference driver, plus --mode,
--optimizers, --seeds, --model-scale, --max-steps, --dtype, ... instead of editing constants in the file)."""
import sys

from supergrok15_b200.race import *  # noqa: F401,F403  (models, data generators, registry, pipelines)
from supergrok15_b200.race import main
from supergrok15_b200.models import MambaModel, Transformer, ViT  # noqa: F401

if __name__ == "__main__":
    sys.exit(main())
