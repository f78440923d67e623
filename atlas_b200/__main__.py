"""``python -m atlas_b200 <command>`` (see :mod:`atlas_b200.cli`)."""
import sys

from .cli import main

sys.exit(main())
