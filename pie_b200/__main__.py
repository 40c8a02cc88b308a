"""`python -m pie_b200 ...` = the `pie` command line."""
import sys

from .server.cli import main

sys.exit(main())
