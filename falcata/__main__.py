"""``python -m falcata`` - the same command line as ``python -m falcata_b200``."""
import sys

from falcata_b200.__main__ import main

if __name__ == "__main__":
    sys.exit(main())
