"""``python -m ironcore`` / the ``ironcore`` console script (reference: ironcore/__main__.py:16-89)."""

import sys

from ironcore_b200.__main__ import main  # noqa: F401

if __name__ == "__main__":
    sys.exit(main())
