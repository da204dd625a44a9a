"""``ironcore inspect`` (reference: ironcore/cli/inspect.py)."""

from ironcore_b200.cli.inspect import (check_integrity, packing_efficiency, render_preview, run_inspect,  # noqa: F401
                                        statistics)
