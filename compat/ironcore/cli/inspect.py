"""``ironcore inspect`` / ``ironcore preprocess --only-inspect`` (reference: ironcore/cli/inspect.py:38-522)."""

from pathlib import Path

from ironcore_b200.cli import inspect as _inspect
from ironcore_b200.cli.inspect import check_integrity, packing_efficiency, render_preview, statistics  # noqa: F401


class Colors:
    """ANSI escape codes used in the previews."""

    RED, GREEN, YELLOW, BLUE = "\033[31m", "\033[32m", "\033[33m", "\033[34m"
    GRAY, DIM, BOLD, RESET = "\033[90m", "\033[2m", "\033[1m", "\033[0m"


def run_inspect(args, tokenizer=None, preview: int = 0, report_dir=None) -> int:
    """``run_inspect(args)`` with ``args.config`` (data YAML) and ``args.preview`` as in the reference, or
    ``run_inspect(data_config, tokenizer, preview, report_dir)`` as in ``ironcore_b200``. Returns the number of
    datasets that failed their integrity checks."""
    if hasattr(args, "all_datasets"):
        return _inspect.run_inspect(args, tokenizer, preview=preview, report_dir=report_dir)
    from ironcore_b200.cli.preprocess import _build_tokenizer   # pylint: disable=protected-access
    from ironcore_b200.data.data_config import UniversalDataConfig

    path = Path(args.config)
    if not path.exists():
        print(f"Error: Configuration file not found: {path}")
        return 1
    dcfg = UniversalDataConfig.from_yaml(path)
    return _inspect.run_inspect(dcfg, _build_tokenizer(dcfg), preview=int(getattr(args, "preview", 0) or 0))
