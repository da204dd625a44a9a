"""``ironcore preprocess --config D [--inspect] [--only-inspect] [--preview N]``.
(Behavioural reference: ironcore/cli/preprocess.py:10-75.)"""

from __future__ import annotations

from pathlib import Path


def _build_tokenizer(dcfg):
    from ..config import default_config
    from ..tokenizer import build_tokenizer

    cfg = default_config()
    cfg.model.tokenizer_type = dcfg.tokenizer_type
    cfg.model.vocab_name_or_path = dcfg.vocab_name_or_path
    return build_tokenizer(cfg)


def run_preprocess(args) -> int:
    from ..data.data_config import UniversalDataConfig
    from ..data.serializer import DataSerializer

    path = Path(args.config)
    if not path.exists():
        print(f"Error: Configuration file not found: {path}")
        return 1
    dcfg = UniversalDataConfig.from_yaml(path)
    tok = _build_tokenizer(dcfg)
    if not getattr(args, "only_inspect", False):
        ser = DataSerializer(dcfg, tok)
        for out in ser.serialize_all():
            print(f"serialized -> {out}")
    if getattr(args, "inspect", False) or getattr(args, "only_inspect", False) or getattr(args, "preview", 0):
        from .inspect import run_inspect

        return run_inspect(dcfg, tok, preview=getattr(args, "preview", 0))
    return 0
