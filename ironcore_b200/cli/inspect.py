"""Integrity checks, statistics, packing-efficiency simulation and previews of preprocessed data.
(Behavioural reference: ironcore/cli/inspect.py:38-522.)"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List

import numpy as np

from ..data.collator import first_fit_decreasing
from ..data.serializer import BIN_NAME, IDX_DTYPE, IDX_NAME

RED, GREEN, DIM, RESET = "\033[31m", "\033[32m", "\033[2m", "\033[0m"


def check_integrity(directory) -> List[str]:
    """Returns a list of problems (empty = healthy)."""
    d = Path(directory)
    problems = []
    for name in (BIN_NAME, IDX_NAME):
        if not (d / name).exists():
            problems.append(f"missing file {name}")
    if problems:
        return problems
    try:
        idx = np.load(d / IDX_NAME, allow_pickle=False)
    except Exception as exc:
        return [f"index unreadable: {exc}"]
    if idx.dtype.names != IDX_DTYPE.names:
        problems.append(f"index fields {idx.dtype.names} != {IDX_DTYPE.names}")
        return problems
    if len(idx) == 0:
        problems.append("index is empty")
        return problems
    off, ln = idx["offset"].astype(np.int64), idx["length"].astype(np.int64)
    if (ln <= 0).any():
        problems.append(f"{int((ln <= 0).sum())} samples have non-positive length")
    if (np.diff(off) < 0).any():
        problems.append("offsets are not monotonic")
    if (off[1:] != off[:-1] + ln[:-1]).any():
        problems.append("offsets are not contiguous (gaps or overlaps)")
    meta = d / "meta.json"
    itemsize = 2
    if meta.exists():
        itemsize = np.dtype(json.loads(meta.read_text())["dtype"]).itemsize
    total = (d / BIN_NAME).stat().st_size // itemsize
    if off[-1] + ln[-1] > total:
        problems.append(f"index points past the end of data.bin ({off[-1] + ln[-1]} > {total})")
    return problems


def statistics(directory) -> Dict:
    idx = np.load(Path(directory) / IDX_NAME, allow_pickle=False)
    ln = idx["length"].astype(np.int64)
    types, counts = np.unique(idx["type"], return_counts=True)
    return {"samples": int(len(idx)), "tokens": int(ln.sum()), "mean_length": float(ln.mean()) if len(ln) else 0.0,
            "median_length": float(np.median(ln)) if len(ln) else 0.0, "max_length": int(ln.max()) if len(ln) else 0,
            "min_length": int(ln.min()) if len(ln) else 0, "types": {str(t): int(c) for t, c in zip(types, counts)}}


def packing_efficiency(directory, seq_len: int, max_samples: int = 20000) -> Dict:
    """First-Fit-Decreasing simulation: fraction of row capacity filled by real tokens."""
    idx = np.load(Path(directory) / IDX_NAME, allow_pickle=False)
    lengths = [int(x) for x in idx["length"][:max_samples]]
    bins = first_fit_decreasing(lengths, seq_len + 1)
    used = sum(min(l, seq_len + 1) for l in lengths)
    cap = len(bins) * (seq_len + 1)
    return {"rows": len(bins), "efficiency": used / cap if cap else 0.0, "samples": len(lengths)}


def render_preview(directory, tokenizer, n: int = 3) -> str:
    """Decoded samples with loss-masked spans dimmed."""
    from ..data.dataset import BinaryDataset

    ds = BinaryDataset(directory)
    lines = []
    for i in range(min(n, len(ds))):
        s = ds.sample(i)
        toks = s["tokens"].tolist()
        masked = np.zeros(len(toks), dtype=bool)
        for a, b in s["mask_ranges"]:
            masked[a:b] = True
        lines.append(f"--- sample {i} ({s['type']}, {len(toks)} tokens, {int(masked.sum())} masked) ---")
        out, cur, buf = [], None, []
        for t, mk in zip(toks, masked):
            if cur is not None and mk != cur:
                out.append((DIM if cur else GREEN) + tokenizer.decode(buf) + RESET)
                buf = []
            cur = mk
            buf.append(t)
        if buf:
            out.append((DIM if cur else GREEN) + tokenizer.decode(buf) + RESET)
        lines.append("".join(out))
    return "\n".join(lines)


def run_inspect(dcfg, tokenizer, preview: int = 0, report_dir=None) -> int:
    report = {}
    bad = 0
    for ds in dcfg.all_datasets():
        d = Path(ds.output_path)
        problems = check_integrity(d)
        entry = {"path": str(d), "problems": problems}
        if not problems:
            entry["stats"] = statistics(d)
            if ds.task_type != "pretrain":
                entry["packing"] = packing_efficiency(d, dcfg.seq_length)
        else:
            bad += 1
        report[ds.name] = entry
        status = f"{GREEN}OK{RESET}" if not problems else f"{RED}FAILED{RESET}: " + "; ".join(problems)
        print(f"[{ds.name}] {status}")
        if not problems:
            print(f"  {entry['stats']}")
            if "packing" in entry:
                print(f"  packing efficiency {entry['packing']['efficiency']:.3f} over {entry['packing']['rows']} rows")
            if preview:
                print(render_preview(d, tokenizer, preview))
    out_dir = Path(report_dir or dcfg.preprocessed_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "inspection_report.json").write_text(json.dumps(report, indent=2))
    md = ["# Data inspection report", ""]
    for name, e in report.items():
        md.append(f"## {name}")
        md.append(f"- path: `{e['path']}`")
        md.append(f"- status: {'OK' if not e['problems'] else 'FAILED: ' + '; '.join(e['problems'])}")
        if "stats" in e:
            md += [f"- {k}: {v}" for k, v in e["stats"].items()]
        md.append("")
    (out_dir / "inspection_report.md").write_text("\n".join(md))
    return 1 if bad else 0
