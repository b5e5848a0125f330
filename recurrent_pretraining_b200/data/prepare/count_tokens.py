"""Token accounting over packed shards: rows, tokens, and per-token-id frequencies of the special tokens (how many
documents, how much padding).  Counterpart of scripts/parquet_token_counter.py and scripts/process_token_counts.py."""
from __future__ import annotations

import argparse
import glob
import json
import os
from collections import Counter


def count_folder(folder: str, column: str = "input_ids", track_ids=()) -> dict:
    import pyarrow.compute as pc
    import pyarrow.parquet as pq

    total_rows = total_tokens = 0
    tracked: Counter = Counter()
    per_file = {}
    for path in sorted(glob.glob(os.path.join(folder, "*.parquet"))):
        pf = pq.ParquetFile(path)
        rows = tokens = 0
        for g in range(pf.num_row_groups):
            col = pf.read_row_group(g, columns=[column]).column(column)
            flat = pc.list_flatten(col)
            rows += len(col)
            tokens += len(flat)
            for t in track_ids:
                tracked[int(t)] += int(pc.sum(pc.equal(flat, t)).as_py() or 0)
        per_file[os.path.basename(path)] = {"rows": rows, "tokens": tokens}
        total_rows += rows
        total_tokens += tokens
    return {"files": len(per_file), "rows": total_rows, "tokens": total_tokens, "tracked": dict(tracked),
            "per_file": per_file}


def category_report(sources: dict, counts: dict) -> dict:
    """Token budget by dataset and by category (the summary of scripts/process_token_counts.py): ``sources`` maps a
    dataset name to its manifest entry (``DataSource``: category, weight ...), ``counts`` maps the name to
    ``(kept_tokens, total_tokens)`` -- kept = what survived packing, the rest was dropped as document tails.  Returns
    the per-dataset rows, the per-category sums with their shares, and the grand total; ``format_category_report``
    prints it."""
    per_dataset, per_category = {}, {}
    for name, src in sources.items():
        kept, total = counts.get(name, (0, 0))
        cat = getattr(src, "category", None) or "generic-text"
        per_dataset[name] = {"kept": kept, "total": total, "category": cat,
                             "dropped_pct": 100.0 * (total - kept) / total if total else float("nan")}
        per_category.setdefault(cat, {"kept": 0, "datasets": []})
        per_category[cat]["kept"] += kept
        per_category[cat]["datasets"].append(name)
    grand = sum(c["kept"] for c in per_category.values())
    for c in per_category.values():
        c["share_pct"] = 100.0 * c["kept"] / grand if grand else float("nan")
        c["datasets"].sort(key=lambda n: -per_dataset[n]["kept"])
    return {"datasets": per_dataset, "categories": per_category, "total_kept": grand}


def format_category_report(report: dict) -> str:
    lines = ["Token counts per dataset:"]
    for i, (name, d) in enumerate(report["datasets"].items()):
        lines.append(f"{i:>3}: {name:<28}: {d['kept'] / 1e9:8.3f}B (dropped: {d['dropped_pct']:.2f}%)")
    lines.append("")
    lines.append("Token counts per category:")
    for cat, c in sorted(report["categories"].items(), key=lambda kv: -kv[1]["kept"]):
        lines.append(f"{cat}: {c['kept'] / 1e9:.3f}B ({c['share_pct']:.2f}%)")
        for name in c["datasets"]:
            kept = report["datasets"][name]["kept"]
            if kept:
                lines.append(f"  - {name}: {kept / 1e9:.3f}B ({100.0 * kept / max(c['kept'], 1):.2f}%)")
    lines.append(f"Total tokens: {report['total_kept'] / 1e12:.4f}T")
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("folder")
    ap.add_argument("--track_ids", type=int, nargs="*", default=[65504, 65505, 65509])
    a = ap.parse_args(argv)
    out = count_folder(a.folder, track_ids=a.track_ids)
    out.pop("per_file")
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
