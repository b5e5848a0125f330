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
