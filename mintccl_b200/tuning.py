"""Measured algorithm choices that override the built-in policy (``MINTCCL_TUNING_FILE``).

The communicator picks algorithm, protocol and CTA count from message size, rank count and where the tensors live
(``parallel/comm.py``); the thresholds in that policy were measured on one kind of box.  A tuning table replaces
them with what a sweep measured on the box at hand:

    python -m torch.distributed.run --nproc-per-node 8 ... mintccl_b200/benchmarks/sweep.py \\
        --algos auto,ring,direct,nvls --ctas 32,64,128 --out sweep.json
    python -m mintccl_b200.tuning sweep.json -o tuning.json
    MINTCCL_TUNING_FILE=tuning.json python train.py

A row says: for this collective on this many ranks, up to this many bytes, on symmetric (or ordinary) tensors, use
this algorithm with this many CTAs / channels.  Rows apply only where the caller left ``algo`` and ``nch`` open.
The reference has no tuning at all: one algorithm (ring) and a fixed grid of 16 CTAs (common.py:85).
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

Key = Tuple[str, int, bool]


class TuningTable:
    def __init__(self, rows: Iterable[dict]):
        self.rows: Dict[Key, List[dict]] = {}
        for r in rows:
            row = {"collective": str(r["collective"]), "nranks": int(r["nranks"]), "max_bytes": int(r["max_bytes"]),
                   "symmetric": bool(r.get("symmetric", True)), "algo": str(r["algo"]),
                   "nch": None if r.get("nch") in (None, 0) else int(r["nch"])}
            self.rows.setdefault((row["collective"], row["nranks"], row["symmetric"]), []).append(row)
        for v in self.rows.values():
            v.sort(key=lambda x: x["max_bytes"])

    # ---------------------------------------------------------------------------------------------- use
    def lookup(self, collective: str, nranks: int, nbytes: int, symmetric: bool = True) -> Optional[Tuple[str, Optional[int]]]:
        """(algo, nch) of the first row whose ``max_bytes`` covers ``nbytes``; None where the table is silent (the
        built-in policy then decides), including beyond the largest measured size."""
        for row in self.rows.get((collective, nranks, symmetric), ()):
            if nbytes <= row["max_bytes"]:
                return row["algo"], row["nch"]
        return None

    # ---------------------------------------------------------------------------------------------- io
    @classmethod
    def load(cls, path: str) -> "TuningTable":
        with open(path) as f:
            d = json.load(f)
        return cls(d["rows"] if isinstance(d, dict) else d)

    @classmethod
    def from_env(cls) -> Optional["TuningTable"]:
        path = os.environ.get("MINTCCL_TUNING_FILE", "")
        return cls.load(path) if path else None

    def dump(self, path: str) -> None:
        rows = [r for k in sorted(self.rows) for r in self.rows[k]]
        with open(path, "w") as f:
            json.dump({"rows": rows}, f, indent=1)

    # ---------------------------------------------------------------------------------------------- build
    @classmethod
    def from_sweep(cls, rows: Iterable[dict], impl: str = "mintccl", symmetric: bool = True) -> "TuningTable":
        """Best (algorithm, CTA count) per collective, rank count and size out of the rows ``benchmarks/sweep.py``
        prints; neighbouring sizes with the same choice merge into one row, and a row reaches up to the geometric
        mean of its last size and the next measured one."""
        best: Dict[Tuple[str, int, int], dict] = {}
        for r in rows:
            if r.get("impl") != impl:
                continue
            k = (r["collective"], int(r["n"]), int(r["bytes"]))
            if k not in best or r["us"] < best[k]["us"]:
                best[k] = r
        out: List[dict] = []
        groups: Dict[Tuple[str, int], List[Tuple[int, dict]]] = {}
        for (coll, n, nbytes), r in best.items():
            groups.setdefault((coll, n), []).append((nbytes, r))
        for (coll, n), items in sorted(groups.items()):
            items.sort()
            for i, (nbytes, r) in enumerate(items):
                choice = (r["algo"], int(r.get("ctas") or 0))
                nxt = items[i + 1][0] if i + 1 < len(items) else None
                upto = int(math.sqrt(nbytes * nxt)) if nxt else nbytes
                if out and out[-1]["collective"] == coll and out[-1]["nranks"] == n and \
                        (out[-1]["algo"], out[-1]["nch"] or 0) == choice:
                    out[-1]["max_bytes"] = upto
                else:
                    out.append({"collective": coll, "nranks": n, "max_bytes": upto, "symmetric": symmetric,
                                "algo": choice[0], "nch": choice[1] or None})
        return cls(out)


def _read_rows(path: str) -> List[dict]:
    """A file written with ``sweep.py --out`` (one JSON object) or its standard output (one JSON object per line)."""
    with open(path) as f:
        text = f.read()
    try:
        d = json.loads(text)
        return d["rows"] if isinstance(d, dict) else d
    except json.JSONDecodeError:
        return [json.loads(l) for l in text.splitlines() if l.startswith("{")]


def main() -> None:
    ap = argparse.ArgumentParser(description="Build a tuning table from sweep results")
    ap.add_argument("sweeps", nargs="+", help="outputs of mintccl_b200/benchmarks/sweep.py (one per rank count)")
    ap.add_argument("-o", "--out", required=True)
    ap.add_argument("--ordinary", action="store_true", help="the sweep ran on ordinary (not symmetric) tensors")
    a = ap.parse_args()
    rows: List[dict] = []
    for p in a.sweeps:
        rows += _read_rows(p)
    t = TuningTable.from_sweep(rows, symmetric=not a.ordinary)
    t.dump(a.out)
    print(f"{sum(len(v) for v in t.rows.values())} rows -> {a.out}")


if __name__ == "__main__":
    main()
