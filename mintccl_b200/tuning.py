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
            if r.get("min_bytes"):
                row["min_bytes"] = int(r["min_bytes"])
            self.rows.setdefault((row["collective"], row["nranks"], row["symmetric"]), []).append(row)
        for v in self.rows.values():
            v.sort(key=lambda x: x["max_bytes"])

    # ---------------------------------------------------------------------------------------------- use
    def lookup(self, collective: str, nranks: int, nbytes: int, symmetric: bool = True) -> Optional[Tuple[str, Optional[int]]]:
        """(algo, nch) of the first row whose ``max_bytes`` covers ``nbytes``; None where the table is silent (the
        built-in policy then decides), including beyond the largest and below the smallest measured size."""
        for row in self.rows.get((collective, nranks, symmetric), ()):
            if nbytes <= row["max_bytes"]:
                if nbytes < row.get("min_bytes", 0):
                    return None     # below the smallest size that was measured
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
        """``MINTCCL_TUNING_FILE``: a table to use; ``none`` (or ``0``): the built-in policy only.  Unset: the table
        shipped with the package (``tuning_b200.json``, measured on HGX B200 boards), if there is one."""
        path = os.environ.get("MINTCCL_TUNING_FILE", "")
        if path.strip().lower() in ("none", "0", "off"):
            return None
        if path:
            return cls.load(path)
        shipped = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuning_b200.json")
        return cls.load(shipped) if os.path.exists(shipped) else None

    def dump(self, path: str) -> None:
        rows = [r for k in sorted(self.rows) for r in self.rows[k]]
        with open(path, "w") as f:
            json.dump({"rows": rows}, f, indent=1)

    # ---------------------------------------------------------------------------------------------- build
    @classmethod
    def from_sweep(cls, rows: Iterable[dict], impl: str = "mintccl", symmetric: Optional[bool] = None,
                   margin: float = 0.05) -> "TuningTable":
        """Best (algorithm, CTA count) per collective, rank count, kind of memory and size out of the rows
        ``benchmarks/sweep.py`` prints.  The automatic choice (``algo == "auto"``) is the yardstick: a row is only
        written where a named algorithm beat it by more than ``margin`` (timing noise must not flip choices), and
        says ``auto`` where nothing did, so that the built-in policy keeps deciding there.  Neighbouring sizes with
        the same choice merge into one row, and a row reaches up to the geometric mean of its last size and the next
        measured one; the first row of a group starts at the smallest measured size (``min_bytes``) when that is not small.  ``symmetric``: None = from each row's ``memory`` field (heap / ordinary)."""
        cands: Dict[Tuple[str, int, bool, int], List[dict]] = {}
        for r in rows:
            if r.get("impl") != impl:
                continue
            # Broadcast and reduce on more than two ranks are tuned from fenced measurements only (sweep.py --sync):
            # consecutive calls of the barrier-free chain overlap one another, so a back-to-back block rates the
            # chain by its steady state and hides the fill that a single call between other work pays in full.
            if r["collective"] in ("broadcast", "reduce") and int(r["n"]) > 2 and not r.get("sync"):
                continue
            sym = symmetric if symmetric is not None else (str(r.get("memory", "heap")) == "heap")
            cands.setdefault((r["collective"], int(r["n"]), sym, int(r["bytes"])), []).append(r)
        groups: Dict[Tuple[str, int, bool], List[Tuple[int, Tuple[str, int]]]] = {}
        for (coll, n, sym, nbytes), rs in cands.items():
            # per algorithm: its own default CTA count unless an explicit count beat that by more than 3 %
            per_algo: Dict[str, Tuple[float, int]] = {}
            for algo_name in {r["algo"] for r in rs}:
                mine = [r for r in rs if r["algo"] == algo_name]
                dflt = [r for r in mine if not r.get("ctas")]
                best = min(mine, key=lambda r: r["us"])
                if dflt and best["us"] >= 0.97 * min(r["us"] for r in dflt):
                    per_algo[algo_name] = (min(r["us"] for r in dflt), 0)
                else:
                    per_algo[algo_name] = (best["us"], int(best.get("ctas") or 0))
            if "ring" in per_algo and per_algo["ring"][1] > 64:
                per_algo["ring"] = (per_algo["ring"][0], 64)   # the FIFOs are laid out for 64 channels: more is the same
            choice = ("auto", 0)
            name = min(per_algo, key=lambda k: per_algo[k][0])
            if name != "auto" and ("auto" not in per_algo or per_algo[name][0] < (1.0 - margin) * per_algo["auto"][0]):
                choice = (name, per_algo[name][1])
            elif "auto" in per_algo and per_algo["auto"][1]:
                choice = ("auto", per_algo["auto"][1])
            groups.setdefault((coll, n, sym), []).append((nbytes, choice))
        out: List[dict] = []
        for (coll, n, sym), items in sorted(groups.items()):
            items.sort()
            if all(c == ("auto", 0) for _, c in items):
                continue
            for i, (nbytes, choice) in enumerate(items):
                nxt = items[i + 1][0] if i + 1 < len(items) else None
                upto = int(math.sqrt(nbytes * nxt)) if nxt else nbytes
                last = out[-1] if out else None
                if last and (last["collective"], last["nranks"], last["symmetric"]) == (coll, n, sym) and \
                        (last["algo"], last["nch"] or 0) == choice:
                    last["max_bytes"] = upto
                else:
                    out.append({"collective": coll, "nranks": n, "max_bytes": upto, "symmetric": sym,
                                "algo": choice[0], "nch": choice[1] or None})
                    if i == 0 and nbytes > 4096:
                        out[-1]["min_bytes"] = nbytes    # a sweep that starts at a large size says nothing below it
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
    ap.add_argument("--ordinary", action="store_true",
                    help="treat every row as measured on ordinary (not symmetric) tensors; default: the rows' own "
                         "`memory` field")
    ap.add_argument("--margin", type=float, default=0.05,
                    help="a named algorithm must beat the automatic choice by this fraction to get a row")
    a = ap.parse_args()
    rows: List[dict] = []
    for p in a.sweeps:
        rows += _read_rows(p)
    t = TuningTable.from_sweep(rows, symmetric=False if a.ordinary else None, margin=a.margin)
    t.dump(a.out)
    print(f"{sum(len(v) for v in t.rows.values())} rows -> {a.out}")


if __name__ == "__main__":
    main()
