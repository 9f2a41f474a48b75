"""Look at dumped rollouts in a terminal (plain-text counterpart of the reference's ``scripts/rollout_viewer.py``).

The trainer writes one ``<step>.jsonl`` per step under ``trainer.rollout_data_dir`` / ``trainer.validation_data_dir``
(fields ``input``, ``output``, ``score``, ``step``).

    python -m verl_b200.utils.rollout_viewer DIR_OR_FILE [--step N] [--grep TEXT] [--min-score X] [--max-score X]
                                            [--sort score|score_desc|length] [--limit K] [--width 120]
"""

from __future__ import annotations

import argparse
import json
import os
import textwrap
from typing import Iterable, Optional


def load(path: str, step: Optional[int] = None) -> list[dict]:
    files = [path] if os.path.isfile(path) else sorted(
        (os.path.join(path, f) for f in os.listdir(path) if f.endswith(".jsonl")),
        key=lambda p: (len(os.path.basename(p)), os.path.basename(p)))
    rows = []
    for f in files:
        with open(f) as fh:
            for line in fh:
                if line.strip():
                    r = json.loads(line)
                    r.setdefault("step", os.path.basename(f).split(".")[0].split("_")[0])
                    rows.append(r)
    if step is not None:
        rows = [r for r in rows if str(r.get("step")) == str(step)]
    return rows


def select(rows: Iterable[dict], grep: Optional[str] = None, min_score: Optional[float] = None,
           max_score: Optional[float] = None, sort: Optional[str] = None, limit: Optional[int] = None) -> list[dict]:
    out = [r for r in rows
           if (grep is None or grep in str(r.get("input", "")) or grep in str(r.get("output", "")))
           and (min_score is None or float(r.get("score", 0)) >= min_score)
           and (max_score is None or float(r.get("score", 0)) <= max_score)]
    if sort in ("score", "score_desc"):
        out.sort(key=lambda r: float(r.get("score", 0)), reverse=sort == "score_desc")
    elif sort == "length":
        out.sort(key=lambda r: len(str(r.get("output", ""))))
    return out[:limit] if limit else out


def render(rows: list[dict], width: int = 120) -> str:
    parts = []
    for i, r in enumerate(rows):
        parts.append(f"--- #{i}  step {r.get('step')}  score {r.get('score')} " + "-" * 20)
        for key in ("input", "output"):
            body = textwrap.fill(str(r.get(key, "")), width=width, initial_indent="  ", subsequent_indent="  ")
            parts.append(f"{key}:\n{body}")
    scores = [float(r.get("score", 0)) for r in rows]
    if scores:
        parts.append(f"=== {len(rows)} rollouts, mean score {sum(scores) / len(scores):.4f}, min {min(scores):.4f}, max {max(scores):.4f}")
    return "\n".join(parts)


def main(argv=None) -> str:
    ap = argparse.ArgumentParser()
    ap.add_argument("path")
    ap.add_argument("--step", type=int)
    ap.add_argument("--grep")
    ap.add_argument("--min-score", type=float)
    ap.add_argument("--max-score", type=float)
    ap.add_argument("--sort", choices=["score", "score_desc", "length"])
    ap.add_argument("--limit", type=int)
    ap.add_argument("--width", type=int, default=120)
    a = ap.parse_args(argv)
    text = render(select(load(a.path, a.step), a.grep, a.min_score, a.max_score, a.sort, a.limit), a.width)
    print(text)
    return text


if __name__ == "__main__":
    main()
