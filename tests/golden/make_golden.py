#!/usr/bin/env python3
"""Writes tests/golden/tiny_{A,B}.json: outputs of the plain implementation
(tests/plain_gpt2.py) on the two tiny random models, in the shape of the reference's
``logits`` probe (src/main.rs:285-312: argmax, first and last four logits, sum) plus greedy
ids.  The reference is Rust and cannot be compiled here (no Rust toolchain), so these values
rest on the formulas as restated in plain_gpt2.py, not on a run of the reference.

    python tests/golden/make_golden.py
"""
import json
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

from make_golden_lib import build_case  # noqa: E402

if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as tmp:
        for name in ("A", "B"):
            case = build_case(name, Path(tmp))
            (HERE / f"tiny_{name}.json").write_text(json.dumps(case, indent=1) + "\n")
            print("wrote", HERE / f"tiny_{name}.json")
