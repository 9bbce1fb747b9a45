"""Extracts the expected outputs of the reference's vectorized-engine script tests into tests/golden/script_outputs.json.

test/api/cli/vectorized/run*.daphne are DaphneDSL scripts that print a few aggregates of rand(...) matrices; the
reference's test (VectorizedPipelineTest.cpp / MultiThreadedOpsTest.cpp) compares what a run prints with run*.txt.  This
script copies, AS TEXT, the printed values (one per line of the .txt) and the seeds and shapes of the rand calls (for
the record); tests/test_script_outputs.py restates each script as a sequence of kernel calls.

    python tests/golden/extract_script_outputs.py /path/to/daphne > tests/golden/script_outputs.json
"""
from __future__ import annotations

import json
import os
import re
import sys
from pathlib import Path

SCRIPTS = ["runRowAgg", "runColAgg", "runFullAgg", "runEwBinary", "runEwUnary", "runMatMult", "runOther",
           "runOuterBinary", "runReorganization", "runIndexing"]
RAND_RE = re.compile(r"(\w+)\s*=\s*rand\(([^)]*)\)\s*;")

if __name__ == "__main__":
    root = Path(sys.argv[1] if len(sys.argv) > 1 else
                os.environ.get("DAPHNE_ROOT") or Path(__file__).resolve().parents[3] / "reference")
    base = root / "test" / "api" / "cli" / "vectorized"
    out = {}
    for name in SCRIPTS:
        src, txt = base / f"{name}.daphne", base / f"{name}.txt"
        if not (src.exists() and txt.exists()):
            continue
        code = re.sub(r"(//|#)[^\n]*", "", src.read_text())
        out[name] = {"file": f"test/api/cli/vectorized/{name}.daphne",
                     "rand": {m.group(1): [a.strip() for a in m.group(2).split(",")] for m in RAND_RE.finditer(code)},
                     "prints": len(re.findall(r"\bprint\(", code)),
                     "expected": [ln.strip() for ln in txt.read_text().splitlines() if ln.strip()]}
        assert out[name]["prints"] == len(out[name]["expected"]), name
    json.dump({"source": "daphne-eu/daphne test/api/cli/vectorized (expected outputs of the script tests)",
               "scripts": out}, sys.stdout, indent=1)
    sys.stderr.write(f"{len(out)} scripts, {sum(len(v['expected']) for v in out.values())} printed values\n")
