"""Transcribe the reference's own known-answer vectors into a JSON fixture.

NNlib.jl is Julia and cannot run where these tests run, but its test-suite
carries literal known-answer vectors for the attention path.  This script reads
those test files AS TEXT from a checkout of the reference (its path is the one argument)
and writes ``nnlib_attention_golden.json`` next to itself:

* ``test/attention.jl`` "specific results": ``ytrue`` (12 values) and ``αtrue``
  (18 values) for ``q = k = v = reshape(1:12, 4, 3, 1) ./ 12, nheads = 2``;
* ``test/softmax.jl`` "softmax with Inf, NaN": the 2x2 input/output tables;
* ``test/softmax.jl`` first tests: ``softmax([0, 0])`` and the -100000 pair.

Run:  python tests/golden/make_golden.py <path-to-an-NNlib.jl-checkout>
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path


def _floats(txt: str):
    return [float(t) for t in re.findall(r"-?\d+\.\d+(?:e-?\d+)?|-?\d+", txt)]


def _jl_matrix(txt: str):
    """'1 2; 3 Inf' -> [[1,2],[3,inf]] (row-major list of rows)."""
    rows = []
    for row in txt.split(";"):
        vals = []
        for tok in row.split():
            tok = tok.strip()
            if tok in ("Inf", "Inf32"):
                vals.append("inf")
            elif tok in ("-Inf", "-Inf32"):
                vals.append("-inf")
            elif tok == "NaN":
                vals.append("nan")
            else:
                vals.append(float(tok))
        rows.append(vals)
    return rows


def main(ref: Path) -> None:
    att = (ref / "test" / "attention.jl").read_text()
    sm = (ref / "test" / "softmax.jl").read_text()
    out = {"source": "FluxML/NNlib.jl test/attention.jl, test/softmax.jl (transcribed as text)"}

    m = re.search(r'@testset "specific results" begin(.*?)\nend', att, re.S)
    block = m.group(1)
    ytrue = _floats(re.search(r"ytrue = \[(.*?)\]", block, re.S).group(1))
    atrue = _floats(re.search(r"αtrue = \[(.*?)\]", block, re.S).group(1))
    assert len(ytrue) == 12 and len(atrue) == 18
    out["attention_specific"] = {
        "input": "q = k = v = reshape(1:12, 4, 3, 1) ./ 12; nheads = 2",
        "q_shape": [4, 3, 1], "nheads": 2,
        "ytrue_shape": [4, 3, 1], "ytrue_colmajor": ytrue,
        "alphatrue_shape": [3, 3, 2, 1], "alphatrue_colmajor": atrue,
        "atol": 1e-5,
        "where": "test/attention.jl:25-34",
    }

    cases = []
    for mm in re.finditer(r"@test softmax\(Float32\[(.*?)\]\) ≈\s+Float32\[(.*?)\]( nans=true)?", sm):
        cases.append({"x": _jl_matrix(mm.group(1)), "y": _jl_matrix(mm.group(2)), "dims": 1,
                      "nans": bool(mm.group(3))})
    mm = re.search(r"@test softmax\(Float32\[(.*?)\]; dims=2\) ≈ Float32\[(.*?)\]", sm)
    cases.append({"x": _jl_matrix(mm.group(1)), "y": _jl_matrix(mm.group(2)), "dims": 2, "nans": False})
    assert len(cases) == 5, len(cases)
    out["softmax_inf_nan"] = {"cases": cases, "where": "test/softmax.jl:61-68"}
    assert "softmax(Int[0, 0]) == [0.5, 0.5]" in sm and "xs = [-100_000.0, -100_000.0]" in sm
    out["softmax_basic"] = {
        "cases": [{"x": [0, 0], "y": [0.5, 0.5]}, {"x": [-100000.0, -100000.0], "y": [0.5, 0.5]}],
        "where": "test/softmax.jl:5,22-23",
    }
    dst = Path(__file__).resolve().parent / "nnlib_attention_golden.json"
    dst.write_text(json.dumps(out, indent=1, ensure_ascii=False) + "\n")
    print("wrote", dst)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of an NNlib.jl checkout>")
    main(Path(sys.argv[1]))
