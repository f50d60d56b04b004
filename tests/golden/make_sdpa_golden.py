"""Extracts the six SDPA golden cases of autorust's tests/attention_golden.rs into a JSON fixture.

The reference file is generated data (tinygrad's outputs for arange-style inputs; generator
py/dump_attention_golden.py:17-45).  This script reads it as text -- nothing of the reference is
executed -- and writes tests/golden/sdpa_golden.json, which the CPU test suite checks the oracle
against with the reference's own tolerance, |a-b| <= 1e-5 * max(|b|, 1) (tests/nn_attention.rs:19-21,54).

Usage:  python tests/golden/make_sdpa_golden.py [path/to/autorust]
"""
from __future__ import annotations

import json
import os
import re
import sys
from pathlib import Path


def parse(text: str) -> list[dict]:
    cases = []
    for block in re.findall(r"SdpaGolden\s*\{(.*?)\n    \},", text, flags=re.S):
        case: dict = {}
        case["name"] = re.search(r'name:\s*"([^"]+)"', block).group(1)
        for field in ("q_shape", "k_shape", "v_shape", "mask_shape", "out_shape"):
            body = re.search(field + r":\s*&\[(.*?)\]", block, flags=re.S).group(1)
            case[field] = [int(x) for x in body.replace("\n", " ").split(",") if x.strip()]
        for field in ("q", "k", "v", "mask", "out"):
            body = re.search(r"\b" + field + r":\s*&\[(.*?)\]", block, flags=re.S).group(1)
            case[field] = [float(x) for x in body.replace("\n", " ").split(",") if x.strip()]
        for field in ("mask_bool", "is_causal", "enable_gqa"):
            case[field] = re.search(field + r":\s*(true|false)", block).group(1) == "true"
        cases.append(case)
    return cases


def main() -> None:
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else
               os.environ.get("AUTORUST_REFERENCE_DIR") or Path(__file__).resolve().parents[3] / "reference")
    text = (ref / "tests" / "attention_golden.rs").read_text()
    cases = parse(text)
    assert len(cases) == 6, f"expected 6 golden cases, found {len(cases)}"
    out = Path(__file__).resolve().parent / "sdpa_golden.json"
    out.write_text(json.dumps({"source": "tests/attention_golden.rs", "rtol": 1e-5, "cases": cases}, indent=1))
    print(f"wrote {out} ({len(cases)} cases: {[c['name'] for c in cases]})")


if __name__ == "__main__":
    main()
