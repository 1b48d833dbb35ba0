"""Checks reference_vectors.json against a checkout of the reference: every number of a case's expected output must
occur, in order, as a literal in the cited line range of the cited test file.  Run where the reference checkout
exists:  python tests/golden/verify_reference_vectors.py <path to the reference repository>"""
import json
import re
import sys
from pathlib import Path

EXPECT_KEYS = ("y", "gx", "gw", "gb", "right", "running_mean", "first_row")


def literals(text):
    return [float(m) for m in re.findall(r"(?<![\w.])-?\d+\.\d*(?:e-?\d+)?(?![\w.]*\()", text)]


def contains_in_order(haystack, needle):
    it = iter(haystack)
    return all(any(abs(h - n) < 1e-12 for h in it) for n in needle)


def main(root):
    cases = json.loads((Path(__file__).parent / "reference_vectors.json").read_text())["cases"]
    bad = 0
    for c in cases:
        path, span = c["source"].rsplit(":", 1)
        lo, hi = (int(v) for v in span.split("-"))
        lines = (Path(root) / path).read_text().splitlines()[lo - 1:hi]
        found = literals("\n".join(lines))
        for key in EXPECT_KEYS:
            if key in c and not contains_in_order(found, [float(v) for v in c[key]]):
                print(f"MISSING  {c['name']}: {key} = {c[key]} not found in {c['source']}")
                bad += 1
    print(f"{len(cases)} cases checked, {bad} problems")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "."))
