"""Writes tests/golden/matmul_kat.json: the known-answer vectors that the reference's own
tests hold for the matmul path (Tests/SwiftRTCoreTests/test_AlgebraicField.swift:551-645:
test_matmul is live; test_batchMatmul / test_leftBatchMatmul / test_rightBatchMatmul are
commented out there but numerically valid).

The literals below were transcribed from that file.  When run with a checkout of the
reference (`python make_kat.py /path/to/reference`), every transcribed number sequence is
also searched, in order, in the text of the corresponding test function, so a typo in the
transcription fails loudly.  Inputs are range-filled Float32 tensors (`array(0..<n, shape)`).
"""
import json
import os
import re
import sys

KAT = {
    "source": "Tests/SwiftRTCoreTests/test_AlgebraicField.swift:551-645",
    "dtype": "float32",
    "cases": {
        "test_matmul": {
            "a_shape": [3, 2], "b_shape": [2, 4],
            "c": [[4, 5, 6, 7], [12, 17, 22, 27], [20, 29, 38, 47]],
            "grad_a": [[6, 22], [6, 22], [6, 22]],
            "grad_b": [[6, 6, 6, 6], [9, 9, 9, 9]],
        },
        "test_batchMatmul": {
            "a_shape": [2, 3, 2], "b_shape": [2, 2, 4],
            "c": [[[4, 5, 6, 7], [12, 17, 22, 27], [20, 29, 38, 47]],
                  [[132, 145, 158, 171], [172, 189, 206, 223], [212, 233, 254, 275]]],
            "grad_a": [[[6, 22], [6, 22], [6, 22]], [[38, 54], [38, 54], [38, 54]]],
            "grad_b": [[[6, 6, 6, 6], [9, 9, 9, 9]], [[24, 24, 24, 24], [27, 27, 27, 27]]],
        },
        # the reference literal lists one batch item of c only (its shapes would give two);
        # that item is what is pinned
        "test_leftBatchMatmul": {
            "a_shape": [2, 3, 2], "b_shape": [2, 4],
            "c_first_item": [[4, 5, 6, 7], [12, 17, 22, 27], [20, 29, 38, 47]],
            "grad_a": [[[6, 22], [6, 22], [6, 22]], [[6, 22], [6, 22], [6, 22]]],
            "grad_b": [[30, 30, 30, 30], [36, 36, 36, 36]],
        },
        "test_rightBatchMatmul": {
            "a_shape": [3, 2], "b_shape": [2, 2, 4],
            "c": [[[4, 5, 6, 7], [12, 17, 22, 27], [20, 29, 38, 47]],
                  [[12, 13, 14, 15], [52, 57, 62, 67], [92, 101, 110, 119]]],
            "grad_a": [[44, 76], [44, 76], [44, 76]],
            "grad_b": [[[6, 6, 6, 6], [9, 9, 9, 9]], [[6, 6, 6, 6], [9, 9, 9, 9]]],
        },
    },
}


def _flat(x):
    if isinstance(x, list):
        for y in x:
            yield from _flat(y)
    else:
        yield x


def verify(reference_root: str) -> None:
    path = os.path.join(reference_root, "Tests/SwiftRTCoreTests/test_AlgebraicField.swift")
    text = open(path).read()
    for name, case in KAT["cases"].items():
        start = text.index("func " + name)
        nxt = text.find("func test_", start + 10)
        body = text[start: nxt if nxt > 0 else len(text)]
        nums = [float(t) for t in re.findall(r"(?<![\w.])\d+(?:\.\d+)?(?![\w.<])", body)]
        for key, val in case.items():
            if key.endswith("shape"):
                continue
            want = [float(v) for v in _flat(val)]
            it = iter(nums)
            if not all(any(w == n for n in it) for w in want):
                raise SystemExit(f"{name}.{key}: transcription not found in {path}")
    print("transcription verified against", path)


if __name__ == "__main__":
    if len(sys.argv) > 1:
        verify(sys.argv[1])
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matmul_kat.json")
    with open(out, "w") as f:
        json.dump(KAT, f, indent=1)
    print("wrote", out)
