"""Writes tests/golden/lstm_kat.json from the golden data of the reference's LSTM test
(Tests/SwiftRTLayerTests/test_Recurrent.swift:97-240): four time steps of a 4 -> 4 LSTM cell
with given fused weights [8 x 16], fused bias [16] and initial state, the hidden state after
every step, the final cell state, and the gradients of sum(final cell) with respect to the
weights, the bias, the inputs and the initial state.

The test body itself is commented out in the reference, but the data is what pins
matmul(_:_:bias:) -- the fused product of LSTMCell.callAsFunction
(Sources/SwiftRTLayers/Recurrent.swift:255-266) -- and the bias gradient (a column sum).

Usage: python make_lstm_kat.py /path/to/reference     (reads the Swift file as text)
"""
import json
import os
import re
import sys

NAMES = ["lstmInputs", "lstmInitialCellFusedWeights", "lstmInitialCellFusedBias", "lstmInitialStateCell",
         "lstmInitialStateHidden", "lstmExpectedStates", "lstmExpectedOutput", "lstmExpectedGradFusedWeights",
         "lstmExpectedGradFusedBias", "lstmExpectedGradX", "lstmExpectedGradInitialStateCell",
         "lstmExpectedGradInitialStateHidden"]


def parse(text: str) -> dict:
    out = {}
    for name in NAMES:
        m = re.search(r"^let " + name + r"\s*=\s*", text, re.M)
        if not m:
            raise SystemExit(f"{name} not found")
        # the literal runs to the next top-level `let` (or the end of the file)
        nxt = re.search(r"^let ", text[m.end():], re.M)
        body = text[m.end(): m.end() + nxt.start()] if nxt else text[m.end():]
        body = re.sub(r"array\(", "", body).replace(")", "")
        body = re.sub(r",\s*\]", "]", body)             # trailing commas
        out[name] = json.loads(body)
    return out


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    path = os.path.join(sys.argv[1], "Tests", "SwiftRTLayerTests", "test_Recurrent.swift")
    data = parse(open(path).read())
    kat = {
        "source": "Tests/SwiftRTLayerTests/test_Recurrent.swift:97-240",
        "dtype": "float32",
        "accuracy": 1e-6,
        "gate_order": ["input", "update", "forget", "output"],
        "inputs": [step[0] for step in data["lstmInputs"]],                  # [T][inputSize]
        "fused_weight": data["lstmInitialCellFusedWeights"],                 # [inputSize + hiddenSize][4 hiddenSize]
        "fused_bias": data["lstmInitialCellFusedBias"],
        "initial_cell": data["lstmInitialStateCell"][0],
        "initial_hidden": data["lstmInitialStateHidden"][0],
        "expected_hidden_per_step": data["lstmExpectedStates"],              # [T][hiddenSize]
        "expected_final_cell": data["lstmExpectedOutput"][0],
        "grad_fused_weight": data["lstmExpectedGradFusedWeights"],
        "grad_fused_bias": data["lstmExpectedGradFusedBias"],
        "grad_inputs": data["lstmExpectedGradX"],
        "grad_initial_cell": data["lstmExpectedGradInitialStateCell"][0],
        "grad_initial_hidden": data["lstmExpectedGradInitialStateHidden"][0],
    }
    assert len(kat["inputs"]) == 4 and len(kat["fused_weight"]) == 8 and len(kat["fused_weight"][0]) == 16
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lstm_kat.json")
    with open(dst, "w") as f:
        json.dump(kat, f, indent=1)
    print(dst)


if __name__ == "__main__":
    main()
