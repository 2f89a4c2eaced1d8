"""Writes reference_known_answers.json: the known-answer vectors that the reference's own test suites hold for the hot
path, transcribed from its test sources (inputs and the expected values they assert; closed forms such as cos(1) are
evaluated here in float64).  The reference stores no other outputs for this path -- its parity tests compare back ends
with each other -- so this file is short.

    TTT = CallaghanDev.ML.TestConsoleApp/Tests/TransformerTests.cs
    RPT = CallaghanDev.ML.TestConsoleApp/Tests/RotaryPositionEmbeddingTests.cs

Run: python tests/golden/make_known_answers.py   (needs nothing but the standard library)
"""
import json
import math
from pathlib import Path

c1, s1, s2, c2 = math.cos(1.0), math.sin(1.0), math.sin(2.0), math.cos(2.0)
cases = {
    "matmul_transpose": {  # TTT:664-674: C = A * B^T, three entries asserted
        "source": "TransformerTests.cs:664-674",
        "A": [[1, 2], [3, 4]], "B": [[5, 6], [7, 8], [9, 10]],
        "expected_entries": [[0, 0, 17.0], [0, 1, 23.0], [1, 2, 67.0]], "tolerance": 1e-6,
    },
    "layernorm_unit_gamma": {  # TTT:676-701: gamma 1, beta 0 -> every row has mean 0 (1e-5) and variance 1 (1e-3)
        "source": "TransformerTests.cs:676-701",
        "input": [[1, 2, 3, 4], [-1, 0, 1, 2]], "row_mean": 0.0, "row_mean_tolerance": 1e-5, "row_variance": 1.0, "row_variance_tolerance": 1e-3,
    },
    "rope_known_values": {  # RPT:156-177: one head of width 2, theta = position
        "source": "RotaryPositionEmbeddingTests.cs:156-177",
        "input": [[1, 0], [1, 0], [0, 1]], "num_heads": 1,
        "expected": [[1.0, 0.0], [c1, s1], [-s2, c2]], "tolerance": 1e-5,
    },
    "rope_heads_independent": {  # RPT:135-154 (position 0 unchanged) and RPT:179-196 (two heads rotate independently)
        "source": "RotaryPositionEmbeddingTests.cs:135-154,179-196",
        "input": [[1, 2, 3, 4], [1, 0, 0, 1]], "num_heads": 2,
        "expected": [[1.0, 2.0, 3.0, 4.0], [c1, s1, -s1, c1]], "tolerance": 1e-5,
    },
}
Path(__file__).with_name("reference_known_answers.json").write_text(json.dumps(cases, indent=1) + "\n")
