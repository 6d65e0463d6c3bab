"""Reads the contraction problem lists of the reference's validation harness (YAML, as text) and writes them
as one JSON fixture next to this script: per file the tensor data types, alphas, betas, lengths and modes.

Run once where the reference tree is mounted:
    python tests/golden/extract_shapes.py /path/to/hipTensor

Sources (paths inside the reference project): test/01_contraction/configs/validation/
    {bilinear,scale,complex_bilinear,complex_scale}_test_params_rank{1..6}.yaml
"""
import json
import os
import sys

import yaml


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    out = {}
    base = os.path.join(ref, "test/01_contraction/configs/validation")
    for kind in ("bilinear", "scale", "complex_bilinear", "complex_scale"):
        for rank in range(1, 7):
            name = "%s_test_params_rank%d.yaml" % (kind, rank)
            doc = yaml.safe_load(open(os.path.join(base, name)))
            out["%s_rank%d" % (kind, rank)] = {
                "source": "test/01_contraction/configs/validation/" + name,
                "types": doc["Tensor Data Types"],  # A, B, C, D, compute
                "alphas": doc["Alphas"],
                "betas": doc.get("Betas", []),
                "lengths": doc["Lengths"],  # per problem: A, B, D
                "modes": doc["Modes"][0],  # A, B, D
            }
            assert len(doc["Modes"]) == 1
    json.dump(out, open(os.path.join(here, "contraction_validation_shapes.json"), "w"), indent=0, separators=(",", ":"))
    print("wrote %d lists" % len(out))


if __name__ == "__main__":
    main(sys.argv[1])
