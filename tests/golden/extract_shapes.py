"""Reads the problem lists of the reference's validation harness (YAML, as text) and writes them as JSON
fixtures next to this script: contractions (per file the tensor data types, alphas, betas, lengths and modes),
permutations (data types, alphas, lengths, operator pairs, permuted dims) and reductions (data types, alphas,
betas, lengths, operators, output dims).

Run once where the reference tree is mounted:
    python tests/golden/extract_shapes.py /path/to/hipTensor

Sources (paths inside the reference project): test/01_contraction/configs/validation/
    {bilinear,scale,complex_bilinear,complex_scale}_test_params_rank{1..6}.yaml
  test/02_permutation/configs/validation/rank{2..6}_test_params.yaml
  test/03_reduction/configs/validation/rank{1..6}_test_params.yaml
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
    perm = {}
    for rank in range(2, 7):
        name = "test/02_permutation/configs/validation/rank%d_test_params.yaml" % rank
        doc = yaml.safe_load(open(os.path.join(ref, name)))
        perm["rank%d" % rank] = {"source": name, "types": doc["Tensor Data Types"], "alphas": doc["Alphas"],
                                 "lengths": doc["Lengths"], "operators": doc["Operators"],
                                 "permuted_dims": doc["Permuted Dims"]}
    json.dump(perm, open(os.path.join(here, "permutation_validation_lists.json"), "w"), indent=0, separators=(",", ":"))
    red = {}
    for rank in range(1, 7):
        name = "test/03_reduction/configs/validation/rank%d_test_params.yaml" % rank
        doc = yaml.safe_load(open(os.path.join(ref, name)))
        red["rank%d" % rank] = {"source": name, "types": doc["Tensor Data Types"], "alphas": doc["Alphas"],
                                "betas": doc["Betas"], "lengths": doc["Lengths"], "operators": doc["Operators"],
                                "output_dims": doc["Output Dims"]}
    json.dump(red, open(os.path.join(here, "reduction_validation_lists.json"), "w"), indent=0, separators=(",", ":"))
    print("wrote %d permutation and %d reduction lists" % (len(perm), len(red)))


if __name__ == "__main__":
    main(sys.argv[1])
