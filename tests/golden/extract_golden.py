"""Reads the known-answer arrays out of the reference's own CPU tests (as text) and
writes them as JSON fixtures next to this script.

Run once where the reference tree is mounted:
    python tests/golden/extract_golden.py /path/to/hipTensor

Sources (paths inside the reference project):
  test/02_permutation/permutation_cpu_impl_test.cpp:82-107
      A[w,h,c,n] = iota, extents w=3 h=2 c=4 n=5, B[c,n,h,w] = 2.1 * A, both layouts
  test/03_reduction/reduction_cpu_impl_test.cpp:73-83
      A[m,h,k,v] = iota, extents m=3 h=5 k=6 v=4, C[k,v] = 1, ADD over {m,h},
      alpha = 1.2, beta = 2.1, C aliases D, both layouts
"""
import json
import os
import re
import sys


def arrays(path):
    text = open(path).read()
    out = []
    for m in re.finditer(r"referenceArray\s*=\s*\{([^}]*)\}", text, re.S):
        vals = [float(tok.rstrip("f")) for tok in re.split(r"[,\s]+", m.group(1).strip()) if tok]
        out.append(vals)
    return out


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    perm = arrays(os.path.join(ref, "test/02_permutation/permutation_cpu_impl_test.cpp"))
    red = arrays(os.path.join(ref, "test/03_reduction/reduction_cpu_impl_test.cpp"))
    assert len(perm) == 2 and len(perm[0]) == 120 and len(perm[1]) == 120
    assert len(red) == 2 and len(red[0]) == 24 and len(red[1]) == 24
    json.dump({"source": "test/02_permutation/permutation_cpu_impl_test.cpp:82-107",
               "modeA": "whcn", "modeB": "cnhw", "extent": {"w": 3, "h": 2, "c": 4, "n": 5},
               "alpha": 2.1, "input": "iota",
               "expected_first_mode_fastest": perm[0], "expected_last_mode_fastest": perm[1]},
              open(os.path.join(here, "permutation_whcn_cnhw.json"), "w"), indent=1)
    json.dump({"source": "test/03_reduction/reduction_cpu_impl_test.cpp:73-83",
               "modeA": "mhkv", "modeC": "kv", "extent": {"m": 3, "h": 5, "k": 6, "v": 4},
               "alpha": 1.2, "beta": 2.1, "op": "ADD", "input": "iota", "C": 1.0,
               "expected_default_build": red[0], "expected_other_layout": red[1]},
              open(os.path.join(here, "reduction_mhkv_kv.json"), "w"), indent=1)


if __name__ == "__main__":
    main(sys.argv[1])
