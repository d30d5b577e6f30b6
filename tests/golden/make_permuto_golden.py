"""Extracts the known answers the reference's own tests hold for the permutohedral encoder and the grid
hashes into tests/golden/permuto_reference.json.

    python tests/golden/make_permuto_golden.py <path to the reference checkout>

Sources (paths inside the reference): tests/neural/permuto-reference-data.slang (forward values, position
gradients, table gradients and the indices they belong to), tests/neural/permuto-encoder-precomputed-
constants.slang (per-level constants), tests/neural/hash-function-test.slang (22 hash values after "BUF")."""
import json
import os
import re
import sys


def arrays(text):
    out = {}
    for m in re.finditer(r"public static const (?:uint|int|float) (\w+)\s*(?:\[[^\]]*\])?\s*=\s*(\{[^}]*\}|[^;]+);", text):
        name, body = m.group(1), m.group(2)
        body = re.sub(r"//[^\n]*", "", body)
        nums = re.findall(r"-?\d+\.\d+|-?\d+", body.replace("f,", ",").replace("f\n", "\n").replace("u", ""))
        vals = [float(n) if "." in n else int(n) for n in nums]
        out[name] = vals if body.strip().startswith("{") else vals[0]
    return out


def main(ref):
    t = os.path.join(ref, "tests", "neural")
    data = arrays(open(os.path.join(t, "permuto-reference-data.slang")).read())
    consts = arrays(open(os.path.join(t, "permuto-encoder-precomputed-constants.slang")).read())
    hashes = [int(v) for v in re.findall(r"// BUF(?:-NEXT)?: (\d+)", open(os.path.join(t, "hash-function-test.slang")).read())]
    assert len(hashes) == 22 and len(data["EXPECTED_FORWARD_VALUES"]) == 128
    assert len(data["EXPECTED_DL_DPOS"]) == 32 and len(data["EXPECTED_DL_DPARAMS"]) == 64
    out = {"verify_positions": data["VERIFY_POSITIONS"], "forward": data["EXPECTED_FORWARD_VALUES"],
           "dl_dpos": data["EXPECTED_DL_DPOS"], "verify_param_indices": data["VERIFY_PARAM_INDICES"],
           "dl_dparams": data["EXPECTED_DL_DPARAMS"],
           "constants": {k: consts[k] for k in ("lc_maxLevel", "lc_offsets", "lc_tableSizes", "lc_scales", "lc_scalesPerDim", "lc_shiftsPerDim")},
           "hashes": hashes,
           "hash_positions": [[42], [17, 53], [137, 281, 419], [523, 661, 797, 937]]}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "permuto_reference.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote permuto_reference.json")


if __name__ == "__main__":
    main(sys.argv[1])
