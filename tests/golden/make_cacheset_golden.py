"""Generates tests/golden/cacheset_cases.json from the reference's cache-set test file: the five
literal cache-set states (cache tags, valid / modified flags, LFU counts and scale, per-row
counters, the ids to update with their increments) and the parameter triples of its randomised
cases, read from the C++ initialisers as text.  Run where a checkout of the reference lies beside
this repository (or pass its path):

    python tests/golden/make_cacheset_golden.py [path/to/reference]

Source: cpp/tests/wholegraph_tensor_ops/cacheset_tests.cu (states :509-720, randomised cases
:722-760 as `Random(base_scale, coverage, update_count)`).
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def parse(text):
    cases = []
    for m in re.finditer(r"static SingleCacheSetTestParam (\w+)\{(.*?)\};\n", text, flags=re.S):
        body, case = m.group(2), {}
        for f in re.finditer(r"\.(\w+)\s*=\s*(\{.*?\}|[^,{}]+?)\s*(?:,\s*(?=\.)|$)", body, flags=re.S):
            key, val = f.group(1), f.group(2).strip()
            if val.startswith("{"):
                items = [x.strip() for x in val.strip("{}").replace("\n", " ").split(",") if x.strip()]
                case[key] = [x == "true" if x in ("true", "false") else int(x.rstrip("L")) for x in items]
            elif val.startswith('"'):
                case[key] = val.strip('"')
            else:   # a scalar, possibly a product such as `564 * 2`
                case[key] = 1
                for factor in val.split("*"):
                    case[key] *= int(factor.strip().rstrip("L"))
        cases.append(case)
    randoms = [[int(a), int(b), int(c)] for a, b, c in
               re.findall(r"SingleCacheSetTestParam\(\)\.Random\((\d+),\s*(\d+),\s*(\d+)\)", text)]
    seen, unique = set(), []
    for r in randoms:
        if tuple(r) not in seen:
            seen.add(tuple(r))
            unique.append(r)
    return {"literal": cases, "random": unique}


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")
    path = os.path.join(ref, "cpp", "tests", "wholegraph_tensor_ops", "cacheset_tests.cu")
    data = parse(open(path).read())
    for c in data["literal"]:
        assert len(c["cache_tag_lids"]) == 32 and len(c["cache_tag_valid"]) == 32 and len(c["cache_lfu_count"]) == 32
        assert len(c["raw_counter"]) == c["cache_set_coverage"], c["name"]
        assert len(c["to_update_gids"]) == c["to_update_id_count"] == len(c["to_update_inc_count"])
    assert [c["name"] for c in data["literal"]] == ["modify_test", "small_test", "medium_test", "large_test",
                                                    "big_number_test"]
    with open(os.path.join(HERE, "cacheset_cases.json"), "w") as f:
        json.dump(data, f, separators=(",", ":"))
    print(len(data["literal"]), "literal states,", len(data["random"]), "random parameter triples")


if __name__ == "__main__":
    main()
