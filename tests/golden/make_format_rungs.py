"""Writes tests/golden/format_rungs.json: every servable format of the reference's runtime contract
(gridbook/runtime_contract.json, the `formats` block) with the superblock size the reference's own
functions give it (gridbook/codec.py:40-41 for v1 layouts, tests/cb_torch_reference.py:194-196 for
the two-tier layout).  Run where the reference checkout is present:

    python tests/golden/make_format_rungs.py <reference root>
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import cb_torch_reference as ref
    from gridbook import codec
    contract = json.load(open(os.path.join(ref_root, "gridbook", "runtime_contract.json")))
    rows = []
    for fam in contract["formats"]:
        for k in fam["rungs"]:
            for version in fam["layout_versions"]:
                is_fp4 = fam["grid"] == "fp4"
                ts = ref.two_tier_v2_type_size(k) if (is_fp4 and version == 2) else codec.type_size(k, is_fp4)
                rows.append({"name": fam["name_pattern"].format(k=k), "grid": fam["grid"], "mode": fam["mode"],
                             "n_sub": fam["n_sub"], "k": k, "layout_version": version, "type_size": int(ts),
                             "served_in_moe": version in fam["moe_layout_versions"]})
    with open(os.path.join(HERE, "format_rungs.json"), "w") as f:
        json.dump({"contract_version": contract.get("contract_version"), "formats": rows}, f, indent=0)
    print(f"{len(rows)} format rungs written")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GRIDBOOK_REFERENCE", ""))
