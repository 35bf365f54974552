"""Writes tests/golden/act_edge_cases.json: the reference codec's activation buckets
(gridbook/codec.py:248-260 group-16 E2M1, 428-437 per-token E4M3) on the rows its kernel test pins
(tests/test_fp4_act_qdq.py:107-149): a NaN, +inf and -inf inside a group, signed zeros, the smallest
bf16 subnormals, and the reciprocal-versus-divide midpoint.  Inputs and outputs are bf16 bit
patterns.  Run where the reference checkout is present:

    python tests/golden/make_act_edge_cases.py <reference root>
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor):
    return [int(v) & 0xFFFF for v in t.to(torch.bfloat16).contiguous().view(torch.int16).flatten().tolist()]


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from gridbook import codec
    nan, inf = float("nan"), float("inf")
    amax = 1.7265625
    cases = {
        "nonfinite": torch.tensor([[nan, 1.0] + [0.0] * 14 + [1.0, -2.0] + [0.5] * 14,
                                   [inf, -1.0] + [0.0] * 14 + [3.0, 0.25] + [0.0] * 14,
                                   [-inf, 1.0] + [0.0] * 14 + [nan] + [1.0] * 15], dtype=torch.bfloat16),
        "signed_zero_subnormal": torch.tensor([0, -32768, 1, -32767] * 8, dtype=torch.int16)
        .view(torch.bfloat16).reshape(1, 32),
        "midpoint": torch.tensor([[amax] + [-amax / 8.0] * 15 + [-amax] + [amax / 8.0] * 15], dtype=torch.bfloat16),
    }
    out = {}
    for name, x in cases.items():
        out[name] = {"shape": list(x.shape), "x": bits(x), "fp4": bits(codec.fp4_group16_act_qdq(x)),
                     "fp8": bits(codec.fp8_dynamic_act_qdq(x))}
    with open(os.path.join(HERE, "act_edge_cases.json"), "w") as f:
        json.dump(out, f, indent=1)
    print({k: v["shape"] for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
