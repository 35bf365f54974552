"""Generate the golden fixtures in this directory from the REFERENCE itself.

Run once in a container that has the reference checked out (it imports the
reference's independent torch decoder and its codec on the CPU):

    python tests/golden/make_golden.py /path/to/reference

Every array written here is an output of reference code
(tests/cb_torch_reference.py, gridbook/codec.py) on seeded inputs that are
stored beside it, so the fixtures can be replayed anywhere without the
reference.  bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import cb_torch_reference as ref
    from gridbook import codec

    torch.manual_seed(0)
    out: dict[str, np.ndarray] = {}

    # ---- 1. FP4 product rungs, two-tier v2 scales, two codebooks by row ----
    for k in (12, 13, 16, 20):
        N, K = 6, 512
        ts = ref.two_tier_v2_type_size(k)
        tabs_a = ref.synth_product_codebook(k, seed=100 + k)
        tabs_b = ref.synth_product_codebook(k, seed=200 + k)
        flat = torch.cat([codec.build_flat_codebook(tabs_a, grid="fp4"),
                          codec.build_flat_codebook(tabs_b, grid="fp4")])
        off = torch.tensor([0, 0, 0, flat.numel() // 2, flat.numel() // 2, 0],
                           dtype=torch.int32)
        qw = ref.synth_two_tier_v2_plane(
            N, K, k, sub_table=codec.TWO_TIER_SUB_TABLE, seed=300 + k)
        compose = codec.build_compose_table(codec.TWO_TIER_SUB_TABLE)
        qwp = codec.pad_qweight(qw)
        codes = ref.extract_codewords(qwp, N=N, K=K, k_bits=k, type_size=ts)
        vals = ref.decode_cb_values(qwp, flat, off, N=N, K=K, k_bits=k, n_sub=2,
                                    type_size=ts)
        w = ref.reconstruct_cb_weight(qwp, flat, off, torch.zeros(1), compose,
                                      N=N, K=K, k_bits=k, n_sub=2, type_size=ts,
                                      is_fp4=True, is_v2=True)
        x = torch.randn(3, K).to(torch.bfloat16)
        xq = codec.fp4_group16_act_qdq(x)
        y = ref.cb_linear_reference(xq, qwp, flat, off, torch.zeros(1), compose,
                                    N=N, K=K, k_bits=k, n_sub=2, type_size=ts,
                                    is_fp4=True, is_v2=True)
        p = f"fp4v2_k{k}_"
        out[p + "qw"] = qw.numpy()
        out[p + "cb"] = bits(flat)
        out[p + "off"] = off.numpy()
        out[p + "codes"] = codes.numpy().astype(np.int32)
        out[p + "vals"] = bits(vals)
        out[p + "w"] = bits(w)
        out[p + "x"] = bits(x)
        out[p + "xq"] = bits(xq)
        out[p + "y"] = bits(y)
    out["compose"] = codec.build_compose_table(codec.TWO_TIER_SUB_TABLE).numpy()
    out["compose_u8"] = codec.build_compose_u8().numpy()
    out["legal_supers"] = ref.two_tier_full_legal_supers(
        codec.TWO_TIER_SUB_TABLE).numpy().astype(np.int32)

    # ---- 2. FP4 v1 scale bytes (pre-decoded plane route of the reference) ----
    k, N, K = 14, 4, 256
    ts = codec.type_size(k, True)
    g = torch.Generator().manual_seed(7)
    qw = torch.randint(0, 256, (N, ts), generator=g, dtype=torch.uint8)
    # scale bytes: finite positive E4M3 only
    qw[:, 4 * k:] = torch.randint(8, 0x77, (N, 16), generator=g, dtype=torch.uint8)
    tabs = ref.synth_product_codebook(k, seed=9)
    flat = codec.build_flat_codebook(tabs, grid="fp4")
    plane = codec.decode_fp4_scale_plane(qw, k)
    off = torch.zeros(N, dtype=torch.int32)
    w = ref.reconstruct_cb_weight(codec.pad_qweight(qw), flat, off, plane,
                                  torch.zeros(1), N=N, K=K, k_bits=k, n_sub=2,
                                  type_size=ts, is_fp4=True, is_v2=False)
    out["fp4v1_k14_qw"] = qw.numpy()
    out["fp4v1_k14_cb"] = bits(flat)
    out["fp4v1_k14_plane"] = plane.numpy()
    out["fp4v1_k14_w"] = bits(w)

    # ---- 3. FP4 signed mode ----
    k, N, K = 13, 3, 256
    ts = ref.two_tier_v2_type_size(k)
    qw = ref.synth_two_tier_v2_plane(N, K, k, sub_table=codec.TWO_TIER_SUB_TABLE,
                                     seed=11)
    mags = torch.tensor(ref.E2M1_MAGNITUDES)
    g = torch.Generator().manual_seed(12)
    flat = mags[torch.randint(0, 8, ((1 << (k - 8)) * 8,), generator=g)].to(
        torch.bfloat16)
    off = torch.zeros(N, dtype=torch.int32)
    w = ref.reconstruct_cb_weight(codec.pad_qweight(qw), flat, off, torch.zeros(1),
                                  codec.build_compose_table(codec.TWO_TIER_SUB_TABLE),
                                  N=N, K=K, k_bits=k, n_sub=1, type_size=ts,
                                  is_fp4=True, is_v2=True)
    out["fp4s_k13_qw"] = qw.numpy()
    out["fp4s_k13_cb"] = bits(flat)
    out["fp4s_k13_w"] = bits(w)

    # ---- 4. FP8 product rungs (n_sub 4 incl. ragged splits; n_sub 2 k16) ----
    for k, n_sub in ((28, 4), (30, 4), (32, 4), (37, 4), (16, 2)):
        N, K = 5, 512
        ts = 4 * k
        g = torch.Generator().manual_seed(400 + k)
        qw = torch.randint(0, 256, (N, (K // 256) * ts), generator=g,
                           dtype=torch.uint8)
        widths = ref._split_widths(k, n_sub)
        subs = [(torch.randn(1 << w_, 8 // n_sub, generator=g) * 4.0)
                .to(torch.float8_e4m3fn).float() for w_ in widths]
        flat = codec.build_flat_codebook(subs, grid="fp8")
        cb8 = codec.flat_codebook_fp8(flat)
        ws = ((torch.rand(N, generator=g) + 0.5) * 0.02).float()
        off = torch.zeros(N, dtype=torch.int32)
        qwp = codec.pad_qweight(qw)
        vals = ref.decode_cb_values(qwp, flat, off, N=N, K=K, k_bits=k,
                                    n_sub=n_sub, type_size=ts)
        w = ref.reconstruct_cb_weight(qwp, flat, off, ws, torch.zeros(1), N=N,
                                      K=K, k_bits=k, n_sub=n_sub, type_size=ts,
                                      is_fp4=False)
        x = torch.randn(2, K).to(torch.bfloat16)
        xq = codec.fp8_dynamic_act_qdq(x)
        y = ref.cb_linear_reference(xq, qwp, flat, off, ws, torch.zeros(1), N=N,
                                    K=K, k_bits=k, n_sub=n_sub, type_size=ts,
                                    is_fp4=False)
        p = f"fp8_k{k}_n{n_sub}_"
        out[p + "qw"] = qw.numpy()
        out[p + "cb"] = bits(flat)
        out[p + "cb8"] = cb8.numpy()
        out[p + "ws"] = ws.numpy()
        out[p + "vals8"] = vals.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        out[p + "w"] = bits(w)
        out[p + "x"] = bits(x)
        out[p + "xq"] = bits(xq)
        out[p + "y"] = bits(y)

    # ---- 5. activation buckets, incl. the exact-midpoint trap ----
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(4, 256, generator=g) * 3).to(torch.bfloat16)
    amax = 1.7265625
    x[0, :16] = torch.tensor([amax, -amax / 8, amax / 8, 0.0] * 4).to(torch.bfloat16)
    x[1, 16:32] = 0.0                                   # all-zero group
    x[2, 0] = 1000.0                                    # outlier token
    out["act_x"] = bits(x)
    out["act_fp4"] = bits(codec.fp4_group16_act_qdq(x))
    out["act_fp8"] = bits(codec.fp8_dynamic_act_qdq(x))
    gs = torch.tensor(0.37, dtype=torch.float32)
    packed, sf, recip = codec.nvfp4_act_quant_ref(x.float(), gs)
    out["act_nvfp4_packed"] = packed.numpy()
    out["act_nvfp4_sf"] = sf.numpy()
    out["act_nvfp4_recip"] = recip.numpy().reshape(1)

    # ---- 6. scale-factor swizzle ----
    sfb = torch.arange(130 * 6, dtype=torch.int32).remainder(251).to(
        torch.uint8).reshape(130, 6)
    out["sf_plain"] = sfb.numpy()
    out["sf_swizzled"] = codec.swizzle_sf_plane(sfb).numpy()

    # ---- 7. routed MoE, per-expert loop chain (FP4 K16 v2) built from the
    #         reference primitives, in the order of tests/test_cuda_gemv.py:329-348
    E, hidden, inter, k, T, topk = 4, 256, 256, 16, 3, 2
    ts = ref.two_tier_v2_type_size(k)
    tabs = ref.synth_product_codebook(k, seed=31)
    flat = codec.build_flat_codebook(tabs, grid="fp4")
    compose = codec.build_compose_table(codec.TWO_TIER_SUB_TABLE)
    w13 = torch.stack([ref.synth_two_tier_v2_plane(
        2 * inter, hidden, k, sub_table=codec.TWO_TIER_SUB_TABLE, seed=40 + e,
        super_span=4) for e in range(E)])
    w2 = torch.stack([ref.synth_two_tier_v2_plane(
        hidden, inter, k, sub_table=codec.TWO_TIER_SUB_TABLE, seed=50 + e,
        super_span=4) for e in range(E)])
    g = torch.Generator().manual_seed(33)
    x = torch.randn(T, hidden, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)])
    tw = torch.rand(T, topk, generator=g).float()

    def lin(xq, stack, e, rows, kin):
        return ref.cb_linear_reference(
            xq, codec.pad_qweight(stack[e].contiguous()), flat,
            torch.zeros(rows, dtype=torch.int32), torch.zeros(1), compose,
            N=rows, K=kin, k_bits=k, n_sub=2, type_size=ts, is_fp4=True,
            is_v2=True)

    ref_out = torch.zeros(T, hidden, dtype=torch.bfloat16)
    for e in range(E):
        sel = ids == e
        if not bool(sel.any()):
            continue
        tok, slot = torch.where(sel)
        xe = codec.fp4_group16_act_qdq(x[tok]).to(torch.bfloat16)
        gu = lin(xe, w13, e, 2 * inter, hidden)
        gate, up = gu.chunk(2, dim=-1)
        a = F.silu(gate) * up
        aq = codec.fp4_group16_act_qdq(a).to(torch.bfloat16)
        oe = lin(aq, w2, e, hidden, inter)
        oe = oe * tw[tok, slot][:, None].to(oe.dtype)
        ref_out.index_add_(0, tok, oe)
    out["moe_w13"] = w13.numpy()
    out["moe_w2"] = w2.numpy()
    out["moe_cb"] = bits(flat)
    out["moe_x"] = bits(x)
    out["moe_ids"] = ids.numpy().astype(np.int32)
    out["moe_tw"] = tw.numpy()
    out["moe_out"] = bits(ref_out)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
