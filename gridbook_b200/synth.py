"""Seeded synthetic weights, activations and routings in the shapes, sizes and value
distributions of the benchmark configurations.  Everything is generated on the host
with numpy so the CUDA path and the CPU checker see the same bytes; the generators
mirror the reference's own fixtures (tests/cb_torch_reference.py:246-304,
tests/test_cuda_gemv.py:105-126, tests/bench_cuda_gemv.py:36-50)."""
from __future__ import annotations

import numpy as np

from .formats import CBFormat

E2M1_MAGS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_GRID = np.array(sorted({v for m in E2M1_MAGS for v in (m, -m)}), dtype=np.float32)  # 15 finite points
TWO_TIER_SUB_TABLE = (1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875,
                      2.0, 2.25, 2.5, 2.75, 3.0, 3.25, 3.5, 3.75)


def _e4m3_values() -> np.ndarray:
    vals = []
    for b in range(256):
        e, m = (b >> 3) & 0xF, b & 7
        if e == 0xF and m == 7:
            continue
        mag = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        vals.append(-mag if b & 0x80 else mag)
    return np.array(sorted(set(vals)), dtype=np.float32)


E4M3_FINITE = _e4m3_values()


def f32_to_e4m3_bytes(x: np.ndarray) -> np.ndarray:
    """Exact E4M3 byte of values that are already on the E4M3 grid."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(mag > 0, mag, 1.0))).astype(np.int32)
    e = np.clip(e, -6, 8)
    sub = mag < 2.0 ** -6
    man = np.where(sub, np.rint(mag * 512), np.rint((mag / np.exp2(e.astype(np.float32)) - 1) * 8)).astype(np.int32)
    byte = np.where(sub, man, ((e + 7) << 3) | man).astype(np.uint8)
    return byte | np.where(np.signbit(x), 0x80, 0).astype(np.uint8)


def compose_table(sub_table=TWO_TIER_SUB_TABLE) -> np.ndarray:
    t = np.asarray(sub_table, dtype=np.float64)
    with np.errstate(over="ignore"):
        return (t[None, :] * np.exp2(np.arange(256, dtype=np.float64)[:, None] - 127.0)
                ).astype(np.float32).reshape(-1)


def legal_supers(span: int | None = None) -> np.ndarray:
    """Super exponents for which every sub code composes to an exact E4M3 value in
    (0, 448]: with the default table that is 2^(E-127) * [1, 3.75] inside [2^-6, 448]."""
    full = np.arange(127 - 6, 127 + 7, dtype=np.int64)     # E in [121, 133]
    if span is None:
        return full
    start = (full.size - span) // 2
    return full[start:start + span]


def make_codebook(fmt: CBFormat, rng: np.random.Generator) -> np.ndarray:
    """Flat fp32 codebook block with on-grid values (tables concatenated row-major)."""
    n = fmt.codebook_elems()
    if fmt.is_fp4:
        pool = E2M1_MAGS if fmt.mode == "signed" else E2M1_GRID
    else:
        pool = E4M3_FINITE
    return pool[rng.integers(0, pool.size, n)].astype(np.float32)


def make_packed(fmt: CBFormat, rows: int, K: int, rng: np.random.Generator,
                super_span: int | None = 4) -> np.ndarray:
    """Random but format-legal packed rows [rows, K/256*type_size] uint8."""
    n_sb = K // 256
    blk = np.empty((rows, n_sb, fmt.type_size), dtype=np.uint8)
    blk[:, :, :4 * fmt.k] = rng.integers(0, 256, (rows, n_sb, 4 * fmt.k), dtype=np.uint8)
    if fmt.is_fp4 and fmt.scale_coding == "v1":
        # log-uniform in [2^-4, 2^2], rounded to E4M3
        s = np.exp2(rng.uniform(-4.0, 2.0, (rows, n_sb, 16))).astype(np.float32)
        e = np.floor(np.log2(s))
        man = np.rint((s / np.exp2(e) - 1.0) * 8.0)
        e = np.where(man == 8, e + 1, e)
        man = np.where(man == 8, 0, man)
        blk[:, :, 4 * fmt.k:] = ((e.astype(np.int32) + 7) << 3 | man.astype(np.int32)).astype(np.uint8)
    elif fmt.is_fp4:
        sup = legal_supers(super_span)
        blk[:, :, 4 * fmt.k] = sup[rng.integers(0, sup.size, (rows, n_sb))].astype(np.uint8)
        blk[:, :, 4 * fmt.k + 1:] = rng.integers(0, 256, (rows, n_sb, 8), dtype=np.uint8)
    return blk.reshape(rows, n_sb * fmt.type_size)


def make_linear(fmt: CBFormat, N: int, K: int, seed: int = 0, *, n_books: int = 1,
                global_scale: float | None = None, super_span: int | None = 4) -> dict:
    """One dense codebook linear.  ``n_books`` > 1 splits the rows into that many
    equal roles with their own codebook block (fused q/k/v or gate/up)."""
    rng = np.random.default_rng(seed)
    books = [make_codebook(fmt, rng) for _ in range(n_books)]
    d = dict(fmt=fmt, N=N, K=K, qw=make_packed(fmt, N, K, rng, super_span),
             cb=np.concatenate(books))
    if n_books > 1:
        per = -(-N // n_books)
        d["cb_row_offset"] = ((np.arange(N) // per) * fmt.codebook_elems()).astype(np.int32)
    else:
        d["cb_row_offset"] = None
    d["compose"] = compose_table() if fmt.scale_coding == "v2" else None
    d["weight_scale"] = None if fmt.is_fp4 else ((rng.random(N) + 0.5) * 0.02).astype(np.float32)
    d["global_scale"] = global_scale
    return d


def make_moe(fmt13: CBFormat, fmt2: CBFormat, E: int, hidden: int, inter: int, seed: int = 0,
             super_span: int | None = 4) -> tuple[dict, dict]:
    """Stacked expert weights: w13 [E, 2*inter, bytes(hidden)], w2 [E, hidden, bytes(inter)]."""
    rng = np.random.default_rng(seed)
    out = []
    for fmt, rows, kin in ((fmt13, 2 * inter, hidden), (fmt2, hidden, inter)):
        d = dict(fmt=fmt, N=rows, K=kin, cb=make_codebook(fmt, rng),
                 qw=make_packed(fmt, E * rows, kin, rng, super_span).reshape(E, rows, -1),
                 compose=compose_table() if fmt.scale_coding == "v2" else None,
                 scale=None if fmt.is_fp4 else ((rng.random((E, rows)) + 0.5) * 0.02).astype(np.float32))
        out.append(d)
    return out[0], out[1]


def bf16_round(x: np.ndarray) -> np.ndarray:
    f = np.ascontiguousarray(x, dtype=np.float32)
    b = f.view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32).reshape(f.shape)


def make_activations(M: int, K: int, seed: int = 0) -> np.ndarray:
    """bf16-valued N(0,1) activations as fp32."""
    return bf16_round(np.random.default_rng(seed + 7919).standard_normal((M, K)).astype(np.float32))


def make_routing(T: int, E: int, topk: int, seed: int = 0):
    """Router logits N(0,1) -> softmax -> top-k -> renormalised weights."""
    rng = np.random.default_rng(seed + 104729)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    ids = np.argsort(-p, axis=1, kind="stable")[:, :topk].astype(np.int32)
    w = np.take_along_axis(p, ids.astype(np.int64), axis=1)
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, w


# ---- host -> device -------------------------------------------------------------
def to_device_weight(d: dict, device, pad_rows: bool = False):
    """Upload one synthetic linear (or expert stack) and wrap it for the kernels."""
    import torch
    from . import kernels

    fmt = d["fmt"]
    qw = torch.from_numpy(np.ascontiguousarray(d["qw"]))
    if pad_rows:
        qw = torch.nn.functional.pad(qw, (0, 16))
    # sixteen readable bytes past the last row, as the kernels' windows want
    flat = torch.zeros(qw.numel() + 16, dtype=torch.uint8, device=device)
    flat[:qw.numel()] = qw.reshape(-1).to(device)
    qw_dev = flat[:qw.numel()].view(qw.shape)
    cb = torch.from_numpy(d["cb"])
    if fmt.is_fp4:
        cb_dev = cb.to(torch.bfloat16).to(device)
    else:
        cb_dev = torch.from_numpy(f32_to_e4m3_bytes(d["cb"])).to(device)
    off = d.get("cb_row_offset")
    comp = d.get("compose")
    ws = d.get("weight_scale", d.get("scale"))
    return kernels.make_weight(
        qw_dev, cb_dev, fmt, d["K"],
        cb_row_offset=None if off is None else torch.from_numpy(off).to(device),
        compose=None if comp is None else torch.from_numpy(comp).to(device),
        weight_scale=None if ws is None else torch.from_numpy(np.ascontiguousarray(ws)).to(device),
        global_scale=1.0 if d.get("global_scale") is None else float(d["global_scale"]))


def bf16_tensor(x: np.ndarray, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).to(device)


# ---- device-side generation (large stacks) ------------------------------------------
def make_packed_device(fmt: CBFormat, rows: int, K: int, gen, device, super_span: int = 4):
    """Same distributions as make_packed, drawn on the device by a seeded torch generator
    (GiB-sized stacks take seconds on the host RNG)."""
    import torch
    n_sb = K // 256
    blk = torch.empty((rows, n_sb, fmt.type_size), dtype=torch.uint8, device=device)
    blk[:, :, :4 * fmt.k] = torch.randint(0, 256, (rows, n_sb, 4 * fmt.k), generator=gen,
                                          dtype=torch.uint8, device=device)
    if fmt.is_fp4 and fmt.scale_coding == "v1":
        u = torch.rand((rows, n_sb, 16), generator=gen, device=device) * 6.0 - 4.0
        blk[:, :, 4 * fmt.k:] = torch.exp2(u).to(torch.float8_e4m3fn).view(torch.uint8)
    elif fmt.is_fp4:
        sup = torch.from_numpy(legal_supers(super_span)).to(device)
        pick = torch.randint(0, sup.numel(), (rows, n_sb), generator=gen, device=device)
        blk[:, :, 4 * fmt.k] = sup[pick].to(torch.uint8)
        blk[:, :, 4 * fmt.k + 1:] = torch.randint(0, 256, (rows, n_sb, 8), generator=gen,
                                                  dtype=torch.uint8, device=device)
    return blk.reshape(rows, n_sb * fmt.type_size)


def codebook_tables(fmt: CBFormat, seed: int):
    """Codebook tables [(rows, dims) fp32 tensors] of one format, on the host."""
    import torch
    flat = make_codebook(fmt, np.random.default_rng(seed))
    out, pos = [], 0
    for r, d in fmt.table_shapes():
        out.append(torch.from_numpy(flat[pos:pos + r * d].reshape(r, d).copy()))
        pos += r * d
    return out
