"""CPU oracle for the gridbook codebook-decode linear / routed MoE hot path.

TEST INFRASTRUCTURE ONLY.  This module is a plain-numpy restatement of the
reference's CPU algorithm.  It is imported by the tests, by the smoke check and
by the CPU-baseline leg of the benchmark, and by nothing that ships: the product
path is the CUDA library and fails closed without it.

Parity is PINNED: every function here is checked against (a) the reference's own
hand-packed known-answer constructions (tests/test_cb_torch_reference.py:20-101,
docs/SPEC.md:224-240) and (b) fixtures produced by importing the reference's
torch oracle and codec in the build container (tests/golden/make_golden.py).
One multiplier is unpinned because the reference has no counterpart for it: the
fp32 "global scale" of the BASELINE-literal format, applied here as an epilogue
multiplier (see ``cb_linear``).

Reference citations (paths inside the reference project):
  * bit extraction           tests/cb_torch_reference.py:33-74
  * value decode             tests/cb_torch_reference.py:77-127, docs/SPEC.md:94-128
  * weight reconstruction    tests/cb_torch_reference.py:130-178
  * linear                   tests/cb_torch_reference.py:307-330
  * compose table            gridbook/codec.py:170-183
  * v1 scale plane           gridbook/codec.py:186-194
  * activation buckets       gridbook/codec.py:248-260, 428-437, 377-425
  * MoE loop chain           tests/test_cuda_gemv.py:329-348
  * routing                  gridbook/moe.py:2400-2411, gridbook/moe_routing.py:99-207
"""
from __future__ import annotations

import numpy as np

SUPERBLOCK = 256
FP4_GROUP = 16
E4M3_MAX = 448.0
TWO_TIER_SUPER_BIAS = 127
TWO_TIER_SUB_TABLE = (1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875,
                      2.0, 2.25, 2.5, 2.75, 3.0, 3.25, 3.5, 3.75)
E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)

MODE_PRODUCT = "product"
MODE_SIGNED = "signed"
MODE_FULL = "full"


# --------------------------------------------------------------------------
# scalar formats
# --------------------------------------------------------------------------
def _e4m3_table() -> np.ndarray:
    """All 256 float8_e4m3fn byte values as fp32 (0x7F / 0xFF are NaN)."""
    out = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        exp = (b >> 3) & 0xF
        man = b & 7
        if exp == 0xF and man == 7:
            val = np.nan
        elif exp == 0:
            val = man * 2.0 ** -9
        else:
            val = (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        out[b] = sign * val
    return out


E4M3_TO_F32 = _e4m3_table()


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return E4M3_TO_F32[np.asarray(b, dtype=np.uint8)]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e4m3fn byte, single rounding, nearest-even, the c10
    conversion torch uses (values >= 480 become NaN 0x7F; callers pre-clamp).
    Restated from the algorithm cited at gridbook/csrc/cb_gemv.cu:103-129."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    sign = bits & 0x80000000
    mag = bits ^ sign
    res = np.zeros(mag.shape, dtype=np.uint64)
    over = mag >= (1087 << 20)
    sub = (~over) & (mag < (121 << 23))
    nrm = ~(over | sub)
    res[over] = 0x7F
    if sub.any():
        magic = np.uint32(141 << 23).view(np.float32)
        fs = mag[sub].astype(np.uint32).view(np.float32) + magic
        res[sub] = fs.view(np.uint32).astype(np.uint64) - (141 << 23)
    if nrm.any():
        m = mag[nrm]
        odd = (m >> 20) & 1
        m = (m + (((7 - 127) << 23) & 0xFFFFFFFF) + 0x7FFFF + odd) & 0xFFFFFFFF
        res[nrm] = (m >> 20) & 0xFF
    return (res | (sign >> 24)).astype(np.uint8)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bfloat16 (ties to even); result kept as fp32."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    nan = np.isnan(f)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32).copy()
    out[nan] = np.nan
    return out.reshape(f.shape)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------
# format arithmetic
# --------------------------------------------------------------------------
def split_widths(k_bits: int, n_sub: int) -> list[int]:
    """Ceil-first sub-index widths (tests/cb_torch_reference.py:26-30)."""
    if n_sub not in (1, 2, 4):
        raise ValueError(f"unsupported sub-codebook count: {n_sub}")
    base, extra = divmod(int(k_bits), int(n_sub))
    return [base + (1 if i < extra else 0) for i in range(n_sub)]


def type_size(k_bits: int, grid: str, scale_coding: str = "v1") -> int:
    """Bytes per 256-weight superblock (docs/SPEC.md:195-214)."""
    if grid == "fp8":
        return 4 * k_bits
    return 4 * k_bits + (9 if scale_coding == "v2" else 16)


def codebook_elems(k_bits: int, n_sub: int, mode: str) -> int:
    """Number of scalar entries in one flat codebook block."""
    if mode == MODE_FULL:
        return (1 << k_bits) * 8
    if mode == MODE_SIGNED:
        return (1 << (k_bits - 8)) * 8
    return sum((1 << w) * (8 // n_sub) for w in split_widths(k_bits, n_sub))


def compose_table(sub_table=TWO_TIER_SUB_TABLE) -> np.ndarray:
    """(256*16,) fp32 ``T[c] * 2**(E-127)`` (gridbook/codec.py:170-183)."""
    t = np.asarray(list(sub_table), dtype=np.float64)
    e = np.arange(256, dtype=np.float64)
    with np.errstate(over="ignore"):
        return (t[None, :] * np.power(2.0, e[:, None] - TWO_TIER_SUPER_BIAS)
                ).astype(np.float32).reshape(-1)


def compose_legal_supers(sub_table=TWO_TIER_SUB_TABLE, span=None) -> np.ndarray:
    """Super exponents whose sixteen sub codes all compose to an exact E4M3
    value in (0, 448] (tests/cb_torch_reference.py:199-243)."""
    t = np.asarray(list(sub_table), dtype=np.float64)
    exact = t[None, :] * np.power(2.0, np.arange(256, dtype=np.float64)[:, None]
                                  - TWO_TIER_SUPER_BIAS)
    with np.errstate(over="ignore"):
        comp = exact.astype(np.float32)
    finite = np.isfinite(comp)
    safe = np.where(finite & (comp < 480.0), comp, 0.0).astype(np.float32)
    trip = e4m3_to_f32(f32_to_e4m3(safe))
    legal = (finite & (comp > 0) & (comp <= E4M3_MAX) & (trip == comp)
             & (comp.astype(np.float64) == exact))
    full = np.nonzero(legal.all(axis=1))[0]
    if span is None:
        return full
    start = (full.size - int(span)) // 2
    return full[start:start + int(span)]


# --------------------------------------------------------------------------
# decode
# --------------------------------------------------------------------------
def extract_codewords(qw: np.ndarray, *, N: int, K: int, k_bits: int,
                      type_size: int) -> np.ndarray:
    """[N, K/256, 32] little-endian ``k_bits`` codewords
    (tests/cb_torch_reference.py:33-74)."""
    qw = np.asarray(qw)
    if qw.dtype != np.uint8 or qw.ndim != 2 or qw.shape[0] != N:
        raise TypeError("qw must be a rank-2 uint8 array with N rows")
    if K <= 0 or K % SUPERBLOCK:
        raise ValueError("K must be a positive multiple of 256")
    if not 0 < k_bits < 57:
        raise ValueError("codewords are 1..56 bits here")
    n_sb = K // SUPERBLOCK
    row_bytes = n_sb * type_size
    if qw.shape[1] < row_bytes:
        raise ValueError(f"packed row has {qw.shape[1]} bytes, needs {row_bytes}")
    padded = np.zeros((N, row_bytes + 8), dtype=np.uint64)
    padded[:, :row_bytes] = qw[:, :row_bytes]
    v = np.arange(32, dtype=np.int64)
    byte_base = (v * k_bits) // 8
    shift = ((v * k_bits) % 8).astype(np.uint64)
    starts = (np.arange(n_sb, dtype=np.int64) * type_size)[:, None] + byte_base[None, :]
    window = np.zeros((N, n_sb, 32), dtype=np.uint64)
    for b in range(8):
        window |= padded[:, starts + b] << np.uint64(8 * b)
    mask = np.uint64((1 << k_bits) - 1)
    return ((window >> shift[None, None, :]) & mask).astype(np.int64)


def decode_values(qw, cb_flat, cb_row_offset, *, N, K, k_bits, n_sub,
                  type_size, mode=None) -> np.ndarray:
    """[N, K] codebook values before any scale
    (tests/cb_torch_reference.py:77-127; ``full`` per docs/SPEC.md:97-101).

    ``mode=None`` keeps the reference's convention: ``n_sub == 1`` is the
    signed layout, anything else is a product split."""
    cb = np.asarray(cb_flat, dtype=np.float32).reshape(-1)
    off = np.asarray(cb_row_offset, dtype=np.int64).reshape(N)
    if mode is None:
        mode = MODE_SIGNED if n_sub == 1 else MODE_PRODUCT
    codes = extract_codewords(qw, N=N, K=K, k_bits=k_bits, type_size=type_size)
    base = off[:, None, None, None]
    local8 = np.arange(8, dtype=np.int64)
    if mode == MODE_FULL:
        vals = cb[base + codes[..., None] * 8 + local8]
    elif mode == MODE_SIGNED:
        mag = codes >> 8
        vals = cb[base + mag[..., None] * 8 + local8]
        neg = ((codes[..., None] >> local8) & 1).astype(bool)
        vals = np.where(neg, -vals, vals)
    else:
        sub_dim = 8 // n_sub
        local = np.arange(sub_dim, dtype=np.int64)
        pieces, bit_off, tbase = [], 0, 0
        for w in split_widths(k_bits, n_sub):
            idx = (codes >> bit_off) & ((1 << w) - 1)
            pieces.append(cb[base + tbase + idx[..., None] * sub_dim + local])
            bit_off += w
            tbase += (1 << w) * sub_dim
        vals = np.concatenate(pieces, axis=-1)
    return vals.reshape(N, K).astype(np.float32)


def fp4_scale_plane(qw, *, N, K, k_bits, type_size, scale_coding,
                    compose=None) -> np.ndarray:
    """[N, K/16] fp32 group scales, from the bytes after each superblock's 4k
    index bytes.  v1: E4M3 bytes (gridbook/codec.py:186-194).  v2: super byte +
    sixteen nibbles through the compose table
    (tests/cb_torch_reference.py:156-170)."""
    n_sb = K // SUPERBLOCK
    blocks = np.asarray(qw)[:, :n_sb * type_size].reshape(N, n_sb, type_size)
    if scale_coding == "v1":
        plane = blocks[:, :, 4 * k_bits:4 * k_bits + 16]
        return e4m3_to_f32(plane).reshape(N, n_sb * 16)
    if scale_coding != "v2":
        raise ValueError(f"unknown fp4 scale coding {scale_coding!r}")
    comp = np.asarray(compose if compose is not None else compose_table(),
                      dtype=np.float32).reshape(256, 16)
    sup = blocks[:, :, 4 * k_bits].astype(np.int64)
    sub = blocks[:, :, 4 * k_bits + 1:4 * k_bits + 9].astype(np.int64)
    codes = np.stack((sub & 0xF, sub >> 4), axis=-1).reshape(N, n_sb, 16)
    return comp[sup[..., None], codes].reshape(N, n_sb * 16)


def reconstruct_weight(qw, cb_flat, cb_row_offset, *, N, K, k_bits, n_sub,
                       type_size, grid, mode=None, scale_coding="v1",
                       compose=None, weight_scale=None) -> np.ndarray:
    """[N, K] served weight = bf16_rn(value * scale), held as fp32
    (tests/cb_torch_reference.py:130-178)."""
    vals = decode_values(qw, cb_flat, cb_row_offset, N=N, K=K, k_bits=k_bits,
                         n_sub=n_sub, type_size=type_size, mode=mode)
    if grid == "fp8":
        s = np.asarray(weight_scale, dtype=np.float32).reshape(N, 1)
        return bf16_round(vals * s)
    plane = fp4_scale_plane(qw, N=N, K=K, k_bits=k_bits, type_size=type_size,
                            scale_coding=scale_coding, compose=compose)
    return bf16_round(vals * np.repeat(plane, 16, axis=1))


def e2m1_codes(values: np.ndarray) -> np.ndarray:
    """E2M1 nibble (bit 3 = sign) of on-grid values (gridbook/codec.py:275-284)."""
    v = np.asarray(values, dtype=np.float32)
    mags = np.asarray(E2M1_MAGNITUDES, dtype=np.float32)
    idx = np.argmax(np.abs(v)[..., None] == mags, axis=-1)
    if not np.array_equal(mags[idx], np.abs(v)):
        raise ValueError("value off the E2M1 grid")
    return (idx + np.where(v < 0, 8, 0)).astype(np.uint8)    # -0.0 encodes as +0, as in the reference


def decode_nvfp4_tile(qw, cb_flat, cb_row_offset, *, N, K, k_bits, n_sub,
                      type_size, mode=None, scale_coding="v1", compose=None):
    """The native NVFP4 view of an FP4-grid layer: packed E2M1 nibbles
    ``[N, K/2]`` (even element in the low nibble, gridbook/codec.py:287-291) and
    the E4M3 group-scale bytes ``[N, K/16]`` (docs/SPEC.md:30-39)."""
    vals = decode_values(qw, cb_flat, cb_row_offset, N=N, K=K, k_bits=k_bits,
                         n_sub=n_sub, type_size=type_size, mode=mode)
    codes = e2m1_codes(vals).astype(np.uint16)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    plane = fp4_scale_plane(qw, N=N, K=K, k_bits=k_bits, type_size=type_size,
                            scale_coding=scale_coding, compose=compose)
    return packed, f32_to_e4m3(plane)


def sf_swizzle_offsets(rows: int, groups: int) -> np.ndarray:
    """Flat offsets of the 128x4 scale-factor atom layout the block-scaled MMA
    reads (gridbook/codec.py:353-363)."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    gpad = (groups + 3) // 4 * 4
    return ((r % 32) * 16 + ((r // 32) % 4) * 4 + (g % 4)
            + (g // 4) * 512 + (r // 128) * (512 * (gpad // 4)))


def swizzle_sf_plane(sf_bytes: np.ndarray) -> np.ndarray:
    """(rows, groups) E4M3 bytes -> flat swizzled plane, zero padded to
    128 rows x 4 groups (gridbook/codec.py:366-374)."""
    rows, groups = sf_bytes.shape
    rpad = (rows + 127) // 128 * 128
    gpad = (groups + 3) // 4 * 4
    out = np.zeros(rpad * gpad, dtype=np.uint8)
    out[sf_swizzle_offsets(rows, groups).reshape(-1)] = sf_bytes.reshape(-1)
    return out


# --------------------------------------------------------------------------
# activation buckets
# --------------------------------------------------------------------------
_F32 = np.float32
_INV6 = _F32(1.0) / _F32(6.0)
_INV448 = _F32(1.0) / _F32(448.0)
_FP4_GRID = np.asarray(sorted({v for a in E2M1_MAGNITUDES for v in (a, -a)}),
                       dtype=np.float32)


def fp4_group16_act_qdq(x: np.ndarray, scale_rule: str = "div") -> np.ndarray:
    """Group-16 E2M1 round-to-nearest QDQ of bf16 activations
    (gridbook/codec.py:248-260).  Input and output are fp32 arrays holding bf16
    values.

    ``scale_rule`` names how ``amax / 6`` is evaluated in fp32.  torch on the
    CPU divides (``"div"``, what the fixtures generated in the build container
    contain); torch on CUDA multiplies by the fp32 reciprocal (``"recip"``),
    which the reference's native kernel reproduces on purpose
    (gridbook/csrc/cb_gemv.cu:485-511).  The two differ by one ulp of the scale
    for some amax, and that moves exact-midpoint elements to the other rung."""
    x = np.asarray(x, dtype=np.float32)
    k = x.shape[-1]
    w = x.reshape(-1, k // FP4_GROUP, FP4_GROUP)
    amax = np.maximum(np.abs(w).max(axis=-1, keepdims=True), _F32(1e-8))
    amax = np.where(np.isnan(w).any(axis=-1, keepdims=True), _F32(np.nan), amax)
    scale = amax / _F32(6.0) if scale_rule == "div" else amax * _INV6
    scale = scale.astype(np.float32)
    with np.errstate(invalid="ignore"):
        xg = (w / scale).astype(np.float32)
        idx = np.searchsorted(_FP4_GRID, xg, side="left")   # bucketize(right=False)
        lo = _FP4_GRID[np.clip(idx - 1, 0, None)]
        hi = _FP4_GRID[np.clip(idx, None, _FP4_GRID.size - 1)]
        q = np.where(np.abs(hi - xg) < np.abs(xg - lo), hi, lo)
        out = (q * scale).astype(np.float32)
    return bf16_round(out).reshape(x.shape)


def fp8_dynamic_act_qdq(x: np.ndarray, scale_rule: str = "div") -> np.ndarray:
    """Per-token dynamic E4M3 QDQ (gridbook/codec.py:428-437); the same two
    scale rules as above (gridbook/csrc/cb_gemv.cu:88-91)."""
    x = np.asarray(x, dtype=np.float32)
    rows = x.reshape(-1, x.shape[-1])
    amax = np.abs(rows).max(axis=-1, keepdims=True)
    s = amax / _F32(448.0) if scale_rule == "div" else amax * _INV448
    scale = np.maximum(s.astype(np.float32), _F32(1.0 / (448.0 * 512.0)))
    q = np.clip((rows / scale).astype(np.float32), -E4M3_MAX, E4M3_MAX)
    deq = (e4m3_to_f32(f32_to_e4m3(q)) * scale).astype(np.float32)
    return bf16_round(deq).reshape(x.shape)


def nvfp4_act_quant(x: np.ndarray, global_scale: float):
    """Native NVFP4 activation quantisation (gridbook/codec.py:377-425):
    returns (packed [M, K/2] u8, sf bytes [M, K/16] u8, 1/global_scale)."""
    x = np.asarray(x, dtype=np.float32)
    m, k = x.shape
    gs = _F32(global_scale)
    xs = (x * gs).astype(np.float32)
    g = xs.reshape(m, k // FP4_GROUP, FP4_GROUP)
    sf = np.minimum((np.abs(g).max(axis=-1) / _F32(6.0)).astype(np.float32),
                    _F32(E4M3_MAX))
    sfb = f32_to_e4m3(sf)
    sff = e4m3_to_f32(sfb)
    nz = sff != 0
    safe = np.where(nz, sff, _F32(1.0))
    xg = np.clip((g / safe[..., None]).astype(np.float32), -6.0, 6.0)
    mag = np.asarray(E2M1_MAGNITUDES, dtype=np.float32)
    xm = np.abs(xg)
    up = np.clip(np.searchsorted(mag, xm, side="left"), None, mag.size - 1)
    lo = np.clip(up - 1, 0, None)
    ld = xm - mag[lo]
    ud = mag[up] - xm
    choose = (ud < ld) | ((ud == ld) & ((up & 1) == 0))
    mi = np.where(choose, up, lo)
    mi = np.where(nz[..., None], mi, 0)
    codes = (mi.astype(np.uint8) | (np.signbit(g).astype(np.uint8) << 3)).reshape(m, k)
    packed = (codes[:, 0::2].astype(np.uint16) | (codes[:, 1::2].astype(np.uint16) << 4))
    return packed.astype(np.uint8), sfb, _F32(1.0) / gs


# --------------------------------------------------------------------------
# linear and MoE
# --------------------------------------------------------------------------
def cb_linear(x, qw, cb_flat, cb_row_offset, *, N, K, k_bits, n_sub, type_size,
              grid, mode=None, scale_coding="v1", compose=None,
              weight_scale=None, global_scale=None) -> np.ndarray:
    """bf16 W, fp32 product, one bf16 rounding of the output
    (tests/cb_torch_reference.py:307-330).  ``x`` is already in its activation
    bucket.  ``global_scale`` (not in the reference, parity unpinned) multiplies
    the fp32 accumulator before the output rounding, like a uniform per-channel
    scale in the reference's scaled epilogue
    (gridbook/csrc/cb_fused_fp4_gemm.cu:90-118)."""
    w = reconstruct_weight(qw, cb_flat, cb_row_offset, N=N, K=K, k_bits=k_bits,
                           n_sub=n_sub, type_size=type_size, grid=grid,
                           mode=mode, scale_coding=scale_coding,
                           compose=compose, weight_scale=weight_scale)
    x = np.asarray(x, dtype=np.float32)
    out = x.reshape(-1, K) @ w.T
    if global_scale is not None:
        out = out * _F32(global_scale)
    return bf16_round(out.astype(np.float32)).reshape(*x.shape[:-1], N)


def act_bucket(x, grid, scale_rule="div"):
    return (fp4_group16_act_qdq if grid == "fp4" else fp8_dynamic_act_qdq)(
        x, scale_rule)


def silu_mul(gate_up: np.ndarray) -> np.ndarray:
    """bf16 ``silu(gate) * up`` on [P, 2I] -> [P, I]; each torch bf16 op rounds
    (tests/test_cuda_gemv.py:336-338: F.silu on bf16, then a bf16 multiply)."""
    g, u = np.split(np.asarray(gate_up, dtype=np.float32), 2, axis=-1)
    with np.errstate(over="ignore"):
        s = bf16_round((g / (_F32(1.0) + np.exp(-g))).astype(np.float32))
    return bf16_round((s * u).astype(np.float32))


def moe_loop_chain(x, topk_ids, topk_w, w13, w2, *, E, hidden, inter, fmt13,
                   fmt2, scale_rule="div") -> np.ndarray:
    """Routed-MoE oracle: the per-expert loop the reference tests use
    (tests/test_cuda_gemv.py:329-348, 434-450).  Per expert, ascending: bucket
    the routed rows, gate_up linear, SiLU*up, bucket, down linear, multiply by
    the bf16 router weight, bf16 ``index_add_``.

    ``w13``/``w2`` are dicts with the packed stack ``qw`` [E, rows, bytes], the
    flat codebook ``cb`` and, per format, ``scale`` [E, rows] / ``compose``;
    ``fmt13``/``fmt2`` carry grid, k_bits, n_sub, type_size, mode, scale_coding
    (the two stages may differ, which the reference refuses:
    gridbook/config.py:1631-1640)."""
    x = np.asarray(x, dtype=np.float32)
    T = x.shape[0]
    out = np.zeros((T, hidden), dtype=np.float32)
    ids = np.asarray(topk_ids)
    wts = np.asarray(topk_w, dtype=np.float32)
    for e in range(E):
        tok, slot = np.nonzero(ids == e)
        if tok.size == 0:
            continue
        xe = act_bucket(x[tok], fmt13["grid"], scale_rule)
        gu = _stage(xe, w13, e, 2 * inter, hidden, fmt13)
        a = silu_mul(gu)
        aq = act_bucket(a, fmt2["grid"], scale_rule)
        oe = _stage(aq, w2, e, hidden, inter, fmt2)
        oe = bf16_round(oe * bf16_round(wts[tok, slot])[:, None])
        for i, t in enumerate(tok):          # index_add_ in bf16, row by row
            out[t] = bf16_round(out[t] + oe[i])
    return out


def _stage(xq, stack, e, rows, k_in, fmt):
    off = stack.get("cb_row_offset")
    if off is None:
        off = np.zeros(rows, dtype=np.int32)
    ws = stack.get("scale")
    return cb_linear(
        xq, stack["qw"][e], stack["cb"], off, N=rows, K=k_in,
        k_bits=fmt["k_bits"], n_sub=fmt["n_sub"], type_size=fmt["type_size"],
        grid=fmt["grid"], mode=fmt.get("mode"),
        scale_coding=fmt.get("scale_coding", "v1"),
        compose=stack.get("compose"),
        weight_scale=None if ws is None else ws[e],
        global_scale=fmt.get("global_scale"))


def route_by_expert(topk_ids: np.ndarray, E: int):
    """Expert-major grouping of the routed (token, slot) pairs: per-expert
    counts, exclusive offsets, and for every sorted position the flat pair index
    ``t * topk + slot`` (stable: token-ascending inside an expert).  Same result
    as the reference's stable argsort + scatter_add histogram
    (gridbook/moe.py:1609-1621, gridbook/moe_routing.py:99-115)."""
    ids = np.asarray(topk_ids, dtype=np.int64).reshape(-1)
    counts = np.bincount(ids, minlength=E).astype(np.int32)
    offsets = np.zeros(E + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    order = np.argsort(ids, kind="stable").astype(np.int32)
    return counts, offsets, order
