"""Load-time format preparation, host side (mirrors gridbook/codec.py): flat codebooks,
the two-tier compose table, row padding and grid validation.  Runs once per layer at
model load; nothing here is on the forward path and nothing here is a dense weight."""
from __future__ import annotations

import os
import sys

import torch

SUPERBLOCK = 256
FP4_GROUP = 16
PAD_BYTES = 16
SCALE_CODING_TWO_TIER = "two_tier"
TWO_TIER_SUPER_BIAS = 127
TWO_TIER_SUB_TABLE = (1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875,
                      2.0, 2.25, 2.5, 2.75, 3.0, 3.25, 3.5, 3.75)
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def type_size(k: int, is_fp4: bool, two_tier: bool = False) -> int:
    """Bytes per superblock (gridbook/codec.py:40-41, docs/SPEC.md:195-214)."""
    return 4 * int(k) + ((9 if two_tier else 16) if is_fp4 else 0)


def assert_cast_lossless(raw: torch.Tensor, cast: torch.Tensor, what: str, prefix: str) -> None:
    """Every table value must survive the cast to the representation the kernels stage
    (gridbook/codec.py:78-107).  Compared in float64, so a float64 sidecar is not rounded before the
    check.  The error names the layer, the cast, how many values moved and the measured maximum
    absolute and relative error; PRISMAQUANT_SKIP_CB_CAST_CHECK=1 turns it into a warning on stderr
    (debugging only), as in the reference."""
    a = raw.reshape(-1).to(torch.float64)
    b = cast.reshape(-1).to(torch.float64)
    sized = a.numel() == b.numel()
    if sized and torch.equal(a, b):
        return
    moved = int((a != b).sum()) if sized else -1
    err = (a - b).abs() if sized else None
    worst = float(err.max()) if sized else -1.0
    rel = float((err / a.abs().clamp_min(1e-12)).max()) if sized else -1.0
    msg = (f"[prismaquant] {prefix}: the {what} codebook cast is LOSSY: {moved} of {a.numel()} table values "
           f"do not survive it (max abs {worst:.3e}, max rel {rel:.3e}). Only values already on the target "
           f"grid cast exactly; a table that is not would make every weight decode against rounded entries. "
           f"PRISMAQUANT_SKIP_CB_CAST_CHECK=1 overrides this (debugging only).")
    if os.environ.get("PRISMAQUANT_SKIP_CB_CAST_CHECK") == "1":
        print("WARNING " + msg, file=sys.stderr, flush=True)
        return
    raise ValueError(msg)


def validate_codebook_grid(raw: torch.Tensor, grid: str, prefix: str = "codebook") -> None:
    """Reject tables that are not exactly on their declared grid (gridbook/codec.py:110-143): a format
    check, not a cast check - 0.53125 survives bf16 but is no E2M1 value."""
    v = raw.reshape(-1).to(torch.float64)
    finite = torch.isfinite(v)
    if not bool(finite.all()):
        raise ValueError(f"[prismaquant] {prefix}: {int((~finite).sum())} of {v.numel()} codebook values are "
                         f"non-finite; {grid} codebooks must be finite and grid-valued")
    if grid == "fp8":
        ok, name = v == v.to(torch.float8_e4m3fn).to(torch.float64), "E4M3"
    elif grid == "fp4":
        mags = torch.tensor(_E2M1, dtype=torch.float64, device=v.device)
        ok, name = (v.abs().unsqueeze(-1) == mags).any(dim=-1), "E2M1"
    else:
        raise ValueError(f"[prismaquant] {prefix}: unknown codebook grid {grid!r}")
    if not bool(ok.all()):
        raise ValueError(f"[prismaquant] {prefix}: {int((~ok).sum())} of {v.numel()} codebook values "
                         f"are off the {name} grid declared by the {grid} format")


def build_flat_codebook(sub_tables: list[torch.Tensor], prefix: str = "codebook",
                        grid: str | None = None) -> torch.Tensor:
    """Concatenate the (2^w, sub_dim) tables row-major into the flat bf16 layout the
    kernels stage (gridbook/codec.py:146-159): entry (idx, j) of table s sits at
    base_s + idx*sub_dim + j.  The input is never rounded before the check."""
    raw = torch.cat([t.reshape(-1).to(torch.float64) for t in sub_tables])
    if grid is not None:
        validate_codebook_grid(raw, grid, prefix)
    flat = torch.cat([t.reshape(-1).to(torch.bfloat16) for t in sub_tables]).contiguous()
    assert_cast_lossless(raw, flat, "bf16 flat", prefix)
    return flat


def flat_codebook_fp8(flat: torch.Tensor, prefix: str = "codebook") -> torch.Tensor:
    """Flat E4M3-grid codebook as raw bytes (gridbook/codec.py:162-167)."""
    f8 = flat.to(torch.float8_e4m3fn).contiguous()
    assert_cast_lossless(flat, f8, "e4m3 flat", prefix)
    return f8.view(torch.uint8)


NVFP4_ACTIVATION_CONTRACT = "nvfp4_w4a4"    # the one static activation contract an fp4 scheme may declare


def static_activation_contract(scheme: dict, prefix: str) -> bool:
    """Whether a scheme declares the static NVFP4 activation contract; a declaration on the fp8 grid
    or of an unknown contract is an error (gridbook/config.py:652-668)."""
    contract = scheme.get("activation_contract")
    if contract is None:
        return False
    if scheme.get("grid") != "fp4":
        raise ValueError(f"{prefix}: activation_contract is fp4-only")
    if contract != NVFP4_ACTIVATION_CONTRACT:
        raise ValueError(f"{prefix}: unsupported activation_contract {contract!r}")
    return True


def loaded_static_activation_scale(values: torch.Tensor, prefix: str) -> float:
    """Gate after loading for a contracted module's `input_global_scale`
    (gridbook/nvfp4_activation_contract.py:719-752): a non-empty 1-D fp32 vector, one slot per
    logical shard, every slot loaded (the parameter starts as NaN) with a finite positive value, and
    all slots the same fp32 BITS - the activation is quantised before the projection split, so one
    module has one scale.  Returns that scale."""
    data = values.detach()
    if data.dtype != torch.float32 or data.ndim != 1 or data.numel() == 0:
        raise ValueError(f"{prefix}.input_global_scale parameter must be nonempty 1-D float32, got "
                         f"dtype={data.dtype}, shape={tuple(data.shape)}")
    host = data.to("cpu").contiguous()
    if not bool(torch.isfinite(host).all()) or not bool((host > 0).all()):
        raise ValueError(f"{prefix}.input_global_scale: every logical shard must load a finite positive scale, "
                         f"got {host.tolist()}")
    bits = host.view(torch.int32)
    if not bool((bits == bits[0]).all()):
        raise ValueError(f"{prefix}: fused logical shards have non-identical input_global_scale values")
    return float(host[0])


def build_compose_table(sub_table=TWO_TIER_SUB_TABLE) -> torch.Tensor:
    """(4096,) fp32 table ``T[c] * 2^(E-127)`` indexed ``E*16 + c``
    (gridbook/codec.py:170-183, docs/SPEC.md:144-177)."""
    t = torch.tensor(list(sub_table), dtype=torch.float64)
    e = torch.arange(256, dtype=torch.float64)
    return (t[None, :] * torch.pow(2.0, e[:, None] - float(TWO_TIER_SUPER_BIAS))
            ).to(torch.float32).reshape(-1).contiguous()


def pad_qweight(qw: torch.Tensor) -> torch.Tensor:
    """Right-pad each row by 16 zero bytes (gridbook/codec.py:200-229).  The kernels
    here do not need the slack per row (they read 16-byte windows of the whole
    buffer), but accept the reference's padded layout through the row stride."""
    return torch.nn.functional.pad(qw.contiguous(), (0, PAD_BYTES), value=0).contiguous()


def pad_superblocks(qw: torch.Tensor, type_size: int, stride: int) -> torch.Tensor:
    """Packed rows [..., n_sb * type_size] with every superblock moved to a `stride`-byte slot (zero
    filled): the resident layout the tensor-core decode kernel needs for superblocks whose size is
    not a multiple of 16 (tiled TMA cannot fetch 73-byte pieces).  Nothing is decoded: the index and
    scale bytes are the shipped ones."""
    if stride < type_size:
        raise ValueError(f"stride {stride} is smaller than the superblock ({type_size} bytes)")
    *lead, row_bytes = qw.shape
    if row_bytes % type_size:
        raise ValueError(f"row of {row_bytes} bytes is not a whole number of {type_size}-byte superblocks")
    n_sb = row_bytes // type_size
    out = torch.zeros((*lead, n_sb, stride), dtype=torch.uint8, device=qw.device)
    out[..., :type_size] = qw.reshape(*lead, n_sb, type_size)
    return out.reshape(*lead, n_sb * stride)


def with_tail_slack(qw: torch.Tensor) -> torch.Tensor:
    """Same bytes in a buffer that stays readable for 16 bytes past the last row, which
    is what the kernels' aligned windows may touch."""
    flat = torch.zeros(qw.numel() + PAD_BYTES, dtype=torch.uint8, device=qw.device)
    flat[:qw.numel()] = qw.reshape(-1)
    return flat[:qw.numel()].view(qw.shape)
