"""Packed-format descriptors (the `scheme` vocabulary of gridbook/config.py:803-957
and docs/SPEC.md:382-460) and their C-ABI mirror."""
from __future__ import annotations

from dataclasses import dataclass, replace

from . import _native as nat

SUPERBLOCK = 256


@dataclass(frozen=True)
class CBFormat:
    grid: str                 # "fp4" | "fp8"
    k: int                    # bits per 8-weight codeword
    n_sub: int = 2            # product sub-indices (1 for signed / full)
    mode: str = "product"     # "product" | "signed" | "full"
    scale_coding: str = "v1"  # fp4: "v1" (16 E4M3 bytes) | "v2" (two-tier); fp8: "none"
    sb_pad: int = 0           # unused bytes after each superblock (0..15): a resident layout, never on disk

    def __post_init__(self):
        if self.grid not in ("fp4", "fp8"):
            raise ValueError(f"unknown grid {self.grid!r}")
        if self.mode not in ("product", "signed", "full"):
            raise ValueError(f"unknown mode {self.mode!r}")
        if self.grid == "fp8":
            object.__setattr__(self, "scale_coding", "none")
        elif self.scale_coding not in ("v1", "v2"):
            raise ValueError(f"fp4 scale coding must be v1 or v2, got {self.scale_coding!r}")
        if self.mode != "product":
            object.__setattr__(self, "n_sub", 1)
        if not 0 <= self.sb_pad <= 15:
            raise ValueError(f"superblock padding must be 0..15 bytes, got {self.sb_pad}")

    @property
    def is_fp4(self) -> bool:
        return self.grid == "fp4"

    @property
    def packed_type_size(self) -> int:
        """Bytes of a superblock as shipped (docs/SPEC.md:195-214)."""
        if not self.is_fp4:
            return 4 * self.k
        return 4 * self.k + (9 if self.scale_coding == "v2" else 16)

    @property
    def type_size(self) -> int:
        """Superblock stride in memory: the shipped bytes plus the resident padding."""
        return self.packed_type_size + self.sb_pad

    def padded(self, stride: int) -> "CBFormat":
        """The same format with superblocks `stride` bytes apart."""
        pad = stride - self.packed_type_size
        if not 0 <= pad <= 15:
            raise ValueError(f"cannot pad {self.packed_type_size}-byte superblocks to {stride}")
        return replace(self, sb_pad=pad)

    @property
    def sub_dim(self) -> int:
        return 8 // self.n_sub if self.mode == "product" else 8

    def widths(self) -> list[int]:
        base, extra = divmod(self.k, self.n_sub)
        return [base + (1 if i < extra else 0) for i in range(self.n_sub)]

    def table_shapes(self) -> list[tuple[int, int]]:
        """(rows, dims) of each codebook table, in flat-layout order."""
        if self.mode == "full":
            return [(1 << self.k, 8)]
        if self.mode == "signed":
            return [(1 << (self.k - 8), 8)]
        return [(1 << w, self.sub_dim) for w in self.widths()]

    def codebook_elems(self) -> int:
        return sum(r * d for r, d in self.table_shapes())

    def row_bytes(self, K: int) -> int:
        if K % SUPERBLOCK:
            raise ValueError(f"in_features {K} not a multiple of {SUPERBLOCK}")
        return (K // SUPERBLOCK) * self.type_size

    def packed_row_bytes(self, K: int) -> int:
        """Shipped (algorithmic) bytes of one row."""
        return (K // SUPERBLOCK) * self.packed_type_size

    def bits_per_weight(self) -> float:
        return self.packed_type_size * 8 / SUPERBLOCK

    def to_native(self) -> nat.GbFormat:
        return nat.GbFormat(
            grid=nat.GRID_FP4 if self.is_fp4 else nat.GRID_FP8,
            mode={"product": nat.MODE_PRODUCT, "signed": nat.MODE_SIGNED,
                  "full": nat.MODE_FULL}[self.mode],
            k_bits=self.k, n_sub=self.n_sub, type_size=self.type_size,
            scale_coding={"none": nat.SCALE_NONE, "v1": nat.SCALE_V1,
                          "v2": nat.SCALE_V2}[self.scale_coding])

    @classmethod
    def from_scheme(cls, scheme: dict) -> "CBFormat":
        """Parse a reference scheme dict (gridbook/linear.py:206-231)."""
        grid = scheme["grid"]
        sc = scheme.get("scale_coding")
        if isinstance(sc, dict):
            sc = sc.get("kind")
        coding = "v2" if sc == "two_tier" else "v1"
        mode = scheme.get("mode", "product")
        n_sub = int(scheme.get("n_sub", 2 if grid == "fp4" else 4))
        if mode == "product" and n_sub == 1:
            mode = "signed"           # the reference encodes signed as n_sub == 1
        fmt = cls(grid=grid, k=int(scheme["k"]), n_sub=n_sub, mode=mode, scale_coding=coding)
        ts = scheme.get("type_size")
        if ts is not None and int(ts) != fmt.packed_type_size:
            raise ValueError(f"scheme type_size {ts} does not match {fmt.packed_type_size} for {fmt}")
        return fmt


# The formats the benchmark configurations name.
NVFP4_LITERAL = CBFormat("fp4", 8, mode="full", scale_coding="v1")       # 48 B / superblock
NVFP4_CB_K16 = CBFormat("fp4", 16, n_sub=2, scale_coding="v2")           # 73 B, reference-native
FP8_CB_K32 = CBFormat("fp8", 32, n_sub=4)                                # 128 B, reference-native
FP8_LITERAL = CBFormat("fp8", 16, n_sub=2)                               # 64 B, 4-element vectors
