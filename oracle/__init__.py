"""CPU restatement of the reference's algorithm for the codebook-decode path.  TEST
INFRASTRUCTURE: imported by the tests, by the smoke check and by the CPU legs of the benchmark
only; nothing in the product package may import it."""


def oracle_kwargs(fmt) -> dict:
    """Keyword arguments of the oracle's decode functions for one packed format (an object with
    the fields of gridbook_b200.formats.CBFormat)."""
    return dict(k_bits=fmt.k, n_sub=fmt.n_sub, type_size=fmt.type_size, grid=fmt.grid, mode=fmt.mode,
                scale_coding=fmt.scale_coding if fmt.is_fp4 else "v1")
