"""IQ2/IQ3 codebooks as the C ABI expects them.

The library embeds no codebook: like the reference's kernels it receives them
from the host through cuda_set_*_grid (src/cuda.rs:9-13, 131-140).  The
reference host takes them from its vendored src/iq2_tables.rs and
src/iq3_tables.rs; this host mirror takes the same numbers from the installed
`gguf` package, which also carries the IQ3_XXS grid the reference lacks.

Layouts: IQ2 grids are u64 = 8 little-endian int8 values, IQ3 grids are
u32 = 4 little-endian uint8 values; the sign table is 128 bytes.
"""
import numpy as np


def _grid_bytes(cls):
    cls.init_grid()
    g = np.asarray(cls.grid, dtype=np.float32).reshape(cls.grid_shape)
    b = g.astype(np.uint8)
    assert np.array_equal(b.astype(np.float32), g)
    return np.ascontiguousarray(b)


def load_tables():
    """dict of numpy arrays: iq2xxs/iq2xs/iq2s (u64), iq3s/iq3xxs (u32), ksigns (u8)."""
    from gguf import quants
    t = {
        "iq2xxs": _grid_bytes(quants.IQ2_XXS).view(np.uint64).reshape(-1),
        "iq2xs": _grid_bytes(quants.IQ2_XS).view(np.uint64).reshape(-1),
        "iq2s": _grid_bytes(quants.IQ2_S).view(np.uint64).reshape(-1),
        "iq3s": _grid_bytes(quants.IQ3_S).view(np.uint32).reshape(-1),
        "iq3xxs": _grid_bytes(quants.IQ3_XXS).view(np.uint32).reshape(-1),
        "ksigns": np.frombuffer(quants.IQ2_XXS.ksigns, dtype=np.uint8).copy(),
    }
    assert t["iq2xxs"].size == 256 and t["iq2xs"].size == 512 and t["iq2s"].size == 1024
    assert t["iq3s"].size == 512 and t["iq3xxs"].size == 256 and t["ksigns"].size == 128
    return t
