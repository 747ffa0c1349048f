"""Row sharding of a quantized matrix over the GPUs of one box.

Output rows of y = W x are independent, so rank g of G owns the rows [g*per, min((g+1)*per, N)) with
per = ceil(N / G); x is replicated and the only exchange is an all-gather of the f32 output slices
(4 * per bytes per rank).  Rows keep their GGUF byte layout, so a shard is a contiguous byte range of
the tensor (row_bytes = ggml_type_size(type, K)) and the plane repack applies to it unchanged.
"""
from .synth import type_size


def shard_rows(n_rows, rank, world):
    """(first row, one past last row, rows per rank slot) of `rank`."""
    per = (n_rows + world - 1) // world
    n0 = min(rank * per, n_rows)
    return n0, min(n0 + per, n_rows), per


def shard_bytes(ggml_type, in_dim, n_rows, rank, world):
    """Byte range [b0, b1) of rank's rows inside the raw GGUF tensor blob."""
    n0, n1, _ = shard_rows(n_rows, rank, world)
    rb = type_size(ggml_type, in_dim)
    return n0 * rb, n1 * rb


def all_gather_rows(y_full, rank, world, per, dist):
    """In-place all-gather: y_full is a [world * per] tensor whose slot `rank` holds this rank's slice."""
    dist.all_gather_into_tensor(y_full, y_full[rank * per:(rank + 1) * per])
    return y_full
