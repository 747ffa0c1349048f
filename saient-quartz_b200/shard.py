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


def exchange_handles(handle, world, dist):
    """Every rank contributes its window handle (bytes); returns all of them concatenated in rank order."""
    if world == 1:
        return bytes(handle)
    got = [None] * world
    dist.all_gather_object(got, bytes(handle))
    return b"".join(got)


class PeerWindow:
    """This rank's exchange window and the peers' mappings (quartz_mgpu_init / quartz_mgpu_attach).

    `lib` is the loaded C library, `dist` torch.distributed (or any object with all_gather_object)
    whose default group spans the ranks of the box.  After construction, `gemv_push` computes this
    rank's row slice of a sharded GEMV and lands it in every rank's window; `wait` completes the
    exchange; `data_ptr` is the device address of the complete vectors.
    """

    def __init__(self, lib, rank, world, data_bytes, dist=None):
        import ctypes as C
        self.lib, self.rank, self.world = lib, rank, world
        n = lib.quartz_mgpu_handle_bytes()
        buf = C.create_string_buffer(n)
        if lib.quartz_mgpu_init(rank, world, data_bytes, buf) != 0:
            raise RuntimeError("quartz_mgpu_init failed: " + _last_error(lib))
        handles = exchange_handles(buf.raw, world, dist)
        if len(handles) != n * world:
            raise RuntimeError("window handle exchange returned %d bytes, expected %d" % (len(handles), n * world))
        if lib.quartz_mgpu_attach(handles) != 0:
            raise RuntimeError("quartz_mgpu_attach failed: " + _last_error(lib))
        self.data_ptr = lib.quartz_mgpu_data()

    def gemv_push(self, ggml_type, d_w, d_x, dst_off, in_dim, rows_local):
        self.lib.cuda_gemv_push(ggml_type, d_w, d_x, dst_off, in_dim, rows_local)

    def push_rows(self, d_src, m, n_local, dst_off, dst_ld):
        self.lib.cuda_push_rows(d_src, m, n_local, dst_off, dst_ld)

    def wait(self, fused=False):
        """All exchanges pushed so far are complete after this: as a kernel of its own, or (fused) inside the
        activation conversion of the next GEMV call."""
        if fused:
            self.lib.quartz_mgpu_fuse_next_wait()
        else:
            self.lib.quartz_mgpu_wait()

    def close(self):
        self.lib.quartz_mgpu_shutdown()


def _last_error(lib):
    try:
        msg = lib.quartz_error_string()
        return msg.decode() if isinstance(msg, bytes) else str(msg)
    except Exception:
        return "unknown"
