"""Seeded synthetic GGUF-layout tensors and activations.

There is no model file and no dataset behind the numbers this project reports:
every weight matrix is drawn here, block by block, in the raw GGUF block layout
the reference uploads verbatim (src/gguf.rs:118-123, row-major [N][K/block]
blocks), with the value distributions the benchmark configuration states:

  * f16 super-block scales d / dmin of the K-quants and IQ formats ~ U[1e-4, 1e-3]
  * f16 d of the 32-weight formats (Q8_0, Q5_0/1, Q4_0/1, IQ4_NL) ~ U[1e-3, 1e-2],
    their f16 m ~ U[-1e-2, 1e-2]
  * Q6_K int8 sub-block scales uniform in -32..31
  * every other byte (packed 6-bit scale codes, quants, grid indices, sign
    bits) uniform in 0..255 -- every bit pattern is a valid code in all formats
  * activations x ~ N(0, 1) in f32

One numpy PCG64 stream per (seed, tensor id); identical on every machine.
"""
import numpy as np

DEFAULT_SEED = 0x5EED0001

# ggml type id -> (name, weights per block, bytes per block); src/gguf.rs:172-188
# plus Q4_0 / Q4_1 / IQ3_XXS, which the reference lacks.
FORMATS = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 30: ("BF16", 1, 2),
    2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 20: ("IQ4_NL", 32, 18),
    10: ("Q2_K", 256, 84), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210),
    16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98),
    21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82),
}
TYPE_BY_NAME = {v[0]: k for k, v in FORMATS.items()}

# byte offsets of the f16 fields inside a block: (offset, lo, hi)
_SMALL = (1e-4, 1e-3)
_BIG = (1e-3, 1e-2)
_MIN = (-1e-2, 1e-2)
_F16_FIELDS = {
    2: [(0, *_BIG)], 3: [(0, *_BIG), (2, *_MIN)], 6: [(0, *_BIG)], 7: [(0, *_BIG), (2, *_MIN)],
    8: [(0, *_BIG)], 20: [(0, *_BIG)],
    10: [(80, *_SMALL), (82, *_SMALL)], 12: [(0, *_SMALL), (2, *_SMALL)], 13: [(0, *_SMALL), (2, *_SMALL)],
    14: [(208, *_SMALL)],
    16: [(0, *_SMALL)], 17: [(0, *_SMALL)], 18: [(0, *_SMALL)], 21: [(0, *_SMALL)], 22: [(0, *_SMALL)],
}


def type_size(ggml_type, n_elems):
    """Byte size of a tensor blob (src/gguf.rs:172-191)."""
    _, be, bb = FORMATS[ggml_type]
    return (n_elems // be) * bb


def algorithmic_bytes(ggml_type, in_dim, out_dim, m=1):
    """Bytes a GEMV/GEMM must move: the weights once, x in, y out (f32)."""
    return type_size(ggml_type, in_dim * out_dim) + 4 * m * in_dim + 4 * m * out_dim


def make_weights(ggml_type, in_dim, out_dim, seed=DEFAULT_SEED, tensor_id=0):
    """uint8 array of out_dim rows in raw GGUF block layout."""
    name, be, bb = FORMATS[ggml_type]
    assert in_dim % be == 0, f"{name}: in_dim {in_dim} not a multiple of {be}"
    rng = np.random.Generator(np.random.PCG64([seed, tensor_id, ggml_type]))
    n = in_dim * out_dim
    if ggml_type == 0:
        return (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).view(np.uint8)
    if ggml_type == 1:
        return (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(np.float16).view(np.uint8)
    if ggml_type == 30:
        w = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).view(np.uint32)
        w = ((w + 0x7FFF + ((w >> 16) & 1)) >> 16).astype(np.uint16)  # round to nearest even
        return w.view(np.uint8)
    nb = n // be
    blocks = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    for off, lo, hi in _F16_FIELDS[ggml_type]:
        v = rng.uniform(lo, hi, size=nb).astype(np.float32).astype(np.float16)
        blocks[:, off:off + 2] = v.view(np.uint8).reshape(nb, 2)
    if ggml_type == 14:
        sc = rng.integers(-32, 32, size=(nb, 16), dtype=np.int8)
        blocks[:, 192:208] = sc.view(np.uint8)
    return blocks.reshape(-1)


def make_x(n, seed=DEFAULT_SEED, tensor_id=1000, rows=1):
    rng = np.random.Generator(np.random.PCG64([seed, tensor_id, 0xA]))
    x = rng.standard_normal(n * rows, dtype=np.float32)
    return x if rows == 1 else x.reshape(rows, n)


# The benchmark's GEMV sweep at Llama-3-8B decode shapes, batch 1:
# (label, ggml type, in_dim, out_dim)
LLAMA3_8B_GEMV_SWEEP = [
    ("q/o  Q4_K 4096->4096", 12, 4096, 4096),
    ("k/v  Q4_K 4096->1024", 12, 4096, 1024),
    ("gate/up Q4_K 4096->14336", 12, 4096, 14336),
    ("down Q6_K 14336->4096", 14, 14336, 4096),
    ("lm_head Q6_K 4096->128256", 14, 4096, 128256),
    ("Q8_0 4096->4096", 8, 4096, 4096),
]
