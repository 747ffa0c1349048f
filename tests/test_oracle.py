"""CPU tests of the oracle (the checker itself): golden vectors, hand-built blocks,
codebook identity with the reference's tables, gemv/gemm consistency."""
import os
import re

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dequant_golden.npz")


def _ref_src():
    from oracle import build as ob
    root = ob.reference_root()
    return os.path.join(root, "src") if root else None


REF = _ref_src()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _formats(pkg):
    from saient_quartz_b200 import synth
    return sorted(synth.FORMATS.items())


def test_dequant_bit_exact_against_golden(pkg, oracle_mod, golden):
    """oracle dequant == gguf-py dequantize, u32 compare, every format."""
    K, N = 512, 6
    for t, (name, be, bb) in _formats(pkg):
        got = oracle_mod.dequant(golden[f"w_{name}"], t, K * N)
        want = golden[f"deq_{name}"]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


def test_gemv_within_tolerance_of_f64(pkg, oracle_mod, golden):
    K, N = 512, 6
    x = golden["x"]
    for t, (name, be, bb) in _formats(pkg):
        w = golden[f"w_{name}"]
        y = oracle_mod.gemv(x, w, t, K, N)
        tol = oracle_mod.tolerance(w, t, K, N, x)
        assert np.all(np.abs(y - golden[f"y64_{name}"]) <= tol), name


def test_type_sizes(pkg, oracle_mod):
    """src/gguf.rs:172-191 sizes, e.g. the benchmark shapes."""
    L = oracle_mod.lib()
    assert L.qz_type_size(12, 4096 * 4096) == 9_437_184
    assert L.qz_type_size(14, 14336 * 4096) == 48_168_960
    assert L.qz_type_size(14, 4096 * 128256) == 430_940_160
    assert L.qz_type_size(8, 4096 * 4096) == 17_825_792
    assert L.qz_type_size(17, 4096 * 14336) == 16_973_824
    assert L.qz_type_size(99, 1024) == 0
    from saient_quartz_b200 import synth
    for t in synth.FORMATS:
        assert L.qz_type_size(t, 4096) == synth.type_size(t, 4096)


def test_f16_conversion_all_bit_patterns(oracle_mod):
    """src/dequant.rs:1329-1349 must equal IEEE half->float for all 65536 inputs."""
    L = oracle_mod.lib()
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([L.qz_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    same = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert same.all()


def test_hand_built_q4_k_block(oracle_mod):
    """d=1, dmin=0.5, sub-block 0 scale 3 / min 2, all low nibbles 5 -> 1*3*5 - 0.5*2 = 14."""
    blk = np.zeros(144, dtype=np.uint8)
    blk[0:2] = np.array([1.0], dtype=np.float16).view(np.uint8)
    blk[2:4] = np.array([0.5], dtype=np.float16).view(np.uint8)
    blk[4] = 3          # scale code of sub-block 0
    blk[8] = 2          # min code of sub-block 0
    blk[16:48] = 0x05   # low nibbles (sub-block 0) = 5, high nibbles (sub-block 1) = 0
    w = oracle_mod.dequant(blk, 12, 256)
    assert np.all(w[:32] == 14.0)
    assert np.all(w[32:64] == 0.0)   # scale/min codes of sub-block 1 are zero
    # sub-block 5 takes its codes from the packed upper part: scales[9] low nibble | scales[1]>>6
    blk2 = blk.copy()
    blk2[4 + 9] = 0x21              # sc5 low 4 bits = 1, m5 low 4 bits = 2
    blk2[4 + 1] |= 0x40             # sc5 high 2 bits = 1 -> sc5 = 17
    blk2[16 + 64:16 + 96] = 0x30    # pair p=2: high nibble (sub-block 5) = 3
    w2 = oracle_mod.dequant(blk2, 12, 256)
    assert np.all(w2[160:192] == 1.0 * 17 * 3 - 0.5 * 2)


def test_hand_built_q6_k_and_q8_0(oracle_mod):
    blk = np.zeros(210, dtype=np.uint8)
    blk[208:210] = np.array([0.25], dtype=np.float16).view(np.uint8)
    blk[192:208] = np.arange(1, 17, dtype=np.int8).view(np.uint8)   # scales 1..16
    blk[0:128] = 0x21          # low nibble 1, high nibble 2
    blk[128:192] = 0b11100100  # two-bit fields 0,1,2,3
    w = oracle_mod.dequant(blk, 14, 256)
    # weights 0..15: ql low nibble 1 | (0<<4) - 32 = -31, scale 1
    assert np.all(w[0:16] == 0.25 * 1 * -31)
    # weights 32..47: ql[l+32] low nibble 1 | (1<<4) = 17 - 32 = -15, scale index 2 -> 3
    assert np.all(w[32:48] == 0.25 * 3 * -15)
    # weights 96..111: high nibble 2 | (3<<4) = 50 - 32 = 18, scale index 6 -> 7
    assert np.all(w[96:112] == 0.25 * 7 * 18)
    q8 = np.zeros(34, dtype=np.uint8)
    q8[0:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
    q8[2:] = np.arange(-16, 16, dtype=np.int8).view(np.uint8)
    assert np.array_equal(oracle_mod.dequant(q8, 8, 32), 0.5 * np.arange(-16, 16, dtype=np.float32))


def test_unsupported_type_is_reported(oracle_mod):
    with pytest.raises(ValueError):
        oracle_mod.dequant(np.zeros(64, np.uint8), 99, 32)
    with pytest.raises(ValueError):
        oracle_mod.gemv(np.zeros(32, np.float32), np.zeros(64, np.uint8), 15, 32, 1)


def test_q4k_gemv_is_the_factored_form(pkg, oracle_mod):
    """src/dequant.rs:659-706 sums d1*sum(x*q) - m1*sum(x) per sub-block: close to, but not
    bitwise, dequant()-then-dot; both within the acceptance bound."""
    from saient_quartz_b200 import synth
    K, N = 1024, 32
    w = synth.make_weights(12, K, N, tensor_id=3)
    x = synth.make_x(K, tensor_id=4)
    y = oracle_mod.gemv(x, w, 12, K, N)
    deq = oracle_mod.dequant(w, 12, K * N).reshape(N, K)
    naive = np.array([np.float32(sum(np.float32(a) * np.float32(b) for a, b in zip(x, r))) for r in deq[:2]])
    tol = oracle_mod.tolerance(w, 12, K, N, x)
    assert np.all(np.abs(y[:2] - naive) <= tol[:2])
    assert np.all(np.abs(y - oracle_mod.gemv_f64(x, w, 12, K, N)) <= tol)


def test_gemm_matches_gemv_per_token(pkg, oracle_mod):
    """src/dequant.rs:143-200: token-major output; n == 1 is gemv itself."""
    from saient_quartz_b200 import synth
    K, N, M = 512, 24, 5
    X = synth.make_x(K, tensor_id=11, rows=M)
    for t in (12, 14, 8, 7, 17):
        w = synth.make_weights(t, K, N, tensor_id=12)
        out = oracle_mod.gemm(X, w, t, K, N, M)
        assert out.shape == (M, N)
        tol = oracle_mod.tolerance(w, t, K, N, X[0]) * 4
        for m in range(M):
            assert np.all(np.abs(out[m] - oracle_mod.gemv(X[m], w, t, K, N)) <= tol)
        one = oracle_mod.gemm(X[:1], w, t, K, N, 1)
        assert np.array_equal(one[0], oracle_mod.gemv(X[0], w, t, K, N))


def test_threads_do_not_change_results(pkg, oracle_mod):
    from saient_quartz_b200 import synth
    K, N = 512, 64
    w = synth.make_weights(14, K, N, tensor_id=5)
    x = synth.make_x(K, tensor_id=6)
    assert np.array_equal(oracle_mod.gemv(x, w, 14, K, N, threads=1), oracle_mod.gemv(x, w, 14, K, N, threads=0))


def test_empty_output(pkg, oracle_mod):
    y = oracle_mod.gemv(np.zeros(256, np.float32), np.zeros(0, np.uint8), 12, 256, 0)
    assert y.shape == (0,)


def test_ksigns_is_parity_table(oracle_mod, tables):
    assert np.array_equal(oracle_mod.ksigns(), tables["ksigns"])


@pytest.mark.skipif(REF is None, reason="reference tree not mounted")
def test_codebooks_equal_reference_tables(tables):
    """The gguf-package codebooks are the numbers in src/iq2_tables.rs / src/iq3_tables.rs."""
    def parse(path, name):
        text = open(path).read()
        m = re.search(r"pub static %s: \[\w+; \d+\] = \[(.*?)\];" % name, text, flags=re.S)
        return [int(v, 0) for v in m.group(1).replace("\n", " ").split(",") if v.strip()]
    iq2 = os.path.join(REF, "iq2_tables.rs")
    assert parse(iq2, "IQ2XXS_GRID") == [int(v) for v in tables["iq2xxs"]]
    assert parse(iq2, "IQ2XS_GRID") == [int(v) for v in tables["iq2xs"]]
    assert parse(iq2, "IQ2S_GRID") == [int(v) for v in tables["iq2s"]]
    assert parse(iq2, "KSIGNS_IQ2XS") == [int(v) for v in tables["ksigns"]]
    assert parse(os.path.join(REF, "iq3_tables.rs"), "IQ3S_GRID") == [int(v) for v in tables["iq3s"]]
