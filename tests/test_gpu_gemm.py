"""GPU parity tests of the complex GEMM, through the C ABI, against the CPU oracle.

The cases re-express the reference's operator tests (test/gemm/mma.cpp: types :351-372, shapes
:402-408 and :426-434, sections :442-520, alpha/beta :645-776; test/cuda/mma.cpp:87-94 all-ones
known answer) and add the BASELINE configurations at sizes the oracle finishes in seconds."""
import os

import numpy as np
import pytest

import gpu_util as gu
import oracle_util as ou
from ccglib_b200 import capi

pytestmark = pytest.mark.gpu

FLOAT_TYPES = [(ou.E4M3, ou.F32), (ou.E5M2, ou.F32), (ou.F16, ou.F16), (ou.F32, ou.F16),
               (ou.F16, ou.F32), (ou.F32, ou.F32), (ou.BF16, ou.F32), (ou.BF16, ou.BF16),
               (ou.F32, ou.BF16)]
TYPE_IDS = ["%s-%s" % (ou.TYPE_NAMES[i], ou.TYPE_NAMES[o]) for i, o in FLOAT_TYPES]
SHAPES = [(128, 256, 64), (100, 60, 40)]  # aligned / unaligned, as in the reference
SECTIONS = [  # (variant, complex axis of C, memory order of C)
    (capi.BASIC, capi.PLANAR, capi.ROW_MAJOR),
    (capi.BASIC, capi.PLANAR, capi.COL_MAJOR),
    (capi.OPT, capi.PLANAR, capi.ROW_MAJOR),
    (capi.OPT, capi.PLANAR, capi.COL_MAJOR),
    (capi.OPT, capi.INTERLEAVED, capi.ROW_MAJOR),
    (capi.OPT, capi.INTERLEAVED, capi.COL_MAJOR),
]
SECTION_IDS = ["basic-row", "basic-col", "opt-row", "opt-col", "opt-inter-row", "opt-inter-col"]


def make_inputs(seed, type_in, B, M, N, K, dist="unit", scale=1.0):
    rng = np.random.default_rng(seed)
    if type_in == ou.INT1:
        kw = (K + 31) // 32
        a = ou.random_storage(rng, (B, 2, M, kw), ou.INT1)
        b = ou.random_storage(rng, (B, 2, N, kw), ou.INT1)
        pad = kw * 32 - K
        if pad:
            mask = np.uint32((1 << (32 - pad)) - 1)
            a[..., -1] &= mask
            b[..., -1] &= mask
        return a, b
    a = ou.random_storage(rng, (B, 2, M, K), type_in, dist, scale)
    b = ou.random_storage(rng, (B, 2, N, K), type_in, dist, scale)
    return a, b


@pytest.mark.parametrize("section", SECTIONS, ids=SECTION_IDS)
@pytest.mark.parametrize("shape", SHAPES, ids=["aligned", "unaligned"])
@pytest.mark.parametrize("types", FLOAT_TYPES, ids=TYPE_IDS)
def test_float_gemm_matches_oracle(types, shape, section):
    type_in, type_out = types
    M, N, K = shape
    variant, c_axis, c_order = section
    B = 3
    a, b = make_inputs(11, type_in, B, M, N, K)
    got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=variant, c_axis=c_axis,
                      c_order=c_order)
    got = gu.canonical_c(got, B, M, N, c_axis, c_order)
    want = gu.oracle_batch(type_in, type_out, a, b, B, M, N, K)
    gu.assert_close_reference_rule(got, want, type_in, type_out)
    gu.assert_close_fp64(got, type_in, type_out, a, b, K)


def test_reference_fixture_batch16_f16():
    # the reference fixture's batch size (test/gemm/mma.cpp:135)
    B, M, N, K = 16, 128, 256, 64
    a, b = make_inputs(12, ou.F16, B, M, N, K)
    got = gu.run_gemm(ou.F16, ou.F32, a, b, B, M, N, K, variant=capi.OPT)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, use_reference=True)
    gu.assert_close_reference_rule(got.reshape(B, 2, M, N), want, ou.F16, ou.F32)
    gu.assert_close_fp64(got.reshape(B, 2, M, N), ou.F16, ou.F32, a, b, K)


@pytest.mark.parametrize("variant", [capi.BASIC, capi.OPT], ids=["basic", "opt"])
@pytest.mark.parametrize("c_order", [capi.ROW_MAJOR, capi.COL_MAJOR], ids=["row", "col"])
@pytest.mark.parametrize("shape", [(64, 64, 256), (100, 60, 288), (130, 300, 1056)],
                         ids=["aligned", "unaligned", "multi-tile"])
def test_int1_gemm_bit_exact(shape, c_order, variant):
    M, N, K = shape
    B = 3
    a, b = make_inputs(13, ou.INT1, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=variant, c_order=c_order)
    got = gu.canonical_c(got, B, M, N, capi.PLANAR, c_order)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K)
    assert np.array_equal(got, want)


def test_int1_interleaved_output_and_k_padding():
    # K not a multiple of 32: padding bits are zero and must not contribute
    # (src/reference/GEMM.cpp:165-200)
    B, M, N, K = 2, 40, 72, 70
    a, b = make_inputs(14, ou.INT1, B, M, N, K)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC)
    assert np.array_equal(got.reshape(B, 2, M, N), want)
    K = 96
    a, b = make_inputs(15, ou.INT1, B, M, N, K)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.OPT,
                      c_axis=capi.INTERLEAVED)
    assert np.array_equal(gu.canonical_c(got, B, M, N, capi.INTERLEAVED, capi.ROW_MAJOR), want)


@pytest.mark.parametrize("M", [255, 256])
def test_alpha_beta_f16(M):
    # test/gemm/mma.cpp:645-700
    B, N, K = 2, 128, 256
    alpha, beta = (0.3, 1.6), (0.8, -1.1)
    a, b = make_inputs(16, ou.F16, B, M, N, K)
    rng = np.random.default_rng(17)
    c0 = rng.random((B, 2, M, N), dtype=np.float32)
    got = gu.run_gemm(ou.F16, ou.F32, a, b, B, M, N, K, variant=capi.BASIC, alpha=alpha, beta=beta,
                      c0=c0)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, alpha, beta, c0)
    gu.assert_close_reference_rule(got.reshape(B, 2, M, N), want, ou.F16, ou.F32)
    # tighter: alpha/beta are applied in float32 on a float32 accumulator
    assert np.allclose(got.reshape(B, 2, M, N), want, rtol=2e-5, atol=2e-3)


@pytest.mark.parametrize("section", [(capi.OPT, capi.INTERLEAVED, capi.COL_MAJOR),
                                     (capi.OPT, capi.PLANAR, capi.COL_MAJOR),
                                     (capi.OPT, capi.INTERLEAVED, capi.ROW_MAJOR)],
                         ids=["inter-col", "planar-col", "inter-row"])
def test_alpha_beta_f16_out_layouts(section):
    variant, c_axis, c_order = section
    B, M, N, K = 2, 100, 60, 40
    alpha, beta = (0.5, 2.5), (0.25, -1.5)
    a, b = make_inputs(18, ou.F16, B, M, N, K)
    rng = np.random.default_rng(19)
    c0 = ou.quantize(rng.random((B, 2, M, N), dtype=np.float32), ou.F16)  # canonical
    # lay c0 out the way the GEMM will read it
    if c_axis == capi.PLANAR:
        c0_dev = c0.transpose(0, 1, 3, 2) if c_order == capi.COL_MAJOR else c0
    else:
        c0_dev = c0.transpose(0, 3, 2, 1) if c_order == capi.COL_MAJOR else c0.transpose(0, 2, 3, 1)
    got = gu.run_gemm(ou.F16, ou.F16, a, b, B, M, N, K, variant=variant, c_axis=c_axis,
                      c_order=c_order, alpha=alpha, beta=beta, c0=np.ascontiguousarray(c0_dev))
    got = gu.canonical_c(got, B, M, N, c_axis, c_order)
    want = gu.oracle_batch(ou.F16, ou.F16, a, b, B, M, N, K, alpha, beta, c0)
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F16)


@pytest.mark.parametrize("path", [dict(CCGLIB_B200_INT1_MXF4="0"),
                                  dict(CCGLIB_B200_INT1_MXF4="0", CCGLIB_B200_PAIR="1"),
                                  dict(CCGLIB_B200_INT1_MXF4="1", CCGLIB_B200_MXF4_NEGATE="0",
                                       CCGLIB_B200_PAIR="0"),
                                  dict(CCGLIB_B200_INT1_MXF4="1", CCGLIB_B200_MXF4_NEGATE="1",
                                       CCGLIB_B200_PAIR="0"),
                                  dict(CCGLIB_B200_INT1_MXF4="1", CCGLIB_B200_MXF4_NEGATE="0",
                                       CCGLIB_B200_PAIR="1"),
                                  dict(CCGLIB_B200_INT1_MXF4="1", CCGLIB_B200_MXF4_NEGATE="1",
                                       CCGLIB_B200_PAIR="1")],
                         ids=["i8", "i8-pair", "mxf4-3planes", "mxf4-negate", "mxf4-3planes-pair",
                              "mxf4-negate-pair"])
def test_int1_every_tensor_path_is_bit_exact(path, monkeypatch):
    """1-bit GEMM runs as signed bytes on the integer MMA kind or as e2m1 nibbles on the
    block-scaled 4-bit kind (unit scale factors), with -Ai from a third plane or from the negate
    bit, on one SM or a CTA pair: all of them must reproduce the oracle exactly, alpha/beta,
    ragged edges and K padding included."""
    for key, value in path.items():
        monkeypatch.setenv(key, value)
    B, M, N, K = 2, 300, 520, 2000
    a, b = make_inputs(31, ou.INT1, B, M, N, K)
    rng = np.random.default_rng(32)
    c0 = rng.integers(-100, 100, size=(B, 2, M, N), dtype=np.int32)
    alpha, beta = (2.0, -3.0), (1.0, 2.0)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC, alpha=alpha,
                      beta=beta, c0=c0)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K, alpha, beta, c0)
    assert np.array_equal(got.reshape(B, 2, M, N), want)
    K = 2016  # the tiled layout holds whole 32-sample words
    a, b = make_inputs(33, ou.INT1, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.OPT,
                      c_axis=capi.INTERLEAVED, c_order=capi.COL_MAJOR)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K)
    assert np.array_equal(gu.canonical_c(got, B, M, N, capi.INTERLEAVED, capi.COL_MAJOR), want)


def test_alpha_beta_int1():
    # test/gemm/mma.cpp:702-776
    B, M, N, K = 2, 256, 128, 256
    alpha, beta = (2.0, 3.0), (-1.0, 2.0)
    a, b = make_inputs(20, ou.INT1, B, M, N, K)
    rng = np.random.default_rng(21)
    c0 = rng.integers(-100, 100, size=(B, 2, M, N), dtype=np.int32)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC, alpha=alpha,
                      beta=beta, c0=c0)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K, alpha, beta, c0)
    assert np.array_equal(got.reshape(B, 2, M, N), want)


@pytest.mark.parametrize("type_in", [ou.F16, ou.BF16, ou.F32, ou.E4M3, ou.E5M2, ou.INT1],
                         ids=lambda t: ou.TYPE_NAMES[t])
def test_all_ones_known_answer(type_in):
    # all-ones input: Re = K - K = 0, Im = 2K (test/cuda/mma.cpp:87-94)
    B, M, N, K = 2, 128, 64, 256
    type_out = ou.INT32 if type_in == ou.INT1 else ou.F32
    if type_in == ou.INT1:
        a = np.full((B, 2, M, K // 32), 0xFFFFFFFF, np.uint32)
        b = np.full((B, 2, N, K // 32), 0xFFFFFFFF, np.uint32)
    else:
        a = ou.quantize(np.ones((B, 2, M, K), np.float32), type_in)
        b = ou.quantize(np.ones((B, 2, N, K), np.float32), type_in)
    got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=capi.BASIC).reshape(B, 2, M, N)
    assert np.all(got[:, 0] == 0)
    assert np.all(got[:, 1] == 2 * K)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("sw_pair", [(64, 0), (128, 0), (128, 1)],
                         ids=["sw64", "sw128", "sw128-pair"])
@pytest.mark.parametrize("types", [(ou.F16, ou.F32), (ou.INT1, ou.INT32), (ou.E4M3, ou.F32),
                                   (ou.F32, ou.F16)],
                         ids=["f16", "int1", "e4m3", "tf32-f16"])
def test_every_tile_configuration(types, sw_pair, bn, monkeypatch):
    """The tile width (128/256 columns), the stage row width (64/128 bytes) and whether two CTAs
    work as a pair on a 256-row tile are chosen by heuristics; force each combination on a
    multi-tile, multi-k-block, ragged problem (odd number of 128-row blocks included)."""
    sw, pair = sw_pair
    monkeypatch.setenv("CCGLIB_B200_BN", str(bn))
    monkeypatch.setenv("CCGLIB_B200_SW", str(sw))
    monkeypatch.setenv("CCGLIB_B200_PAIR", str(pair))
    type_in, type_out = types
    B, M, N = 2, 300, 520  # 3 blocks of 128 rows: the second CTA pair is half empty
    K = 1056 if type_in == ou.INT1 else 712
    a, b = make_inputs(22, type_in, B, M, N, K, dist="uniform")
    for variant in (capi.BASIC, capi.OPT):
        got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=variant).reshape(B, 2, M, N)
        if type_in == ou.INT1:
            assert np.array_equal(got, gu.oracle_batch(type_in, type_out, a, b, B, M, N, K))
        else:
            gu.assert_close_fp64(got, type_in, type_out, a, b, K)


def test_l2_prefetch_cursor_does_not_change_results(monkeypatch):
    monkeypatch.setenv("CCGLIB_B200_PREFETCH", "5")
    B, M, N, K = 3, 300, 520, 200  # 4 k-blocks per tile: the cursor runs into later tiles
    a, b = make_inputs(30, ou.BF16, B, M, N, K, dist="uniform")
    for variant in (capi.BASIC, capi.OPT):
        got = gu.run_gemm(ou.BF16, ou.F32, a, b, B, M, N, K, variant=variant).reshape(B, 2, M, N)
        gu.assert_close_fp64(got, ou.BF16, ou.F32, a, b, K)


def test_interleaved_input_through_transpose():
    # BASELINE config 2 in miniature: interleaved complex input -> Transpose -> opt GEMM
    B, M, N, K = 2, 200, 300, 100
    a, b = make_inputs(23, ou.F16, B, M, N, K, dist="normal", scale=1.0 / np.sqrt(K))
    a_il = np.ascontiguousarray(a.transpose(0, 2, 3, 1))
    b_il = np.ascontiguousarray(b.transpose(0, 2, 3, 1))
    got = gu.run_gemm(ou.F16, ou.F32, a_il, b_il, B, M, N, K, variant=capi.OPT,
                      in_axis=capi.INTERLEAVED).reshape(B, 2, M, N)
    gu.assert_close_fp64(got, ou.F16, ou.F32, a, b, K)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K)
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F32)


def test_config1_basic_f16_1024_cubed():
    # BASELINE config 1 at full size, against the reference's own CPU GEMM where it was built
    B, M, N, K = 1, 1024, 1024, 1024
    a, b = make_inputs(1001, ou.F16, B, M, N, K, dist="uniform")
    got = gu.run_gemm(ou.F16, ou.F32, a, b, B, M, N, K, variant=capi.BASIC).reshape(B, 2, M, N)
    want = gu.oracle_batch(ou.F16, ou.F32, a, b, B, M, N, K, use_reference=True)
    gu.assert_close_reference_rule(got, want, ou.F16, ou.F32)
    ratio = gu.assert_close_fp64(got, ou.F16, ou.F32, a, b, K)
    print("config1 accumulation error / (sqrt(2K) u S) = %.3f" % ratio)


LONG_K = [
    ("f16-K8192", ou.F16, ou.F32, 2, 256, 512, 8192, "normal"),      # config 2's K
    ("e4m3-K16384", ou.E4M3, ou.F32, 1, 256, 256, 16384, "fp8"),      # config 4's K
    ("e5m2-K16384", ou.E5M2, ou.F32, 1, 256, 256, 16384, "fp8"),
    ("bf16-c5", ou.BF16, ou.F32, 4, 256, 2048, 512, "uniform"),      # config 5's item shape
    ("tf32-c5", ou.F32, ou.F32, 4, 256, 2048, 512, "uniform"),
]


@pytest.mark.parametrize("case", LONG_K, ids=[c[0] for c in LONG_K])
def test_baseline_shapes_fp64_gate(case):
    _, type_in, type_out, B, M, N, K, dist = case
    if dist == "fp8":
        # N(0,1) clamped to +-4, scaled to +-0.5 * max finite value, rounded to the fp8 type
        rng = np.random.default_rng(24)
        fmax = 448.0 if type_in == ou.E4M3 else 57344.0
        gen = lambda shape: ou.quantize(
            (np.clip(rng.standard_normal(shape), -4, 4) / 4 * 0.5 * fmax).astype(np.float32),
            type_in)
        a, b = gen((B, 2, M, K)), gen((B, 2, N, K))
    else:
        a, b = make_inputs(25, type_in, B, M, N, K, dist=dist,
                           scale=1.0 / np.sqrt(K) if dist == "normal" else 1.0)
    got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K, variant=capi.OPT).reshape(B, 2, M, N)
    ratio = gu.assert_close_fp64(got, type_in, type_out, a, b, K)
    print("%s accumulation error / (sqrt(2K) u S) = %.3f" % (case[0], ratio))


@pytest.mark.parametrize("types", [(ou.F16, ou.F32), (ou.BF16, ou.F32), (ou.F32, ou.F32),
                                   (ou.E4M3, ou.F32)], ids=["f16", "bf16", "tf32", "e4m3"])
def test_same_sign_inputs_show_the_truncation_bias_and_stay_inside_the_gate(types):
    """All-positive operands make the running sum of the imaginary part grow to |c|; the tensor
    core's truncating adder then loses a fraction of a unit in the last place per MMA
    instruction, always downwards.  The gate's bias term covers it; the measured share of that
    term is printed."""
    type_in, type_out = types
    B, M, N, K = 1, 256, 256, 4096
    a, b = make_inputs(71, type_in, B, M, N, K, dist="unit")
    got = gu.run_gemm(type_in, type_out, a, b, B, M, N, K).reshape(B, 2, M, N)
    gu.assert_close_fp64(got, type_in, type_out, a, b, K)
    c64, s = ou.double_gemm(type_in, a[0], b[0])
    im_err = got[0, 1].astype(np.float64) - c64[1]
    steps = 2.0 * K / gu.MMA_K[type_in]
    share = np.abs(im_err) / (steps * 2.0 ** -23 * np.abs(c64[1]))
    print("%s: bias %.3g of |c| (mean signed error %.3g), %.2f of the gate's bias term at most" % (
        ou.TYPE_NAMES[type_in], float(np.abs(im_err).max() / np.abs(c64[1]).max()),
        float(im_err.mean()), float(share.max())))
    assert float(im_err.mean()) <= 0.0  # truncation: never above the exact sum on positive data


def test_int1_config3_k65536_bit_exact():
    # BASELINE config 3's K (65536 bits) on one 128 x 256 output tile per batch item
    B, M, N, K = 2, 128, 256, 65536
    a, b = make_inputs(26, ou.INT1, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.OPT).reshape(B, 2, M, N)
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K)
    assert np.array_equal(got, want)


def _step_rows(points, K):
    """Packed 1-bit rows whose sample k is +1 (bit set) for k < points[r] and -1 after."""
    kw = K // 32
    word = np.arange(kw, dtype=np.int64)[None, :]
    p = np.asarray(points, dtype=np.int64)[:, None]
    full = word < p // 32
    part = word == p // 32
    partial = ((np.uint64(1) << (p % 32).astype(np.uint64)) - np.uint64(1)).astype(np.uint32)
    return np.where(full, np.uint32(0xFFFFFFFF), np.where(part, partial, np.uint32(0)))


def _step_dot(p, q, K):
    """sum_k a(k) b(k) for two such rows: they agree except between the two steps."""
    return K - 2 * np.abs(np.asarray(p, np.int64)[:, None] - np.asarray(q, np.int64)[None, :])


CORRELATED = [
    ("k65536-single", 128, 128, 65536, {}),
    ("k65536-pair", 256, 224, 65536, {}),
    ("k65536-3planes", 256, 192, 65536, dict(CCGLIB_B200_MXF4_NEGATE="0")),
    ("k2^22-pair", 256, 128, 1 << 22, {}),
    ("k2^22-single", 128, 128, 1 << 22, dict(CCGLIB_B200_PAIR="0")),
    ("k2^22+1024-i8", 128, 128, (1 << 22) + 1024, {}),
]


@pytest.mark.parametrize("case", CORRELATED, ids=[c[0] for c in CORRELATED])
def test_int1_correlated_inputs_large_sums_bit_exact(case, monkeypatch):
    """Correlated 1-bit input (what a correlator's autocorrelations look like) drives the sums to
    +-2K, where random signs only reach sqrt(2K): all-ones rows, rows that are +1 up to a step
    and -1 after it, and their negations.  The default tensor route accumulates in float32, so
    every partial sum up to 2K = 2^23 must be held exactly; the answer is known in closed form
    (rows with steps at p and q agree in K - |p - q| samples)."""
    _, M, N, K, env = case
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    rng = np.random.default_rng(41)

    def points(rows):
        p = rng.integers(0, K + 1, rows)
        p[:4] = [K, K, 0, K // 2]  # all +1, all +1, all -1, half and half
        return p

    pa_re, pa_im, pb_re, pb_im = points(M), points(M), points(N), points(N)
    pa_im[0], pb_re[0], pb_im[0] = 0, K, K  # row 0 x column 0: Re = K - (-K) = 2K, Im = 0
    pa_im[1], pb_re[1], pb_im[1] = K, K, K  # row 1 x column 1: Re = 0, Im = 2K
    a = np.stack([_step_rows(pa_re, K), _step_rows(pa_im, K)])[None]
    b = np.stack([_step_rows(pb_re, K), _step_rows(pb_im, K)])[None]
    want_re = _step_dot(pa_re, pb_re, K) - _step_dot(pa_im, pb_im, K)
    want_im = _step_dot(pa_re, pb_im, K) + _step_dot(pa_im, pb_re, K)
    assert want_re[0, 0] == 2 * K and want_im[1, 1] == 2 * K
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, 1, M, N, K, variant=capi.BASIC).reshape(2, M, N)
    assert np.array_equal(got[0], want_re)
    assert np.array_equal(got[1], want_im)


def test_int1_correlated_closed_form_agrees_with_oracle():
    # the closed form used above, checked against the CPU oracle at a size it finishes quickly
    M, N, K = 40, 24, 2048
    rng = np.random.default_rng(42)
    pts = [rng.integers(0, K + 1, r) for r in (M, M, N, N)]
    a = np.stack([_step_rows(pts[0], K), _step_rows(pts[1], K)])[None]
    b = np.stack([_step_rows(pts[2], K), _step_rows(pts[3], K)])[None]
    want = gu.oracle_batch(ou.INT1, ou.INT32, a, b, 1, M, N, K)[0]
    assert np.array_equal(want[0], _step_dot(pts[0], pts[2], K) - _step_dot(pts[1], pts[3], K))
    assert np.array_equal(want[1], _step_dot(pts[0], pts[3], K) + _step_dot(pts[1], pts[2], K))
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, 1, M, N, K, variant=capi.BASIC).reshape(2, M, N)
    assert np.array_equal(got, want)


def test_tf32_ignores_low_mantissa_bits():
    """float32 input is consumed as tf32: the 13 low mantissa bits are dropped (truncation), which
    is what the reference assumes (kernels/gemm_kernel_float.cu:80-81) and why its tests mask
    their inputs (test/gemm/mma.cpp:32-38).  Unmasked input must give the masked result."""
    B, M, N, K = 1, 128, 128, 64
    rng = np.random.default_rng(27)
    a = rng.uniform(-1, 1, (B, 2, M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (B, 2, N, K)).astype(np.float32)
    got = gu.run_gemm(ou.F32, ou.F32, a, b, B, M, N, K, variant=capi.BASIC)
    got_masked = gu.run_gemm(ou.F32, ou.F32, ou.mask_tf32(a), ou.mask_tf32(b), B, M, N, K,
                             variant=capi.BASIC)
    assert np.array_equal(got, got_masked)


def test_staged_batch_chunks(monkeypatch):
    """1-bit input is re-staged through plan-owned scratch in batch chunks; force several chunks."""
    monkeypatch.setenv("CCGLIB_B200_SCRATCH_MB", "1")
    B, M, N, K = 5, 128, 256, 1024  # 0.6 MiB of staged bytes per item -> one item per chunk
    a, b = make_inputs(28, ou.INT1, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC).reshape(B, 2, M, N)
    assert np.array_equal(got, gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K))


@pytest.mark.parametrize("type_in,type_out,K", [(ou.INT1, ou.INT32, 1056), (ou.F16, ou.F32, 100)])
def test_staged_two_lanes(monkeypatch, type_in, type_out, K):
    """Staged plans with several chunks alternate them over two internal streams; the result must
    equal the single-lane one bit for bit, run after run, and match the oracle."""
    import torch

    B, M, N = 7, 200, 264
    a, b = make_inputs(31, type_in, B, M, N, K)
    d_a, d_b = gu.dev(a), gu.dev(b)
    outs = []
    for lanes in ("1", "2"):
        monkeypatch.setenv("CCGLIB_B200_LANES", lanes)
        monkeypatch.setenv("CCGLIB_B200_LANE_WAVES", "0")  # small chunks qualify
        plan = capi.GemmPlan(B, M, N, K, type_in, type_out, variant=capi.BASIC)
        assert plan.launches == (3 * 7 if lanes == "2" else 3)
        for _ in range(2):
            d_c = gu.dev_empty(B * 2 * M * N * 4, 0xFF)
            plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), gu.stream_handle())
            torch.cuda.synchronize()
            gu.check_device_status()
            outs.append(d_c)
        plan.close()
    for other in outs[1:]:
        assert torch.equal(outs[0], other)
    dt = np.int32 if type_out == ou.INT32 else np.float32
    got = gu.host(outs[-1], dt).reshape(B, 2, M, N)
    if type_in == ou.INT1:
        assert np.array_equal(got, gu.oracle_batch(type_in, type_out, a, b, B, M, N, K))
    else:
        gu.assert_close_fp64(got, type_in, type_out, a, b, K)


def test_staged_two_lanes_by_default_on_a_large_batch():
    """A 1-bit batch of many tile waves is split into chunks over two lanes without any override."""
    B, M, N, K = 64, 1024, 1024, 256
    plan = capi.GemmPlan(B, M, N, K, ou.INT1, ou.INT32, variant=capi.BASIC)
    launches = plan.launches
    plan.close()
    assert launches >= 6 and launches % 3 == 0  # at least two chunks of (expand A, expand B, GEMM)
    a, b = make_inputs(33, ou.INT1, B, M, N, K)
    got = gu.run_gemm(ou.INT1, ou.INT32, a, b, B, M, N, K, variant=capi.BASIC).reshape(B, 2, M, N)
    assert np.array_equal(got, gu.oracle_batch(ou.INT1, ou.INT32, a, b, B, M, N, K))


def test_run_twice_same_plan_is_deterministic():
    import torch

    B, M, N, K = 2, 256, 256, 512
    a, b = make_inputs(29, ou.F16, B, M, N, K)
    d_a, d_b = gu.dev(a), gu.dev(b)
    d_c1 = gu.dev_empty(B * 2 * M * N * 4, 0)
    d_c2 = gu.dev_empty(B * 2 * M * N * 4, 0)
    plan = capi.GemmPlan(B, M, N, K, ou.F16, ou.F32, variant=capi.BASIC)
    plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c1.data_ptr(), gu.stream_handle())
    plan.run(d_a.data_ptr(), d_b.data_ptr(), d_c2.data_ptr(), gu.stream_handle())
    torch.cuda.synchronize()
    gu.check_device_status()
    assert torch.equal(d_c1, d_c2)


def test_verbose_prints_the_plan_geometry(monkeypatch, capfd):
    # the counterpart of the reference's DEBUG print of its launch geometry (src/mma/GEMM.cpp:84-95)
    monkeypatch.setenv("CCGLIB_B200_VERBOSE", "1")
    plan = capi.GemmPlan(2, 300, 520, 1056, ou.INT1, ou.INT32, variant=capi.BASIC)
    plan.close()
    err = capfd.readouterr().err
    assert "ccglib_b200 plan: batch 2 M 300 N 520 K 1056" in err and "CTA pair" in err
