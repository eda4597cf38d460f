"""Pins the CPU oracle against the golden vectors and host reference loops held by the
reference's own tests (src/ternary_gemm_test.cpp, src/int8_act_test.cpp, src/t1_58_test.cpp).
Runs without a GPU."""
import numpy as np
import pytest


# ---- src/ternary_gemm_test.cpp:69-99 -------------------------------------------------
def test_trit_layout_constants(orc):
    assert orc.trit_words_per_row(16) == 1
    assert orc.trit_words_per_row(17) == 2
    assert orc.trit_words_per_row(1) == 1
    assert orc.trit_bytes_per_row(512) == 128  # 0.25 B / weight


GOLD_W16 = [1.0, -1.0, 0.0, 0.4, -0.4, 1.0, -1.0, 0.0, 0.9, -0.9, 0.1, -0.1, 0.6, -0.6, 0.0, 0.0]
GOLD_CODES16 = [3, 1, 2, 2, 2, 3, 1, 2, 3, 1, 2, 2, 3, 1, 2, 2]


def test_trit_golden_codes_and_bit_order(orc):
    word = orc.trit_pack_row(np.array(GOLD_W16, np.float32), 1.0)
    assert word.shape == (1,)
    for j in range(16):
        assert (int(word[0]) >> (2 * j)) & 3 == GOLD_CODES16[j]


def test_trit_tail_padding_is_code_two(orc):
    w2 = orc.trit_pack_row(np.array(GOLD_W16[:5], np.float32), 1.0)
    for i in range(5):
        assert orc.trit_at(w2, i) == orc.trit_value_of(GOLD_CODES16[i])
    for i in range(5, 16):
        assert orc.trit_at(w2, i) == 0.0  # tail = trit 0, not the undefined code 0


def test_trit_threshold_is_strict(orc):
    # |w| == 0.5*tau goes to 0 (compute_layer_bitlinear.hpp:657-667)
    assert orc.trit_code_of(0.5, 1.0) == 2
    assert orc.trit_code_of(-0.5, 1.0) == 2
    assert orc.trit_code_of(np.nextafter(np.float32(0.5), np.float32(1)), 1.0) == 3
    assert orc.trit_code_of(-np.nextafter(np.float32(0.5), np.float32(1)), 1.0) == 1


# ---- src/t1_58_test.cpp:211-252 (known latent, tau and trits) -------------------------
RAW_W = np.array([[1.0, 0.3, -0.3, 0.3], [0.4, -0.4, 0.1, -0.1], [0.7, 0.6, 0.5, 0.1]], np.float32)
KX = np.array([[1.0, -2.0], [0.5, 1.0], [-1.0, 0.25], [2.0, -0.5]], np.float32)


def test_bitlinear_known_tau_and_trits(orc):
    tau = orc.absmean_tau(RAW_W)
    assert np.allclose(tau, [0.475, 0.25, 0.475], atol=1e-6)
    packed = orc.trit_pack(RAW_W, tau)
    trits = orc.trit_unpack(packed, 4)
    want = np.array([[1, 1, -1, 1], [1, -1, 0, 0], [1, 1, 1, 0]], np.int8)
    assert np.array_equal(trits, want)
    # row 0: absmean keeps the 0.3 entries (absmax would zero them)
    assert trits[0, 1] == 1 and trits[0, 2] == -1


def test_bitlinear_known_forward_and_grads(orc):
    tau = orc.absmean_tau(RAW_W)
    packed = orc.trit_pack(RAW_W, tau)
    wq = orc.trit_unpack(packed, 4).astype(np.float64)
    y = orc.matmul_q(packed, tau, KX, 4)
    ref = (wq @ KX.astype(np.float64)) * tau.astype(np.float64)[:, None]
    assert np.abs(y - ref).max() < 1e-5
    dY = np.array([[0.5, -0.25], [1.0, 0.75], [-0.5, 0.25]], np.float32)
    # dX = wq^T (dY * tau): matmul_q_t with tau per storage row inside the sum
    dx = orc.matmul_q_t(packed, tau, dY, 4)
    ref_dx = wq.T @ (dY.astype(np.float64) * tau.astype(np.float64)[:, None])
    assert np.abs(dx - ref_dx).max() < 1e-5


# ---- src/ternary_gemm_test.cpp:188-251, 529-539 (generators and odd shapes) ------------
def _gen(rows, k, n):
    r = np.arange(rows)[:, None]
    c = np.arange(k)[None, :]
    W = (0.13 * ((r * 7 + c * 3) % 11) - 0.6).astype(np.float32)
    kk = np.arange(k)[:, None]
    nn_ = np.arange(n)[None, :]
    X = (0.21 * ((kk + 2 * nn_) % 9) - 0.8).astype(np.float32)
    return W, X


@pytest.mark.parametrize("rows,k,n", [(7, 40, 3), (5, 17, 1), (64, 64, 8), (65, 100, 7), (130, 48, 3)])
def test_matmul_q_matches_host_reference(orc, rows, k, n):
    W, X = _gen(rows, k, n)
    tau = (np.abs(W.astype(np.float64)).sum(1) / k).astype(np.float32)
    packed = orc.trit_pack(W, tau)
    # packed words == row-wise pack_row
    for r in range(rows):
        assert np.array_equal(packed[r], orc.trit_pack_row(W[r], float(tau[r])))
    trit = orc.trit_unpack(packed, k).astype(np.float64)
    want = np.where(W > 0.5 * tau[:, None], 1, np.where(W < -0.5 * tau[:, None], -1, 0))
    assert np.array_equal(trit, want)
    ref = ((tau[:, None] * trit.astype(np.float32)).astype(np.float64)) @ X.astype(np.float64)
    got = orc.matmul_q(packed, tau, X, k)
    assert np.abs(got - ref).max() <= 1e-5 + 1e-4 * np.abs(ref).max()


@pytest.mark.parametrize("rows,m,n", [(40, 7, 3), (17, 5, 2), (64, 33, 4)])
def test_matmul_q_t_matches_host_reference(orc, rows, m, n):
    W, _ = _gen(rows, m, n)
    _, B = _gen(1, rows, n)
    tau = (np.abs(W.astype(np.float64)).sum(1) / m).astype(np.float32)
    packed = orc.trit_pack(W, tau)
    trit = orc.trit_unpack(packed, m).astype(np.float32)
    ref = ((tau[:, None] * trit).astype(np.float64)).T @ B.astype(np.float64)
    got = orc.matmul_q_t(packed, tau, B, m)
    assert np.abs(got - ref).max() <= 1e-5 + 1e-4 * np.abs(ref).max()


# ---- src/int8_act_test.cpp:86-168 (quantise rule, byte order, unpack) -------------------
def test_i8_quantize_rule(orc):
    assert orc.i8_quantize(1.0, 0.0) == 0            # s == 0 -> 0
    assert orc.i8_quantize(float("nan"), 1.0) == 0   # NaN -> 0
    assert orc.i8_quantize(0.5, 1.0) == 1            # round half away from zero
    assert orc.i8_quantize(-0.5, 1.0) == -1
    assert orc.i8_quantize(2.5, 1.0) == 3
    assert orc.i8_quantize(-2.5, 1.0) == -3
    assert orc.i8_quantize(1000.0, 1.0) == 127       # clamp to [-127, 127]
    assert orc.i8_quantize(-1000.0, 1.0) == -127
    assert orc.i8_quantize(0.49999997, 1.0) == 0


def test_i8_container_layout(orc):
    rng = np.random.default_rng(11)
    m, n = 5, 7  # n not a multiple of 4
    x = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    s = np.abs(x).max(0)
    x[:, 0] = 0.0
    s[0] = 0.0
    x[1, 1] = np.nan
    packed = orc.quantize_i8(x, s, True)
    assert packed.shape == (m, 2)
    for r in range(m):
        for c in range(n):
            want = orc.i8_quantize(float(x[r, c]), float(s[c]))
            assert orc.i8_at(packed[r], c) == want
            assert (int(packed[r, c // 4]) >> (8 * (c % 4))) & 0xFF == (want & 0xFF)  # little endian
        assert (int(packed[r, 1]) >> 24) == 0  # tail byte is 0
    assert np.all(packed.view(np.uint32)[:, 0] & 0xFF == 0)  # the s == 0 column
    up = orc.unpack_i8(packed, n)
    assert up.shape == (m, n)
    assert np.all(up == np.round(up)) and up.min() >= -127 and up.max() <= 127


# ---- src/int8_act_test.cpp:170-238 (integer reference, shapes 130x17x6 and 512x256x8) ----
@pytest.mark.parametrize("out,k,n,seed", [(130, 17, 6, 3), (512, 256, 8, 4), (64, 65, 67, 5)])
def test_matmul_q_i8_integer_reference(orc, out, k, n, seed):
    rng = np.random.default_rng(seed)
    W = rng.uniform(-1, 1, (out, k)).astype(np.float32)
    tau = (np.abs(W.astype(np.float64)).sum(1) / k).astype(np.float32)
    X = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    s = np.abs(X).max(0).astype(np.float32)
    packed = orc.trit_pack(W, tau)
    xq = orc.quantize_i8(X, s, True)
    y, acc = orc.matmul_q_i8(packed, tau, xq, s, k, n)
    trit = orc.trit_unpack(packed, k).astype(np.int64)
    q = orc.unpack_i8(xq, n).astype(np.int64)
    ref_acc = trit @ q
    assert np.array_equal(acc, ref_acc)
    ref_y = (tau[:, None] * s[None, :]) * ref_acc.astype(np.float32)
    assert np.array_equal(y.view(np.uint32), ref_y.astype(np.float32).view(np.uint32))  # bitwise


def test_token_major_variant_equals_reference_layout(orc):
    rng = np.random.default_rng(9)
    t, k, out = 9, 128, 70
    W = rng.normal(0, 0.02, (out, k)).astype(np.float32)
    tau = orc.absmean_tau(W)
    packed = orc.trit_pack(W, tau)
    X = rng.normal(0, 1, (t, k)).astype(np.float32)
    q, s = orc.act_quant_tm(X)
    s_ref = orc.col_absmax_scale(X.T.copy())
    assert np.array_equal(s, s_ref)
    xq = orc.quantize_i8(X.T.copy(), s, True)
    assert np.array_equal(orc.unpack_i8(xq, t).T.astype(np.int8), q)
    y_tm, acc_tm = orc.bitlinear_i8_tm(packed, tau, None, q, s)
    y_ref, acc_ref = orc.matmul_q_i8(packed, tau, xq, s, k, t)
    assert np.array_equal(acc_tm, acc_ref.T)
    assert np.array_equal(y_tm.view(np.uint32), y_ref.T.copy().view(np.uint32))


def test_forward_quant_error_bound(orc):
    # src/int8_act_test.cpp:262-290: |Y_int8 - Y_float| <= tau_m * s_n * K * 0.5
    rng = np.random.default_rng(5)
    k, out, b = 64, 32, 8
    W = rng.uniform(-0.3, 0.3, (out, k)).astype(np.float32)
    tau = orc.absmean_tau(W)
    packed = orc.trit_pack(W, tau)
    X = rng.uniform(-1, 1, (k, b)).astype(np.float32)
    s = orc.col_absmax_scale(X)
    y0 = orc.matmul_q(packed, tau, X, k)
    y1, _ = orc.matmul_q_i8(packed, tau, orc.quantize_i8(X, s, True), s, k, b)
    bound = tau[:, None].astype(np.float64) * s[None, :] * k * 0.5
    assert (np.abs(y1.astype(np.float64) - y0) / bound).max() <= 1.0
