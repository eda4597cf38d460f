"""Parity of the CUDA ternary-linear operators with the CPU oracle, through the C-ABI.
Integer results and scaled outputs must be bit-exact; float-accumulating matmul_q/_t use the
reference's own tolerances (src/ternary_gemm_test.cpp:267,513)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a, eng):
    return torch.from_numpy(np.ascontiguousarray(a)).to(eng.device)


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def _gen(rows, k, n):
    r = np.arange(rows)[:, None]
    c = np.arange(k)[None, :]
    W = (0.13 * ((r * 7 + c * 3) % 11) - 0.6).astype(np.float32)
    kk = np.arange(k)[:, None]
    nn_ = np.arange(n)[None, :]
    X = (0.21 * ((kk + 2 * nn_) % 9) - 0.8).astype(np.float32)
    return W, X


def test_describe(eng):
    assert "ternary_gemm=true" in eng.describe()


# shapes of src/ternary_gemm_test.cpp:529-539 style: K not a multiple of 16, rows crossing 64
@pytest.mark.parametrize("rows,k,n", [(7, 40, 3), (5, 17, 1), (64, 64, 8), (65, 100, 7), (129, 48, 3), (130, 256, 5)])
def test_trit_pack_and_matmul_q(eng, orc, rows, k, n):
    W, X = _gen(rows, k, n)
    tau = (np.abs(W.astype(np.float64)).sum(1) / k).astype(np.float32)
    d_packed = eng.trit_pack(_dev(W, eng), _dev(tau, eng))
    packed = orc.trit_pack(W, tau)
    assert np.array_equal(_u32(d_packed), packed)
    ref = orc.matmul_q(packed, tau, X, k)
    got = eng.matmul_q(d_packed, _dev(tau, eng), _dev(X, eng), k).cpu().numpy()
    assert np.abs(got - ref).max() <= 1e-5 + 1e-4 * np.abs(ref).max()


@pytest.mark.parametrize("rows,m,n", [(40, 7, 3), (17, 5, 2), (64, 33, 4), (100, 130, 6)])
def test_matmul_q_t(eng, orc, rows, m, n):
    W, _ = _gen(rows, m, n)
    _, B = _gen(1, rows, n)
    tau = (np.abs(W.astype(np.float64)).sum(1) / m).astype(np.float32)
    packed = orc.trit_pack(W, tau)
    ref = orc.matmul_q_t(packed, tau, B, m)
    got = eng.matmul_q_t(_dev(packed.view(np.int32), eng), _dev(tau, eng), _dev(B, eng), m).cpu().numpy()
    assert np.abs(got - ref).max() <= 1e-5 + 1e-4 * np.abs(ref).max()


def test_absmean_tau(eng, orc):
    rng = np.random.default_rng(1)
    W = rng.normal(0, 0.02, (70, 300)).astype(np.float32)
    got = eng.absmean_tau(_dev(W, eng)).cpu().numpy()
    ref = orc.absmean_tau(W)
    assert np.abs(got - ref).max() <= 1e-6  # src/t1_58_test.cpp:291


def test_trit_pack_threshold_ties(eng, orc):
    # entries exactly at +-0.5*tau must become 0 (strict compares)
    tau = np.array([1.0, 0.25, 0.475], np.float32)
    W = np.stack([np.array([0.5, -0.5, 0.50000006, -0.50000006, 0, 1, -1, 0.4] * 3, np.float32) * t
                  for t in tau])
    got = _u32(eng.trit_pack(_dev(W, eng), _dev(tau, eng)))
    assert np.array_equal(got, orc.trit_pack(W, tau))


def test_quantize_i8_rules_and_layout(eng, orc):
    rng = np.random.default_rng(11)
    m, n = 5, 7
    x = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    s = np.abs(x).max(0)
    x[:, 0] = 0.0
    s[0] = 0.0
    x[1, 1] = np.nan
    got = _u32(eng.quantize_i8(_dev(x, eng), _dev(s, eng), True))
    assert np.array_equal(got, orc.quantize_i8(x, s, True))
    # row scale variant
    sr = np.abs(np.nan_to_num(x)).max(1).astype(np.float32)
    got = _u32(eng.quantize_i8(_dev(x, eng), _dev(sr, eng), False))
    assert np.array_equal(got, orc.quantize_i8(x, sr, False))
    # half-way cases round away from zero
    xs = np.array([[0.5, -0.5, 1.5, -1.5, 2.5, 126.5, 127.5, -300.0]], np.float32)
    one = np.ones(8, np.float32)
    got = _u32(eng.quantize_i8(_dev(xs, eng), _dev(one, eng), True))
    assert np.array_equal(got, orc.quantize_i8(xs, one, True))


def test_unpack_i8_roundtrip(eng, orc):
    rng = np.random.default_rng(23)
    x = rng.uniform(-1, 1, (3, 6)).astype(np.float32)
    s = np.maximum(0.3, np.abs(x[0]) + 0.1).astype(np.float32)
    packed = orc.quantize_i8(x, s, True)
    got = eng.unpack_i8(_dev(packed.view(np.int32), eng), 6).cpu().numpy()
    assert np.array_equal(got, orc.unpack_i8(packed, 6))


def test_col_absmax_scale(eng, orc):
    rng = np.random.default_rng(2)
    x = rng.normal(0, 1, (130, 9)).astype(np.float32)
    got = eng.col_absmax_scale(_dev(x, eng)).cpu().numpy()
    assert np.array_equal(got, orc.col_absmax_scale(x))


# src/int8_act_test.cpp:475-476 shapes + one crossing every boundary
@pytest.mark.parametrize("out,k,n,seed", [(130, 17, 6, 3), (512, 256, 8, 4), (64, 65, 67, 5)])
def test_matmul_q_i8_reference_layout_bitwise(eng, orc, out, k, n, seed):
    rng = np.random.default_rng(seed)
    W = rng.uniform(-1, 1, (out, k)).astype(np.float32)
    tau = (np.abs(W.astype(np.float64)).sum(1) / k).astype(np.float32)
    X = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    s = np.abs(X).max(0).astype(np.float32)
    d_packed = eng.trit_pack(_dev(W, eng), _dev(tau, eng))
    d_xq = eng.quantize_i8(_dev(X, eng), _dev(s, eng), True)
    y, acc = eng.matmul_q_i8(d_packed, _dev(tau, eng), d_xq, _dev(s, eng), k, n, want_acc=True)
    y_ref, acc_ref = orc.matmul_q_i8(orc.trit_pack(W, tau), tau, orc.quantize_i8(X, s, True), s, k, n)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(_u32(y), y_ref.view(np.uint32))


def _case_tm(orc, t, k, out, seed, ternary_iid=False):
    rng = np.random.default_rng(seed)
    if ternary_iid:
        trits = rng.integers(-1, 2, (out, k)).astype(np.float32)
        tau = np.full(out, rng.uniform(0.01, 0.1), np.float32)  # per-tensor scale fed per row
        W = trits * tau[:, None]
    else:
        W = rng.normal(0, 0.02, (out, k)).astype(np.float32)
        tau = orc.absmean_tau(W)
    X = rng.normal(0, 1, (t, k)).astype(np.float32)
    bias = rng.normal(0, 0.05, out).astype(np.float32)
    return W, tau, X, bias


@pytest.mark.parametrize("t,k,out", [
    (1, 64, 32), (1, 256, 33), (3, 128, 100), (8, 256, 64),
    # one to four tokens run on the CUDA-core GEMV: K beyond one chunk of 32 blocks, ragged row counts, one group of rows
    (2, 2112, 77), (4, 5632, 300), (1, 2048, 1000), (2, 64, 8), (4, 4096, 5), (1, 8640, 129), (9, 320, 48), (16, 512, 130),
    (17, 192, 96), (32, 1024, 256), (33, 256, 64), (64, 448, 200), (65, 256, 129),
    (130, 384, 257), (300, 2048, 384),
])
def test_bitlinear_fwd_tm_bitwise(eng, orc, t, k, out):
    _bitwise_case(eng, orc, t, k, out)


# shapes with enough row slabs for the persistent weight streamer with register-resident activations (it takes over from
# about 19 000 output rows per launch): 4, 8 and 12 blocks of K per warp, one and two token tiles, ragged rows, warps
# without any block of their own (K 192)
@pytest.mark.parametrize("t,k,out", [(1, 2560, 19000), (8, 3200, 19000), (16, 2048, 19010), (12, 4096, 19001), (7, 5632, 19003),
                                     (3, 192, 20000), (2, 2048, 19040)])
def test_bitlinear_fwd_tm_bitwise_on_the_streamer(eng, orc, t, k, out):
    _bitwise_case(eng, orc, t, k, out)


def _bitwise_case(eng, orc, t, k, out):
    W, tau, X, bias = _case_tm(orc, t, k, out, seed=t * 1000 + k + out)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref, acc_ref = orc.bitlinear_i8_tm(packed, tau, bias, q_ref, s_ref)
    q, s, qsum = eng.act_quant_tm(_dev(X, eng))
    assert np.array_equal(eng.actq_to_plain(q).cpu().numpy(), q_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(qsum.cpu().numpy(), q_ref.astype(np.int32).sum(1))
    y, acc = eng.bitlinear_fwd_tm(_dev(packed.view(np.int32), eng), _dev(tau, eng), _dev(bias, eng),
                                  q, s, qsum, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(_u32(y), y_ref.view(np.uint32))
    # without bias, bf16 output = rounding of the same f32 value
    y_nb = eng.bitlinear_fwd_tm(_dev(packed.view(np.int32), eng), _dev(tau, eng), None, q, s, qsum,
                                out_dtype=torch.bfloat16)
    y_nb_ref = orc.bitlinear_i8_tm(packed, tau, None, q_ref, s_ref, want_acc=False)
    assert torch.equal(y_nb.cpu(), torch.from_numpy(y_nb_ref).to(torch.bfloat16))


# the operator sweep of the benchmark configuration: M in {1,16,64,256,2048},
# (K,N) in {(2048,2048),(2048,5632),(5632,2048)}, iid ternary weights, int32 accumulators bit-exact
@pytest.mark.parametrize("k,out", [(2048, 2048), (2048, 5632), (5632, 2048)])
@pytest.mark.parametrize("t", [1, 16, 64, 256, 2048])
def test_operator_sweep_accumulators_bit_exact(eng, orc, t, k, out):
    W, tau, X, _ = _case_tm(orc, t, k, out, seed=4, ternary_iid=True)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref, acc_ref = orc.bitlinear_i8_tm(packed, tau, None, q_ref, s_ref)
    q, s, qsum = eng.act_quant_tm(_dev(X, eng))
    y, acc = eng.bitlinear_fwd_tm(_dev(packed.view(np.int32), eng), _dev(tau, eng), None, q, s, qsum,
                                  want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(_u32(y), y_ref.view(np.uint32))


@pytest.mark.parametrize("k,out", [(2048, 2048), (2048, 5632), (5632, 2048)])
@pytest.mark.parametrize("t", [64, 256, 2048])
def test_operator_sweep_on_the_tcgen05_path(eng, orc, t, k, out):
    """Same sweep through the Blackwell tensor-core forward (used from 64 tokens up): Y bitwise."""
    W, tau, X, _ = _case_tm(orc, t, k, out, seed=4, ternary_iid=True)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref = orc.bitlinear_i8_tm(packed, tau, None, q_ref, s_ref, want_acc=False)
    q, s, _ = eng.act_quant_tm(_dev(X, eng))
    w8, _ = eng.expand_weights(_dev(packed.view(np.int32), eng), k, want_bf16=False)
    y = eng.bitlinear_fwd_tc(w8, _dev(tau, eng), None, q, s)
    eng.check_device_errors()
    assert np.array_equal(_u32(y), y_ref.view(np.uint32))


def test_stack_equals_single(eng, orc):
    rng = np.random.default_rng(7)
    n_mats, t, k, out = 5, 4, 256, 96
    X = rng.normal(0, 1, (t, k)).astype(np.float32)
    q, s, qsum = eng.act_quant_tm(_dev(X, eng))
    Ws = rng.normal(0, 0.02, (n_mats, out, k)).astype(np.float32)
    taus = np.stack([orc.absmean_tau(w) for w in Ws])
    packs = np.stack([orc.trit_pack(w, tq) for w, tq in zip(Ws, taus)])
    bias = rng.normal(0, 0.05, (n_mats, out)).astype(np.float32)
    y = torch.empty((n_mats, t, out), device=eng.device, dtype=torch.float32)
    eng.bitlinear_fwd_tm_stack(_dev(packs.view(np.int32), eng), _dev(taus, eng), _dev(bias, eng), q, s, qsum, y)
    for i in range(n_mats):
        yi = eng.bitlinear_fwd_tm(_dev(packs[i].view(np.int32), eng), _dev(taus[i], eng), _dev(bias[i], eng),
                                  q, s, qsum)
        assert torch.equal(y[i], yi)


def test_host_entry_point(eng, orc):
    W, tau, X, bias = _case_tm(orc, 16, 512, 192, seed=3)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref = orc.bitlinear_i8_tm(packed, tau, bias, q_ref, s_ref, want_acc=False)
    h_x = torch.from_numpy(X).pin_memory()
    h_y = torch.empty((16, 192), dtype=torch.float32).pin_memory()
    eng.bitlinear_fwd_host(_dev(packed.view(np.int32), eng), _dev(tau, eng), _dev(bias, eng), h_x, h_y)
    assert np.array_equal(h_y.numpy().view(np.uint32), y_ref.view(np.uint32))


def test_bad_arguments_are_rejected(eng, pkg):
    x = torch.zeros((2, 100), device=eng.device)
    with pytest.raises(pkg.NnbError):
        eng.act_quant_tm(x)  # k not a multiple of 64


@pytest.mark.parametrize("t,k,out", [(5, 64, 33), (130, 192, 100), (300, 256, 257)])
def test_bitlinear_backward_gemms(eng, orc, t, k, out):
    """dX = matmul_q_t and dW = ((dY*s) Q^T)*tau against the reference formulas
    (src/t1_58_test.cpp:345-403, src/int8_act_test.cpp:327-359)."""
    W, tau, X, _ = _case_tm(orc, t, k, out, seed=t + k)
    packed = orc.trit_pack(W, tau)
    trit = orc.trit_unpack(packed, k).astype(np.float64)
    q_ref, s_ref = orc.act_quant_tm(X)
    dY = np.random.default_rng(1).normal(0, 1, (t, out)).astype(np.float32)
    dx_ref = (dY.astype(np.float64) * tau[None, :]) @ trit
    dw_ref = ((dY.astype(np.float64) * s_ref[:, None]).T @ q_ref.astype(np.float64)) * tau[:, None]
    q, s, _ = eng.act_quant_tm(_dev(X, eng))
    for exact, tol in ((True, 1e-5), (False, 2e-2)):
        dx = eng.bitlinear_dx_tm(_dev(dY, eng), _dev(packed.view(np.int32), eng), _dev(tau, eng), k, exact=exact)
        assert np.abs(dx.cpu().numpy() - dx_ref).max() <= tol * np.abs(dx_ref).max()
        dw = torch.zeros((out, k), device=eng.device)
        eng.bitlinear_dw_tm(_dev(dY, eng), q, s, _dev(tau, eng), dw, exact=exact)
        assert np.abs(dw.cpu().numpy() - dw_ref).max() <= tol * np.abs(dw_ref).max()
        eng.bitlinear_dw_tm(_dev(dY, eng), q, s, _dev(tau, eng), dw, exact=exact)  # accumulates
        assert np.abs(dw.cpu().numpy() - 2 * dw_ref).max() <= tol * 2 * np.abs(dw_ref).max()
