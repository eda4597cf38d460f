"""Host-side row codecs of the model-file format (no GPU): the base-3 disk form of ternary rows and the dequantisation
rule L = trit * (tau * K / n), restating src/ternary_gemm_test.cpp:658-735 ([8]: formula bitwise, re-pack with the same tau
reproduces the container bit for bit, per-row absmean(L) == tau within 2e-6, an all-zero row stays zero, an all-non-zero
row has magnitude tau) on the reference's rows and K in {17, 32, 37}."""
import ctypes as C

import numpy as np
import pytest


def _rows(K, ki):
    i = np.arange(K)
    r0 = (0.13 * ((i * 7 + ki) % 11) - 0.7).astype(np.float32)
    r1 = np.zeros(K, np.float32)
    r2 = np.where(i % 2 == 0, 0.8, -0.55).astype(np.float32)
    r3 = (1e-3 * (i % 3)).astype(np.float32)
    return [r0, r1, r2, r3]


@pytest.mark.parametrize("ki,K", [(0, 17), (1, 32), (2, 37)])
def test_dequant_fixed_point_and_base3_round_trip(pkg, orc, ki, K):
    lib = pkg.lib()
    wpr = (K + 15) // 16
    for which, w in enumerate(_rows(K, ki)):
        tau = np.float32(np.abs(w.astype(np.float64)).sum() / K)
        words = orc.trit_pack(w[None, :], np.array([tau], np.float32)).reshape(-1).copy()
        assert words.size == wpr
        trits = orc.trit_unpack(words[None, :], K)[0].astype(np.float32)
        lat = np.zeros(K, np.float32)
        lib.nnb_trit_dequant_row(words.ctypes.data_as(C.c_void_p), K, C.c_float(tau), lat.ctypes.data_as(C.c_void_p))
        s = np.float32(lib.nnb_trit_latent_row_scale(words.ctypes.data_as(C.c_void_p), K, C.c_float(tau)))
        assert np.array_equal(lat, trits * s)  # (1) the formula, bitwise
        again = orc.trit_pack(lat[None, :], np.array([tau], np.float32)).reshape(-1)
        assert np.array_equal(again, words)  # (2) the same trits
        if tau > 0:
            mean = np.abs(lat.astype(np.float64)).sum() / K
            if np.any(trits != 0):
                assert abs(mean - tau) / tau <= 2e-6  # (3) the quantiser's fixed point
        if which == 1:
            assert not lat.any()
        if which == 2:
            assert s == tau
        # base-3 disk form: ceil(K/5) bytes per row, values <= 242, exact round trip (tail padded with code 2)
        nb = lib.nnb_trit_base3_bytes_per_row(K)
        assert nb == (K + 4) // 5
        b3 = np.zeros(nb, np.uint8)
        lib.nnb_trit_pack_row_base3(words.ctypes.data_as(C.c_void_p), K, b3.ctypes.data_as(C.c_void_p))
        assert b3.max() <= 242
        back = np.zeros(wpr, np.uint32)
        lib.nnb_trit_unpack_row_base3(b3.ctypes.data_as(C.c_void_p), K, back.ctypes.data_as(C.c_void_p))
        assert np.array_equal(back, words)
