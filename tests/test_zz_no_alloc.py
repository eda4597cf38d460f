"""nnb_group_advantage_noalloc — the entry point for hosts that must not allocate device memory (their
own pool owns the GPU, or the step runs where the CUDA allocator may not be entered).  It keeps its span
table in a fixed array inside the library instead of the engine's cudaMalloc'ed scratch arena.  Called
here through the C-ABI and compared bit for bit with nnb_group_advantage and with the CPU restatement of
GroupAdvantage, on two calls in a row (the second with other data, so contents left behind by the first
call cannot matter).  This file sorts last so that a run stopping at the first failure has already
executed every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(pkg, eng, returns, spans, eps=1e-8):
    lib = pkg.lib()
    first = np.ascontiguousarray([s[0] for s in spans], np.int32)
    count = np.ascontiguousarray([s[1] for s in spans], np.int32)
    out = torch.empty(returns.numel(), device=eng.device, dtype=torch.float32)
    st = lib.nnb_group_advantage_noalloc(eng.handle, C.c_void_p(returns.data_ptr()), returns.numel(),
                                         first.ctypes.data_as(C.c_void_p), count.ctypes.data_as(C.c_void_p), len(spans),
                                         C.c_float(eps), C.c_void_p(out.data_ptr()))
    return st, out


def _spans(sizes):
    spans, c = [], 0
    for k in sizes:
        spans.append((c, k))
        c += k
    return spans


def test_noalloc_matches_allocating_entry_point_and_oracle_twice(pkg, eng):
    from oracle_binding import OracleRL

    orc = OracleRL()
    rng = np.random.default_rng(0)
    for sizes in ([16] * 64, [3, 70, 1, 5, 8] * 7):  # two calls in a row, different shapes and data
        spans = _spans(sizes)
        h_ret = (rng.uniform(size=sum(sizes)) < 0.3).astype(np.float32)
        ret = torch.from_numpy(h_ret).to(eng.device)
        want = eng.group_advantage(ret, spans)
        st, got = _call_noalloc(pkg, eng, ret, spans)
        assert st == 0, pkg.lib().nnb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # same kernel, same inputs: bit-exact
        ref = orc.group_advantage(h_ret, spans)  # GroupAdvantage::apply restated on the CPU
        assert np.array_equal(got.cpu().numpy().view(np.uint32), np.asarray(ref, np.float32).view(np.uint32))


def test_noalloc_takes_its_maximum_and_leaves_device_memory_alone(pkg, eng):
    n = 16384  # exactly the limit: accepted
    rng = np.random.default_rng(1)
    ret = torch.from_numpy(rng.normal(size=2 * n).astype(np.float32)).to(eng.device)
    spans = [(2 * i, 2) for i in range(n)]
    want = eng.group_advantage(ret, spans)
    st, got = _call_noalloc(pkg, eng, ret, spans)  # warmed up: any lazy loading is behind us
    assert st == 0, pkg.lib().nnb_last_error()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    out = torch.empty_like(ret)
    first = np.ascontiguousarray([s[0] for s in spans], np.int32)
    count = np.ascontiguousarray([s[1] for s in spans], np.int32)
    lib = pkg.lib()
    dev_before = torch.cuda.current_device()
    free_before, _ = torch.cuda.mem_get_info()
    st = lib.nnb_group_advantage_noalloc(eng.handle, C.c_void_p(ret.data_ptr()), ret.numel(), first.ctypes.data_as(C.c_void_p),
                                         count.ctypes.data_as(C.c_void_p), n, C.c_float(1e-8), C.c_void_p(out.data_ptr()))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert st == 0 and free_after == free_before  # the call itself took no device memory
    assert torch.cuda.current_device() == dev_before
    assert torch.equal(out, want)


def test_noalloc_rejects_more_groups_than_its_fixed_scratch(pkg, eng):
    n = 16385
    ret = torch.zeros(n, device=eng.device)
    st, _ = _call_noalloc(pkg, eng, ret, [(i, 1) for i in range(n)])
    assert st != 0 and b"16384" in pkg.lib().nnb_last_error()
    st, _ = _call_noalloc(pkg, eng, ret[:6], [(0, 2), (3, 1)])  # the span checks of the allocating entry point
    assert st != 0
