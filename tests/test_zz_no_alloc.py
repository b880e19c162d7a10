"""syn_gemm_noalloc against syn_gemm (producer role), through the C ABI.

Who needs the no-alloc entry point: hosts that cannot call cudaMalloc when the GEMM runs - all GPU
memory already belongs to their own pool, or an allocation's device-wide synchronisation is not
acceptable at that point.  The scratch (per-wave tile counters) then comes from a fixed array
inside the library instead of from the caller.

The test runs the same flag-raising GEMM through both entry points, twice in a row, and expects
identical outputs, identical flags, and the usual tolerance against the fp32 product."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(entry, a, b, c, flags, counters, epoch, status):
    from syncopate_b200 import _lib as L

    M, K = a.shape
    N = b.shape[0]
    g = L.GemmArgs()
    g.a, g.b, g.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.dtype = L.SYN_DTYPE_BF16
    g.producer_signal_ptr = flags.data_ptr()
    g.producer_counter_ptr = counters.data_ptr() if counters is not None else None
    g.signal_value = epoch
    g.status = status.data_ptr()
    offs = [[256, 0], [0, 0], [384, 0], [128, 0]]
    sched, keep = L.make_schedule(offs, [[128, N]] * 4, [2, 0, 3, 1])
    rc = getattr(L.lib(), entry)(C.byref(g), None, C.byref(sched), None)
    assert rc == 0, f"{entry} returned {rc}"
    torch.cuda.synchronize()


def test_noalloc_entry_point_matches_the_regular_one_twice():
    torch.manual_seed(7)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    counters = torch.zeros(64, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):  # two calls in a row: the shared scratch must be clean for the second
        c_ref = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        c_new = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        f_ref = torch.zeros(4, dtype=torch.int64, device="cuda")
        f_new = torch.zeros(4, dtype=torch.int64, device="cuda")
        _run("syn_gemm", a, b, c_ref, f_ref, counters, epoch, status)
        _run("syn_gemm_noalloc", a, b, c_new, f_new, None, epoch, status)
        assert status.tolist() == [0, 0, 0, 0]
        assert torch.equal(c_new, c_ref)
        assert f_new.tolist() == f_ref.tolist() == [epoch] * 4
        err = ((c_new.float() - ref).norm() / ref.norm()).item()
        assert err < 1e-2


def test_noalloc_rejects_more_waves_than_its_scratch_holds():
    from syncopate_b200 import _lib as L

    a = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    g = L.GemmArgs()
    g.a, g.b, g.c = a.data_ptr(), a.data_ptr(), c.data_ptr()
    g.M, g.N, g.K = 128, 128, 64
    g.dtype = L.SYN_DTYPE_BF16
    g.producer_signal_ptr = flags.data_ptr()
    sched, keep = L.make_schedule([[0, 0]] * 65, [[128, 128]] * 65, [0] * 65)
    assert L.lib().syn_gemm_noalloc(C.byref(g), None, C.byref(sched), None) == -9  # SYN_ERR_TOO_LARGE
