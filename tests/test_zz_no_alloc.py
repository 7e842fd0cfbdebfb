"""GPU test of the allocation-free partition entry point, pspmm_split_csr_device_static.

It exists for hosts that may not create device memory when they need a PCSR partition (fully
pre-partitioned serving processes, code locked inside another framework's pool, plug-ins called
where allocation is forbidden): its scratch is a fixed array inside the library.  The test calls
it through the C ABI twice in a row, a large matrix and then a smaller one so that the second
call runs over the first call's leftovers, and requires the same bits as the scratch-taking
entry point pspmm_split_csr_device.  The file name sorts last on purpose: it runs after every
other test, and it also passes on its own in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _split_both_ways(lib, check, rowPtr_dev, gran):
    n = rowPtr_dev.shape[0] - 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    nseg = ctypes.c_int64(0)
    host_rp = rowPtr_dev.cpu()
    check(lib.pspmm_split_count(p(host_rp), n, gran, ctypes.byref(nseg)))
    S = nseg.value
    # existing entry point: caller-provided scratch
    need = ctypes.c_size_t(0)
    check(lib.pspmm_split_device_scratch_bytes(n, ctypes.byref(need)))
    scratch = torch.empty((need.value + 7) // 8, dtype=torch.int64, device=rowPtr_dev.device)
    a_rps = torch.full((S + 1,), -7, dtype=torch.int32, device=rowPtr_dev.device)
    a_tr = torch.full((S,), -7, dtype=torch.int32, device=rowPtr_dev.device)
    check(lib.pspmm_split_csr_device(p(rowPtr_dev), n, gran, p(a_rps), p(a_tr), S, p(scratch), need.value, stream))
    # new entry point: no scratch argument, nothing allocated inside
    b_rps = torch.full((S + 1,), -9, dtype=torch.int32, device=rowPtr_dev.device)
    b_tr = torch.full((S,), -9, dtype=torch.int32, device=rowPtr_dev.device)
    # One call first, so that loading the kernels and looking up the built-in array are behind us;
    # then the driver's own count of free device memory must not move across a second call
    # (torch's allocator statistics would miss an allocation made inside the library).
    check(lib.pspmm_split_csr_device_static(p(rowPtr_dev), n, gran, p(b_rps), p(b_tr), S, stream))
    torch.cuda.synchronize()
    b_rps.fill_(-9)
    b_tr.fill_(-9)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    check(lib.pspmm_split_csr_device_static(p(rowPtr_dev), n, gran, p(b_rps), p(b_tr), S, stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before, "the entry point took %d bytes of device memory" % (free_before - free_after)
    assert torch.cuda.memory_allocated() == allocated_before
    return (a_rps, a_tr), (b_rps, b_tr)


def test_static_scratch_split_matches_scratch_taking_entry_point():
    assert torch.cuda.is_available()
    from paramspmm_ae_b200 import _lib, synth
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    big = synth.rmat(18, 3_000_000, seed=5, device=dev)          # 262,144 rows, hub rows, empty rows
    small = synth.powerlaw_graph(3001, 24000, seed=1).to(dev)    # fewer tiles than the call before
    for m, gran in ((big, 32), (small, 7)):
        (a_rps, a_tr), (b_rps, b_tr) = _split_both_ways(lib, _lib.check, m.rowPtr, gran)
        assert torch.equal(a_rps, b_rps)
        assert torch.equal(a_tr, b_tr)
        assert int(b_rps[-1]) == m.nnz and int(b_rps[0]) == 0


def test_static_scratch_split_rejects_oversized_input():
    from paramspmm_ae_b200 import _lib
    lib = _lib.lib()
    fake = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    too_many_rows = 16_777_216 + 1
    rc = lib.pspmm_split_csr_device_static(fake, too_many_rows, 32, fake, fake, 10, ctypes.c_void_p(0))
    assert rc == _lib.PSPMM_E_RANGE
    with pytest.raises(_lib.PspmmError, match="built-in scratch"):
        _lib.check(rc)
    assert lib.pspmm_split_csr_device_static(ctypes.c_void_p(0), 5, 32, fake, fake, 1, ctypes.c_void_p(0)) == _lib.PSPMM_E_ARG
