"""octexB200QueryCodesStatic: the cell codes of a batch computed with the library's fixed scratch
array instead of allocated buffers.

The call exists for programs that may not allocate device memory at the point where they need the
codes (all device memory owned by one arena, a serving loop that cannot take cudaMalloc's
device-wide synchronisation, a stream capture open elsewhere in the process).  Its answer has to be
the one the allocating path gives, so this test runs the normal search with its intermediates kept
(octexB200Search + octexB200Fetch "codes") and the static-scratch call on the same queries, twice
in a row with different batches: the second call finds the first call's bytes in the shared array
and must not be disturbed by them.  Integer results: compared for equality.

The file name sorts last on purpose, so that a run stopping at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def static_codes(idx, meta, q_dev, out=None):
    """The call on torch's current stream; ``out`` (device int64 [m, copies, levels]) is made here
    unless the caller brings it."""
    import torch
    from octex_b200 import _lib
    m = q_dev.shape[0]
    if out is None:
        out = torch.full((m, meta["copies"], len(meta["spacings"])), -7, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = _lib.lib().octexB200QueryCodesStatic(idx._h, C.c_void_p(q_dev.data_ptr()), C.c_int64(m),
                                              C.c_void_p(out.data_ptr()), C.c_void_p(stream))
    _lib.check(rc)
    torch.cuda.current_stream().synchronize()
    return out.cpu().numpy()


def test_static_scratch_matches_allocating_path(small_index):
    import torch
    import octex_b200
    from octex_b200 import _lib
    arrays, meta, _, queries = small_index
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(taps=True)
    C_, L = meta["copies"], len(meta["spacings"])
    batches = (queries[:200], np.ascontiguousarray(queries[100:300][::-1]), queries[:7])
    for batch in batches:  # calls in a row on the same shared array, sizes differ
        q_dev = torch.as_tensor(batch, device="cuda")
        idx.search(q_dev, 10, read=8, starts=16, waves=0)
        want = idx.fetch("codes", np.int64, (len(batch), C_, L))
        got = static_codes(idx, meta, q_dev)
        assert np.array_equal(got, want)
    # an empty batch is a success that touches nothing
    empty = torch.zeros((0, meta["dim"]), device="cuda")
    assert static_codes(idx, meta, empty).shape == (0, C_, L)
    # a batch whose intermediates do not fit the fixed array is refused with a message, and the
    # next call still works
    per_query = 2 * 64 * ((meta["dim"] + 63) // 64) + 4 * meta["sketch_width"] + 16 * meta["blocks"] * C_
    too_many = (32 << 20) // per_query + 1000
    big = torch.zeros((too_many, meta["dim"]), device="cuda")
    out = torch.zeros((too_many, C_, L), dtype=torch.int64, device="cuda")
    rc = _lib.lib().octexB200QueryCodesStatic(idx._h, C.c_void_p(big.data_ptr()), C.c_int64(too_many),
                                              C.c_void_p(out.data_ptr()), C.c_void_p(0))
    assert rc == _lib.CUVS_ERROR
    text = _lib.lib().cuvsGetLastErrorText().decode()
    assert "static scratch holds" in text and "queries per call" in text
    q_dev = torch.as_tensor(queries[:64], device="cuda")
    idx.search(q_dev, 10, read=8, starts=16, waves=0)
    assert np.array_equal(static_codes(idx, meta, q_dev), idx.fetch("codes", np.int64, (64, C_, L)))
    idx.close()


def test_static_scratch_on_a_four_block_index(wide_index):
    """An index whose search projects on the tensor cores by default.  The static-scratch call
    projects in dimension order, so its codes are those of the search under
    ``set_projection(ordered=True)`` exactly, and those of the default search up to the few
    coordinates the two summation orders round to neighbouring fp16 values.  The calls are made on
    a stream of their own, and from the second call on the free device memory must not move: the
    call allocates nothing."""
    import torch
    import octex_b200
    arrays, meta, _, queries = wide_index
    idx = octex_b200.attach(arrays, meta, borrow=False)
    idx.set_debug(taps=True)
    C_, L = meta["copies"], len(meta["spacings"])
    q_dev = torch.as_tensor(queries, device="cuda")
    nq = len(queries)
    idx.set_projection(ordered=True)
    idx.search(q_dev, 10, read=8, starts=16, waves=0)
    want_ordered = idx.fetch("codes", np.int64, (nq, C_, L))
    idx.set_projection(ordered=False)
    idx.search(q_dev, 10, read=8, starts=16, waves=0)
    codes_tc = idx.fetch("codes", np.int64, (nq, C_, L))
    side = torch.cuda.Stream()
    out = torch.empty((nq, C_, L), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        got = static_codes(idx, meta, q_dev, out)  # the first call on this GPU may load the module
        free0 = torch.cuda.mem_get_info()[0]
        for _ in range(3):
            out.fill_(-7)
            got = static_codes(idx, meta, q_dev, out)
            assert torch.cuda.mem_get_info()[0] == free0, "a later call changed the free device memory"
            assert np.array_equal(got, want_ordered)
    differ = float((got != codes_tc).mean())
    print(f"codes that differ from the tensor-core search's: {differ:.5f}")
    assert differ <= 0.05
    idx.close()
