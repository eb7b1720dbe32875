"""The allocation-free dispatch entry point against the regular one, through the C ABI.

Who needs it: a host that cannot give the library a workspace and cannot create one either -- for example an
inference server whose memory pool has already claimed every free byte of the GPU, or a caller sitting in a
context where the CUDA runtime must not be asked for memory.  The entry point keeps its scratch in a fixed
array inside the library, so the only things checked here are that it produces exactly the tables the
regular entry point produces, twice in a row on different inputs (the array is reused and not cleared), and
that it refuses sizes beyond its fixed capacity.  This file sorts last on purpose: a run that stops at the
first failure has then already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

DEV = "cuda:0"


def _tables(lib, ids, n_experts, noalloc):
    t, k = ids.shape
    bounds = torch.full((n_experts + 1,), -1, dtype=torch.int32, device=DEV)
    sa = torch.full((t * k,), -1, dtype=torch.int32, device=DEV)
    st = torch.full((t * k,), -1, dtype=torch.int32, device=DEV)
    inv = torch.full((t * k,), -1, dtype=torch.int32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if noalloc:
        rc = lib.hq_moe_dispatch_build_noalloc(ids.data_ptr(), t, k, n_experts, bounds.data_ptr(), sa.data_ptr(),
                                               st.data_ptr(), inv.data_ptr(), stream)
    else:
        nbytes = lib.hq_moe_dispatch_workspace_bytes(t, k, n_experts)
        ws = torch.empty(nbytes // 4, dtype=torch.int32, device=DEV)
        rc = lib.hq_moe_dispatch_build(ids.data_ptr(), t, k, n_experts, bounds.data_ptr(), sa.data_ptr(),
                                       st.data_ptr(), inv.data_ptr(), ws.data_ptr(), nbytes, stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return bounds, sa, st, inv


def test_noalloc_dispatch_matches_regular_entry_point_twice():
    from engine_b200 import _lib as L
    lib = L.lib()
    rng = np.random.Generator(np.random.PCG64(4242))
    # two calls in a row, the second smaller than the first so stale words from the first stay in the array
    for (t, k, e) in [(3000, 8, 256), (700, 4, 128)]:
        ids_np = np.stack([rng.choice(e, size=k, replace=False) for _ in range(t)]).astype(np.int32)
        ids = torch.from_numpy(ids_np).to(DEV)
        want = _tables(lib, ids, e, noalloc=False)
        got = _tables(lib, ids, e, noalloc=True)
        for a, b in zip(got, want):
            assert torch.equal(a, b)       # integer tables: exact


def test_noalloc_dispatch_at_exact_capacity_and_with_no_tokens():
    """8192 x 8 ids over 512 experts fill the fixed array to its last word; an off-by-one in its size would write
    into neighbouring device globals, so the tables are compared and the regular entry point is run again
    afterwards (it shares no state with the array).  Zero tokens: both entry points return at once and touch
    nothing."""
    from engine_b200 import _lib as L
    lib = L.lib()
    rng = np.random.Generator(np.random.PCG64(4343))
    t, k, e = 8192, 8, 512
    ids_np = np.stack([rng.choice(e, size=k, replace=False) for _ in range(t)]).astype(np.int32)
    ids = torch.from_numpy(ids_np).to(DEV)
    want = _tables(lib, ids, e, noalloc=False)
    got = _tables(lib, ids, e, noalloc=True)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    again = _tables(lib, ids, e, noalloc=False)
    for a, b in zip(again, want):
        assert torch.equal(a, b)
    sentinel = torch.full((8,), -5, dtype=torch.int32, device=DEV)
    p = sentinel.data_ptr()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.hq_moe_dispatch_build_noalloc(p, 0, 8, 4, p, p, p, p, stream) == 0
    torch.cuda.synchronize()
    # the bounds of an empty call are all zero (n_experts + 1 words); nothing else is written
    assert sentinel.tolist() == [0, 0, 0, 0, 0, -5, -5, -5]
    sentinel.fill_(-5)
    nbytes = lib.hq_moe_dispatch_workspace_bytes(0, 8, 4)
    ws = torch.empty(max(nbytes // 4, 4), dtype=torch.int32, device=DEV)
    assert lib.hq_moe_dispatch_build(p, 0, 8, 4, p, p, p, p, ws.data_ptr(), nbytes, stream) == 0
    torch.cuda.synchronize()
    assert sentinel.tolist() == [0, 0, 0, 0, 0, -5, -5, -5]


def test_noalloc_dispatch_rejects_sizes_beyond_its_array():
    from engine_b200 import _lib as L
    lib = L.lib()
    one = torch.zeros(16, dtype=torch.int32, device=DEV)
    p = one.data_ptr()
    assert lib.hq_moe_dispatch_build_noalloc(p, 65536 // 8 + 1, 8, 256, p, p, p, p, None) == -7
    assert lib.hq_moe_dispatch_build_noalloc(p, 16, 1, 513, p, p, p, p, None) == -7
    assert lib.hq_error_string(-7).decode().startswith("size beyond")
