"""The allocation-free embedding backward against the workspace version (runs last).

Some callers hold all device memory themselves (a fixed VRAM budget, or a rule against cudaMalloc
inside a step) and cannot give the library a workspace; for them eisen_embedding_bwd_static keeps
its integer scratch in a fixed array inside the library.  Both entry points run the same kernels in
the same order, so the outputs must agree bit for bit, on the first call and on a second call that
reuses the array with different ids.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import eisen_b200 as eb  # noqa: E402


def _run_pair(seed, n, vocab, dim):
    dev = torch.device("cuda:0")
    s = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(seed)
    ids = torch.from_numpy(rng.integers(0, vocab, n).astype(np.int32)).to(dev)
    g = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32)).to(dev)
    dw0 = torch.from_numpy(rng.standard_normal((vocab, dim)).astype(np.float32)).to(dev)  # accumulate into non-zero
    dw_ws, dw_st = dw0.clone(), dw0.clone()
    ws = torch.empty(eb.lib().eisen_embedding_bwd_workspace_bytes(n, vocab), dtype=torch.uint8, device=dev)
    eb.call("eisen_embedding_bwd", s, g.data_ptr(), eb.F32, ids.data_ptr(), dw_ws.data_ptr(), ws.data_ptr(), n, dim, vocab)
    eb.call("eisen_embedding_bwd_static", s, g.data_ptr(), eb.F32, ids.data_ptr(), dw_st.data_ptr(), n, dim, vocab)
    torch.cuda.synchronize()
    a, b = dw_ws.cpu().numpy(), dw_st.cpu().numpy()
    assert (a == b).all()
    ref = dw0.cpu().numpy().astype(np.float64)
    np.add.at(ref, ids.cpu().numpy(), g.cpu().numpy().astype(np.float64))
    assert np.abs(b - ref).max() < 1e-4


def test_static_matches_workspace_on_two_calls_in_a_row():
    _run_pair(1, 4096, 1000, 96)
    # second call: other ids, more rows, a smaller vocabulary: stale contents must not leak in
    _run_pair(2, 16384, 257, 64)


@pytest.mark.parametrize("n", [1, 4097])
def test_static_odd_number_of_ids(n):
    # an odd id count once put the (id, first position) list on a 4-byte boundary
    _run_pair(3, n, 1000, 64)


def test_static_rejects_sizes_beyond_the_built_in_scratch():
    dev = torch.device("cuda:0")
    x = torch.zeros(8, device=dev)
    ids = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = eb.lib().eisen_embedding_bwd_static(torch.cuda.current_stream().cuda_stream, x.data_ptr(), eb.F32,
                                             ids.data_ptr(), x.data_ptr(), 65537, 1, 8)
    assert rc == 5 and b"65536" in eb.lib().eisen_last_error()
    rc = eb.lib().eisen_embedding_bwd_static(torch.cuda.current_stream().cuda_stream, x.data_ptr(), eb.F32,
                                             ids.data_ptr(), x.data_ptr(), 8, 1, 131073)
    assert rc == 5
