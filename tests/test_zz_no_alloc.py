"""monofab_pack_pairs_static — the pack for callers that cannot allocate.

A process that keeps a persistent kernel on the GPU, or one that was given a
fixed memory budget, cannot call cudaMalloc when a batch arrives; this entry
point therefore keeps its scratch in an array inside the library.  The test
calls it through the C ABI twice in a row (the second time on a smaller, different
batch, so that stale scratch from the first call would show) and requires the
same bits as monofab_pack_pairs, whose scratch the caller provides.  It lives in
its own file, collected last, and passes alone in a fresh process as well as
after the rest of the suite.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(ids, w, E, x):
    from tests.test_gpu_moe import run_pack_pairs
    a = run_pack_pairs("monofab_pack_pairs", ids, w, E, x, with_scratch=True)
    b = run_pack_pairs("monofab_pack_pairs_static", ids, w, E, x, with_scratch=False)
    return a, b


def test_static_pack_matches_pack_with_caller_scratch_twice():
    from tests.test_gpu_moe import check_pack_against_oracle, random_routing
    for T, E, K, H, seed in [(1500, 128, 8, 256, 1), (77, 16, 4, 64, 2)]:
        ids, w = random_routing(T, E, K, seed)
        x = torch.randn(T, H).to(torch.bfloat16)
        a, b = _both(ids, w, E, x)
        for key in ("counts", "starts", "pair_token", "pair_pos"):
            assert torch.equal(a[key], b[key]), key
        assert np.array_equal(a["pair_weight"].numpy().view(np.int32), b["pair_weight"].numpy().view(np.int32))
        assert torch.equal(a["xp"].view(torch.int16), b["xp"].view(torch.int16))
        check_pack_against_oracle(b, ids, w, E, x)


def test_static_pack_rejects_sizes_beyond_its_scratch():
    from monoserve_b200 import _C
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = _C.lib.monofab_pack_pairs_static(z.data_ptr(), z.data_ptr(), 4097, 8, 2, 0, None, None, z.data_ptr(),
                                          z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None)
    assert rc == -1
    msg = _C.lib.monofab_last_error().decode()
    assert "4096" in msg and "monofab_pack_pairs" in msg
