"""The bounded-wait path of the tcgen05 kernels, exercised by a kernel made for it: two warps
wait on an mbarrier nobody arrives at, with the time limit cut to a millisecond.  The wait has to
give up, the status word has to carry the time-out bit, and the context has to stay usable.
(The reference has nothing to compare with here: its kernels never wait on each other.)"""
import pytest
import torch

from flaxattention_b200 import _cabi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("limit_ns", [1_000_000, 5_000_000])
def test_wait_that_nothing_satisfies_runs_out_and_reports(limit_ns):
    dev = torch.device("cuda", 0)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gave_up = torch.zeros(2, dtype=torch.int32, device=dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream(dev)
    _cabi.selftest_bounded_wait(limit_ns, status.data_ptr(), gave_up.data_ptr(), waited.data_ptr(), stream.cuda_stream)
    torch.cuda.synchronize(dev)  # returns without an error: the kernel ended by itself
    assert int(status.item()) & 1 == 1, "the time-out bit is set"
    assert gave_up.tolist() == [64, 0], "every thread's wait reported failure"
    ns = int(waited.item())
    assert limit_ns <= ns < 50 * limit_ns, ns
    # the context is intact: an attention call right after gives the usual answer
    import flaxattention_b200 as fa
    q = torch.randn(1, 2, 128, 64, device=dev, dtype=torch.float16)
    out = fa.flax_attention(q, q, q)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), q.float(), q.float())
    assert torch.allclose(out.float(), ref, atol=2e-3, rtol=2e-3)


def test_limit_outside_the_accepted_range_is_refused():
    with pytest.raises(_cabi.FlaxAttnError):
        _cabi.selftest_bounded_wait(10, 0, 0, 0)
