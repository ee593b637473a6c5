"""A wait that nothing satisfies runs out of its time budget, reports ERR_WAIT_TIMEOUT and leaves the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_times_out_and_context_survives():
    from trl_b200.ops import cuda as K

    dev = torch.device("cuda")
    K.check_status(dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    K.bounded_wait_selftest(flag, expect=1, budget_ms=50)  # nobody sets the flag
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="code=1 site=999"):
        K.check_status(dev)
    K.check_status(dev)  # the error word was cleared by the failed check
    flag.fill_(1)
    K.bounded_wait_selftest(flag, expect=1, budget_ms=50)  # satisfied at once: no error
    x = torch.randn(64, 512, device=dev).to(torch.bfloat16)
    w = torch.ones(512, device=dev, dtype=torch.bfloat16)
    y = K.rmsnorm_infer(x, w, 1e-6)  # the context still runs kernels
    torch.cuda.synchronize()
    K.check_status(dev)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert (y.float() - ref).abs().max().item() < 3e-2
