"""The allocation-free prefill convolution (scratch built into the library) gives the same result as the
entry point that takes a caller-allocated scratch tensor.  Collected last on purpose: it exercises the
library-wide static array, so a failure here cannot hide behind, or cause, failures elsewhere."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _hist_from(xp, Lh):
    B, T, d = xp.shape
    h = torch.zeros(B, d, 2, Lh, dtype=xp.dtype)
    for p in range(2):
        n = (T - p + 1) // 2
        h[:, :, p, :n] = xp[:, p::2].transpose(1, 2)
    return h


@pytest.mark.parametrize("dt,tc", [(torch.bfloat16, True), (torch.float32, False)])
def test_static_scratch_matches_caller_scratch_twice(dt, tc):
    """Two calls in a row (different data, second one smaller so stale scratch contents remain beyond it)
    must each equal the ordinary entry point; a host that cannot cudaMalloc gets identical numbers."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from flash_stu_2_b200 import ops
    dev = torch.device("cuda:0")
    torch.manual_seed(11)
    for (B, T, d, t0) in [(3, 700, 64, 0), (2, 333, 48, 101)]:
        L = T + 5
        Lh = ((L + 1) // 2 + 7) // 8 * 8
        xp = torch.randn(B, T, d).to(dt)
        fp = (torch.randn(L, d) / math.sqrt(L)).to(dt)
        x0 = torch.randn(B, T - t0, d).to(dt)
        hist = _hist_from(xp, Lh).to(dev)
        taps = ops.taps_even(fp.to(dev), Lh)
        yT = torch.empty(B, d, 2, ((T + 1) // 2 + 7) // 8 * 8, dtype=dt, device=dev)
        want = ops.conv_prefill_approx(hist, taps, yT, x0.clone().to(dev), t0, T, use_tensor_cores=tc)
        got = ops.conv_prefill_approx_static(hist, taps, x0.clone().to(dev), t0, T, use_tensor_cores=tc)
        torch.cuda.synchronize()
        ops.check_status()
        a, b = got.float().cpu(), want.float().cpu()
        err = float((a - b).abs().max() / b.abs().max())
        assert err <= (1e-6 if dt == torch.float32 else 2e-2), err
        assert torch.equal(got.cpu(), want.cpu())  # same kernels, same order: bit-identical


def test_static_scratch_rejects_oversize():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from flash_stu_2_b200 import ops
    dev = torch.device("cuda:0")
    B, d, Lh = 8, 1024, 4096                      # 8*1024*2*4096 bf16 = 128 MiB of scratch > 32 MiB
    hist = torch.zeros(B, d, 2, Lh, dtype=torch.bfloat16, device=dev)
    taps = torch.zeros(d, Lh, dtype=torch.bfloat16, device=dev)
    x = torch.zeros(B, 8192, d, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="32 MiB"):
        ops.conv_prefill_approx_static(hist, taps, x, 0, 8192, use_tensor_cores=True)
