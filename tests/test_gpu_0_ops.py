"""Kernel-level parity on a B200: every C-ABI op against the CPU oracle / an fp32 torch statement of the op.
Tolerances: fp32 1e-3 relative (observed far below), bf16 2e-2 relative, as the parity bar states."""
import math

import pytest
import torch

from oracle import stu_oracle as O
from parity import close

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-3, torch.bfloat16: 2e-2}


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")




@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 32), (3, 7, 1024), (2, 50)])
def test_rmsnorm(dt, shape):
    from flash_stu_2_b200 import ops
    torch.manual_seed(0)
    x = (torch.randn(*shape) * 3).to(dt)
    w = torch.randn(shape[-1]).to(dt)
    y = ops.rmsnorm(x.to(dev()), w.to(dev()))
    ref = O.rmsnorm(x, w)
    close(y, ref, (1e-6 if dt == torch.float32 else 2 ** -7))


def _lin_ref(x, W, W2, resid, epi, dt):
    acc = x.double() @ W.double().t()
    if epi == 0:
        return acc.to(dt)
    if epi == 1:
        return (resid.float() + acc.to(dt).float()).to(dt)
    g = torch.nn.functional.gelu(acc.to(dt).float(), approximate="tanh").to(dt)
    return (g.float() * (x.double() @ W2.double().t()).to(dt).float()).to(dt)


@pytest.mark.parametrize("backend", [1, 2, 3])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_linear_backends(backend, dt, epi):
    from flash_stu_2_b200 import ops
    if backend == 2 and dt != torch.bfloat16:
        pytest.skip("tcgen05 path is bf16 only")
    torch.manual_seed(1)
    shapes = [(300, 200, 136), (128, 128, 64), (257, 520, 1032)] if backend != 3 else [(8, 200, 136), (33, 72, 1024), (2, 50, 64)]
    for (M, N, K) in shapes:
        x = torch.randn(M, K).to(dt)
        W = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        W2 = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        resid = torch.randn(M, N).to(dt)
        ref = _lin_ref(x, W, W2, resid, epi, dt)
        y = ops.linear(x.to(dev()), W.to(dev()), W2=W2.to(dev()) if epi == 2 else None,
                       resid=resid.to(dev()) if epi == 1 else None, epilogue=epi, backend=backend)
        ops.check_status()
        close(y, ref, TOL[dt] / 2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_linear_narrow_output_long_rows(dt):
    """Decode linears whose output is narrow and whose rows are long (down projections of a wide MLP): bf16 splits K
    across a thread-block cluster and reduces through distributed shared memory, fp32 across the warps of a CTA."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(4)
    for (M, N, K, epi) in [(5, 512, 6144, 1), (20, 384, 4096, 0), (2, 512, 6144, 1), (8, 760, 8200, 0)]:
        x = torch.randn(M, K).to(dt)
        W = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        resid = torch.randn(M, N).to(dt)
        ref = _lin_ref(x, W, None, resid, epi, dt)
        y = ops.linear(x.to(dev()), W.to(dev()), resid=resid.to(dev()) if epi == 1 else None, epilogue=epi, backend=3)
        ops.check_status()
        close(y, ref, TOL[dt] / 2)


@pytest.mark.parametrize("epi", [0, 1, 2])
def test_linear_17_to_64_rows(epi):
    """Decode linears of 17..64 token rows (bf16).  Store / residual: 32 output features per CTA, operands streamed
    through registers, K over a cluster of up to 4 CTAs.  Gate/up at up to 32 rows: the kernel that stages the
    activation rows in shared memory by bulk copies and has every weight load in flight at once (16 gate + 16 up rows
    per CTA, K over a cluster of up to 8 CTAs).  Ragged N, K and M included (K not a multiple of 32 falls back to the
    8-feature kernel)."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    torch.manual_seed(8)
    for (M, N, K) in [(32, 1536, 6144), (32, 1536, 1536), (32, 4608, 1536), (17, 72, 1024), (48, 1000, 2056),
                      (64, 3072, 512), (33, 40, 264), (32, 6144, 1536), (25, 1000, 12288), (20, 40, 264),
                      (32, 104, 8192), (16, 1024, 49152), (11, 200, 8200), (20, 4750, 1504), (32, 9601, 544)]:
        if epi == 2 and M > 32 and N * K > 4e6:
            continue
        x = torch.randn(M, K).to(dt)
        W = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        W2 = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        resid = torch.randn(M, N).to(dt)
        ref = _lin_ref(x, W, W2, resid, epi, dt)
        y = ops.linear(x.to(dev()), W.to(dev()), W2=W2.to(dev()) if epi == 2 else None,
                       resid=resid.to(dev()) if epi == 1 else None, epilogue=epi, backend=3)
        ops.check_status()
        close(y, ref, TOL[dt] / 2, what=f"{M}x{N}x{K}")


@pytest.mark.parametrize("epi", [0, 1])
def test_linear_wide_tensor_core_tiles(epi):
    """Outputs with at least two waves of 128 x 256 tiles take the wide-tile tcgen05 kernel; ragged M, N and K."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(5)
    dt = torch.bfloat16
    for (M, N, K) in [(20000, 520, 136), (9000, 1024, 264), (38000, 776, 64)]:
        x = torch.randn(M, K).to(dt)
        W = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        resid = torch.randn(M, N).to(dt)
        ref = _lin_ref(x, W, None, resid, epi, dt)
        y = ops.linear(x.to(dev()), W.to(dev()), resid=resid.to(dev()) if epi == 1 else None, epilogue=epi, backend=2)
        ops.check_status()
        close(y, ref, TOL[dt] / 2)


def test_bounded_wait_expiry_is_reported_and_the_context_survives():
    """Failure detection inside the tcgen05 GEMM: with the copies of its first pipeline stage dropped (test hook) the
    consumer's bounded wait runs out after the shortened limit; the kernel reports status 3, frees its tensor memory
    and returns, the host raises, and the next GEMM on the same context is correct.  Nothing faults or hangs."""
    import time
    from flash_stu_2_b200 import _lib, ops
    lib = _lib.load()
    torch.manual_seed(21)
    dt = torch.bfloat16
    x = torch.randn(128, 64).to(dt)
    W = (torch.randn(128, 64) / 8).to(dt)
    xd, Wd = x.to(dev()), W.to(dev())
    ref = _lin_ref(x, W, None, None, 0, dt)
    close(ops.linear(xd, Wd, backend=2), ref, TOL[dt] / 2)      # the healthy kernel first
    ops.check_status()
    assert lib.stu_test_inject_wait_expiry(100) == 0
    try:
        t0 = time.monotonic()
        ops.linear(xd, Wd, backend=2)
        torch.cuda.synchronize()
        assert time.monotonic() - t0 < 5.0                           # returned by itself, within the shortened bound
        with pytest.raises(RuntimeError, match="status 3"):
            ops.check_status()
    finally:
        assert lib.stu_test_inject_wait_expiry(0) == 0
    close(ops.linear(xd, Wd, backend=2), ref, TOL[dt] / 2)      # same context, same kernel, healthy again
    big = torch.randn(300, 136).to(dt)
    Wb = (torch.randn(200, 136) / 12).to(dt)
    close(ops.linear(big.to(dev()), Wb.to(dev()), backend=2), _lin_ref(big, Wb, None, None, 0, dt), TOL[dt] / 2)
    ops.check_status()


def test_linear_fused_norm_decode():
    """RMSNorm fused into the mma.sync token-step linears (every row count up to 64; callers use it up to 16 rows)."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(2)
    for (M, N, K, epi) in [(8, 4096, 1024, 2), (32, 1536, 1536, 0), (5, 104, 64, 1), (48, 4608, 1536, 0),
                           (20, 1000, 520, 1), (64, 72, 2048, 0), (32, 6144, 1536, 2), (19, 200, 512, 2),
                           (16, 1536, 3072, 0), (12, 6144, 1504, 2), (32, 1536, 4104, 0), (64, 6144, 3072, 2)]:
        dt = torch.bfloat16
        x = torch.randn(M, K).to(dt)
        nw = torch.randn(K).to(dt)
        W = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        W2 = (torch.randn(N, K) / math.sqrt(K)).to(dt)
        resid = torch.randn(M, N).to(dt)
        ref = _lin_ref(O.rmsnorm(x, nw), W, W2, resid, epi, dt)
        y = ops.linear(x.to(dev()), W.to(dev()), W2=W2.to(dev()) if epi == 2 else None,
                       resid=resid.to(dev()) if epi == 1 else None, epilogue=epi, norm_w=nw.to(dev()))
        ops.check_status()
        close(y, ref, 1e-2, what=f"{M}x{N}x{K}")


def test_linear_transposed_small_k():
    """phi @ M_filters: K = num_eigh = 24 inner dimension, weight given as [K, N]."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(3)
    for dt in (torch.float32, torch.bfloat16):
        phi = torch.randn(130, 24).to(dt)
        Mf = torch.randn(24, 72).to(dt)
        y = ops.linear(phi.to(dev()), Mf.to(dev()), transposed_weight=True, backend=1)
        close(y, (phi.double() @ Mf.double()).to(dt), TOL[dt] / 4)


def _hist_from(xp, Lh):
    B, T, d = xp.shape
    h = torch.zeros(B, d, 2, Lh, dtype=xp.dtype)
    for p in range(2):
        n = (T - p + 1) // 2
        h[:, :, p, :n] = xp[:, p::2].transpose(1, 2)
    return h


@pytest.mark.parametrize("dt,tc", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("shape", [(2, 64, 16, 0), (3, 300, 40, 0), (9, 1100, 8, 0), (2, 1301, 8, 655)])
def test_conv_prefill_matches_fft_oracle(dt, tc, shape):
    """x += conv_plus + conv_minus of the reference (FFT, fp32) == 2 * even-tap direct sum."""
    from flash_stu_2_b200 import ops
    B, T, d, t0 = shape
    torch.manual_seed(4)
    L = T + 3
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    xp = torch.randn(B, T, d).to(dt)
    fp = (torch.randn(L, d) / math.sqrt(L)).to(dt)
    x0 = torch.randn(B, T, d).to(dt)
    n = O.fft_length(L)
    plus, minus = O.convolve(xp, fp, n, True, True)
    ref = (x0.float() + (plus + minus).float()).to(dt)
    hist = _hist_from(xp, Lh).to(dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    yT = torch.full((B, d, 2, ((T + 1) // 2 + 7) // 8 * 8), float("nan"), dtype=dt, device=dev())
    x = x0[:, t0:].contiguous().to(dev())
    ops.conv_prefill_approx(hist, taps, yT, x, t0, T, use_tensor_cores=tc)
    # bf16: the reference rounds each branch before the add, the kernel rounds the folded sum once
    # bf16: the reference rounds each branch before adding them, the kernel rounds the folded sum once; on rows whose
    # largest value is small that is up to two bf16 ulps of the branch magnitude (observed 1.75e-2 per row)
    close(x, ref[:, t0:], (2e-5 if dt == torch.float32 else 1.5e-2), row_tol=(2e-5 if dt == torch.float32 else 2e-2))


@pytest.mark.parametrize("shape", [(2, 250, 16, 0), (3, 700, 24, 0), (9, 1100, 8, 0), (2, 1301, 8, 655),
                                   (1, 8800, 8, 0), (2, 9001, 8, 8300)])
def test_conv_prefill_tcgen05_matches_fft_oracle(shape):
    """The tcgen05 prefill convolution against the reference's FFT convolution (fp32): histories of one and of two
    accumulator-sized superblocks (more than 4096 positions per parity), more than 8 sequences, a resumed prefill
    (t0 > 0), and NaN in the cache past the valid positions, which must not reach any output."""
    from flash_stu_2_b200 import ops
    B, T, d, t0 = shape
    torch.manual_seed(4)
    L = T + 3
    Lh = ((L + 1) // 2 + 127) // 128 * 128
    xp = torch.randn(B, T, d).bfloat16()
    fp = (torch.randn(L, d) / math.sqrt(L)).bfloat16()
    x0 = torch.randn(B, T, d).bfloat16()
    plus, minus = O.convolve(xp, fp, O.fft_length(L), True, True)
    ref = (x0.float() + (plus + minus).float()).bfloat16()
    hist = _hist_from(xp, Lh)
    for p in range(2):
        hist[:, :, p, (T - p + 1) // 2:] = float("nan")
    hist = hist.to(dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    taps8 = ops.taps_rev8(taps)
    yT = torch.full((B, d, 2, ((T + 1) // 2 + 7) // 8 * 8), float("nan"), dtype=torch.bfloat16, device=dev())
    x = x0[:, t0:].contiguous().to(dev())
    assert ops.conv_prefill_tc5_supported(hist, x)
    ops.conv_prefill_approx_tc5(hist, taps8, yT, x, t0, T)
    ops.check_status()
    # the reference rounds each branch to bf16 before adding them; over thousands of positions the branches grow
    # against their sum, so a row of 8 channels sees up to three ulps of that rounding
    close(x, ref[:, t0:], 1.5e-2, row_tol=(2e-2 if T < 4096 else 3e-2))
    # and against the mma.sync kernel on the same operands: same products, fp32 sums in another order
    hist0 = torch.nan_to_num(hist, nan=0.0)
    x2 = x0[:, t0:].contiguous().to(dev())
    ops.conv_prefill_approx(hist0, taps, torch.zeros_like(yT), x2, t0, T, use_tensor_cores=True)
    close(x, x2, 8e-3, row_tol=1.6e-2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_history_scatter_epilogue(dt):
    from flash_stu_2_b200 import ops
    torch.manual_seed(5)
    for backend, (B, T, d, t0) in [(1, (2, 37, 24, 5)), (0, (2, 256, 128, 32)), (0, (3, 100, 64, 7))]:
        Lh = ((t0 + T + 1) // 2 + 7) // 8 * 8
        x = torch.randn(B, T, d).to(dt)
        Mi = (torch.randn(d, d) / math.sqrt(d)).to(dt)
        xp = (x.double() @ Mi.double()).to(dt)
        hist = torch.zeros(B, d, 2, Lh, dtype=dt, device=dev())
        ops.linear(x.reshape(B * T, d).to(dev()), Mi.t().contiguous().to(dev()), out=hist, epilogue=3, hist_T=T,
                   hist_t0=t0, hist_Lh=Lh, backend=backend)
        ops.check_status()
        full = torch.zeros(B, t0 + T, d, dtype=dt)
        full[:, t0:] = xp
        close(hist, _hist_from(full, Lh), TOL[dt] / 2)


def _decode_fixture(dt, B, T, d, L, seed=6):
    import math as _m
    torch.manual_seed(seed)
    x = torch.randn(B, T, d).to(dt)
    nw = (1 + 0.1 * torch.randn(d)).to(dt)
    Mi = (torch.randn(d, d) / _m.sqrt(d)).to(dt)
    fp = (torch.randn(L, d) / 8).to(dt)
    xn = O.rmsnorm(x, nw)
    xp = xn @ Mi
    plus, minus = O.convolve(xp, fp, O.fft_length(L), True, True)
    return x, nw, Mi, fp, xp, x + (plus + minus)


@pytest.mark.parametrize("dt,tc", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("shape", [(3, 45, 64, 64), (9, 70, 40, 160), (10, 300, 256, 600)])
def test_decode_step_equals_prefill_row(dt, tc, shape):
    """S3: the fused decode kernel at time t reproduces row t of the full-prefix layer half
    (CUDA-core kernel and, for bf16, the tensor-core kernel fed by the reversed tap table)."""
    from flash_stu_2_b200 import ops
    B, T, d, L = shape
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, T, d, L)
    hist = torch.zeros(B, d, 2, Lh, dtype=dt, device=dev())
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    taps8 = ops.taps_rev8(taps) if tc else None
    MinT = Mi.t().contiguous().to(dev())
    outs = []
    for t in range(T):
        out = torch.empty(B, d, dtype=dt, device=dev())
        ops.decode_approx(x[:, t].contiguous().to(dev()), nw.to(dev()), MinT, hist, taps, pos, out, taps8=taps8)
        outs.append(out.cpu())
    ops.check_status()
    got = torch.stack(outs, 1)
    assert pos[:, 0].tolist() == [T] * B and int(pos[0, 1]) == 0
    close(got, ref, (1e-5 if dt == torch.float32 else 1.5e-2))
    close(hist, _hist_from(xp, Lh), (1e-5 if dt == torch.float32 else 1e-2))


@pytest.mark.parametrize("shape", [(3, 45, 64, 64), (9, 70, 40, 160), (8, 300, 256, 600), (17, 140, 1024, 300)])
def test_decode_step_shared_tap_kernel(shape):
    """Batches at one common position: the kernel that owns 8 channels x 8 sequences per CTA (taps staged once
    in shared memory, projection and tap contraction as MMAs with the sequences as rows) reproduces the
    full-prefix rows; a ragged batch under the same flag is refused with status 6 and leaves the cache alone."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    B, T, d, L = shape
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, T, d, L)
    hist = torch.zeros(B, d, 2, Lh, dtype=dt, device=dev())
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    taps8 = ops.taps_rev8(taps)
    MinT = Mi.t().contiguous().to(dev())
    xd, nwd = x.to(dev()), nw.to(dev())
    outs = []
    for t in range(T):
        out = torch.empty(B, d, dtype=dt, device=dev())
        ops.decode_approx(xd[:, t].contiguous(), nwd, MinT, hist, taps, pos, out, taps8=taps8,
                          flags=ops.FLAG_UNIFORM_POS)
        outs.append(out)
    ops.check_status()
    got = torch.stack(outs, 1).cpu()
    assert pos[:, 0].tolist() == [T] * B and int(pos[0, 1]) == 0
    close(got, ref, 1.5e-2)
    close(hist, _hist_from(xp, Lh), 1e-2)
    if B > 1:
        pos[:, 0] = 5
        pos[1, 0] = 4          # ragged inside the first group of eight sequences
        before = hist.clone()
        ops.decode_approx(xd[:, 5].contiguous(), nwd, MinT, hist, taps, pos, out, taps8=taps8,
                          flags=ops.FLAG_UNIFORM_POS)
        with pytest.raises(RuntimeError, match="status 6"):
            ops.check_status()
        assert torch.equal(before[:2], hist[:2])


@pytest.mark.parametrize("shape", [(3, 45, 64, 64), (9, 70, 40, 160), (8, 300, 256, 600), (17, 140, 1024, 300),
                                   (5, 1300, 64, 2700)])
def test_decode_step_pipelined_kernel(shape):
    """The persistent bulk-copy pipeline form of the fused decode step (one CTA per SM, history and taps through a
    shared-memory ring, a row of 8 sequences x 8 channels summed inside one CTA in slice order): every step's row
    equals the full-prefix row; positions advance; a ragged batch is refused with status 6; channel shards of the same
    kernel concatenate to exactly the whole layer's output (the sum order does not depend on the grid)."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    B, T, d, L = shape
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, T, d, L)
    hist = torch.zeros(B, d, 2, Lh, dtype=dt, device=dev())
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    taps8 = ops.taps_rev8(taps)
    MinT = Mi.t().contiguous().to(dev())
    xd, nwd = x.to(dev()), nw.to(dev())
    # two channel shards fed the same inputs (stale values beyond the position must not matter: poison the tails)
    half = d // 2
    shards = []
    for r in range(2):
        sl = slice(r * half, (r + 1) * half)
        shards.append((MinT[sl].contiguous(), torch.full((B, half, 2, Lh), 3.0, dtype=dt, device=dev()),
                       ops.taps_rev8(taps[sl].contiguous()), torch.zeros(B, 2, dtype=torch.int32, device=dev())))
    outs = []
    for t in range(T):
        xt = xd[:, t].contiguous()
        out = torch.empty(B, d, dtype=dt, device=dev())
        ops.decode_approx_pipelined(xt, nwd, MinT, hist, taps8, pos, out)
        outs.append(out)
        if half % 8 == 0 and t % 7 == 0:
            ys = []
            for (Ms, hs, t8s, ps) in shards:
                ps[:, 0] = t
                if t:   # the shard caches follow the whole layer's (only steps t % 7 == 0 run through the shards)
                    sl = slice(0, half) if Ms is shards[0][0] else slice(half, d)
                    for par in range(2):
                        n = (t - par + 1) // 2
                        hs[:, :, par, :n] = hist[:, sl, par, :n]
                y = torch.empty(B, half, dtype=dt, device=dev())
                ops.decode_approx_pipelined(xt, nwd, Ms, hs, t8s, ps, y, add_residual=False)
                ys.append(y)
            sharded = (xt.float() + torch.cat(ys, 1).float()).to(dt)
            assert torch.equal(sharded, out), t
    ops.check_status()
    got = torch.stack(outs, 1).cpu()
    assert pos[:, 0].tolist() == [T] * B and int(pos[0, 1]) == 0
    close(got, ref, 1.5e-2)
    close(hist, _hist_from(xp, Lh), 1e-2)
    if B > 1:
        pos[:, 0] = 5
        pos[1, 0] = 4
        before = hist.clone()
        ops.decode_approx_pipelined(xd[:, 5].contiguous(), nwd, MinT, hist, taps8, pos, out)
        with pytest.raises(RuntimeError, match="status 6"):
            ops.check_status()
        assert torch.equal(before, hist)


@pytest.mark.parametrize("world", [2, 4])
def test_peer_exchange_of_the_token_step_with_all_ranks_emulated_on_one_gpu(world):
    """The fused exchanges of a tensor-parallel token step with every rank's buffers on this GPU: the channel-shard
    decode kernel stores its outputs straight into all inboxes (all-gather), the down projection stores its partial
    rows into all inboxes (all-reduce), and the combine kernel of every rank ends with the residual stream (and the
    next RMSNorm) the unfused path computes.  All producing kernels are launched before the first combine, so no
    kernel ever waits for one that has not run.  Repeated steps reuse the same inboxes and counters."""
    from flash_stu_2_b200 import ops
    from flash_stu_2_b200.peer import GATHER, REDUCE, PeerExchange
    dt = torch.bfloat16
    B, d, L, inter = 8, 64 * world, 40, 128 * world
    dl, il = d // world, inter // world
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    torch.manual_seed(11)
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, 6, d, L)
    taps = ops.taps_even(fp.to(dev()), Lh)
    MinT = Mi.t().contiguous().to(dev())
    nwd = nw.to(dev())
    Wd = (torch.randn(d, inter) / math.sqrt(inter)).to(dt).to(dev())
    norm2 = (1 + 0.1 * torch.randn(d)).to(dt).to(dev())
    exs = PeerExchange.emulate([GATHER, REDUCE], B, d, world)
    try:
        ranks = []
        for r in range(world):
            sl = slice(r * dl, (r + 1) * dl)
            ranks.append(dict(MinT=MinT[sl].contiguous(), taps8=ops.taps_rev8(taps[sl].contiguous()),
                              hist=torch.zeros(B, dl, 2, Lh, dtype=dt, device=dev()),
                              pos=torch.zeros(B, 2, dtype=torch.int32, device=dev()),
                              hist_ref=torch.zeros(B, dl, 2, Lh, dtype=dt, device=dev()),
                              pos_ref=torch.zeros(B, 2, dtype=torch.int32, device=dev()),
                              Wd=Wd[:, r * il:(r + 1) * il].contiguous()))
        for t in range(6):
            xt = x[:, t].contiguous().to(dev())
            h = (torch.randn(B, inter) / 2).to(dt).to(dev())
            # ---- unfused: shard outputs gathered, partial products reduced (bf16 sums as a collective would form them)
            ys = []
            for rk in ranks:
                y = torch.empty(B, dl, dtype=dt, device=dev())
                ops.decode_approx_pipelined(xt, nwd, rk["MinT"], rk["hist_ref"], rk["taps8"], rk["pos_ref"], y,
                                            add_residual=False)
                ys.append(y)
            x1 = (xt.float() + torch.cat(ys, 1).float()).to(dt)
            n1 = ops.rmsnorm(x1, norm2)
            parts = [ops.linear(h[:, r * il:(r + 1) * il].contiguous(), rk["Wd"]) for r, rk in enumerate(ranks)]
            x2 = (x1.float() + torch.stack(parts).float().sum(0).to(dt).float()).to(dt)
            # ---- fused: every rank's producers first, then every rank's combine
            xs = [xt.clone() for _ in range(world)]
            xn = [torch.empty_like(xt) for _ in range(world)]
            for r, rk in enumerate(ranks):
                ops.decode_approx_push(xs[r], nwd, rk["MinT"], rk["hist"], rk["taps8"], rk["pos"], exs[r].dest(0), d)
            for r in range(world):
                exs[r].combine(0, xs[r], norm_w=norm2, xn=xn[r])
            for r, rk in enumerate(ranks):
                ops.linear_push(h[:, r * il:(r + 1) * il].contiguous(), rk["Wd"], exs[r].dest(1), d)
            for r in range(world):
                x_mid = xs[r].clone()
                exs[r].combine(1, xs[r])
                assert torch.equal(x_mid, x1), (t, r)
                close(xn[r], n1, 8e-3, what="next RMSNorm")   # the row sums are formed in another order
                if world == 2:
                    assert torch.equal(xs[r], x2), (t, r)    # two bf16 partials: one rounding either way
                else:
                    close(xs[r], x2, 8e-3)
            ops.check_status()
            for r in range(world):
                for e in range(2):
                    flags, epoch = exs[r].counters(e)
                    assert flags == [t + 1] * world and epoch == t + 1
        # a sender that never arrives: the bounded wait runs out, status 10, x untouched, the context stays usable
        before = xs[0].clone()
        ops.decode_approx_push(xs[0], nwd, ranks[0]["MinT"], ranks[0]["hist"], ranks[0]["taps8"], ranks[0]["pos"],
                               exs[0].dest(0), d)
        exs[0].combine(0, xs[0], wait_ms=50)
        with pytest.raises(RuntimeError, match="status 10"):
            ops.check_status()
        assert torch.equal(xs[0], before)
    finally:
        for ex in exs:
            ex.close()


@pytest.mark.parametrize("world", [2, 4])
def test_single_launch_exchange_kernel_with_the_other_ranks_stood_in_by_host_copies(world):
    """The exchange kernel (push + wait + combine + RMSNorm, one CTA per row) for every rank of a group on one GPU.
    What the other ranks would have delivered is copied into the rank's inbox from the host before its kernel runs,
    so the kernel never waits for another launch; its own rows must land in every other rank's inbox all the same."""
    from flash_stu_2_b200 import ops
    from flash_stu_2_b200.peer import GATHER, REDUCE, PeerExchange
    dt = torch.bfloat16
    B, d = 5, 128 * world
    dl = d // world
    torch.manual_seed(12)
    exs = PeerExchange.emulate([GATHER, REDUCE], B, d, world)
    norm = (1 + 0.1 * torch.randn(d)).to(dt).to(dev())
    try:
        for t in range(3):
            x0 = torch.randn(B, d).to(dt).to(dev())
            slices = [torch.randn(B, dl).to(dt).to(dev()) for _ in range(world)]
            parts = [(torch.randn(B, d) / 2).to(dt).to(dev()) for _ in range(world)]
            x1 = (x0.float() + torch.cat(slices, 1).float()).to(dt)
            x2 = (x1.float() + torch.stack(parts).float().sum(0).to(dt).float()).to(dt)
            for r in range(world):
                for s_ in range(world):
                    if s_ != r:
                        exs[r].fake_arrival(0, s_, slices[s_], t + 1)
                        exs[r].fake_arrival(1, s_, parts[s_], t + 1)
            for r in range(world):
                x = x0.clone()
                xn = torch.empty_like(x)
                exs[r].exchange(0, x, slices[r], norm_w=norm, xn=xn)
                assert torch.equal(x, x1), (t, r)
                close(xn, ops.rmsnorm(x1, norm), 8e-3)
                exs[r].exchange(1, x, parts[r])
                if world == 2:
                    assert torch.equal(x, x2), (t, r)
                else:
                    close(x, x2, 8e-3)
            ops.check_status()
        # nobody else arrives for a further step (counters put back below the row's epoch): bounded wait, status 10,
        # x untouched
        for s_ in range(1, world):
            exs[0].fake_arrival(0, s_, slices[s_], 0)
        x = x0.clone()
        exs[0].exchange(0, x, slices[0], wait_ms=50)
        with pytest.raises(RuntimeError, match="status 10"):
            ops.check_status()
        assert torch.equal(x, x0)
    finally:
        for ex in exs:
            ex.close()


@pytest.mark.parametrize("shape", [(17, 60, 256, 300), (32, 40, 128, 700), (9, 530, 64, 1100)])
def test_decode_step_with_the_projection_done_by_the_caller(shape):
    """Larger batches: rmsnorm + one GEMM give the projected input of the whole batch, the pipeline kernel only appends
    it, streams the history and adds the residual.  Every step's row equals the full-prefix row, the cache equals the
    projected inputs, positions advance."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    B, T, d, L = shape
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    x, nw, Mi, fp, xp_ref, ref = _decode_fixture(dt, B, T, d, L)
    hist = torch.full((B, d, 2, Lh), 3.0, dtype=dt, device=dev())   # stale values beyond the position must not matter
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    taps8 = ops.taps_rev8(ops.taps_even(fp.to(dev()), Lh))
    MinT = Mi.t().contiguous().to(dev())
    xd, nwd = x.to(dev()), nw.to(dev())
    outs = []
    for t in range(T):
        xt = xd[:, t].contiguous()
        xp = ops.linear(ops.rmsnorm(xt, nwd), MinT)
        out = torch.empty(B, d, dtype=dt, device=dev())
        ops.decode_approx_projected(xt, xp, hist, taps8, pos, out)
        outs.append(out)
    ops.check_status()
    assert pos[:, 0].tolist() == [T] * B and int(pos[0, 1]) == 0
    close(torch.stack(outs, 1).cpu(), ref, 1.5e-2)
    want = _hist_from(xp_ref, Lh)
    for p_ in range(2):
        n = (T - p_ + 1) // 2
        close(hist[:, :, p_, :n], want[:, :, p_, :n], 1e-2)


def test_decode_step_channel_shards_tile_the_layer():
    """Tensor-parallel form of the fused decode step: two ranks' channel shards (own history, own rows of
    M_inputs^T, own taps) give, concatenated and added to the input, exactly the whole-layer kernel's output."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    B, T, d, L = 5, 40, 64, 96
    Lh = ((L + 1) // 2 + 7) // 8 * 8
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, T, d, L)
    taps = ops.taps_even(fp.to(dev()), Lh)
    MinT = Mi.t().contiguous().to(dev())
    xd, nwd = x.to(dev()), nw.to(dev())
    hist = torch.zeros(B, d, 2, Lh, dtype=dt, device=dev())
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    taps8 = ops.taps_rev8(taps)
    halves = []
    for r in range(2):
        sl = slice(r * d // 2, (r + 1) * d // 2)
        halves.append((MinT[sl].contiguous(), torch.zeros(B, d // 2, 2, Lh, dtype=dt, device=dev()),
                       ops.taps_rev8(taps[sl].contiguous()), torch.zeros(B, 2, dtype=torch.int32, device=dev())))
    for t in range(T):
        xt = xd[:, t].contiguous()
        whole = torch.empty(B, d, dtype=dt, device=dev())
        ops.decode_approx(xt, nwd, MinT, hist, taps, pos, whole, taps8=taps8, flags=ops.FLAG_UNIFORM_POS)
        ys = []
        for (Ms, hs, t8s, ps) in halves:
            y = torch.empty(B, d // 2, dtype=dt, device=dev())
            ops.decode_approx_shard(xt, nwd, Ms, hs, t8s, ps, y)
            ys.append(y)
        sharded = (xt.float() + torch.cat(ys, 1).float()).to(dt)
        assert torch.equal(sharded, whole), t
    ops.check_status()
    assert torch.equal(torch.cat([h[1] for h in halves], 1), hist)
    assert halves[0][3][:, 0].tolist() == [T] * B


@pytest.mark.parametrize("tc", [False, True])
def test_decode_step_with_ragged_positions(tc):
    """Sequences of one batch at different positions (what _reorder_cache / ragged prompts produce)."""
    from flash_stu_2_b200 import ops
    dt = torch.bfloat16
    B, T, d, L = 5, 50, 32, 64
    Lh = 32
    x, nw, Mi, fp, xp, ref = _decode_fixture(dt, B, T, d, L, seed=9)
    where = [7, 30, 30, 1, 49]
    hist_full = _hist_from(xp, Lh)
    hist = torch.zeros_like(hist_full)
    for b, t in enumerate(where):  # rows hold only the first t projected inputs
        for p in range(2):
            n = (t - p + 1) // 2
            hist[b, :, p, :n] = hist_full[b, :, p, :n]
    hist = hist.to(dev())
    pos = torch.zeros(B, 2, dtype=torch.int32)
    pos[:, 0] = torch.tensor(where, dtype=torch.int32)
    pos = pos.to(dev())
    taps = ops.taps_even(fp.to(dev()), Lh)
    taps8 = ops.taps_rev8(taps) if tc else None
    xin = torch.stack([x[b, t] for b, t in enumerate(where)]).to(dev())
    out = torch.empty(B, d, dtype=dt, device=dev())
    ops.decode_approx(xin, nw.to(dev()), Mi.t().contiguous().to(dev()), hist, taps, pos, out, taps8=taps8)
    ops.check_status()
    want = torch.stack([ref[b, t] for b, t in enumerate(where)])
    assert pos[:, 0].tolist() == [t + 1 for t in where]
    close(out, want, 1.5e-2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [(2, 40, 4, 8, 8), (1, 70, 2, 64, 16), (2, 33, 3, 128, 100)])
def test_attention_prefill_and_cached_decode(dt, cfg):
    from flash_stu_2_b200 import ops
    B, T, H, hd, w = cfg
    d = H * hd
    torch.manual_seed(7)
    x = torch.randn(B, T, d).to(dt)
    p = {"attn.c_attn.weight": (torch.randn(3 * d, d) / math.sqrt(d)).to(dt),
         "attn.c_proj.weight": torch.eye(d).to(dt)}
    ref, _ = O.attention(x, p, H, w, 50.0)
    qkv = (x @ p["attn.c_attn.weight"].t()).to(dev())
    slopes = O.alibi_slopes(H).float().to(dev())
    W = w + 1
    kr = torch.zeros(B, W, d, dtype=dt, device=dev())
    vr = torch.zeros_like(kr)
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    T1 = T - 5
    y1 = ops.swa_forward(qkv[:, :T1].contiguous(), kr, vr, pos, slopes, H, w, 50.0, update_cache=True)
    ys = [y1]
    for t in range(T1, T):
        ys.append(ops.swa_forward(qkv[:, t:t + 1].contiguous(), kr, vr, pos, slopes, H, w, 50.0, update_cache=True))
    got = torch.cat(ys, 1)
    assert pos[:, 0].tolist() == [T] * B
    close(got, ref, (1e-4 if dt == torch.float32 else 1.5e-2))
    # uncached call over the whole sequence
    dummy = torch.zeros(1, 1, 1, dtype=dt, device=dev())
    y = ops.swa_forward(qkv, dummy, dummy, torch.zeros(B, 2, dtype=torch.int32, device=dev()), slopes, H, w, 50.0,
                        update_cache=False)
    close(y, ref, (1e-4 if dt == torch.float32 else 1.5e-2))


@pytest.mark.parametrize("cfg", [(2, 300, 2, 100), (1, 700, 3, 256), (3, 260, 2, 1024), (2, 1031, 2, 77), (1, 128, 1, 16)])
def test_attention_prefill_on_tcgen05_matches_oracle(cfg):
    """Prefill from position 0, bf16, head dimension 128: the tcgen05 kernel (S and O in tensor memory, lazy row
    maximum) against the fp32 oracle and against the mma.sync kernel; ragged last query tile, windows shorter and
    longer than a key tile, the ring and the positions afterwards, then cached steps on top of it."""
    from flash_stu_2_b200 import ops
    B, T, H, w = cfg
    hd, dt = 128, torch.bfloat16
    d = H * hd
    torch.manual_seed(13)
    x = torch.randn(B, T, d).to(dt)
    p = {"attn.c_attn.weight": (torch.randn(3 * d, d) / math.sqrt(d)).to(dt),
         "attn.c_proj.weight": torch.eye(d).to(dt)}
    ref, _ = O.attention(x, p, H, w, 50.0)
    qkv = (x @ p["attn.c_attn.weight"].t()).to(dev())
    slopes = O.alibi_slopes(H).float().to(dev())
    W = w + 1
    T1 = T - 3
    q1 = qkv[:, :T1].contiguous()
    assert ops.swa_prefill_tc5_supported(q1, H, 0) or T1 < 128
    kr, vr = torch.zeros(B, W, d, dtype=dt, device=dev()), torch.zeros(B, W, d, dtype=dt, device=dev())
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    kr2, vr2, pos2 = torch.zeros_like(kr), torch.zeros_like(vr), torch.zeros_like(pos)
    y1 = ops.swa_prefill_tc5(q1, kr, vr, pos, slopes, H, w, 50.0, update_cache=True)
    y2 = ops.swa_forward(q1, kr2, vr2, pos2, slopes, H, w, 50.0, update_cache=True)
    ops.check_status()
    close(y1, ref[:, :T1], 1.5e-2, what="tcgen05 vs oracle")
    close(y1, y2, 1.5e-2, what="tcgen05 vs mma.sync")
    assert torch.equal(kr, kr2) and torch.equal(vr, vr2) and torch.equal(pos, pos2)
    ys = [y1]
    for t in range(T1, T):
        ys.append(ops.swa_forward(qkv[:, t:t + 1].contiguous(), kr, vr, pos, slopes, H, w, 50.0, update_cache=True))
    close(torch.cat(ys, 1), ref, 1.5e-2)
    # a sequence that is not at position 0 is refused on the device
    ops.swa_prefill_tc5(q1, kr, vr, pos, slopes, H, w, 50.0, update_cache=False)
    with pytest.raises(RuntimeError, match="status 11"):
        ops.check_status()


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [(2, 300, 2, 64, 100), (1, 700, 3, 128, 256), (3, 260, 2, 128, 1024)])
def test_attention_chunked_prefill_across_many_key_tiles(dt, cfg):
    """Windows spanning several 64-key tiles, a second prefill chunk whose older keys come from the ring, then
    cached single-token steps (tensor-core prefill kernel and memory-bound decode kernel for bf16)."""
    from flash_stu_2_b200 import ops
    B, T, H, hd, w = cfg
    d = H * hd
    torch.manual_seed(11)
    x = torch.randn(B, T, d).to(dt)
    p = {"attn.c_attn.weight": (torch.randn(3 * d, d) / math.sqrt(d)).to(dt),
         "attn.c_proj.weight": torch.eye(d).to(dt)}
    ref, _ = O.attention(x, p, H, w, 50.0)
    qkv = (x @ p["attn.c_attn.weight"].t()).to(dev())
    slopes = O.alibi_slopes(H).float().to(dev())
    W = w + 1
    kr = torch.zeros(B, W, d, dtype=dt, device=dev())
    vr = torch.zeros_like(kr)
    pos = torch.zeros(B, 2, dtype=torch.int32, device=dev())
    cuts = [0, 131, T - 6]
    ys = [ops.swa_forward(qkv[:, a:b].contiguous(), kr, vr, pos, slopes, H, w, 50.0, update_cache=True)
          for a, b in zip(cuts[:-1], cuts[1:])]
    for t in range(T - 6, T):
        ys.append(ops.swa_forward(qkv[:, t:t + 1].contiguous(), kr, vr, pos, slopes, H, w, 50.0, update_cache=True))
    got = torch.cat(ys, 1)
    assert pos[:, 0].tolist() == [T] * B and int(pos[0, 1]) == 0
    close(got, ref, (1e-4 if dt == torch.float32 else 1.5e-2))


def test_sampling_matches_oracle():
    from flash_stu_2_b200 import ops
    torch.manual_seed(8)
    B, V = 6, 50257
    for dt in (torch.float32, torch.bfloat16):
        logits = (torch.randn(B, V) * 3).to(dt)
        out = torch.zeros(B, dtype=torch.int64, device=dev())
        ops.sample(logits.to(dev()), 1.0, None, None, False, None, out)
        assert torch.equal(out.cpu(), logits.float().argmax(-1))
        # (temperature, top_k, top_p): candidate-list path (top_k <= 1024), and the full-vocabulary filters: nucleus
        # without top-k, a top-k wider than the candidate list, and a nucleus inside such a top-k
        for (temp, k, p) in [(0.8, 40, None), (0.8, 5, 0.9), (1.3, 1, None), (1.0, None, None), (0.9, None, 0.9),
                             (1.0, None, 0.35), (0.7, 3000, None), (1.1, 5000, 0.8), (1.0, 1024, 0.95)]:
            u = torch.rand(B)
            z = O.filter_logits(logits, temp, k, p)
            want = O.pick_token(z, True, u).view(-1)
            ops.sample(logits.to(dev()), temp, k, p, True, u.to(dev()), out)
            ops.check_status()
            got = out.cpu()
            # the draw may differ only where u lands within rounding of a CDF boundary; require the
            # chosen token to be inside the filtered support and almost all draws identical
            assert all(torch.isfinite(z[b, got[b]]) for b in range(B)), (temp, k, p, got.tolist())
            if dt == torch.float32:
                frac = float((got == want).float().mean())
                assert frac >= 0.8, f"{frac:.2f} of the fp32 draws equal the oracle's ({got.tolist()} vs {want.tolist()})"


def test_sampling_row_with_a_nan_logit_draws_uniformly():
    """The reference replaces the distribution of a row whose softmax is not finite by a uniform one
    (flash_stu/model.py:293-296); the kernel takes the row's uniform for it and leaves the other rows alone."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(9)
    B, V = 4, 1000
    logits = torch.randn(B, V)
    logits[2, 17] = float("nan")
    u = torch.tensor([0.3, 0.9, 0.25, 0.5])
    out = torch.zeros(B, dtype=torch.int64, device=dev())
    ops.sample(logits.to(dev()), 1.0, 50, None, True, u.to(dev()), out)
    ops.check_status()
    got = out.cpu()
    assert int(got[2]) == int(0.25 * V)
    z = O.filter_logits(logits[[0, 1, 3]], 1.0, 50, None)
    assert all(torch.isfinite(z[i, got[b]]) for i, b in enumerate((0, 1, 3)))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_full_variant_building_blocks(dt):
    """to_history, the three Toeplitz matrices, the causal GEMM flag and the combine step against plain torch."""
    from flash_stu_2_b200 import ops
    torch.manual_seed(12)
    B, T, d, K, L, t0 = 2, 301, 40, 5, 320, 0
    S = ((T + 1) // 2 + 7) // 8 * 8
    x = torch.randn(B, T, d).to(dt)
    phi = (torch.randn(L, K) / 4).to(dt)
    hist = torch.zeros(B, d, 2, S, dtype=dt, device=dev())
    ops.to_history(x.to(dev()), hist, t0)
    assert torch.equal(hist.cpu(), _hist_from(x, S))
    Tz = torch.empty(3, S, S, dtype=dt, device=dev())
    ops.toeplitz(phi.to(dev()), 3, Tz)
    m = torch.arange(S)[:, None]
    s_ = torch.arange(S)[None, :]
    for kind, off in ((0, 0), (1, 1), (2, -1)):
        j = 2 * (m - s_) + off
        ok = (m >= s_) & (j >= 0) & (j < L)
        want = torch.where(ok, phi[:, 3][j.clamp(0, L - 1)], torch.zeros((), dtype=dt))
        assert torch.equal(Tz[kind].cpu(), want), kind
    rows = hist.view(B * d * 2, S)
    dense = ops.linear(rows, Tz[0], backend=0)
    causal = ops.linear(rows, Tz[0], epilogue=ops.EPI_STORE | ops.EPI_FLAG_CAUSAL, backend=0)
    ops.check_status()
    close(causal, dense, 1e-6)
    ref = (rows.cpu().double() @ Tz[0].cpu().double().t()).to(dt)
    close(causal, ref, TOL[dt] / 2)
    # E, Q -> U for one filter
    E = torch.randn(B * d * 2, S).to(dt)
    Q = torch.randn(B * d * 2, S).to(dt)
    U = torch.zeros(B * T, 2 * K * d, dtype=dt, device=dev())
    ops.full_combine(E.to(dev()), Q.to(dev()), U, B, d, K, 3, True, t0, T)
    Ev = E.view(B, d, 2, S)
    Qv = Q.view(B, d, 2, S)
    want = torch.zeros(B, T, 2, K, d, dtype=dt)
    for p in range(2):
        n = (T - p + 1) // 2
        want[:, p::2, 0, 3] = (Ev[:, :, p, :n].float() + Qv[:, :, p, :n].float()).to(dt).transpose(1, 2)
        want[:, p::2, 1, 3] = (Ev[:, :, p, :n].float() - Qv[:, :, p, :n].float()).to(dt).transpose(1, 2)
    assert torch.equal(U.cpu().view(B, T, 2, K, d), want)


@pytest.mark.parametrize("name,tol", [("std_full_float32", 1e-3), ("std_full_bfloat16", 2e-2),
                                       ("hankelL_full_float32", 1e-3), ("std_approx_float32", 1e-3),
                                       ("std_approx_bfloat16", 2e-2), ("hankelL_approx_float32", 1e-3),
                                       ("hankelL_approx_bfloat16", 2e-2), ("hankelL_full_bfloat16", 2e-2)])
def test_stu_operator_matches_reference_golden(golden, name, tol):
    """STU.forward (operator output, no residual) against the reference module's own outputs."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    r = golden("stu_modules")[name]
    dt = r["x"].dtype
    L, K = r["phi"].shape
    d = r["x"].shape[2]
    cfg = F.FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx="_approx_" in name,
                           use_hankel_L=name.startswith("hankelL"), torch_dtype=dt, n_layers=1, vocab_size=1)
    m = F.STU(cfg, r["phi"].clone(), r["n"])
    with torch.no_grad():
        for k, v in r["params"].items():
            getattr(m, k).copy_(v)
    m = m.to(dev())
    with torch.no_grad():
        y = m(r["x"].to(dev()))
        T = r["T_short"]
        ys = m(r["x"][:, :T].contiguous().to(dev()))
    ops.check_status()
    close(y, r["y_full"], tol)
    close(ys, r["y_short"], tol)


@pytest.mark.parametrize("name,tol", [("tiled16_approx_float32", 1e-3), ("tiled20_approx_float32", 1e-3),
                                       ("tiled16_approx_bfloat16", 2e-2), ("tiled20_approx_bfloat16", 2e-2)])
def test_stu_operator_with_block_diagonal_tiling_matches_reference_golden(golden, name, tol):
    """d_in_tile / d_out_tile (flash_stu/modules/stu.py:123-191): only the diagonal blocks of M_inputs take part
    (tile 16 divides the width, tile 20 leaves a ragged last block)."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    r = golden("variants")[name]
    dt = r["x"].dtype
    L, K = r["phi"].shape
    d = r["x"].shape[2]
    cfg = F.FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=True, torch_dtype=dt, n_layers=1, vocab_size=1,
                           d_in_tile=r["tile"][0], d_out_tile=r["tile"][1])
    m = F.STU(cfg, r["phi"].clone(), r["n"])
    with torch.no_grad():
        for k, v in r["params"].items():
            getattr(m, k).copy_(v)
    m = m.to(dev())
    with torch.no_grad():
        y = m(r["x"].to(dev()))
    ops.check_status()
    close(y, r["y"], tol)


def test_mini_stu_spectral_matches_reference_golden(golden):
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    r = golden("mini_stu")["spectral_fp32"]
    L, K = r["phi"].shape
    m = F.MiniSTU(seq_len=L, num_filters=K, input_dim=r["x"].shape[2], output_dim=r["y"].shape[2],
                  precomputed_filters=r["phi"])
    m.load_state_dict(r["params"])
    m = m.to(dev())
    with torch.no_grad():
        y = m(r["x"].to(dev()))
    ops.check_status()
    close(y, r["y"], 1e-3)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-3), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("shape", [(2, 48, 6, 10), (3, 200, 64, 32)])
def test_mini_stu_lds_prefill_and_recurrent_decode(golden, dt, tol, shape):
    """MiniSTU(backend='lds'): prefill (convolution with the LDS impulse responses) and the recurrent decode
    steps against the float64 recurrence of the reference (mini_stu/stu_lds.py) on the same rounded inputs."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    B, T, din, dout = shape
    g = golden("mini_stu")["lds_fp64"]
    torch.manual_seed(13)
    m = F.MiniSTU(seq_len=T, num_filters=24, input_dim=din, output_dim=dout, backend="lds", dtype=dt)
    x = torch.randn(B, T, din).to(dt)
    Mr = m.distill_stu.M.detach().clone()
    Cr = m.lds_module.C.detach().clone()
    assert torch.equal(m.lds_module.A, g["A"]) and torch.equal(Cr, g["C"].to(dt))
    want = O.lds_forward(x.double(), g["A"], g["B_vec"], Cr.double(), g["h0"], Mr.double())
    m = m.to(dev())
    T1 = T - 9
    with torch.no_grad():
        y_all = m(x.to(dev()))
        y1, cache = m(x[:, :T1].to(dev()), use_cache=True)
        state_scan = cache[0].clone()
        rows = [y1]
        for t in range(T1, T):
            yt, cache = m(x[:, t:t + 1].to(dev()), past_key_value=cache, use_cache=True)
            rows.append(yt)
        # the convolution form of the same prefill (full-length impulse responses): same rows within tolerance, and
        # its final-state kernel gives bit for bit the state the chunked scan hands to the recurrent decode
        F.MiniSTU.chunked_scan_prefill = False
        try:
            y_conv, cache_conv = m(x[:, :T1].to(dev()), use_cache=True)
        finally:
            F.MiniSTU.chunked_scan_prefill = True
    ops.check_status()
    assert torch.equal(cache_conv[0], state_scan)
    close(y_conv, want[:, :T1], tol)
    close(y_all, want, tol)
    got = torch.cat(rows, 1)
    close(got, want, tol)
    if shape == (2, 48, 6, 10) and dt == torch.float32:
        # the reference module's own output (float64 run of MiniSTU(backend='lds')) with its M
        m2 = F.MiniSTU(seq_len=T, num_filters=24, input_dim=din, output_dim=dout, backend="lds", dtype=dt)
        with torch.no_grad():
            m2.distill_stu.M.copy_(g["M"].to(dt))
        m2 = m2.to(dev())
        with torch.no_grad():
            y2 = m2(g["x"].to(dt).to(dev()))
        close(y2, g["y"], 1e-3)
