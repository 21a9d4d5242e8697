"""FlashSTUBlock on a B200 against the reference's own outputs (tests/golden/blocks.pt) and the
size-independent properties of the cached token loop."""
import os

import pytest
import torch

from oracle import stu_oracle as O
from parity import close

pytestmark = pytest.mark.gpu


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def make_block(r, dt, approx=True):
    approx = approx and not r.get("_full", False)
    import flash_stu_2_b200 as F
    cfg = F.FlashSTUConfig(n_embd=r["d"], seq_len=r["L"], num_eigh=r["K"], use_approx=approx, use_attn=False,
                           mlp_scale=4, torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=1)
    blk = F.FlashSTUBlock(config=cfg, phi=r["sd"]["phi"].clone(), n=r["n"])
    blk.load_state_dict(r["sd"])
    return blk.to(dev()).eval()


ALL_BLOCKS = [("approx_float32", 1e-3), ("approx_bfloat16", 2e-2), ("full_float32", 1e-3), ("full_bfloat16", 2e-2)]


@pytest.mark.parametrize("name,tol", ALL_BLOCKS)
def test_block_forward_matches_reference_golden(golden, name, tol):
    from flash_stu_2_b200 import ops
    r = dict(golden("blocks")[name], _full=name.startswith("full"))
    dt = r["x"].dtype
    blk = make_block(r, dt)
    x = r["x"].clone().to(dev())
    with torch.no_grad():
        y = blk(x)
    ops.check_status()
    assert y.data_ptr() == x.data_ptr()  # in place on the caller's tensor, like the reference
    close(y.cpu(), r["y"], tol)


@pytest.mark.parametrize("name,tol", ALL_BLOCKS)
def test_block_cached_decode_equals_prefill_rows(golden, name, tol):
    """prefill T1 tokens with a cache, then single-token steps: every row equals the full forward."""
    from flash_stu_2_b200 import ops
    r = dict(golden("blocks")[name], _full=name.startswith("full"))
    dt = r["x"].dtype
    blk = make_block(r, dt)
    x = r["x"].to(dev())
    T = x.shape[1]
    T1 = T - 17
    with torch.no_grad():
        y1, cache = blk(x[:, :T1].clone(), use_cache=True)
        rows = [y1]
        for t in range(T1, T):
            yt, cache = blk(x[:, t:t + 1].clone(), past_key_value=cache, use_cache=True)
            rows.append(yt)
    ops.check_status()
    got = torch.cat(rows, 1).cpu()
    assert int(cache[1][0, 0]) == T
    close(got, r["y"], tol)


def test_block_tensor_core_and_cuda_core_convolutions_agree(golden):
    import flash_stu_2_b200 as F
    r = golden("blocks")["approx_bfloat16"]
    blk = make_block(r, torch.bfloat16)
    x = r["x"].to(dev())
    with torch.no_grad():
        a = blk(x.clone())
        F.STU.tensor_core_conv = False
        try:
            b = blk(x.clone())
        finally:
            F.STU.tensor_core_conv = True
    close(a.cpu(), b.cpu(), 4e-3)


def test_block_properties_at_benchmark_width():
    """d_model=1024, K=24 as in the benchmark block, shorter context (L=2048, B=2): prefix consistency,
    causality and chunked prefill == one-shot prefill, checked against the oracle on one sequence."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    torch.manual_seed(1)
    L, K, d, B = 2048, 24, 1024, 2
    dt = torch.bfloat16
    phi = O.spectral_filters(L, K, dtype=dt)
    cfg = F.FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_attn=False, mlp_scale=4, torch_dtype=dt, n_layers=1,
                           vocab_size=1, n_heads=1)
    blk = F.FlashSTUBlock(config=cfg, phi=phi, n=O.fft_length(L))
    for n_, p in blk.named_parameters():
        if ".stu.M_" in n_:
            torch.nn.init.xavier_normal_(p)
    sd = {k: v.clone() for k, v in blk.state_dict().items()}
    blk = blk.to(dev()).eval()
    x = torch.randn(B, L, d).to(dt)
    with torch.no_grad():
        full = blk(x.clone().to(dev())).cpu()
        T = 1000
        short = blk(x[:, :T].clone().to(dev())).cpu()
        y1, cache = blk(x[:, :768].clone().to(dev()), use_cache=True)
        y2, cache = blk(x[:, 768:1500].clone().to(dev()), past_key_value=cache, use_cache=True)
        y3, cache = blk(x[:, 1500:1501].clone().to(dev()), past_key_value=cache, use_cache=True)
    ops.check_status()
    close(short, full[:, :T], 1e-6)          # prefix consistency (same kernels, same order)
    chunked = torch.cat([y1.cpu(), y2.cpu(), y3.cpu()], 1)
    close(chunked, full[:, :1501], 2e-2)
    lsd = {k[len("layer."):]: v for k, v in sd.items() if k.startswith("layer.")}
    ref = O.stu_layer(x[:1], lsd, sd["phi"], O.fft_length(L), True)
    close(full[:1], ref, 2e-2)


def test_overlapped_decode_launches_equal_plain_launches(golden):
    """The decode kernels launched with programmatic stream serialization (prefetch of weights / history while
    the preceding kernel drains) give bit-identical rows to plain stream-ordered launches, eagerly and when the
    token step is replayed from a captured CUDA graph."""
    from flash_stu_2_b200 import ops
    r = golden("blocks")["approx_bfloat16"]
    blk = make_block(r, torch.bfloat16)
    x = r["x"].to(dev())
    T = x.shape[1]
    T1 = T - 24

    def run(overlap, graph):
        ops.overlap_decode = overlap
        try:
            with torch.no_grad():
                _, cache = blk(x[:, :T1].clone(), use_cache=True)
                step = torch.empty_like(x[:, :1])
                rows = []
                g = None
                if graph:
                    # two eager steps first (derived weights, scratch), then capture one step and rewind
                    for t in range(T1, T1 + 2):
                        step.copy_(x[:, t:t + 1])
                        blk(step, past_key_value=cache, use_cache=True)
                    cache[1][:, 0] = T1
                    cache[1]._host_t = T1
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        blk(step, past_key_value=cache, use_cache=True)
                    cache[1][:, 0] = T1
                    cache[1]._host_t = T1
                for t in range(T1, T):
                    step.copy_(x[:, t:t + 1])
                    if g is not None:
                        g.replay()
                    else:
                        blk(step, past_key_value=cache, use_cache=True)
                    rows.append(step.clone())
                torch.cuda.synchronize()
                assert int(cache[1][0, 0]) == T
            return torch.cat(rows, 1).cpu()
        finally:
            ops.overlap_decode = True

    plain = run(False, False)
    assert torch.equal(run(True, False), plain)
    assert torch.equal(run(True, True), plain)
    ops.check_status()
    close(plain, r["y"][:, T1:], 2e-2)


@pytest.mark.parametrize("approx", [True, False])
def test_benchmark_block_at_full_size_against_the_oracle(approx):
    """The benchmark block at its full size (d_model=1024, K=24, L=8192, bf16; both STU variants), two sequences:
    a prefill over all 8192 positions and the last 24 positions again as cached single-token steps, against the
    CPU oracle on the same weights and inputs (bf16 tolerance 2e-2)."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    torch.manual_seed(1)
    L, K, d, B = 8192, 24, 1024, 2
    dt = torch.bfloat16
    fpath = os.path.join(os.path.dirname(F.__file__), "data", f"phi_{L}_{K}.pt")
    phi = F.load_spectral_filters(fpath, device="cpu", dtype=dt, verify_shape=(L, K))
    cfg = F.FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_attn=False, use_approx=approx, mlp_scale=4,
                           torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=16)
    blk = F.FlashSTUBlock(config=cfg, phi=phi, n=O.fft_length(L))
    for n_, p in blk.named_parameters():
        if ".stu.M_" in n_:
            torch.nn.init.xavier_normal_(p)
    sd = {k: v.clone() for k, v in blk.state_dict().items()}
    blk = blk.to(dev()).eval()
    x = torch.randn(B, L, d).to(dt)
    S = 24
    with torch.no_grad():
        full = blk(x.clone().to(dev())).cpu()
        y1, cache = blk(x[:, :L - S].clone().to(dev()), use_cache=True)
        rows = []
        for t in range(L - S, L):
            yt, cache = blk(x[:, t:t + 1].clone().to(dev()), past_key_value=cache, use_cache=True)
            rows.append(yt.cpu())
    ops.check_status()
    lsd = {k[len("layer."):]: v for k, v in sd.items() if k.startswith("layer.")}
    # one sequence at a time: the full variant's FFT stack takes 10 GB of host memory per sequence
    ref = torch.cat([O.stu_layer(x[b:b + 1], lsd, sd["phi"], O.fft_length(L), approx) for b in range(B)])
    close(full, ref, 2e-2)
    close(torch.cat(rows, 1), ref[:, L - S:], 2e-2)
    close(y1.cpu(), ref[:, :L - S], 2e-2)


def test_cache_laid_out_for_fewer_positions_than_the_filters(golden):
    """config.cache_len: a block whose filters span seq_len positions but whose caches and tap tables are laid out
    for fewer gives the same rows as the full-capacity block, and refuses positions beyond its capacity."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    r = golden("blocks")["approx_bfloat16"]
    x = r["x"].to(dev())
    T = x.shape[1]
    cap = T - 40
    cfg = F.FlashSTUConfig(n_embd=r["d"], seq_len=r["L"], num_eigh=r["K"], use_attn=False, mlp_scale=4,
                           torch_dtype=torch.bfloat16, n_layers=1, vocab_size=1, n_heads=1, cache_len=cap)
    blk = F.FlashSTUBlock(config=cfg, phi=r["sd"]["phi"].clone(), n=r["n"])
    blk.load_state_dict(r["sd"])
    blk = blk.to(dev()).eval()
    with torch.no_grad():
        y1, cache = blk(x[:, :cap - 5].clone(), use_cache=True)
        rows = [y1]
        for t in range(cap - 5, cap):
            yt, cache = blk(x[:, t:t + 1].clone(), past_key_value=cache, use_cache=True)
            rows.append(yt)
        with pytest.raises(ValueError, match="capacity"):
            blk(x[:, cap:cap + 1].clone(), past_key_value=cache, use_cache=True)
    ops.check_status()
    assert cache[0].shape[3] < (r["L"] + 1) // 2
    close(torch.cat(rows, 1).cpu(), r["y"][:, :cap], 2e-2)


@pytest.mark.parametrize("name,tol", [("sandwich_approx_float32", 1e-3), ("sandwich_approx_bfloat16", 2e-2)])
def test_stu_layer_with_the_mlp_sandwich_matches_reference_golden(golden, name, tol):
    """stu_enable_mlp_sandwich (in_proj -> SiLU -> STU on the hidden width -> out_proj): the whole input, a shorter
    input, and prefill + cached single-token steps (bf16: the steps read their position on the device) against the
    reference's own outputs."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    r = golden("variants")[name]
    dt = r["x"].dtype
    cfg = F.FlashSTUConfig(n_embd=r["d"], seq_len=r["L"], num_eigh=r["K"], use_approx=True, use_attn=False,
                           mlp_scale=4, torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=1,
                           stu_enable_mlp_sandwich=True, stu_mlp_hidden_size=r["hidden"])
    blk = F.FlashSTUBlock(config=cfg, phi=r["sd"]["phi"].clone(), n=r["n"])
    blk.load_state_dict(r["sd"])
    blk = blk.to(dev()).eval()
    x = r["x"].to(dev())
    T, Ts = x.shape[1], r["T_short"]
    with torch.no_grad():
        close(blk(x.clone()).cpu(), r["y"], tol)
        close(blk(x[:, :Ts].clone()).cpu(), r["y_short"], tol)
        T1 = T - 9
        y1, cache = blk(x[:, :T1].clone(), use_cache=True)
        rows = [y1]
        for t in range(T1, T):
            yt, cache = blk(x[:, t:t + 1].clone(), past_key_value=cache, use_cache=True)
            rows.append(yt)
    ops.check_status()
    assert int(cache[1][0, 0]) == T
    close(torch.cat(rows, 1).cpu(), r["y"], tol)


@pytest.mark.parametrize("name", ["mini_mlp_relu2", "mini_mlp_gelu3", "mini_mlp_tanh2", "mini_mlp_single"])
def test_mini_stu_with_post_mlp_matches_reference_golden(golden, name):
    from flash_stu_2_b200 import MiniSTU, ops
    r = golden("variants")[name]
    L, din = r["x"].shape[1], r["x"].shape[2]
    dout = r["y"].shape[2]
    m = MiniSTU(seq_len=L, num_filters=r["phi"].shape[1], input_dim=din, output_dim=dout, use_mlp=True,
                dtype=torch.float32, precomputed_filters=r["phi"], **r["kw"])
    m.load_state_dict(r["sd"])
    m = m.to(dev())
    with torch.no_grad():
        y = m(r["x"].to(dev()))
    ops.check_status()
    close(y.cpu(), r["y"], 1e-3)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-3), (torch.bfloat16, 2e-2)])
def test_single_branch_approx_block_cached_steps_equal_prefill_rows(dt, tol):
    """use_hankel_L with use_approx (one convolution branch over ALL taps: the even taps act on the same time parity,
    the odd taps on the other one a step earlier): the layer's output against the oracle, and prefill + cached
    single-token steps against the full forward."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    torch.manual_seed(31)
    L, K, d, B = 96, 8, 32, 3
    phi = O.spectral_filters(L, K, use_hankel_L=True)
    cfg = F.FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=True, use_hankel_L=True, use_attn=False,
                           mlp_scale=4, torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=1)
    blk = F.FlashSTUBlock(config=cfg, phi=phi.to(dt), n=O.fft_length(L))
    with torch.no_grad():
        for name, p in blk.named_parameters():
            if p.dim() >= 2:
                torch.nn.init.xavier_normal_(p)
    sd = {k[len("layer."):]: v.detach().clone() for k, v in blk.state_dict().items() if k.startswith("layer.")}
    x = torch.randn(B, L, d).to(dt)
    want = O.stu_layer(x, sd, phi.to(dt), O.fft_length(L), True, use_hankel_L=True)
    blk = blk.to(dev()).eval()
    xd = x.to(dev())
    with torch.no_grad():
        close(blk(xd.clone()).cpu(), want, tol)
        T1 = L - 11
        y1, cache = blk(xd[:, :T1].clone(), use_cache=True)
        rows = [y1]
        for t in range(T1, L):
            yt, cache = blk(xd[:, t:t + 1].clone(), past_key_value=cache, use_cache=True)
            rows.append(yt)
    ops.check_status()
    assert int(cache[1][0, 0]) == L
    close(torch.cat(rows, 1).cpu(), want, tol)
