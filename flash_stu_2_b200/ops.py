"""Tensor-level wrappers around the C-ABI: torch supplies device memory and streams, nothing else.

Every function takes CUDA tensors, launches on torch's current stream and returns without
synchronising.  Device-side problems (bounded waits that ran out, out-of-range token ids or
positions) are recorded in a per-process status word; `check_status()` reads it (one sync).
"""
from typing import Optional

import torch

from . import _lib

EPI_STORE, EPI_RESID, EPI_GELU_MUL, EPI_HIST = 0, 1, 2, 3
EPI_FLAG_CAUSAL = 0x100  # OR-ed into the epilogue: the weight is lower triangular
# Overlapped (programmatic dependent) launches of the decode kernels: OR-ed into the epilogue code of linear() and
# passed as flags to decode_approx().  FLAG_OVERLAP: the kernel may start while its predecessor in the stream is
# still running and fetches its constants (weights; history and taps) meanwhile; FLAG_EARLY_TRIGGER: it lets its
# own successor start at once.  The decode paths of the layers use them when overlap_decode is True: the MLP kernels
# overlap their weight fetch with the drain of the kernel before them (measured 1.3 us per layer step on a B200);
# the STU decode kernel only triggers early - letting it start early made the step slower, its history loads
# compete with the down projection it would overlap.
FLAG_OVERLAP = 0x200
FLAG_EARLY_TRIGGER = 0x400
FLAG_UNIFORM_POS = 0x800  # decode_approx: every sequence of the batch stands at the same position (checked on device)
overlap_decode = True
# early_decode: additionally launch the pipelined STU decode kernel overlapped with the kernel before it (the down
# projection of the previous layer, which then triggers early): its history stream needs nothing that kernel writes,
# only its projection waits.
early_decode = True
# fused_step: a cached token step of an approx STU layer with at most 8 sequences at one position runs as ONE
# persistent kernel (STU sub-layer and MLP) that already streams the next position's history partial sums.
fused_step = True
BACKEND_AUTO, BACKEND_SIMT, BACKEND_TCGEN05, BACKEND_SKINNY = 0, 1, 2, 3
RMS_EPS = float(torch.finfo(torch.float32).eps)  # what torch.nn.RMSNorm(eps=None) resolves to

_status = {}
launch_count = 0  # kernels launched through this module (bench.py reports it)


def _count(n=1):
    global launch_count
    launch_count += n


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"flash_stu_2_b200 kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flash_stu_2_b200 has no CPU path: tensors must live on a CUDA device")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = w
        with torch.cuda.device(key):   # the library keeps one word per device, registered with that device current
            _lib.check(_lib.load().stu_set_status_word(w.data_ptr()), "stu_set_status_word")
    return _status[key]


STATUS_TEXT = {1: "token id outside the vocabulary", 2: "position outside the cache capacity (seq_len)",
               3: "a bounded mbarrier wait ran out inside the tcgen05 GEMM", 4: "more top-k ties than the candidate list holds and the vocabulary does not fit in shared memory",
               5: "top_p without top_k (<= 1024) needs the vocabulary row in shared memory (at most 51712 entries)",
               6: "decode step told that all sequences share one position, but the cached positions differ",
               7: "a bounded pipeline wait ran out inside the decode kernel",
               8: "the fused token-step kernel found no partial sums for the current position in its workspace",
               9: "a bounded pipeline wait ran out inside the tcgen05 prefill convolution",
               10: "a tensor-parallel rank waited in vain for another rank's sub-layer output",
               11: "tcgen05 attention prefill: a bounded wait ran out, or a sequence was not at position 0"}


def check_status(device=None):
    """Raise if any kernel flagged a device-side problem since the last check (synchronises)."""
    for key, w in _status.items():
        v = int(w.item())
        if v:
            w.zero_()
            raise RuntimeError(f"flash_stu_2_b200 device status {v}: {STATUS_TEXT.get(v, 'unknown')}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = RMS_EPS, out: Optional[torch.Tensor] = None):
    _cuda(x, weight)
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    o2 = out.reshape(-1, d)
    rc = _lib.load().stu_rmsnorm(x2.data_ptr(), weight.data_ptr(), o2.data_ptr(), x2.shape[0], d, x2.stride(0),
                                 o2.stride(0), eps, _dt(x), _stream())
    _lib.check(rc, "stu_rmsnorm")
    _count()
    return out.reshape(x.shape)


ACT_NONE, ACT_RELU, ACT_GELU, ACT_TANH, ACT_SILU = 0, 1, 2, 3, 4


def bias_act(y: torch.Tensor, bias: Optional[torch.Tensor], act: int = ACT_NONE):
    """In place: y[..., c] = act(y[..., c] + bias[c]) (bias may be None)."""
    _cuda(y, bias)
    cols = y.shape[-1]
    y2 = y.view(-1, cols)
    assert y2.stride(1) == 1 and (bias is None or (bias.shape == (cols,) and bias.is_contiguous()))
    rc = _lib.load().stu_bias_act(y2.data_ptr(), _p(bias), y2.shape[0], cols, y2.stride(0), act, _dt(y), _stream())
    _lib.check(rc, "stu_bias_act")
    _count()
    return y


def embed(ids: torch.Tensor, table: torch.Tensor):
    _cuda(ids, table)
    ids = ids.contiguous().to(torch.int64)
    out = torch.empty(*ids.shape, table.shape[1], dtype=table.dtype, device=table.device)
    rc = _lib.load().stu_embed(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1],
                               table.shape[0], status_word(table.device).data_ptr(), _dt(table), _stream())
    _lib.check(rc, "stu_embed")
    _count()
    return out


def can_fuse_norm(M: int, N: int, K: int, epilogue: int, dtype: torch.dtype) -> bool:
    code = 1 if dtype == torch.bfloat16 else 0
    return bool(_lib.load().stu_linear_can_fuse_norm(M, N, K, epilogue, code))


def linear(x: torch.Tensor, W: torch.Tensor, *, W2: Optional[torch.Tensor] = None,
           resid: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, epilogue: int = EPI_STORE,
           norm_w: Optional[torch.Tensor] = None, eps: float = RMS_EPS, backend: int = BACKEND_AUTO,
           transposed_weight: bool = False, hist_T: int = 0, hist_t0: int = 0, hist_Lh: int = 0):
    """y = epilogue(x @ W^T) for x [M,K] and W [N,K] (or W [K,N] with transposed_weight=True)."""
    _cuda(x, W, W2, resid, out, norm_w)
    assert x.dim() == 2 and W.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    if transposed_weight:
        assert W.shape[0] == K
        N, w_rs, w_ks = W.shape[1], W.stride(1), W.stride(0)
    else:
        assert W.shape[1] == K, (W.shape, K)
        N, w_rs, w_ks = W.shape[0], W.stride(0), W.stride(1)
    if W2 is not None:
        assert W2.shape == W.shape and W2.stride() == W.stride()
    if (epilogue & 0xff) == EPI_HIST:
        assert out is not None
        y_rs = 0
    else:
        if out is None:
            out = torch.empty(M, N, dtype=x.dtype, device=x.device)
        assert out.shape == (M, N) and out.stride(1) == 1
        y_rs = out.stride(0)
    r_rs = 0
    if resid is not None:
        assert resid.shape == (M, N) and resid.stride(1) == 1
        r_rs = resid.stride(0)
    status_word(x.device)   # the tcgen05 GEMM reports an expired device-side wait through the registered word
    rc = _lib.load().stu_linear(x.data_ptr(), x.stride(0), W.data_ptr(), w_rs, w_ks, _p(W2), _p(resid), r_rs,
                                out.data_ptr(), y_rs, M, N, K, epilogue, hist_T, hist_t0, hist_Lh, _p(norm_w), eps,
                                _dt(x), backend, _stream())
    _lib.check(rc, "stu_linear")
    _count()
    return out


def taps_even(fp: torch.Tensor, Lh: int):
    """fp [L, d] (phi @ M_filters in the model dtype) -> even taps, channel-major [d, Lh]."""
    _cuda(fp)
    fp = fp.contiguous()
    L, d = fp.shape
    taps = torch.zeros(d, Lh, dtype=fp.dtype, device=fp.device)
    rc = _lib.load().stu_taps_even(fp.data_ptr(), taps.data_ptr(), L, d, Lh, _dt(fp), _stream())
    _lib.check(rc, "stu_taps_even")
    _count()
    return taps


def taps_rev8(taps: torch.Tensor):
    """Reversed tap table in all eight 16-byte alignments, [8, d, Lh+8] (bf16; feeds the tensor-core decode kernel)."""
    _cuda(taps)
    d, Lh = taps.shape
    out = torch.empty(8, d, Lh + 8, dtype=taps.dtype, device=taps.device)
    rc = _lib.load().stu_taps_rev8(taps.data_ptr(), out.data_ptr(), d, Lh, _dt(taps), _stream())
    _lib.check(rc, "stu_taps_rev8")
    _count()
    return out


def conv_prefill_approx(hist, taps, yT, x, t0: int, t_end: int, use_tensor_cores: bool):
    """x[b, t-t0, c] += 2 * sum_{j even} fp[j,c] * hist[b,c,t-j] for t in [t0, t_end)."""
    _cuda(hist, taps, yT, x)
    B, d, _, Lh = hist.shape
    assert hist.is_contiguous() and yT.is_contiguous() and taps.shape == (d, Lh) and taps.is_contiguous()
    assert x.shape == (B, t_end - t0, d) and x.stride(2) == 1
    rc = _lib.load().stu_conv_prefill_approx(hist.data_ptr(), taps.data_ptr(), yT.data_ptr(), x.data_ptr(),
                                             x.stride(0), x.stride(1), B, d, Lh, yT.shape[3], t0, t_end, _dt(x),
                                             int(use_tensor_cores), _stream())
    _lib.check(rc, "stu_conv_prefill_approx")
    _count(2)
    return x


def conv_prefill_tc5_supported(hist, x) -> bool:
    """The tcgen05 prefill convolution takes bf16 histories tiled in 128-position blocks."""
    return x.dtype == torch.bfloat16 and hist.shape[3] % 128 == 0


def conv_prefill_approx_tc5(hist, taps8, yT, x, t0: int, t_end: int):
    """conv_prefill_approx on the tcgen05 tensor cores; taps8 is the reversed tap table of taps_rev8."""
    _cuda(hist, taps8, yT, x)
    B, d, _, Lh = hist.shape
    assert hist.is_contiguous() and yT.is_contiguous() and taps8.shape == (8, d, Lh + 8) and taps8.is_contiguous()
    assert x.shape == (B, t_end - t0, d) and x.stride(2) == 1
    rc = _lib.load().stu_conv_prefill_approx_tc5(hist.data_ptr(), taps8.data_ptr(), yT.data_ptr(), x.data_ptr(),
                                                 x.stride(0), x.stride(1), B, d, Lh, yT.shape[3], t0, t_end,
                                                 status_word(x.device).data_ptr(), _dt(x), _stream())
    _lib.check(rc, "stu_conv_prefill_approx_tc5")
    _count(2)
    return x


def set_programmatic_launch(on: bool) -> bool:
    """Programmatic (overlapped) launches of the token-step kernels on or off for the launches that follow; returns the
    previous setting.  A captured CUDA graph keeps the setting it was captured with."""
    return bool(_lib.load().stu_set_programmatic_launch(int(bool(on))))


def conv_prefill_timeline(words: Optional[torch.Tensor]):
    """Register (or, with None, remove) the int64 tensor of 128 words that receives the tcgen05 convolution's
    device-side time stamps; see stu_conv_prefill_set_timeline."""
    if words is not None:
        _cuda(words)
        assert words.dtype == torch.int64 and words.numel() >= 128 and words.is_contiguous()
    _lib.check(_lib.load().stu_conv_prefill_set_timeline(None if words is None else words.data_ptr()),
               "stu_conv_prefill_set_timeline")


def conv_prefill_approx_static(hist, taps, x, t0: int, t_end: int, use_tensor_cores: bool):
    """conv_prefill_approx without a caller-provided scratch tensor: for hosts that cannot allocate device
    memory when they call (all HBM already owned by their own pool, or a no-allocation steady state).
    The scratch is a 32 MiB array built into the library; larger problems raise."""
    _cuda(hist, taps, x)
    B, d, _, Lh = hist.shape
    assert hist.is_contiguous() and taps.shape == (d, Lh) and taps.is_contiguous()
    assert x.shape == (B, t_end - t0, d) and x.stride(2) == 1
    rc = _lib.load().stu_conv_prefill_approx_static(hist.data_ptr(), taps.data_ptr(), x.data_ptr(), x.stride(0),
                                                    x.stride(1), B, d, Lh, t0, t_end, _dt(x), int(use_tensor_cores),
                                                    _stream())
    _lib.check(rc, "stu_conv_prefill_approx_static")
    _count(2)
    return x


def decode_approx(x, norm_w, MinT, hist, taps, pos, out, eps: float = RMS_EPS, taps8=None, flags: int = 0):
    """One fused decode step of an approx STU layer (norm, projection, cache append, taps, residual).
    With taps8 (bf16) a tensor-core kernel runs, otherwise the CUDA-core one.  flags: FLAG_UNIFORM_POS selects the
    kernel for batches at one common position (taps shared between sequences); FLAG_EARLY_TRIGGER lets an
    overlapped successor (the MLP's gate/up kernel) start fetching its weights while this kernel runs."""
    _cuda(x, norm_w, MinT, hist, taps, pos, out, taps8)
    B, d, _, Lh = hist.shape
    assert x.shape == (B, d) and out.shape == (B, d) and x.stride(1) == 1 and out.stride(1) == 1
    assert pos.dtype == torch.int32 and pos.shape == (B, 2) and pos.is_contiguous()
    assert x.data_ptr() != out.data_ptr()
    rc = _lib.load().stu_decode_approx(x.data_ptr(), x.stride(0), norm_w.data_ptr(), MinT.data_ptr(), hist.data_ptr(),
                                       taps.data_ptr(), _p(taps8), pos.data_ptr(), out.data_ptr(), out.stride(0), B, d,
                                       Lh, eps,
                                       status_word(x.device).data_ptr(), _dt(x) | flags, _stream())
    _lib.check(rc, "stu_decode_approx")
    _count()
    return out


def decode_approx_shard(x, norm_w, MinT, hist, taps8, pos, out, eps: float = RMS_EPS, add_residual: bool = False,
                        flags: int = 0):
    """Fused decode step for the d_ch channels of a tensor-parallel rank: x [B,d_in] (full layer input), MinT
    [d_ch,d_in], hist [B,d_ch,2,Lh], taps8 [8,d_ch,Lh+8] -> out [B,d_ch] (the STU output, plus x when add_residual)."""
    _cuda(x, norm_w, MinT, hist, taps8, pos, out)
    B, dch, _, Lh = hist.shape
    d_in = x.shape[1]
    assert x.shape[0] == B and MinT.shape == (dch, d_in) and out.shape == (B, dch) and x.stride(1) == 1
    assert out.stride(1) == 1 and taps8.shape == (8, dch, Lh + 8) and pos.dtype == torch.int32
    rc = _lib.load().stu_decode_approx_shard(x.data_ptr(), x.stride(0), norm_w.data_ptr(), MinT.data_ptr(),
                                             hist.data_ptr(), taps8.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                             out.stride(0), B, d_in, dch, Lh, eps, int(add_residual),
                                             status_word(x.device).data_ptr(), _dt(x) | flags, _stream())
    _lib.check(rc, "stu_decode_approx_shard")
    _count()
    return out


def decode_approx_projected(x, xp, hist, taps8, pos, out, add_residual: bool = True):
    """Decode step of an approx STU sub-layer whose projected input xp [B, d_ch] the caller computed as one GEMM:
    appends xp to the cache, out = (x +) taps . history.  With overlap_decode the kernel starts its history stream
    while the projection before it is still running and lets its own successor start at once."""
    _cuda(xp, hist, taps8, pos, out)
    flags = (FLAG_OVERLAP | FLAG_EARLY_TRIGGER) if overlap_decode else 0
    B, dch, _, Lh = hist.shape
    assert xp.shape == (B, dch) and out.shape == (B, dch) and xp.stride(1) == 1 and out.stride(1) == 1
    assert hist.is_contiguous() and taps8.is_contiguous() and (x is not None or not add_residual)
    rc = _lib.load().stu_decode_approx_projected(_p(x), x.stride(0) if x is not None else 0, xp.data_ptr(),
                                                 xp.stride(0), hist.data_ptr(), taps8.data_ptr(), pos.data_ptr(),
                                                 out.data_ptr(), out.stride(0), B, dch, Lh, int(add_residual),
                                                 status_word(xp.device).data_ptr(), _dt(xp) | flags, _stream())
    _lib.check(rc, "stu_decode_approx_projected")
    _count()
    return out


def linear_push(x: torch.Tensor, W: torch.Tensor, dest: int, dest_row_stride: int):
    """x[M,K] @ W[N,K]^T stored into every tensor-parallel rank's inbox through the exchange descriptor at device
    address `dest` (peer.PeerExchange.dest); M <= 64, bf16."""
    _cuda(x, W)
    M, K = x.shape
    N = W.shape[0]
    assert W.shape[1] == K and x.stride(1) == 1 and W.stride(1) == 1
    rc = _lib.load().stu_linear_push(x.data_ptr(), x.stride(0), W.data_ptr(), W.stride(0), M, N, K, dest,
                                     dest_row_stride, _dt(x), _stream())
    _lib.check(rc, "stu_linear_push")
    _count()


def decode_approx_push(x, norm_w, MinT, hist, taps8, pos, dest: int, dest_row_stride: int, eps: float = RMS_EPS):
    """decode_approx_pipelined for a channel shard whose outputs go into every rank's inbox (see linear_push)."""
    _cuda(x, norm_w, MinT, hist, taps8, pos)
    B, d_ch, _, Lh = hist.shape
    d_in = x.shape[1]
    assert MinT.shape == (d_ch, d_in) and MinT.is_contiguous() and hist.is_contiguous() and taps8.is_contiguous()
    rc = _lib.load().stu_decode_approx_push(x.data_ptr(), x.stride(0), norm_w.data_ptr(), MinT.data_ptr(),
                                            hist.data_ptr(), taps8.data_ptr(), pos.data_ptr(), dest, dest_row_stride,
                                            B, d_in, d_ch, Lh, eps, status_word(x.device).data_ptr(), _dt(x),
                                            _stream())
    _lib.check(rc, "stu_decode_approx_push")
    _count()


def peer_combine(x, inbox: int, slot_stride: int, in_row_stride: int, slots: int, flags: int, n_ranks: int,
                 epoch: int, norm_w=None, xn=None, eps: float = RMS_EPS, wait_ms: int = 0):
    """x += sum of this rank's inbox blocks once every sender has arrived; optionally xn = RMSNorm(x) * norm_w."""
    _cuda(x)
    rows, d = x.shape
    assert x.stride(1) == 1 and (norm_w is None or (xn is not None and xn.shape == x.shape and xn.stride(1) == 1))
    rc = _lib.load().stu_peer_combine(x.data_ptr(), x.stride(0), inbox, slot_stride, in_row_stride, slots, flags,
                                      n_ranks, epoch, _p(norm_w), _p(xn), xn.stride(0) if xn is not None else 0, eps,
                                      rows, d, status_word(x.device).data_ptr(), wait_ms, _dt(x), _stream())
    _lib.check(rc, "stu_peer_combine")
    _count()


def peer_exchange(xchg: int, x, src, gather: bool, slot_stride: int, norm_w=None, xn=None, eps: float = RMS_EPS,
                  wait_ms: int = 0):
    """One exchange of a tensor-parallel token step in one launch: src (this rank's rows) into every rank's inbox,
    wait for the other ranks' rows, x += their sum, optionally xn = RMSNorm(x) * norm_w (peer.PeerExchange.exchange)."""
    _cuda(x, src)
    rows, d = x.shape
    assert src.shape[0] == rows and x.stride(1) == 1 and src.stride(1) == 1
    assert norm_w is None or (xn is not None and xn.shape == x.shape and xn.stride(1) == 1)
    rc = _lib.load().stu_peer_exchange(xchg, x.data_ptr(), x.stride(0), src.data_ptr(), src.stride(0), src.shape[1],
                                       int(gather), slot_stride, _p(norm_w), _p(xn),
                                       xn.stride(0) if xn is not None else 0, eps, rows, d,
                                       status_word(x.device).data_ptr(), wait_ms, _dt(x), _stream())
    _lib.check(rc, "stu_peer_exchange")
    _count()


def decode_approx_pipelined(x, norm_w, MinT, hist, taps8, pos, out, eps: float = RMS_EPS, add_residual: bool = True,
                            flags: int = 0):
    """The fused decode step of an approx STU layer (or of a channel shard: MinT [d_ch, d_in], add_residual=False) as
    the bulk-copy pipeline kernel: bf16, every sequence at the same position."""
    _cuda(x, norm_w, MinT, hist, taps8, pos, out)
    B, dch, _, Lh = hist.shape
    d_in = x.shape[1]
    assert x.shape[0] == B and MinT.shape == (dch, d_in) and out.shape == (B, dch) and x.stride(1) == 1
    assert out.stride(1) == 1 and taps8.shape == (8, dch, Lh + 8) and pos.dtype == torch.int32 and pos.is_contiguous()
    assert hist.is_contiguous() and taps8.is_contiguous() and x.data_ptr() != out.data_ptr()
    rc = _lib.load().stu_decode_approx_pipelined(x.data_ptr(), x.stride(0), norm_w.data_ptr(), MinT.data_ptr(),
                                                 hist.data_ptr(), taps8.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                                 out.stride(0), B, d_in, dch, Lh, eps, int(add_residual),
                                                 status_word(x.device).data_ptr(), _dt(x) | flags, _stream())
    _lib.check(rc, "stu_decode_approx_pipelined")
    _count()
    return out


def block_step_workspace(d: int, I: int, device) -> torch.Tensor:
    """Zeroed workspace of block_decode_step for one layer's cache (partial sums carried from one token step to the
    next, grid-barrier words, the step's intermediate rows)."""
    n = int(_lib.load().stu_block_step_workspace_bytes(d, I))
    return torch.zeros((n + 255) // 256 * 256, dtype=torch.uint8, device=device)


def block_decode_step(x, stu_norm_w, MinT, hist, taps8, pos, mlp_norm_w, Wg, Wu, Wd, out, workspace, mode: int,
                      eps_stu: float = RMS_EPS, eps_mlp: float = RMS_EPS):
    """One cached token step of a whole approx STU layer (STU sub-layer + MLP, both residuals) in one persistent
    kernel; mode 1 only prepares the partial sums of the current position (first step after a prefill)."""
    _cuda(x, stu_norm_w, MinT, hist, taps8, pos, mlp_norm_w, Wg, Wu, Wd, out, workspace)
    B, d, _, Lh = hist.shape
    I = Wg.shape[0]
    assert x.shape == (B, d) and out.shape == (B, d) and x.stride(1) == 1 and out.stride(1) == 1
    assert MinT.shape == (d, d) and Wg.shape == (I, d) and Wu.shape == (I, d) and Wd.shape == (d, I)
    assert all(w.is_contiguous() for w in (MinT, Wg, Wu, Wd, hist, taps8, pos)) and pos.dtype == torch.int32
    rc = _lib.load().stu_block_decode_step(x.data_ptr(), x.stride(0), stu_norm_w.data_ptr(), MinT.data_ptr(),
                                           hist.data_ptr(), taps8.data_ptr(), pos.data_ptr(), mlp_norm_w.data_ptr(),
                                           Wg.data_ptr(), Wu.data_ptr(), Wd.data_ptr(), out.data_ptr(), out.stride(0),
                                           B, d, I, Lh, eps_stu, eps_mlp, workspace.data_ptr(), workspace.numel(), mode,
                                           status_word(x.device).data_ptr(), _dt(x), _stream())
    _lib.check(rc, "stu_block_decode_step")
    _count()
    return out


def to_history(x, hist, t0: int):
    """x [B,T,d] -> hist[b][c][t&1][t>>1] for t in [t0, t0+T)."""
    _cuda(x, hist)
    B, T, d = x.shape
    assert hist.is_contiguous() and hist.shape[:3] == (B, d, 2) and x.stride(2) == 1
    rc = _lib.load().stu_to_history(x.data_ptr(), x.stride(0), x.stride(1), hist.data_ptr(), B, d, hist.shape[3], t0,
                                    t0 + T, _dt(x), _stream())
    _lib.check(rc, "stu_to_history")
    _count()


def toeplitz(phi, k: int, out):
    """out [3,S,S] <- the three Toeplitz matrices (even / odd->parity 1 / odd->parity 0) of filter column k."""
    _cuda(phi, out)
    L, K = phi.shape
    assert phi.is_contiguous() and out.is_contiguous() and out.shape[0] == 3 and out.shape[1] == out.shape[2]
    col = phi[:, k]
    rc = _lib.load().stu_toeplitz(col.data_ptr(), K, L, out.data_ptr(), out.shape[1], out.shape[2], _dt(phi), _stream())
    _lib.check(rc, "stu_toeplitz")
    _count()


def full_combine(E, Q, U, B: int, d: int, K: int, k: int, both_signs: bool, t0: int, t_end: int):
    _cuda(E, Q, U)
    assert E.shape == Q.shape and E.is_contiguous() and Q.is_contiguous() and U.stride(1) == 1
    rc = _lib.load().stu_full_combine(E.data_ptr(), Q.data_ptr(), E.shape[1], U.data_ptr(), U.stride(0), B, d, K, k,
                                      int(both_signs), t0, t_end, _dt(E), _stream())
    _lib.check(rc, "stu_full_combine")
    _count()


def full_decode_prepare(x2d, hist, phi, pos, PhiT):
    _cuda(x2d, hist, phi, pos, PhiT)
    B, d, _, Lh = hist.shape
    L, K = phi.shape
    assert PhiT.shape == (2 * K, Lh) and PhiT.is_contiguous() and phi.is_contiguous() and x2d.stride(1) == 1
    rc = _lib.load().stu_full_decode_prepare(x2d.data_ptr(), x2d.stride(0), hist.data_ptr(), phi.data_ptr(),
                                             pos.data_ptr(), PhiT.data_ptr(), B, d, K, L, Lh,
                                             status_word(x2d.device).data_ptr(), _dt(x2d), _stream())
    _lib.check(rc, "stu_full_decode_prepare")
    _count()


def full_decode_combine(G, pos, U, B: int, d: int, K: int, both_signs: bool, Lh: int, advance: bool = True):
    _cuda(G, pos, U)
    assert G.stride(1) == 1 and U.is_contiguous()
    rc = _lib.load().stu_full_decode_combine(G.data_ptr(), G.stride(0), pos.data_ptr(), U.data_ptr(), B, d, K,
                                             int(both_signs), Lh, int(advance), _dt(G), _stream())
    _lib.check(rc, "stu_full_decode_combine")
    _count(2 if advance else 1)


def lds_final_state(hist, h, A32, B32, T: int):
    """h[b,i,:] <- LDS state after the T inputs stored in hist [B,d,2,Lh] (float64 state [B,d,D])."""
    _cuda(hist, h, A32, B32)
    B, d, _, Lh = hist.shape
    assert hist.is_contiguous() and h.is_contiguous() and h.dtype == torch.float64 and A32.dtype == torch.float64
    rc = _lib.load().stu_lds_final_state(hist.data_ptr(), h.data_ptr(), A32.data_ptr(), B32.data_ptr(), B, d, Lh, T,
                                         h.shape[2], _dt(hist), _stream())
    _lib.check(rc, "stu_lds_final_state")
    _count()


def lds_chunk_scan(x, A64, B64, Vs, Z, hfin, Ck: int, unit_b: bool = False):
    """Chunked scan of the distilled LDS over x [B,T,d]: float64 recurrence per (sequence, channel); at every chunk
    start the carried state goes, rotated into the balanced basis (Vs [D,R] float64), into the leading columns of
    Z [B, nchunks, d, KZ], the chunk's inputs into the trailing Ck columns; hfin [B,d,D] float64 = the final state.
    unit_b: the caller has checked that every entry of B64 is exactly 1 (B*x is then x, bit for bit)."""
    _cuda(x, A64, B64, Vs, Z, hfin)
    B, T, d = x.shape
    D, R = Vs.shape
    assert x.stride(2) == 1 and Z.is_contiguous() and hfin.is_contiguous() and Vs.is_contiguous()
    assert A64.dtype == torch.float64 and Vs.dtype == torch.float64 and hfin.dtype == torch.float64
    KZ = (3 * R if x.dtype == torch.bfloat16 else R) + Ck
    assert Z.shape == (B, (T + Ck - 1) // Ck, d, KZ) and Z.dtype == x.dtype and hfin.shape == (B, d, D)
    rc = _lib.load().stu_lds_chunk_scan(x.data_ptr(), x.stride(0), x.stride(1), A64.data_ptr(), B64.data_ptr(),
                                        Vs.data_ptr(), Z.data_ptr(), hfin.data_ptr(), B, d, T, D, R, Ck,
                                        _dt(x) | (0x1000 if unit_b else 0), _stream())
    _lib.check(rc, "stu_lds_chunk_scan")
    _count()


def lds_chunk_features(W, Zb, U2, d: int, Ck: int, F: int):
    """U2[c*Ck + tau, f*d + i] = sum_k W[tau*F + f, k] * Zb[c*d + i, k]: the LDS features of one sequence, one GEMM over
    all its chunks, scattered straight into the [tokens, F*d] operand of the contraction with M."""
    _cuda(W, Zb, U2)
    Mrows, KZ = W.shape
    N = Zb.shape[0]
    assert Mrows == Ck * F and Zb.shape[1] == KZ and W.is_contiguous() and Zb.is_contiguous() and U2.is_contiguous()
    assert N % d == 0 and U2.shape == (N // d * Ck, F * d) and U2.dtype == W.dtype == Zb.dtype
    status_word(W.device)
    rc = _lib.load().stu_linear(W.data_ptr(), KZ, Zb.data_ptr(), KZ, 1, None, None, Ck * F * d, U2.data_ptr(), d,
                                Mrows, N, KZ, 5, d, 0, 0, None, 0.0, _dt(W), BACKEND_AUTO, _stream())
    _lib.check(rc, "stu_linear (LDS feature scatter)")
    _count()


def lds_decode_features(x2d, h, A32, B32, C, U):
    """One recurrent LDS step for every channel: h <- A*h + B*x; U[b, f*d+i] = (h @ C)[f]."""
    _cuda(x2d, h, A32, B32, C, U)
    B, d = x2d.shape
    D, F = C.shape
    assert h.shape == (B, d, D) and h.is_contiguous() and h.dtype == torch.float64 and A32.dtype == torch.float64
    assert C.is_contiguous() and U.is_contiguous() and x2d.stride(1) == 1
    rc = _lib.load().stu_lds_decode_features(x2d.data_ptr(), x2d.stride(0), h.data_ptr(), A32.data_ptr(), B32.data_ptr(),
                                             C.data_ptr(), U.data_ptr(), B, d, D, F, _dt(x2d), _stream())
    _lib.check(rc, "stu_lds_decode_features")
    _count()


def swa_forward(qkv, k_ring, v_ring, pos, slopes, H: int, window: int, softcap: float, update_cache: bool):
    """Sliding-window attention for the Tn tokens in qkv [B,Tn,3d] against the ring cache; returns [B,Tn,d]."""
    _cuda(qkv, k_ring, v_ring, pos, slopes)
    B, Tn, d3 = qkv.shape
    d = d3 // 3
    assert qkv.is_contiguous() and slopes.dtype == torch.float32 and pos.dtype == torch.int32
    W = max(int(k_ring.shape[1]), window + 1)  # an uncached call passes a dummy ring that is never read
    assert not update_cache or (k_ring.shape == (B, W, d) and k_ring.is_contiguous() and v_ring.is_contiguous())
    out = torch.empty(B, Tn, d, dtype=qkv.dtype, device=qkv.device)
    rc = _lib.load().stu_swa_forward(qkv.data_ptr(), k_ring.data_ptr(), v_ring.data_ptr(), pos.data_ptr(),
                                     slopes.data_ptr(), out.data_ptr(), B, Tn, H, d // H, W, window, float(softcap or 0.0),
                                     int(update_cache), _dt(qkv), _stream())
    _lib.check(rc, "stu_swa_forward")
    _count(2 if update_cache else 1)
    return out


swa_tc5 = True   # switch: prefills from position 0 with head dimension 128 (bf16) use the tcgen05 attention kernel


def swa_prefill_tc5_supported(qkv, H: int, t0: int) -> bool:
    d = qkv.shape[2] // 3
    return swa_tc5 and qkv.dtype == torch.bfloat16 and d // H == 128 and t0 == 0 and qkv.shape[1] >= 128


def swa_prefill_tc5(qkv, k_ring, v_ring, pos, slopes, H: int, window: int, softcap: float, update_cache: bool):
    """swa_forward for a prefill that starts at position 0 (bf16, head dimension 128) on the tcgen05 tensor cores."""
    _cuda(qkv, k_ring, v_ring, pos, slopes)
    B, Tn, d3 = qkv.shape
    d = d3 // 3
    assert qkv.is_contiguous() and slopes.dtype == torch.float32 and pos.dtype == torch.int32 and d // H == 128
    W = max(int(k_ring.shape[1]), window + 1)
    assert not update_cache or (k_ring.shape == (B, W, d) and k_ring.is_contiguous() and v_ring.is_contiguous())
    lib = _lib.load()
    vt = torch.empty(lib.stu_swa_prefill_scratch_elems(B, Tn, H, 128), dtype=qkv.dtype, device=qkv.device)
    out = torch.empty(B, Tn, d, dtype=qkv.dtype, device=qkv.device)
    rc = lib.stu_swa_prefill_tc5(qkv.data_ptr(), vt.data_ptr(), k_ring.data_ptr(), v_ring.data_ptr(), pos.data_ptr(),
                                 slopes.data_ptr(), out.data_ptr(), B, Tn, H, 128, W, window, float(softcap or 0.0),
                                 int(update_cache), status_word(qkv.device).data_ptr(), _dt(qkv), _stream())
    _lib.check(rc, "stu_swa_prefill_tc5")
    _count(3 if update_cache else 2)
    return out


def sample(logits, temperature: float, top_k: Optional[int], top_p: Optional[float], do_sample: bool,
           uniforms: Optional[torch.Tensor], out: torch.Tensor, out_stride: int = 1):
    """Pick one token per row of logits [B,V]; writes int64 ids to out[b*out_stride]."""
    _cuda(logits, uniforms, out)
    B, V = logits.shape
    assert logits.stride(1) == 1 and out.dtype == torch.int64
    rc = _lib.load().stu_sample(logits.data_ptr(), logits.stride(0), B, V, float(temperature), int(top_k or 0),
                                float(top_p if top_p is not None else -1.0), int(do_sample), _p(uniforms),
                                out.data_ptr(), out_stride, status_word(logits.device).data_ptr(), _dt(logits),
                                _stream())
    _lib.check(rc, "stu_sample")
    _count()
    return out
