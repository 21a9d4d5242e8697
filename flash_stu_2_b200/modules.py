"""Operators of the token loop with the reference's class names, constructor signatures and
state-dict keys (flash_stu/modules/{stu,attention,swiglu}.py), running on the CUDA kernels.

Cache entries are tuples of tensors with the batch on dim 0 (so FlashSTU._reorder_cache keeps
working): STU layers hold the projected input history, attention layers a ring of the last
window+1 keys/values.  The reference's STU layers hold no cache at all (layers/stu_layer.py:99-119);
the cached decode defined here equals the reference's full-prefix forward row by row.
"""
import math
from typing import Optional, Tuple

import os

import torch
import torch.nn as nn

from . import ops
from .filters import nearest_power_of_two


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


_SM_COUNT = {}


def _sm_count(device) -> int:
    key = torch.device(device).index
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


def new_pos(batch: int, device) -> torch.Tensor:
    """[B,2] int32: column 0 = tokens cached so far, column 1 (row 0) = arrival counter used by kernels."""
    p = torch.zeros(batch, 2, dtype=torch.int32, device=device)
    p._host_t = 0
    p._uniform = True
    return p


def host_pos(pos: torch.Tensor) -> int:
    """Host-side mirror of pos[0,0]; falls back to a device read when the tensor was re-created
    (e.g. by _reorder_cache), which also re-checks whether all sequences share one position."""
    t = getattr(pos, "_host_t", None)
    if t is None:
        col = pos[:, 0].tolist()
        t = int(col[0])
        pos._host_t = t
        pos._uniform = all(v == t for v in col)
    return t


def uniform_pos(pos: torch.Tensor) -> bool:
    return getattr(pos, "_uniform", False)


class RMSNorm(nn.Module):
    """torch.nn.RMSNorm(dim, dtype) arithmetic (the reference's non-Triton branch,
    flash_stu/layers/stu_layer.py:17-36): fp32 statistics, eps = finfo(float32).eps."""

    def __init__(self, dim: int, eps: Optional[float] = None, dtype=None):
        super().__init__()
        self.eps = ops.RMS_EPS if eps is None else eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class MLP(nn.Module):
    """Gated tanh-GELU MLP, down(gelu_tanh(gate(x)) * up(x)) (flash_stu/modules/swiglu.py:4-29)."""

    def __init__(self, config, dtype=None):
        super().__init__()
        dtype = dtype if dtype is not None else config.torch_dtype
        if config.bias:
            raise NotImplementedError("bias=True has no kernel here (the reference default is bias=False)")
        self.hidden_size = config.n_embd
        self.intermediate_size = config.n_embd * config.mlp_scale
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False, dtype=dtype)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False, dtype=dtype)
        self.dropout = nn.Dropout(config.dropout)

    def apply_residual(self, xn2d: torch.Tensor, resid2d: torch.Tensor, out2d: torch.Tensor,
                       norm_w: Optional[torch.Tensor] = None, eps: float = ops.RMS_EPS, overlap: bool = False):
        """out = resid + down(gelu(gate(xn)) * up(xn)); with norm_w, xn is RMS-normalised inside the kernel.
        overlap (decode steps): both kernels fetch their weights while the kernel before them is still running."""
        ov = ops.FLAG_OVERLAP if (overlap and ops.overlap_decode) else 0
        h = ops.linear(xn2d, self.gate_proj.weight, W2=self.up_proj.weight, epilogue=ops.EPI_GELU_MUL | ov,
                       norm_w=norm_w, eps=eps)
        # early_decode: the down projection releases its successor at once, so that an STU decode kernel that follows
        # streams its history while this kernel runs (the successor's projection still waits for this output)
        ovd = ov | (ops.FLAG_EARLY_TRIGGER if (ov and ops.early_decode) else 0)
        return ops.linear(h, self.down_proj.weight, resid=resid2d, out=out2d, epilogue=ops.EPI_RESID | ovd)

    def forward(self, x):
        x2 = x.reshape(-1, x.shape[-1])
        h = ops.linear(x2, self.gate_proj.weight, W2=self.up_proj.weight, epilogue=ops.EPI_GELU_MUL)
        return ops.linear(h, self.down_proj.weight).reshape(x.shape)


class STU(nn.Module):
    """Spectral transform unit (flash_stu/modules/stu.py:12-120), approx and full variants on CUDA kernels.

    forward(x) returns the operator output like the reference.  Layers call `add_to_residual`,
    which also maintains the decode cache: entry = (hist [B,d,2,Lh], pos [B,2])."""

    def __init__(self, config, phi, n, feature_dim=None) -> None:
        super().__init__()
        self.config = config
        self.register_buffer("phi", phi, persistent=False)
        self.n = n
        self.K = config.num_eigh
        self.d_in = feature_dim if feature_dim is not None else config.n_embd
        self.d_out = self.d_in
        self.use_hankel_L = config.use_hankel_L
        self.use_approx = config.use_approx
        # block-diagonal tiling of the approx variant (flash_stu/modules/stu.py:123-191): only the diagonal
        # tile x tile blocks of M_inputs take part; the full variant ignores the switch, as the reference does
        self.tile = None
        if self.use_approx and (getattr(config, "d_in_tile", None) is not None
                                or getattr(config, "d_out_tile", None) is not None):
            tile = min(config.d_in_tile or self.d_in, config.d_out_tile or self.d_out)
            if tile < self.d_in:
                self.tile = int(tile)
        dt = config.torch_dtype
        if self.use_approx:
            self.M_inputs = nn.Parameter(torch.empty(self.d_in, self.d_out, dtype=dt))
            self.M_filters = nn.Parameter(torch.empty(self.K, self.d_in, dtype=dt))
        else:
            self.M_phi_plus = nn.Parameter(torch.empty(self.K, self.d_in, self.d_out, dtype=dt))
            if not self.use_hankel_L:
                self.M_phi_minus = nn.Parameter(torch.empty(self.K, self.d_in, self.d_out, dtype=dt))
        self._prep_key = None
        self._prep = None
        # optional cap on the positions a cache (and the tap tables) are laid out for: a model whose filters span
        # 32768 positions but that will only ever see 9216 keeps 9216-position histories (config.cache_len)
        self.cache_len = getattr(config, "cache_len", None)

    # ---- derived, cached per parameter version: M_inputs^T (K-major rows) and the even-tap table
    @property
    def seq_len(self) -> int:
        return self.phi.shape[0]

    @property
    def capacity(self) -> int:
        """Positions this operator can hold: seq_len (the filters have seq_len taps), or config.cache_len if smaller."""
        return min(self.seq_len, self.cache_len) if self.cache_len else self.seq_len

    @property
    def Lh(self) -> int:
        return _round_up((self.capacity + 1) // 2, 8)

    def prepared(self):
        if not self.use_approx:
            return self.prepared_full()
        key = (self.M_inputs._version, self.M_filters._version, self.phi._version, self.M_inputs.data_ptr(),
               self.M_filters.data_ptr(), self.phi.data_ptr())
        if self._prep_key != key:
            with torch.no_grad():
                # only the taps of positions a cache can hold are ever used
                phi = self.phi[:self.capacity].to(self.M_filters.dtype).contiguous()
                Min = self.M_inputs.detach()
                if self.tile is not None:
                    # tiling: x_tile @ M_inputs[i:e, i:e] per diagonal block == x @ (M_inputs with the off-diagonal
                    # blocks zeroed); the zeros add nothing to the fp32 sums
                    blk = torch.arange(self.d_in, device=Min.device) // self.tile
                    Min = Min * (blk[:, None] == blk[None, :]).to(Min.dtype)
                MinT = Min.t().contiguous()
                # fp = phi @ M_filters, rounded to the model dtype as in the reference (stu.py:88)
                fp = ops.linear(phi, self.M_filters.detach(), transposed_weight=True, backend=ops.BACKEND_SIMT)
                if self.use_hankel_L:
                    # single branch (stu_utils.py:229-246): y[t] = sum over ALL taps.  Even taps act on the same
                    # time parity, odd taps on the other one a step earlier; the kernels return twice an even-tap
                    # sum, so both tables are halved (exact) and the odd taps are stored at even positions.
                    half = (fp.float() * 0.5).to(fp.dtype)
                    taps = ops.taps_even(half, self.Lh)
                    self._taps_odd = ops.taps_even(half[1:].contiguous(), self.Lh)
                    taps8 = None
                else:
                    taps = ops.taps_even(fp, self.Lh)
                    taps8 = ops.taps_rev8(taps) if taps.dtype == torch.bfloat16 else None
            self._prep, self._prep_key = (MinT, taps, taps8), key
        return self._prep

    def prepared_full(self):
        """(phi [L,K] contiguous in the model dtype, Mcat [d_out, nsign*K*d_in]): the two M_phi tensors as one
        K-major weight whose column order (sign, k, i) matches the U operand the kernels build."""
        mats = [self.M_phi_plus] + ([] if self.use_hankel_L else [self.M_phi_minus])
        key = tuple(m._version for m in mats) + tuple(m.data_ptr() for m in mats) + (self.phi._version, self.phi.data_ptr())
        if self._prep_key != key:
            with torch.no_grad():
                phi = self.phi.to(self.M_phi_plus.dtype).contiguous()
                Mcat = torch.cat([m.detach().reshape(self.K * self.d_in, self.d_out) for m in mats], dim=0).t().contiguous()
            self._prep, self._prep_key = (phi, Mcat), key
        return self._prep

    @property
    def param_dtype(self):
        return (self.M_inputs if self.use_approx else self.M_phi_plus).dtype

    def new_cache(self, batch: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        hist = torch.zeros(batch, self.d_in, 2, self.Lh, dtype=self.param_dtype, device=device)
        return hist, new_pos(batch, device)

    # ------------------------------------------------------------------ full variant
    def full_forward(self, xn: torch.Tensor, resid: Optional[torch.Tensor], out: torch.Tensor, entry=None,
                     use_cache: bool = False):
        """out[B,T,d_out] = (resid +) sum_k U+[..,k,:] @ M_phi_plus[k] + U-[..,k,:] @ M_phi_minus[k] for the T new
        positions of xn [B,T,d_in]; the cache holds the history of xn."""
        B, T, d = xn.shape
        phi, Mcat = self.prepared_full()
        K, nsign = self.K, (1 if self.use_hankel_L else 2)
        t0 = 0
        if entry is not None:
            hist, pos = entry
            t0 = host_pos(pos)
        elif use_cache:
            hist, pos = self.new_cache(B, xn.device)
        else:
            pos = None
            hist = torch.zeros(B, d, 2, _round_up((T + 1) // 2, 8), dtype=xn.dtype, device=xn.device)
        if t0 + T > self.capacity:
            raise ValueError(f"sequence position {t0 + T} exceeds the capacity {self.capacity} (seq_len={self.seq_len}: "
                             f"the filters have seq_len taps; cache_len={self.cache_len})")
        Lh = hist.shape[3]
        ops.to_history(xn, hist, t0)
        S = _round_up((t0 + T + 1) // 2, 8)
        rows = hist.view(B * d * 2, Lh)[:, :S]
        even_in = hist.view(B * d, 2, Lh)[:, 0, :S]
        odd_in = hist.view(B * d, 2, Lh)[:, 1, :S]
        Tz = torch.empty(3, S, S, dtype=xn.dtype, device=xn.device)
        E = torch.empty(B * d * 2, S, dtype=xn.dtype, device=xn.device)
        Q = torch.empty(B * d * 2, S, dtype=xn.dtype, device=xn.device)
        U = torch.empty(B * T, nsign * K * d, dtype=xn.dtype, device=xn.device)
        causal = ops.EPI_STORE | ops.EPI_FLAG_CAUSAL
        for k in range(K):
            ops.toeplitz(phi, k, Tz)
            ops.linear(rows, Tz[0], out=E, epilogue=causal)
            ops.linear(even_in, Tz[1], out=Q.view(B * d, 2, S)[:, 1], epilogue=causal)  # parity-1 outputs
            ops.linear(odd_in, Tz[2], out=Q.view(B * d, 2, S)[:, 0], epilogue=causal)   # parity-0 outputs
            ops.full_combine(E, Q, U, B, d, K, k, nsign == 2, t0, t0 + T)
        o2 = out.view(B * T, self.d_out)
        if resid is not None:
            ops.linear(U, Mcat, resid=resid.view(B * T, self.d_out), out=o2, epilogue=ops.EPI_RESID)
        else:
            ops.linear(U, Mcat, out=o2)
        if pos is not None:
            pos[:, 0] += T
            pos._host_t = t0 + T
            return hist, pos
        return None

    def full_decode_step(self, xn2d: torch.Tensor, resid2d: torch.Tensor, out2d: torch.Tensor, entry):
        """One cached token of the full variant: out = resid + STU(xn) at the cached position."""
        hist, pos = entry
        phi, Mcat = self.prepared_full()
        B, d, _, Lh = hist.shape
        K, nsign = self.K, (1 if self.use_hankel_L else 2)
        t = host_pos(pos)
        if t + 1 > self.capacity:
            raise ValueError(f"sequence position {t + 1} exceeds the capacity {self.capacity} (seq_len={self.seq_len})")
        key = (B, xn2d.device, xn2d.dtype)
        if getattr(self, "_dec_scratch_key", None) != key:
            self._dec_scratch = (torch.zeros(2 * K, Lh, dtype=xn2d.dtype, device=xn2d.device),
                                 torch.empty(B * d * 2, 2 * K, dtype=xn2d.dtype, device=xn2d.device),
                                 torch.empty(B, nsign * K * d, dtype=xn2d.dtype, device=xn2d.device))
            self._dec_scratch_key = key
        PhiT, G, U = self._dec_scratch
        ops.full_decode_prepare(xn2d, hist, phi, pos, PhiT)
        ops.linear(hist.view(B * d * 2, Lh), PhiT, out=G)
        ops.full_decode_combine(G, pos, U, B, d, K, nsign == 2, Lh, advance=True)
        ops.linear(U, Mcat, resid=resid2d, out=out2d, epilogue=ops.EPI_RESID)
        pos._host_t = t + 1
        return hist, pos

    def add_to_residual(self, xn: torch.Tensor, x: torch.Tensor, entry=None, use_cache: bool = False):
        """x += STU(xn) for xn, x [B,T,d] (x contiguous).  Returns the cache entry when use_cache."""
        if not self.use_approx:
            return self.full_forward(xn, x, x, entry, use_cache)
        B, T, d = xn.shape
        MinT, taps, taps8 = self.prepared()
        t0 = 0
        if entry is not None:
            hist, pos = entry
            t0 = host_pos(pos)
        elif use_cache:
            hist, pos = self.new_cache(B, xn.device)
        else:
            pos = None
            hist = torch.empty(B, d, 2, self.Lh, dtype=xn.dtype, device=xn.device)
        if t0 + T > self.capacity:
            raise ValueError(f"sequence position {t0 + T} exceeds the capacity {self.capacity} (seq_len={self.seq_len}: "
                             f"the filters have seq_len taps; cache_len={self.cache_len})")
        Lh = hist.shape[3]
        ops.linear(xn.reshape(B * T, d), MinT, out=hist, epilogue=ops.EPI_HIST, hist_T=T, hist_t0=t0, hist_Lh=Lh)
        yT = torch.empty(B, d, 2, _round_up((t0 + T + 1) // 2, 8), dtype=xn.dtype, device=xn.device)
        if STU.tensor_core_conv and STU.tcgen05_conv and taps8 is not None and ops.conv_prefill_tc5_supported(hist, x):
            ops.conv_prefill_approx_tc5(hist, taps8, yT, x, t0, t0 + T)
        else:
            ops.conv_prefill_approx(hist, taps, yT, x, t0, t0 + T,
                                    use_tensor_cores=(xn.dtype == torch.bfloat16 and STU.tensor_core_conv))
        if self.use_hankel_L:
            # odd taps: the even-tap sum of the odd-tap table at time t - 1 goes to output row t
            s0, s1 = max(t0 - 1, 0), t0 + T - 1
            if s1 > s0:
                r0 = s0 + 1 - t0
                ops.conv_prefill_approx(hist, self._taps_odd, yT, x[:, r0:r0 + (s1 - s0)], s0, s1,
                                        use_tensor_cores=(xn.dtype == torch.bfloat16 and STU.tensor_core_conv))
        if pos is not None:
            pos[:, 0] += T
            pos._host_t = t0 + T
            return hist, pos
        return None

    tensor_core_conv = True    # class switches used by tests to compare the tensor-core and CUDA-core kernels
    tcgen05_conv = True        # ... and, of the tensor-core ones, the tcgen05 kernel against the mma.sync kernel
    tensor_core_decode = True
    shared_tap_decode = True   # batches at one common position: the kernel with 8 channels x 8 sequences per CTA
    pipelined_decode = True    # ... and, of those, the persistent bulk-copy pipeline kernel
    # from this batch size on, the token's projection is one GEMM of its own (STU_B200_PROJECTED_MIN_BATCH overrides)
    projected_decode_min_batch = int(os.environ.get("STU_B200_PROJECTED_MIN_BATCH", "16"))

    def decode_step(self, x2d: torch.Tensor, norm_w: torch.Tensor, eps: float, entry, out2d: torch.Tensor):
        """out = x + STU(rmsnorm(x)) for one new token per sequence; appends to the cache."""
        hist, pos = entry
        MinT, taps, taps8 = self.prepared()
        t = host_pos(pos)
        if t + 1 > self.capacity:
            raise ValueError(f"sequence position {t + 1} exceeds the capacity {self.capacity} (seq_len={self.seq_len})")
        B, d, _, Lh = hist.shape
        if self.use_hankel_L:
            # single branch: a one-position prefill (its position is a host argument: not replayable from a graph)
            out2d.copy_(x2d)
            self.add_to_residual(ops.rmsnorm(x2d, norm_w, eps).view(B, 1, d), out2d.view(B, 1, d), entry, True)
            return hist, pos
        # rows of 8 sequences x 8 channels, slices of 256 cached positions per parity: the pipeline kernel pays a
        # per-row projection latency, which only long rows (or one row per SM) hide
        rows, nsl = (B + 7) // 8 * (d // 8), ((t >> 1) + 255) // 256
        if (B >= STU.projected_decode_min_batch and STU.pipelined_decode and STU.tensor_core_decode
                and STU.shared_tap_decode and taps8 is not None and uniform_pos(pos) and d % 8 == 0
                and x2d.shape[1] % 8 == 0):
            # larger batches: the projection of the whole batch as one GEMM, then the pipeline kernel as a pure stream
            if ops.can_fuse_norm(B, d, x2d.shape[1], ops.EPI_STORE, x2d.dtype):
                xp = ops.linear(x2d, MinT, norm_w=norm_w, eps=eps)
            else:
                # token step: MinT is nobody's output here, so its tiles may be requested while the norm kernel runs
                xp = ops.linear(ops.rmsnorm(x2d, norm_w, eps), MinT,
                                epilogue=ops.EPI_STORE | (ops.FLAG_OVERLAP if ops.overlap_decode else 0))
            ops.decode_approx_projected(x2d, xp, hist, taps8, pos, out2d)
        elif (STU.pipelined_decode and STU.tensor_core_decode and STU.shared_tap_decode and taps8 is not None
                and uniform_pos(pos) and d % 8 == 0 and x2d.shape[1] % 8 == 0
                and (nsl >= 8 or rows <= _sm_count(x2d.device))):
            # batch at one common position: the bulk-copy pipeline kernel
            ops.decode_approx_pipelined(x2d, norm_w, MinT, hist, taps8, pos, out2d, eps,
                                        flags=(ops.FLAG_EARLY_TRIGGER if ops.overlap_decode else 0) |
                                              (ops.FLAG_OVERLAP if (ops.overlap_decode and ops.early_decode) else 0))
        else:
            ops.decode_approx(x2d, norm_w, MinT, hist, taps, pos, out2d, eps,
                              taps8=taps8 if STU.tensor_core_decode else None,
                              flags=(ops.FLAG_EARLY_TRIGGER if ops.overlap_decode else 0) |
                                    (ops.FLAG_UNIFORM_POS if (uniform_pos(pos) and STU.shared_tap_decode) else 0))
        pos._host_t = t + 1
        return hist, pos

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.use_approx:
            y = torch.empty(*x.shape[:2], self.d_out, dtype=x.dtype, device=x.device)
            self.full_forward(x.contiguous(), None, y)
            return y
        y = torch.zeros_like(x, memory_format=torch.contiguous_format)
        self.add_to_residual(x.contiguous(), y)
        return y


class Attention(nn.Module):
    """Causal sliding-window multi-head attention with ALiBi slopes (x0.25) and tanh soft-capping
    (flash_stu/modules/attention.py:16-105).  Cache entry = (k_ring [B,W,d], v_ring [B,W,d], pos [B,2])
    with W = window+1 slots, exact because older keys can never be attended."""

    def __init__(self, config):
        super().__init__()
        assert config.n_embd % config.n_heads == 0
        if config.bias:
            raise NotImplementedError("bias=True has no kernel here (the reference default is bias=False)")
        self.n_heads = config.n_heads
        self.head_dim = config.n_embd // config.n_heads
        if self.head_dim > 128:
            raise NotImplementedError("head_dim > 128 has no kernel here")
        self.bsz = config.bsz
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=False, dtype=config.torch_dtype)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=False, dtype=config.torch_dtype)
        self.c_proj.SCALE_INIT = 1
        self.dropout = config.dropout
        self.resid_dropout = nn.Dropout(self.dropout)
        self.register_buffer("alibi_slopes", self._get_alibi_slopes(self.n_heads), persistent=False)
        ws = config.window_size
        self.window_size = ws
        self.window = int(ws[0] if isinstance(ws, (tuple, list)) else ws)
        self.softcap = config.softcap

    @staticmethod
    def _generate_slopes(n: int):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]

    def _get_alibi_slopes(self, n_heads: int, interpolation_factor: float = 0.25):
        if math.log2(n_heads).is_integer():
            slopes = self._generate_slopes(n_heads)
        else:
            n = nearest_power_of_two(n_heads, round_up=False)
            slopes = self._generate_slopes(n) + self._generate_slopes(2 * n)[0::2][: n_heads - n]
        return torch.tensor(slopes, dtype=torch.float32) * interpolation_factor

    def new_cache(self, batch: int, device):
        d = self.n_heads * self.head_dim
        W = self.window + 1
        dt = self.c_attn.weight.dtype
        return (torch.zeros(batch, W, d, dtype=dt, device=device), torch.zeros(batch, W, d, dtype=dt, device=device),
                new_pos(batch, device))

    def attend(self, xn: torch.Tensor, entry=None, use_cache: bool = False, norm_w=None, eps: float = 0.0):
        """Heads merged, before c_proj: returns (y [B,T,d], entry).  With norm_w, xn is the un-normalised layer input
        and the RMSNorm is applied inside the c_attn kernel (token steps)."""
        B, T, d = xn.shape
        if norm_w is not None:
            qkv = ops.linear(xn.reshape(B * T, d), self.c_attn.weight, norm_w=norm_w, eps=eps).view(B, T, 3 * d)
        else:
            ov = ops.FLAG_OVERLAP if (T == 1 and ops.overlap_decode) else 0   # token step: weights fetched early
            qkv = ops.linear(xn.reshape(B * T, d), self.c_attn.weight, epilogue=ops.EPI_STORE | ov).view(B, T, 3 * d)
        if entry is None and use_cache:
            entry = self.new_cache(B, xn.device)
        if entry is not None:
            k_ring, v_ring, pos = entry
            t0 = host_pos(pos)
            attend = ops.swa_prefill_tc5 if ops.swa_prefill_tc5_supported(qkv, self.n_heads, t0) else ops.swa_forward
            y = attend(qkv, k_ring, v_ring, pos, self.alibi_slopes, self.n_heads, self.window, self.softcap,
                       update_cache=True)
            pos._host_t = t0 + T
            return y, entry
        dummy = torch.zeros(1, 1, 1, dtype=xn.dtype, device=xn.device)
        attend = ops.swa_prefill_tc5 if ops.swa_prefill_tc5_supported(qkv, self.n_heads, 0) else ops.swa_forward
        y = attend(qkv, dummy, dummy, new_pos(B, xn.device), self.alibi_slopes, self.n_heads, self.window,
                   self.softcap, update_cache=False)
        return y, None

    def forward(self, x, past_key_value=None, use_cache=True):
        B, T, d = x.shape
        y, entry = self.attend(x.contiguous(), past_key_value, use_cache)
        y = ops.linear(y.reshape(B * T, d), self.c_proj.weight).view(B, T, d)
        if use_cache:
            return y, entry
        return y
