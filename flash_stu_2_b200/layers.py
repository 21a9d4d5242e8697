"""Residual layers (flash_stu/layers/stu_layer.py:28-119, flash_stu/layers/attention_layer.py:29-87):
x += op(norm(x)); x += mlp(norm(x)), in place on the caller's tensor as in the reference."""
import torch
import torch.nn as nn

from . import ops
from .modules import MLP, STU, Attention, RMSNorm


def _inplace_target(x: torch.Tensor):
    """The kernels write a contiguous [B,T,d] buffer; a strided caller tensor is copied back at the end."""
    return x if x.is_contiguous() else x.contiguous()


class STULayer(nn.Module):
    def __init__(self, config, phi, n):
        super().__init__()
        self.config = config
        self.stu_norm = RMSNorm(config.n_embd, dtype=config.torch_dtype)
        # STU sandwich (flash_stu/layers/stu_layer.py:39-63,83-88): up-projection, SiLU, the STU on the hidden width,
        # down-projection
        self.stu_mlp_enabled = bool(config.stu_enable_mlp_sandwich)
        if self.stu_mlp_enabled:
            if config.bias:
                raise NotImplementedError("bias=True has no kernel here (the reference default is bias=False)")
            self.stu_mlp_hidden_size = (config.stu_mlp_hidden_size if config.stu_mlp_hidden_size is not None
                                        else config.intermediate_size)
            self.stu_mlp_in_proj = nn.Linear(config.n_embd, self.stu_mlp_hidden_size, bias=False,
                                             dtype=config.torch_dtype)
            self.stu_mlp_act = nn.SiLU()
            self.stu = STU(config, phi, n, feature_dim=self.stu_mlp_hidden_size)
            self.stu_mlp_out_proj = nn.Linear(self.stu_mlp_hidden_size, config.n_embd, bias=False,
                                              dtype=config.torch_dtype)
        else:
            self.stu = STU(config, phi, n)
        self.mlp_norm = RMSNorm(config.n_embd, dtype=config.torch_dtype)
        self.mlp = MLP(config, dtype=config.torch_dtype)
        self._scratch = {}

    def _fused_decode(self, x2, entry):
        """The whole token step as one persistent kernel (bf16, B <= 8, one common position).  The kernel leaves the
        history partial sums of the NEXT position in a workspace kept with the cache's position tensor; when the
        workspace holds none for the current position (first step after a prefill, a rewound or reordered cache) a
        mode-1 launch computes them first."""
        from .modules import host_pos
        hist, pos = entry
        stu = self.stu
        MinT, taps, taps8 = stu.prepared()
        B, d = x2.shape
        t = host_pos(pos)
        if t + 1 > stu.capacity:
            raise ValueError(f"sequence position {t + 1} exceeds the capacity {stu.capacity} (seq_len={stu.seq_len})")
        ahead = getattr(pos, "_ahead", None)
        if ahead is None or ahead[0].device != x2.device:
            ahead = [ops.block_step_workspace(d, self.mlp.intermediate_size, x2.device), 0 if t == 0 else -1]
            pos._ahead = ahead
        ws = ahead[0]
        args = (x2, self.stu_norm.weight, MinT, hist, taps8, pos, self.mlp_norm.weight, self.mlp.gate_proj.weight,
                self.mlp.up_proj.weight, self.mlp.down_proj.weight, x2, ws)
        if ahead[1] != t:
            ops.block_decode_step(*args, mode=1, eps_stu=self.stu_norm.eps, eps_mlp=self.mlp_norm.eps)
        ops.block_decode_step(*args, mode=0, eps_stu=self.stu_norm.eps, eps_mlp=self.mlp_norm.eps)
        ahead[1] = t + 1
        pos._host_t = t + 1
        return hist, pos

    def _sandwich(self, xc, past_key_value, use_cache):
        """x += out_proj(STU(silu(in_proj(norm(x))))) for any number of new positions; the cache holds the projected
        history of the hidden width.  Token steps on a bf16 batch at one position read their position on the device
        (the projection is a GEMM, the pipeline kernel appends and streams); other token steps are a one-position
        prefill, whose position is a host argument."""
        from .modules import host_pos, uniform_pos
        B, T, d = xc.shape
        Hs = self.stu_mlp_hidden_size
        x2 = xc.view(B * T, d)
        xn = ops.rmsnorm(x2, self.stu_norm.weight, self.stu_norm.eps)
        h = ops.linear(xn, self.stu_mlp_in_proj.weight)
        ops.bias_act(h, None, ops.ACT_SILU)
        entry = past_key_value
        taps8 = self.stu.prepared()[2] if self.stu.use_approx else None
        if (T == 1 and entry is not None and taps8 is not None and uniform_pos(entry[1]) and Hs % 8 == 0
                and STU.pipelined_decode):
            hist, pos = entry
            t = host_pos(pos)
            if t + 1 > self.stu.capacity:
                raise ValueError(f"sequence position {t + 1} exceeds the capacity {self.stu.capacity}")
            xp = ops.linear(h, self.stu.prepared()[0])
            y = torch.empty(B, Hs, dtype=xc.dtype, device=xc.device)
            ops.decode_approx_projected(None, xp, hist, taps8, pos, y, add_residual=False)
            pos._host_t = t + 1
        else:
            y3 = torch.zeros(B, T, Hs, dtype=xc.dtype, device=xc.device)
            if self.stu.use_approx:
                entry = self.stu.add_to_residual(h.view(B, T, Hs), y3, entry, use_cache)
            else:
                entry = self.stu.full_forward(h.view(B, T, Hs), None, y3, entry, use_cache)
            y = y3.view(B * T, Hs)
        ops.linear(y, self.stu_mlp_out_proj.weight, resid=x2, out=x2, epilogue=ops.EPI_RESID)
        return entry

    def _can_fuse(self, x, entry):
        from .modules import uniform_pos
        B, _, d = x.shape
        # the kernel passes the MLP weights through 32 KB shared-memory slots: 16 rows of d and 8 rows of I values
        return (ops.fused_step and self.stu.use_approx and not self.stu.use_hankel_L and x.dtype == torch.bfloat16 and B <= 8 and d % 8 == 0
                and d <= 1024 and self.mlp.intermediate_size <= 4096
                and self.mlp.intermediate_size % 8 == 0 and STU.pipelined_decode and STU.tensor_core_decode
                and STU.shared_tap_decode and uniform_pos(entry[1]))

    def _decode(self, x, entry):
        B, _, d = x.shape
        if self._can_fuse(x, entry):
            return self._fused_decode(x.view(B, d), entry)
        key = (B, x.device, x.dtype)
        if key not in self._scratch:
            self._scratch = {key: torch.empty(B, d, dtype=x.dtype, device=x.device)}
        mid = self._scratch[key]
        x2 = x.view(B, d)
        if self.stu.use_approx:
            entry = self.stu.decode_step(x2, self.stu_norm.weight, self.stu_norm.eps, entry, mid)
        else:
            xn = ops.rmsnorm(x2, self.stu_norm.weight, self.stu_norm.eps)
            entry = self.stu.full_decode_step(xn, x2, mid, entry)
        inter = self.mlp.intermediate_size
        if ops.can_fuse_norm(B, inter, d, ops.EPI_GELU_MUL, x.dtype):
            self.mlp.apply_residual(mid, mid, x2, norm_w=self.mlp_norm.weight, eps=self.mlp_norm.eps, overlap=True)
        else:
            self.mlp.apply_residual(ops.rmsnorm(mid, self.mlp_norm.weight, self.mlp_norm.eps), mid, x2, overlap=True)
        return entry

    def forward(self, x: torch.Tensor, past_key_value=None, use_cache=False):
        xc = _inplace_target(x)
        B, T, d = xc.shape
        if self.stu_mlp_enabled:
            entry = self._sandwich(xc, past_key_value, use_cache)
            x2 = xc.view(B * T, d)
            self.mlp.apply_residual(ops.rmsnorm(x2, self.mlp_norm.weight, self.mlp_norm.eps), x2, x2)
        elif T == 1 and past_key_value is not None:
            entry = self._decode(xc, past_key_value)
        else:
            xn = ops.rmsnorm(xc, self.stu_norm.weight, self.stu_norm.eps)
            entry = self.stu.add_to_residual(xn, xc, past_key_value, use_cache)
            x2 = xc.view(B * T, d)
            xn2 = ops.rmsnorm(x2, self.mlp_norm.weight, self.mlp_norm.eps)
            self.mlp.apply_residual(xn2, x2, x2)
        if xc is not x:
            x.copy_(xc)
        if use_cache:
            return x, entry
        return x


class AttentionLayer(nn.Module):
    def __init__(self, config) -> None:
        super().__init__()
        self.config = config
        self.attn_norm = RMSNorm(config.n_embd, dtype=config.torch_dtype)
        self.attn = Attention(config)
        self.mlp_norm = RMSNorm(config.n_embd, dtype=config.torch_dtype)
        self.mlp = MLP(config, dtype=config.torch_dtype)

    def forward(self, x: torch.Tensor, past_key_value=None, use_cache=True):
        xc = _inplace_target(x)
        B, T, d = xc.shape
        x2 = xc.view(B * T, d)
        if T == 1 and ops.can_fuse_norm(B, 3 * d, d, ops.EPI_STORE, x.dtype):
            y, entry = self.attn.attend(xc, past_key_value, use_cache, norm_w=self.attn_norm.weight,
                                        eps=self.attn_norm.eps)
        else:
            xn = ops.rmsnorm(xc, self.attn_norm.weight, self.attn_norm.eps)
            y, entry = self.attn.attend(xn, past_key_value, use_cache)
        ov = ops.FLAG_OVERLAP if (T == 1 and ops.overlap_decode) else 0   # token step: weights fetched early
        ops.linear(y.view(B * T, d), self.attn.c_proj.weight, resid=x2, out=x2, epilogue=ops.EPI_RESID | ov)
        inter = self.mlp.intermediate_size
        if T == 1 and ops.can_fuse_norm(B, inter, d, ops.EPI_GELU_MUL, x.dtype):
            self.mlp.apply_residual(x2, x2, x2, norm_w=self.mlp_norm.weight, eps=self.mlp_norm.eps, overlap=True)
        else:
            self.mlp.apply_residual(ops.rmsnorm(x2, self.mlp_norm.weight, self.mlp_norm.eps), x2, x2, overlap=(T == 1))
        if xc is not x:
            x.copy_(xc)
        if use_cache:
            return x, entry
        return x
