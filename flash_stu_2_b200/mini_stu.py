"""MiniSTU (mini_stu/stu.py:12-275): the bare full-variant spectral transform with its own input and
output widths, same constructor signature and parameter names (M_phi_plus, M_phi_minus) as the reference.
The spectral backend runs on the kernels of the full STU variant; the distilled-LDS backend and the
optional post-MLP are not built here yet and raise."""
from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn as nn

from .filters import get_spectral_filters, nearest_power_of_two
from .modules import STU


class MiniSTU(nn.Module):
    def __init__(
        self,
        seq_len: int,
        num_filters: int,
        input_dim: int,
        output_dim: int,
        use_hankel_L: bool = False,
        use_flash_fft: bool = True,
        use_mlp: bool = False,
        mlp_hidden_dim: Optional[int] = None,
        mlp_num_layers: int = 2,
        mlp_dropout: float = 0.0,
        mlp_activation: str = "relu",
        dtype: torch.dtype = torch.float32,
        device: Optional[torch.device] = None,
        precomputed_filters: Optional[torch.Tensor] = None,
        backend: str = "spectral",
    ):
        super().__init__()
        if backend != "spectral":
            raise NotImplementedError("MiniSTU(backend='lds') has no kernel here yet")
        if use_mlp:
            raise NotImplementedError("MiniSTU(use_mlp=True) (plain post-MLP) is not part of this implementation")
        self.seq_len, self.num_filters = seq_len, num_filters
        self.input_dim, self.output_dim = input_dim, output_dim
        self.use_hankel_L, self.use_mlp, self.dtype, self.backend = use_hankel_L, use_mlp, dtype, backend
        self.device = device or torch.device("cpu")
        if precomputed_filters is not None:
            phi = precomputed_filters.to(self.device, dtype)
        else:
            phi = get_spectral_filters(seq_len, num_filters, use_hankel_L, self.device, dtype)
        self.register_buffer("phi", phi, persistent=False)
        self.n = nearest_power_of_two(seq_len * 2 - 1, round_up=True)
        scale = (num_filters * input_dim) ** -0.5
        self.M_phi_plus = nn.Parameter(torch.randn(num_filters, input_dim, output_dim, dtype=dtype, device=self.device) * scale)
        if not use_hankel_L:
            self.M_phi_minus = nn.Parameter(
                torch.randn(num_filters, input_dim, output_dim, dtype=dtype, device=self.device) * scale)
        self.mlp = None
        cfg = SimpleNamespace(num_eigh=num_filters, n_embd=input_dim, use_hankel_L=use_hankel_L, use_approx=False,
                              torch_dtype=dtype, d_in_tile=None, d_out_tile=None)
        inner = STU(cfg, phi, self.n)
        inner.d_out = output_dim
        # the operator shares this module's parameters; it is kept out of the module tree so that the
        # state dict has exactly the reference's keys
        del inner.M_phi_plus
        inner.M_phi_plus = self.M_phi_plus
        if not use_hankel_L:
            del inner.M_phi_minus
            inner.M_phi_minus = self.M_phi_minus
        object.__setattr__(self, "_op", inner)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 2:
            x = x.unsqueeze(0)
        assert x.dim() == 3, f"Expected x with shape [B, L, I] or [L, I]; got {tuple(x.shape)}"
        x = x.to(self.M_phi_plus.dtype)
        op = self._op
        if op.phi.device != self.phi.device:
            op.phi = self.phi
        return op(x)

    def get_num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
