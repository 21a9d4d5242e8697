"""FlashSTUBlock: one standalone STU or attention layer (flash_stu/blocks/block.py:11-150), same two
construction modes (from a config, or from d_model / sequence_length / ... keywords)."""
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from .config import FlashSTUConfig
from .filters import get_spectral_filters, nearest_power_of_two
from .layers import AttentionLayer, STULayer


class FlashSTUBlock(nn.Module):
    def __init__(
        self,
        config: Optional[FlashSTUConfig] = None,
        phi: Optional[torch.Tensor] = None,
        n: Optional[int] = None,
        d_model: Optional[int] = None,
        sequence_length: Optional[int] = None,
        num_filters: Optional[int] = None,
        attention_window: Optional[int] = None,
        use_attention: bool = False,
        use_flash_fft: bool = True,
        attention_config: Optional[Dict[str, Any]] = None,
        n_heads: Optional[int] = None,
        mlp_scale: int = 4,
        dropout: float = 0.0,
        bias: bool = False,
        torch_dtype: torch.dtype = torch.bfloat16,
        stu_enable_mlp_sandwich: bool = False,
        stu_mlp_hidden_size: Optional[int] = None,
        **kwargs,
    ):
        super().__init__()
        if config is not None:
            self.config = config
        else:
            if d_model is None:
                raise ValueError("d_model is required when config is not provided")
            if sequence_length is None:
                raise ValueError("sequence_length is required when config is not provided")
            fields = dict(
                n_embd=d_model, seq_len=sequence_length, num_eigh=num_filters if num_filters else 24,
                window_size=attention_window if attention_window else sequence_length // 4,
                use_flash_fft=use_flash_fft, n_heads=n_heads if n_heads else max(1, d_model // 64),
                mlp_scale=mlp_scale, dropout=dropout, bias=bias, torch_dtype=torch_dtype, use_attn=use_attention,
                use_approx=kwargs.get("use_approx", True), use_hankel_L=kwargs.get("use_hankel_L", False),
                softcap=50.0, n_layers=1, bsz=1, vocab_size=1, stu_enable_mlp_sandwich=stu_enable_mlp_sandwich,
                stu_mlp_hidden_size=stu_mlp_hidden_size,
            )
            for key, value in (attention_config or {}).items():
                if key in fields:
                    fields[key] = value
            self.config = FlashSTUConfig(**fields)
            phi, n = None, None
        if phi is None:
            phi = get_spectral_filters(self.config.seq_len, self.config.num_eigh, use_hankel_L=self.config.use_hankel_L,
                                       dtype=self.config.torch_dtype, load_from=self.config.filter_path)
        self.register_buffer("phi", phi, persistent=True)
        self.n = n if n is not None else nearest_power_of_two(self.config.seq_len * 2 - 1, round_up=True)
        if use_attention or self.config.use_attn:
            self.layer = AttentionLayer(self.config)
        else:
            self.layer = STULayer(self.config, self.phi, self.n)

    def forward(self, x: torch.Tensor, past_key_value=None, use_cache=False):
        return self.layer(x, past_key_value=past_key_value, use_cache=use_cache)

    @property
    def is_attention_block(self) -> bool:
        return isinstance(self.layer, AttentionLayer)

    def get_num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
