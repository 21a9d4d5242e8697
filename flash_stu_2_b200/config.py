"""FlashSTUConfig: the hyper-parameter object of the reference (flash_stu/config.py:71-132), field for
field, so that configs and checkpoints written for the reference construct this implementation."""
from typing import Optional, Tuple, Union

import torch
from transformers import PretrainedConfig


class FlashSTUConfig(PretrainedConfig):
    """Hyper-parameters of a Flash STU model (alternating STU / sliding-window attention layers).

    Same constructor signature and attribute names as the reference class.  Switches whose code
    path has no CUDA kernel here (use_flash_fft is ignored: there is a single convolution path;
    tiling and bias terms raise at module construction) are kept so that
    existing configs load.
    """
    model_type = "FlashSTU"

    def __init__(
        self,
        bsz: int = 1,
        n_embd: int = 1536,
        n_heads: int = 8,
        n_layers: int = 26,
        seq_len: int = 8192,
        window_size: Union[int, Tuple[int, int]] = 1024,
        vocab_size: int = 200064,
        mlp_scale: int = 12,
        bias: bool = False,
        dropout: float = 0.0,
        num_eigh: int = 24,
        use_hankel_L: bool = False,
        use_flash_fft: bool = True,
        use_approx: bool = True,
        use_attn: bool = True,
        use_cache: bool = True,
        use_gradient_checkpointing: bool = False,
        softcap: float = 50.0,
        torch_dtype: torch.dtype = torch.bfloat16,
        tie_word_embeddings: bool = True,
        stu_enable_mlp_sandwich: bool = False,
        stu_mlp_hidden_size: Optional[int] = None,
        filter_path: Optional[str] = None,
        d_in_tile: Optional[int] = None,
        d_out_tile: Optional[int] = None,
        cache_len: Optional[int] = None,
        **kwargs,
    ):
        # transformers >= 5 serialises a model's dtype under the key `dtype` (and drops `torch_dtype` from the dict it
        # hands back to this constructor): a checkpoint written from a float32 model must not come back as the
        # bfloat16 default, so an explicit `dtype` wins over an unset / default `torch_dtype`
        dtype_kw = kwargs.get("dtype")
        if isinstance(dtype_kw, str):
            dtype_kw = getattr(torch, dtype_kw.replace("torch.", ""), None)
        if isinstance(dtype_kw, torch.dtype) and (torch_dtype is None or torch_dtype == torch.bfloat16):
            torch_dtype = dtype_kw
        super().__init__(tie_word_embeddings=tie_word_embeddings, **kwargs)
        for name, value in dict(
            bsz=bsz, n_embd=n_embd, n_heads=n_heads, n_layers=n_layers, seq_len=seq_len, window_size=window_size,
            vocab_size=vocab_size, mlp_scale=mlp_scale, bias=bias, dropout=dropout, num_eigh=num_eigh,
            use_hankel_L=use_hankel_L, use_flash_fft=use_flash_fft, use_approx=use_approx, use_attn=use_attn,
            use_cache=use_cache, use_gradient_checkpointing=use_gradient_checkpointing, softcap=softcap,
            stu_enable_mlp_sandwich=stu_enable_mlp_sandwich, stu_mlp_hidden_size=stu_mlp_hidden_size,
            filter_path=filter_path, d_in_tile=d_in_tile, d_out_tile=d_out_tile, cache_len=cache_len,
        ).items():
            setattr(self, name, value)
        self.hidden_size = n_embd
        self.intermediate_size = n_embd * mlp_scale
        self.hidden_act = "swish"
        if torch_dtype is None:
            torch_dtype = torch.float32
        elif isinstance(torch_dtype, str):
            torch_dtype = getattr(torch, torch_dtype)
        self.torch_dtype = torch_dtype

    def to_dict(self):
        out = super().to_dict()
        dt = getattr(self, "torch_dtype", None)
        if isinstance(dt, torch.dtype):
            out["torch_dtype"] = str(dt).replace("torch.", "")
            out["dtype"] = out["torch_dtype"]
        return out
