"""flash_stu_2_b200: the Flash STU token loop (prefill + cached decode) on hand-written sm_100a kernels.

Drop-in for the public names of the reference packages `flash_stu` and `mini_stu`:
    from flash_stu_2_b200 import FlashSTU, FlashSTUConfig, FlashSTUBlock, STU, Attention, get_spectral_filters
"""
from .config import FlashSTUConfig
from .filters import (get_hankel, get_spectral_filters, load_spectral_filters, nearest_power_of_two,
                      save_spectral_filters)
from .modules import MLP, STU, Attention, RMSNorm
from .layers import AttentionLayer, STULayer
from .block import FlashSTUBlock
from .model import FlashSTU
from .mini_stu import MiniSTU

__all__ = ["FlashSTU", "MiniSTU", "FlashSTUConfig", "FlashSTUBlock", "STU", "Attention", "MLP", "RMSNorm", "STULayer",
           "AttentionLayer", "get_spectral_filters", "get_hankel", "save_spectral_filters", "load_spectral_filters",
           "nearest_power_of_two"]
