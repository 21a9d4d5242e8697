"""Pre-compute spectral filter files shipped with the package (host eigh is O(L^3): ~1 min for L=8192).

    python flash_stu_2_b200/data/make_filters.py 8192 24

writes flash_stu_2_b200/data/phi_<L>_<K>.pt in the reference's filter-file format
(flash_stu/utils/stu_utils.py:62-72), loadable through FlashSTUConfig(filter_path=...)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from flash_stu_2_b200.filters import get_spectral_filters, save_spectral_filters  # noqa: E402

if __name__ == "__main__":
    L, K = int(sys.argv[1]), int(sys.argv[2])
    phi = get_spectral_filters(L, K, dtype=torch.float32, device="cpu")
    assert torch.isfinite(phi).all()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), f"phi_{L}_{K}.pt")
    save_spectral_filters(phi, out, metadata={"seq_len": L, "K": K, "use_hankel_L": False})
    print(out, os.path.getsize(out))
