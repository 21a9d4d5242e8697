"""Spectral filters: the input data of the STU path (flash_stu/utils/stu_utils.py:18-193,
flash_stu/utils/numerics.py:3-6).  Generation is an init-time float64 eigendecomposition of the Hankel matrix:
on the GPU when the filters are wanted there (what the reference does, stu_utils.py:146-193 - at seq_len 32768
the host eigh takes hours), on the host otherwise; the `.pt` file format {phi, shape, dtype, metadata} is the
reference's."""
import math
from pathlib import Path
from typing import Any, Dict, Optional

import numpy as np
import torch


def nearest_power_of_two(x: int, round_up: bool = False) -> int:
    return 1 << (math.ceil(math.log2(x)) if round_up else math.floor(math.log2(x)))


def get_hankel(seq_len: int, use_hankel_L: bool = False) -> np.ndarray:
    idx = np.arange(1, seq_len + 1, dtype=np.float64)
    s = idx[:, None] + idx[None, :]
    if use_hankel_L:
        return ((-1.0) ** (s - 2.0) + 1.0) * (8.0 / ((s + 3.0) * (s - 1.0) * (s + 1.0)))
    return 2.0 / (s ** 3 - s)


def save_spectral_filters(phi: torch.Tensor, save_path: str, metadata: Optional[Dict[str, Any]] = None) -> None:
    path = Path(save_path)
    if path.suffix != ".pt":
        path = path.with_suffix(".pt")
    path.parent.mkdir(parents=True, exist_ok=True)
    cpu = phi.detach().cpu()
    blob = {"phi": cpu, "shape": list(cpu.shape), "dtype": str(cpu.dtype)}
    if metadata is not None:
        blob["metadata"] = metadata
    torch.save(blob, path)


def load_spectral_filters(load_path: str, device: Optional[torch.device] = None,
                          dtype: Optional[torch.dtype] = None, verify_shape: Optional[tuple] = None) -> torch.Tensor:
    path = Path(load_path)
    if not path.exists():
        raise FileNotFoundError(f"Filter file not found: {path}")
    blob = torch.load(path, map_location="cpu", weights_only=False)
    phi = blob["phi"] if isinstance(blob, dict) else blob
    if verify_shape is not None and tuple(phi.shape) != tuple(verify_shape):
        raise ValueError(f"Filter shape mismatch: expected {tuple(verify_shape)}, got {tuple(phi.shape)}")
    if dtype is not None:
        phi = phi.to(dtype=dtype)
    if device is None:
        device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return phi.to(device=device)


def get_spectral_filters(seq_len: int, K: int, use_hankel_L: bool = False, device: Optional[torch.device] = None,
                         dtype: torch.dtype = torch.bfloat16, load_from: Optional[str] = None) -> torch.Tensor:
    """Top-K eigenvectors of the Hankel matrix scaled by sigma**0.25, shape [seq_len, K]; or the
    content of `load_from`.  Eigenvalues below float64 eigh noise can come out negative for large K;
    they are clamped to zero instead of producing NaN filters."""
    if load_from is not None:
        return load_spectral_filters(load_from, device=device, dtype=dtype, verify_shape=(seq_len, K))
    if device is None:
        device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    device = torch.device(device)
    if device.type == "cuda":
        return spectral_filters_on_device(seq_len, K, use_hankel_L, device, dtype)
    sigma, phi = np.linalg.eigh(get_hankel(seq_len, use_hankel_L))
    sigma, phi = np.clip(sigma[-K:], 0.0, None), phi[:, -K:]
    phi = phi * sigma ** 0.25
    return torch.tensor(phi, device=device, dtype=dtype)


def top_eigenpairs_subspace(Z: torch.Tensor, K: int, sweeps: int = 40, oversample: int = 16):
    """The K largest eigenpairs (ascending, like eigh) of a symmetric positive semi-definite matrix by block power
    iteration with re-orthonormalisation and a final Rayleigh-Ritz step, all in float64 on Z's device.  Eigenvalues
    below the float64 noise of the largest one come out as noise, exactly as they do from a dense solver."""
    n = Z.shape[0]
    p = min(n, K + oversample)
    g = torch.Generator(device="cpu").manual_seed(0)
    X = torch.randn(n, p, dtype=torch.float64, generator=g).to(Z.device)
    for _ in range(sweeps):
        X, _ = torch.linalg.qr(Z @ X)
    T = X.T @ (Z @ X)
    w, V = torch.linalg.eigh((T + T.T) * 0.5)
    return w[-K:], X @ V[:, -K:]


def spectral_filters_on_device(seq_len: int, K: int, use_hankel_L: bool, device: torch.device,
                               dtype: torch.dtype) -> torch.Tensor:
    """The same filters with the Hankel matrix built and decomposed on the GPU (float64 torch.linalg.eigh, as
    flash_stu/utils/stu_utils.py:189-193).  Eigenvector signs are whatever the solver returns; columns are made
    reproducible by flipping each so that its largest-magnitude entry is positive."""
    idx = torch.arange(1, seq_len + 1, dtype=torch.float64, device=device)
    s = idx[:, None] + idx[None, :]
    if use_hankel_L:
        Z = ((-1.0) ** (s - 2.0) + 1.0) * (8.0 / ((s + 3.0) * (s - 1.0) * (s + 1.0)))
    else:
        Z = 2.0 / (s ** 3 - s)
    del s
    try:
        sigma, phi = torch.linalg.eigh(Z)
        sigma, phi = sigma[-K:], phi[:, -K:]
    except RuntimeError:
        # the dense solver refuses very large matrices (seq_len 32768 on this stack): only K eigenpairs are
        # wanted and the spectrum decays geometrically, so block power iteration gets them in O(L^2 K) per sweep
        sigma, phi = top_eigenpairs_subspace(Z, K)
    del Z
    sigma = sigma.clamp_min(0.0)
    pick = phi.abs().argmax(dim=0)
    phi = phi * torch.sign(phi.gather(0, pick[None, :]))
    return (phi * sigma ** 0.25).to(dtype)
