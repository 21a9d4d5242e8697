"""Deterministic synthetic weights for full-size parity fixtures.

A full-size model (147 M parameters for the 12-layer d=512 configuration) cannot travel as a fixture, so the script
that runs the reference and the test that runs the kernels both fill the state dict with this function: every
tensor comes from one seeded CPU generator, visited in sorted key order, so the two sides hold bit-identical
weights.  Scales follow the reference's initialiser (normal, std 0.02; RMSNorm weights 1; flash_stu/model.py:437-452).
"""
import torch


def fill_state_dict(shapes: dict, seed: int, dtype=torch.float32, std: float = 0.02, skip=("phi",)):
    """shapes: {key: torch.Size}.  Returns {key: tensor}; keys in `skip` are left out; tied keys (lm_head.weight)
    reuse tok_emb.weight."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    out = {}
    for key in sorted(shapes):
        if key in skip or key == "lm_head.weight":
            continue
        shape = tuple(shapes[key])
        if key.endswith("norm.weight"):
            out[key] = torch.ones(shape, dtype=dtype)
        else:
            out[key] = (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)
    if "lm_head.weight" in shapes:
        out["lm_head.weight"] = out["tok_emb.weight"]
    return out


C1_CONFIG = dict(n_embd=512, n_layers=12, n_heads=8, seq_len=2048, window_size=512, vocab_size=50257, mlp_scale=12,
                 num_eigh=24, use_approx=True, use_attn=True, softcap=50.0)
C1_SEED = 1234
