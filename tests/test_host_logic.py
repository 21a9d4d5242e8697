"""Host-side mirror of the reference API: construction, state-dict keys, filters, cache plumbing."""
import os

import pytest
import torch

import flash_stu_2_b200 as F
from oracle import stu_oracle as O


def _cfg(tmp_path, **kw):
    L, K = kw.pop("seq_len", 64), kw.pop("num_eigh", 8)
    phi = F.get_spectral_filters(L, K, dtype=torch.float32, device="cpu")
    fp = os.path.join(tmp_path, "phi.pt")
    F.save_spectral_filters(phi, fp, metadata={"seq_len": L, "K": K})
    base = dict(n_embd=32, n_layers=4, n_heads=4, seq_len=L, window_size=8, vocab_size=97, mlp_scale=4, num_eigh=K,
                torch_dtype=torch.float32, filter_path=fp)
    base.update(kw)
    return F.FlashSTUConfig(**base)


def test_filters_match_oracle_and_roundtrip(tmp_path):
    phi = F.get_spectral_filters(64, 8, dtype=torch.float32, device="cpu")
    ref = O.spectral_filters(64, 8)
    assert torch.allclose(phi, ref, rtol=0, atol=0)
    p = os.path.join(tmp_path, "sub", "f")
    F.save_spectral_filters(phi, p)
    back = F.load_spectral_filters(p + ".pt", device="cpu", dtype=torch.bfloat16, verify_shape=(64, 8))
    assert back.dtype == torch.bfloat16 and torch.equal(back, phi.bfloat16())
    with pytest.raises(ValueError):
        F.load_spectral_filters(p + ".pt", device="cpu", verify_shape=(64, 9))
    assert F.nearest_power_of_two(2 * 8192 - 1, round_up=True) == 16384


def test_state_dict_keys_match_reference(tmp_path, golden):
    g = golden("models")
    for name in ("stu_only_approx_fp32", "hybrid_approx_fp32", "stu_only_full_fp32"):
        r = g[name]
        m = F.FlashSTU(_cfg(str(tmp_path), use_attn=r["cfg"]["use_attn"], use_approx=r["cfg"]["use_approx"]))
        assert set(m.state_dict().keys()) == set(r["sd"].keys())
        m.load_state_dict(r["sd"])
        assert m.tok_emb.weight is m.lm_head.weight
    blk = F.FlashSTUBlock(d_model=64, sequence_length=128, num_filters=8, torch_dtype=torch.float32)
    assert set(blk.state_dict().keys()) == set(golden("blocks")["approx_float32"]["sd"].keys())
    assert not blk.is_attention_block and blk.get_num_params() > 0


def test_layer_alternation_and_alibi(tmp_path, golden):
    m = F.FlashSTU(_cfg(str(tmp_path)))
    kinds = [type(l).__name__ for l in m.layers]
    assert kinds == ["STULayer", "AttentionLayer", "STULayer", "AttentionLayer"]
    m2 = F.FlashSTU(_cfg(str(tmp_path), use_attn=False))
    assert all(type(l).__name__ == "STULayer" for l in m2.layers)
    for H, s in golden("alibi_slopes").items():
        cfg = _cfg(str(tmp_path), n_embd=8 * H, n_heads=H)
        assert torch.allclose(F.Attention(cfg).alibi_slopes.double(), s.double(), rtol=1e-6, atol=0)


def test_unsupported_switches_fail_loudly(tmp_path):
    for kw in (dict(bias=True), dict(stu_enable_mlp_sandwich=True, bias=True)):
        with pytest.raises(NotImplementedError):
            F.FlashSTU(_cfg(str(tmp_path), use_attn=False, **kw))
    # the sandwich itself constructs, with the reference's parameter names
    m = F.FlashSTU(_cfg(str(tmp_path), use_attn=False, stu_enable_mlp_sandwich=True, stu_mlp_hidden_size=24))
    keys = set(m.state_dict())
    assert {"layers.0.stu_mlp_in_proj.weight", "layers.0.stu_mlp_out_proj.weight"} <= keys
    assert m.layers[0].stu.M_inputs.shape == (24, 24)


def test_model_refuses_cpu(tmp_path):
    m = F.FlashSTU(_cfg(str(tmp_path)))
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(1, 4, dtype=torch.long))


def test_reorder_cache_keeps_structure():
    hist, pos = torch.arange(24.).view(3, 2, 2, 2), torch.tensor([[5, 0]] * 3, dtype=torch.int32)
    kv = (torch.arange(12.).view(3, 2, 2), torch.arange(12.).view(3, 2, 2), pos.clone())
    out = F.FlashSTU._reorder_cache(((hist, pos), kv, None), torch.tensor([2, 0, 0]))
    assert out[2] is None and torch.equal(out[0][0][0], hist[2]) and out[1][2].shape == (3, 2)


def test_checkpoint_round_trip_and_vocabulary_resize(tmp_path):
    """save_pretrained / from_pretrained (flash_stu/model.py:338-366) keep every tensor, the dtype and the
    tok_emb / lm_head tie; resize_token_embeddings keeps the tie and updates the config."""
    import os
    import torch
    import flash_stu_2_b200 as F
    from oracle import stu_oracle as O
    L, K = 64, 8
    fp = os.path.join(str(tmp_path), "phi.pt")
    F.save_spectral_filters(O.spectral_filters(L, K), fp)
    cfg = F.FlashSTUConfig(n_embd=32, n_layers=4, n_heads=4, seq_len=L, window_size=8, vocab_size=97, mlp_scale=4,
                           num_eigh=K, torch_dtype=torch.bfloat16, filter_path=fp, use_attn=True)
    torch.manual_seed(0)
    m = F.FlashSTU(cfg)
    ckpt = os.path.join(str(tmp_path), "ckpt")
    m.save_pretrained(ckpt)
    m2 = F.FlashSTU.from_pretrained(ckpt)
    assert m2.config.torch_dtype == torch.bfloat16 and next(m2.parameters()).dtype == torch.bfloat16
    # a float32 model comes back as float32 (not as the bfloat16 default of the config class), bit for bit
    m32 = F.FlashSTU(F.FlashSTUConfig(n_embd=32, n_layers=2, n_heads=4, seq_len=L, window_size=8, vocab_size=97,
                                      mlp_scale=4, num_eigh=K, torch_dtype=torch.float32, filter_path=fp))
    ck32 = os.path.join(str(tmp_path), "ckpt32")
    m32.save_pretrained(ck32)
    r32 = F.FlashSTU.from_pretrained(ck32)
    assert r32.config.torch_dtype == torch.float32
    assert all(v.dtype == torch.float32 and torch.equal(v, m32.state_dict()[k]) for k, v in r32.state_dict().items())
    # buffers that are not part of a checkpoint (the STU layers' filters, the ALiBi slopes) are re-derived on load
    assert all(torch.equal(l.stu.phi, r32.phi) for l in r32.layers if hasattr(l, "stu"))
    assert all(torch.equal(a.attn.alibi_slopes, b.attn.alibi_slopes)
               for a, b in zip(m2.layers, m.layers) if hasattr(a, "attn"))
    sd1, sd2 = m.state_dict(), m2.state_dict()
    assert set(sd1) == set(sd2) and all(torch.equal(sd1[k], sd2[k]) for k in sd1)
    assert m2.lm_head.weight.data_ptr() == m2.tok_emb.weight.data_ptr()
    m2.resize_token_embeddings(101)
    assert m2.tok_emb.weight.shape == (101, 32) and m2.lm_head.weight.shape == (101, 32)
    assert m2.config.vocab_size == 101 and m2.lm_head.weight.data_ptr() == m2.tok_emb.weight.data_ptr()
    assert torch.equal(m2.tok_emb.weight[:97], sd1["tok_emb.weight"])
    # beam reordering of a cache (flash_stu/model.py:404-426): every tensor of every layer entry, batch on dim 0
    hist = torch.arange(2 * 3 * 2 * 8, dtype=torch.float32).view(2, 3, 2, 8)
    pos = torch.tensor([[5, 0], [7, 0]], dtype=torch.int32)
    out = F.FlashSTU._reorder_cache(((hist, pos), None), torch.tensor([1, 0]))
    assert torch.equal(out[0][0], hist[[1, 0]]) and out[0][1][:, 0].tolist() == [7, 5] and out[1] is None


def test_block_power_iteration_reproduces_the_leading_hankel_eigenpairs():
    """top_eigenpairs_subspace (used for filters when the dense solver refuses the matrix) against numpy eigh."""
    import numpy as np
    import torch
    from flash_stu_2_b200.filters import get_hankel, top_eigenpairs_subspace
    L, K = 384, 16
    Zn = get_hankel(L)
    w, V = top_eigenpairs_subspace(torch.tensor(Zn), K)
    wr, Vr = np.linalg.eigh(Zn)
    assert np.allclose(w.numpy()[-10:], wr[-10:], rtol=1e-9, atol=1e-15)
    assert (V[:, -8:].abs() - torch.tensor(Vr[:, -8:]).abs()).abs().max() < 1e-9
    assert torch.allclose(V.T @ V, torch.eye(K, dtype=torch.float64), atol=1e-10)
