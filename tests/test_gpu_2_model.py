"""FlashSTU.forward / generate on a B200 against the reference's outputs (tests/golden/models.pt).
Attention inside the hybrid fixtures comes from the fp32 restatement of flash_attn_func (the reference
has no CPU attention), so hybrid parity is pinned to that restatement, STU-only parity to the reference."""
import os

import pytest
import torch

from oracle import stu_oracle as O

pytestmark = pytest.mark.gpu


def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def build(r, tmp_path):
    import flash_stu_2_b200 as F
    dt = getattr(torch, r["dtype"])
    fp = os.path.join(str(tmp_path), "phi.pt")
    F.save_spectral_filters(r["sd"]["phi"].float(), fp)
    m = F.FlashSTU(F.FlashSTUConfig(filter_path=fp, torch_dtype=dt, **r["cfg"]))
    m.load_state_dict(r["sd"])
    return m.to(dev()).eval()


@pytest.mark.parametrize("name", ["stu_only_approx_fp32", "stu_only_full_fp32", "hybrid_approx_fp32", "hybrid_approx_bf16"])
def test_logits_match_reference(golden, tmp_path, name):
    from flash_stu_2_b200 import ops
    r = golden("models")[name]
    m = build(r, tmp_path)
    tol = 1e-3 if r["dtype"] == "float32" else 2e-2
    with torch.no_grad():
        full = m(r["ids"].to(dev()), use_cache=False).logits.cpu()
        T = r["T_short"]
        short = m(r["ids"][:, :T].to(dev()), use_cache=False).logits.cpu()
    ops.check_status()
    assert O.rel_err(full, r["logits_full"]) <= tol, O.rel_err(full, r["logits_full"])
    assert O.rel_err(short, r["logits_short"]) <= tol


@pytest.mark.parametrize("name", ["stu_only_approx_fp32", "stu_only_full_fp32", "hybrid_approx_fp32"])
def test_greedy_generate_is_token_exact(golden, tmp_path, name):
    """fp32 greedy decoding with the cache reproduces the reference's no-cache loop token for token."""
    from flash_stu_2_b200 import ops
    r = golden("models")[name]
    m = build(r, tmp_path)
    want = r["gen_greedy"]
    got_cached = m.generate(r["gen_prompt"].to(dev()), max_length=want.shape[1], do_sample=False, use_cache=True)
    got_nocache = m.generate(r["gen_prompt"].to(dev()), max_length=want.shape[1], do_sample=False, use_cache=False)
    ops.check_status()
    assert torch.equal(got_cached.cpu(), want)
    assert torch.equal(got_nocache.cpu(), want)


@pytest.mark.parametrize("name", ["hybrid_approx_fp32", "hybrid_approx_bf16"])
def test_cached_logits_and_sampling_follow_oracle(golden, tmp_path, name):
    from flash_stu_2_b200 import ops
    r = golden("models")[name]
    m = build(r, tmp_path)
    tol = 1e-3 if r["dtype"] == "float32" else 2e-2
    T0, new = 9, 10
    torch.manual_seed(0)
    u = torch.rand(new, r["ids"].shape[0])
    prompt = r["ids"][:, :T0]
    want, want_logits = O.generate(prompt, r["sd"], r["cfg"], T0 + new, temperature=0.8, top_k=5, do_sample=True,
                                   uniforms=u, return_logits=True)
    got, got_logits = m.generate(prompt.to(dev()), max_length=T0 + new, temperature=0.8, top_k=5, do_sample=True,
                                 uniforms=u, return_logits=True)
    ops.check_status()
    got, got_logits = got.cpu(), got_logits.cpu()
    # compare logits step by step while the sampled prefixes agree
    agree = 0
    for s in range(new):
        assert O.rel_err(got_logits[:, s], want_logits[:, s]) <= tol, (s, O.rel_err(got_logits[:, s], want_logits[:, s]))
        if not torch.equal(got[:, : T0 + s + 1], want[:, : T0 + s + 1]):
            break
        agree += 1
    if r["dtype"] == "float32":
        assert agree == new, (got, want)
    else:
        assert agree >= 1
