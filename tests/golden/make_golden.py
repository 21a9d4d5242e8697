"""Generate the golden fixtures in this folder by running the *reference's own modules* on CPU.

Run once, in a container that has the reference checkout, with REFERENCE_ROOT pointing at it:

    REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py

Nothing in the test-suite or the product imports the reference; the fixtures written here
(*.pt, a few hundred KB in total) are what travels.  Shims applied to make the unmodified
reference run without a GPU:
  * `liger_kernel` masked so the torch RMSNorm branch is taken (layers/stu_layer.py:17-25);
  * filters computed on CPU with numpy eigh (same formula as utils/stu_utils.py:189-193) and
    passed through `filter_path`, which skips the CUDA assert (stu_utils.py:175-185);
  * use_flash_fft=False (torch.fft branch);
  * for inputs shorter than seq_len every STU module's cached `sgn` buffer is sliced to the
    input length before the call (the buffer is otherwise unusable, modules/stu.py:30-33);
  * hybrid models: the reference's Attention asserts CUDA and calls flash-attn, so a stand-in
    class with the same parameters and init hooks, computing the documented flash_attn_func
    arithmetic in fp32, is substituted.  Fixtures that involve it are marked
    `attention_pinned=False`.
"""
import math
import os
import sys
import tempfile

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
sys.modules["liger_kernel"] = None
REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (hazan-lab/flash-stu-2)")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

from flash_stu.utils.stu_utils import get_hankel, save_spectral_filters  # noqa: E402
from flash_stu.utils.numerics import nearest_power_of_two  # noqa: E402
import flash_stu.modules.attention as ref_attention  # noqa: E402
import flash_stu.layers.attention_layer as ref_attention_layer  # noqa: E402
import flash_stu.model as ref_model  # noqa: E402


def make_phi(L, K, hankel_L=False):
    sigma, phi = np.linalg.eigh(get_hankel(L, hankel_L))
    sigma, phi = sigma[-K:], phi[:, -K:]
    phi = phi * sigma ** 0.25
    return torch.tensor(phi, dtype=torch.float32)


class AttnStandIn(nn.Module):
    """Same parameters / SCALE_INIT hook as flash_stu.modules.attention.Attention; slopes from
    the reference's own (unbound) helper methods; flash_attn_func written out in fp32."""

    def __init__(self, config):
        super().__init__()
        self.n_heads = config.n_heads
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=config.bias, dtype=config.torch_dtype)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=config.bias, dtype=config.torch_dtype)
        self.c_proj.SCALE_INIT = 1
        self.window_size = config.window_size
        self.softcap = config.softcap
        self.device = torch.device("cpu")
        self.alibi_slopes = ref_attention.Attention._get_alibi_slopes(self, self.n_heads)

    _generate_slopes = ref_attention.Attention._generate_slopes

    def forward(self, x, past_key_value=None, use_cache=True):
        B, T, d = x.shape
        H, hd = self.n_heads, d // self.n_heads
        q, k, v = torch.chunk(self.c_attn(x), 3, dim=2)
        q, k, v = (t.view(B, T, H, hd) for t in (q, k, v))
        if past_key_value is not None:
            k = torch.cat([past_key_value[0], k], 1)
            v = torch.cat([past_key_value[1], v], 1)
        Tk = k.shape[1]
        i = torch.arange(T)[:, None] + Tk - T
        j = torch.arange(Tk)[None, :]
        s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(hd)
        s = self.softcap * torch.tanh(s / self.softcap) - self.alibi_slopes[None, :, None, None] * (i - j).abs()[None, None]
        s = s.masked_fill(~((j <= i) & (j >= i - self.window_size))[None, None], float("-inf"))
        y = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v.float()).to(x.dtype).reshape(B, T, d)
        y = self.c_proj(y)
        return (y, (k, v)) if use_cache else y


ref_attention_layer.Attention = AttnStandIn
ref_model.Attention = AttnStandIn

from flash_stu import FlashSTU, FlashSTUConfig, FlashSTUBlock  # noqa: E402
from flash_stu.modules.stu import STU  # noqa: E402


def set_len(module, T, full):
    for s in module.modules():
        if isinstance(s, STU):
            s.sgn = full[id(s)][:, :T]


def full_sgn(module):
    return {id(s): s.sgn.clone() for s in module.modules() if isinstance(s, STU)}


def sd_of(module):
    return {k: v.detach().clone() for k, v in module.state_dict().items()}


def save(name, obj):
    path = os.path.join(HERE, name + ".pt")
    torch.save(obj, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def golden_stu_modules(tmp):
    """Bare STU operator: approx / full / Hankel-L, fp32 and bf16, T == seq_len and T < seq_len."""
    out = {}
    L, K, d, B = 64, 8, 32, 2
    for hankel_L in (False, True):
        phi32 = make_phi(L, K, hankel_L)
        for dt in (torch.float32, torch.bfloat16):
            for approx in (True, False):
                torch.manual_seed(10 + int(approx) + 2 * int(hankel_L))
                cfg = FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=approx, use_hankel_L=hankel_L,
                                     use_flash_fft=False, torch_dtype=dt, n_layers=1, vocab_size=1)
                n = nearest_power_of_two(L * 2 - 1, round_up=True)
                m = STU(cfg, phi32.to(dt), n)
                for p in m.parameters():
                    nn.init.xavier_normal_(p)
                full = full_sgn(m)
                x = torch.randn(B, L, d).to(dt)
                rec = {"phi": phi32.to(dt), "x": x, "n": n,
                       "params": {k: v.detach().clone() for k, v in m.named_parameters()}}
                with torch.no_grad():
                    rec["y_full"] = m(x).clone()
                    T = 37
                    set_len(m, T, full)
                    rec["T_short"] = T
                    rec["y_short"] = m(x[:, :T].contiguous()).clone()
                out[f"{'hankelL' if hankel_L else 'std'}_{'approx' if approx else 'full'}_{str(dt).split('.')[-1]}"] = rec
    save("stu_modules", out)


def golden_models(tmp):
    out = {}
    # --- STU-only model, approx and full, fp32
    for name, kw in (("stu_only_approx_fp32", dict(use_approx=True, use_attn=False)),
                     ("stu_only_full_fp32", dict(use_approx=False, use_attn=False)),
                     ("hybrid_approx_fp32", dict(use_approx=True, use_attn=True)),
                     ("hybrid_approx_bf16", dict(use_approx=True, use_attn=True, torch_dtype=torch.bfloat16))):
        L, K, d, V = 64, 8, 32, 97
        dt = kw.pop("torch_dtype", torch.float32)
        phi = make_phi(L, K)
        fp = os.path.join(tmp, f"phi_{L}_{K}.pt")
        save_spectral_filters(phi, fp)
        torch.manual_seed(0)
        cfgd = dict(n_embd=d, n_layers=4, n_heads=4, seq_len=L, window_size=8, vocab_size=V, mlp_scale=4,
                    num_eigh=K, use_flash_fft=False, torch_dtype=dt, softcap=50.0, **kw)
        m = FlashSTU(FlashSTUConfig(filter_path=fp, **cfgd)).eval()
        full = full_sgn(m)
        ids = torch.randint(0, V, (2, L))
        rec = {"cfg": {k: v for k, v in cfgd.items() if k != "torch_dtype"}, "dtype": str(dt).split(".")[-1],
               "ids": ids, "sd": sd_of(m), "attention_pinned": not kw["use_attn"]}
        with torch.no_grad():
            rec["logits_full"] = m(ids, use_cache=False).logits.clone()
            T = 21
            set_len(m, T, full)
            rec["T_short"] = T
            rec["logits_short"] = m(ids[:, :T], use_cache=False).logits.clone()
            # greedy generate through the reference's own loop, no cache, sgn re-sliced per step
            T0, new = 9, 12
            orig_forward = m.forward

            def fwd(input_ids, *a, **k):
                set_len(m, input_ids.shape[1], full)
                return orig_forward(input_ids, *a, **k)

            m.forward = fwd
            rec["gen_prompt"] = ids[:, :T0].clone()
            rec["gen_greedy"] = m.generate(ids[:, :T0], max_length=T0 + new, do_sample=False, use_cache=False).clone()
            # sampling filters: capture the probabilities the reference hands to multinomial
            captured = []
            real_multinomial = torch.multinomial

            def fake_multinomial(probs, num_samples=1, **k):
                captured.append(probs.clone())
                return probs.argmax(-1, keepdim=True)

            torch.multinomial = fake_multinomial
            try:
                g = m.generate(ids[:, :T0], max_length=T0 + 4, temperature=0.8, top_k=5, top_p=0.9,
                               do_sample=True, use_cache=False)
            finally:
                torch.multinomial = real_multinomial
            rec["gen_filtered"] = g.clone()
            rec["filtered_probs"] = torch.stack(captured, 1)
            rec["filter_args"] = dict(temperature=0.8, top_k=5, top_p=0.9)
            m.forward = orig_forward
        out[name] = rec
    save("models", out)


def golden_blocks(tmp):
    out = {}
    L, K, d = 128, 8, 64
    phi = make_phi(L, K)
    for approx in (True, False):
        for dt in (torch.bfloat16, torch.float32):
            torch.manual_seed(1)
            cfg = FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=approx, use_attn=False, mlp_scale=4,
                                 use_flash_fft=False, torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=1)
            n = nearest_power_of_two(L * 2 - 1, round_up=True)
            blk = FlashSTUBlock(config=cfg, phi=phi.to(dt), n=n)
            for name, p in blk.named_parameters():
                if ".stu.M_" in name:
                    nn.init.xavier_normal_(p)
            x = torch.randn(3, L, d).to(dt)
            with torch.no_grad():
                y = blk(x.clone())
            out[f"{'approx' if approx else 'full'}_{str(dt).split('.')[-1]}"] = {
                "x": x, "y": y.clone(), "sd": sd_of(blk), "n": n, "L": L, "K": K, "d": d}
    save("blocks", out)


def golden_mini(tmp):
    from mini_stu import MiniSTU
    out = {}
    torch.manual_seed(2)
    L, K, din, dout = 64, 8, 12, 20
    phi = make_phi(L, K)
    m = MiniSTU(seq_len=L, num_filters=K, input_dim=din, output_dim=dout, use_flash_fft=False,
                dtype=torch.float32, precomputed_filters=phi)
    x = torch.randn(2, L, din)
    with torch.no_grad():
        y = m(x)
    out["spectral_fp32"] = {"x": x, "y": y.clone(), "phi": phi, "n": m.n,
                            "params": {k: v.detach().clone() for k, v in m.named_parameters()}}
    # LDS backend: only float64 executes on CPU in the reference
    torch.manual_seed(3)
    T, din, dout = 48, 6, 10
    m = MiniSTU(seq_len=T, num_filters=24, input_dim=din, output_dim=dout, backend="lds", dtype=torch.float64)
    x = torch.randn(2, T, din, dtype=torch.float64)
    with torch.no_grad():
        y = m(x)
    lds = m.lds_module
    out["lds_fp64"] = {"x": x, "y": y.clone(), "A": lds.A.clone(), "B_vec": lds.B_vec.clone(), "C": lds.C.clone(),
                       "h0": lds.h0.clone(), "M": m.distill_stu.M.detach().clone()}
    save("mini_stu", out)
    # The distilled LDS parameters the lds backend loads (mini_stu/stu.py:88-96), re-saved as plain tensors.
    raw = torch.load(os.path.join(REF, "mini_stu", "phi_lds.pt"), map_location="cpu", weights_only=False)["model_state_dict"]
    save("lds_params", {k: v.clone() for k, v in raw.items()})


def golden_slopes():
    out = {}
    for H in (1, 2, 4, 8, 12, 16, 24):
        s = AttnStandIn.__new__(AttnStandIn)
        nn.Module.__init__(s)
        s.device = torch.device("cpu")
        out[H] = ref_attention.Attention._get_alibi_slopes(s, H).clone()
    save("alibi_slopes", out)


def golden_c1_full(tmp):
    """The 12-layer d=512 fp32 configuration at full size (6 STU + 6 sliding-window layers, vocabulary 50257,
    seq_len 2048, mlp_scale 12): batch 2, prompt 128, 128 greedy tokens through the reference's own generate()
    (no cache, sgn re-sliced per step).  Weights are synthetic (synth_weights.fill_state_dict) so that the test
    can rebuild them; the fixture holds the filters, the prompt, the generated ids, the margin between the two
    largest logits at every step and a sample of the logits at the last prompt position."""
    sys.path.insert(0, HERE)
    from synth_weights import fill_state_dict, C1_CONFIG, C1_SEED
    cfg = dict(C1_CONFIG)
    L, K = cfg["seq_len"], cfg["num_eigh"]
    phi = make_phi(L, K)
    fp = os.path.join(tmp, f"phi_{L}_{K}.pt")
    save_spectral_filters(phi, fp)
    m = FlashSTU(FlashSTUConfig(filter_path=fp, use_flash_fft=False, torch_dtype=torch.float32, **cfg)).eval()
    shapes = {k: v.shape for k, v in m.state_dict().items()}
    sd = fill_state_dict(shapes, C1_SEED)
    missing = m.load_state_dict(sd, strict=False)
    assert set(missing.missing_keys) <= {"phi"} and not missing.unexpected_keys, missing
    full = full_sgn(m)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg["vocab_size"], (2, 128), generator=g)
    margins, first_logits = [], []
    orig_forward = m.forward

    def fwd(input_ids, *a, **k):
        set_len(m, input_ids.shape[1], full)
        out = orig_forward(input_ids, *a, **k)
        last = out.logits[:, -1].float()
        top2 = last.topk(2, dim=-1).values
        margins.append((top2[:, 0] - top2[:, 1]).clone())
        if not first_logits:
            first_logits.append(last.clone())
        return out

    m.forward = fwd
    with torch.no_grad():
        gen = m.generate(ids, max_length=256, do_sample=False, use_cache=False)
    rec = {"phi": m.state_dict()["phi"].clone(), "prompt": ids, "gen_greedy": gen.clone(),
           "margins": torch.stack(margins, 1), "logits_prompt_end_sample": first_logits[0][:, ::16].clone(),
           "logits_prompt_end_top": first_logits[0].topk(32, dim=-1), "shapes": {k: tuple(v) for k, v in shapes.items()},
           "attention_pinned": False}
    rec["logits_prompt_end_top"] = (rec["logits_prompt_end_top"].values.clone(), rec["logits_prompt_end_top"].indices.clone())
    save("c1_full", rec)


def golden_variants(tmp):
    """Inference variants next to the benchmark configurations: the STU layer with the MLP sandwich
    (flash_stu/layers/stu_layer.py:39-63,83-88: in_proj -> SiLU -> STU on the hidden width -> out_proj), full-length
    and shorter inputs, fp32 and bf16; MiniSTU with the post-MLP (mini_stu/stu.py:171-211) in its three shapes."""
    from mini_stu import MiniSTU
    out = {}
    L, K, d, Hs = 128, 8, 64, 96
    phi = make_phi(L, K)
    for dt in (torch.float32, torch.bfloat16):
        torch.manual_seed(21)
        cfg = FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=True, use_attn=False, mlp_scale=4,
                             use_flash_fft=False, torch_dtype=dt, n_layers=1, vocab_size=1, n_heads=1,
                             stu_enable_mlp_sandwich=True, stu_mlp_hidden_size=Hs)
        n = nearest_power_of_two(L * 2 - 1, round_up=True)
        blk = FlashSTUBlock(config=cfg, phi=phi.to(dt), n=n)
        for name, p in blk.named_parameters():
            if ".stu.M_" in name:
                nn.init.xavier_normal_(p)
        full = full_sgn(blk)
        x = torch.randn(3, L, d).to(dt)
        T = 51
        with torch.no_grad():
            y = blk(x.clone()).clone()
            set_len(blk, T, full)
            y_short = blk(x[:, :T].clone()).clone()
        out[f"sandwich_approx_{str(dt).split('.')[-1]}"] = {
            "x": x, "y": y, "y_short": y_short, "T_short": T, "sd": sd_of(blk), "n": n, "L": L, "K": K, "d": d,
            "hidden": Hs}
    # block-diagonal tiling of the approx operator (flash_stu/modules/stu.py:123-191)
    L, K, d = 64, 8, 48
    phi32 = make_phi(L, K)
    for dt in (torch.float32, torch.bfloat16):
        for tile in (16, 20):
            torch.manual_seed(23)
            cfg = FlashSTUConfig(n_embd=d, seq_len=L, num_eigh=K, use_approx=True, use_flash_fft=False, torch_dtype=dt,
                                 n_layers=1, vocab_size=1, d_in_tile=tile, d_out_tile=None if tile == 16 else 32)
            n = nearest_power_of_two(L * 2 - 1, round_up=True)
            m = STU(cfg, phi32.to(dt), n)
            for p in m.parameters():
                nn.init.xavier_normal_(p)
            x = torch.randn(2, L, d).to(dt)
            with torch.no_grad():
                y = m(x).clone()
            out[f"tiled{tile}_approx_{str(dt).split('.')[-1]}"] = {
                "phi": phi32.to(dt), "x": x, "n": n, "y": y, "tile": (cfg.d_in_tile, cfg.d_out_tile),
                "params": {k: v.detach().clone() for k, v in m.named_parameters()}}
    L, K, din, dout = 64, 8, 12, 20
    phi = make_phi(L, K)
    for name, kw in (("mini_mlp_relu2", dict(mlp_num_layers=2, mlp_activation="relu")),
                     ("mini_mlp_gelu3", dict(mlp_num_layers=3, mlp_activation="gelu", mlp_hidden_dim=24)),
                     ("mini_mlp_tanh2", dict(mlp_num_layers=2, mlp_activation="tanh", mlp_hidden_dim=16)),
                     ("mini_mlp_single", dict(mlp_num_layers=1))):
        torch.manual_seed(22)
        m = MiniSTU(seq_len=L, num_filters=K, input_dim=din, output_dim=dout, use_flash_fft=False, use_mlp=True,
                    dtype=torch.float32, precomputed_filters=phi, **kw)
        x = torch.randn(2, L, din)
        with torch.no_grad():
            y = m(x)
        out[name] = {"x": x, "y": y.clone(), "phi": phi, "kw": kw, "sd": sd_of(m)}
    save("variants", out)


if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as tmp:
        if len(sys.argv) > 1 and sys.argv[1] == "variants":
            golden_variants(tmp)
            raise SystemExit(0)
        golden_stu_modules(tmp)
        golden_models(tmp)
        golden_blocks(tmp)
        golden_mini(tmp)
        golden_slopes()
        golden_c1_full(tmp)
        golden_variants(tmp)
