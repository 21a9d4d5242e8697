"""Pin the CPU oracle against outputs of the reference's own modules (tests/golden/*.pt)."""
import torch

from oracle import stu_oracle as O


def _close(a, b, tol):
    assert a.shape == b.shape
    err = O.rel_err(a, b)
    assert err <= tol, err


def test_stu_operator_matches_reference(golden):
    g = golden("stu_modules")
    assert len(g) == 8
    for name, r in g.items():
        hankel_L = name.startswith("hankelL")
        approx = "_approx_" in name
        tol = 0.0 if "float32" in name else 0.0  # same ops, same machine arithmetic -> bit-equal
        y = O.stu_forward(r["x"], r["phi"], r["params"], r["n"], approx, hankel_L)
        _close(y, r["y_full"], 1e-6 if "float32" in name else 1e-2)
        T = r["T_short"]
        ys = O.stu_forward(r["x"][:, :T].contiguous(), r["phi"], r["params"], r["n"], approx, hankel_L)
        _close(ys, r["y_short"], 1e-6 if "float32" in name else 1e-2)
        # causality / prefix consistency of the reference function itself
        _close(ys.float(), r["y_full"][:, :T].float(), 2e-6 if "float32" in name else 2e-2)


def test_fft_conv_equals_direct_sum(golden):
    r = golden("stu_modules")["std_approx_float32"]
    xp = r["x"] @ r["params"]["M_inputs"]
    fp = r["phi"] @ r["params"]["M_filters"]
    plus, minus = O.convolve(xp, fp, r["n"], True, True)
    _close(plus.double(), O.convolve_direct(xp, fp, minus=False), 1e-5)
    _close(minus.double(), O.convolve_direct(xp, fp, minus=True), 1e-5)
    # even-tap identity used by the kernels: plus + minus == 2 * (even taps only)
    fe = fp.clone()
    fe[1::2] = 0
    _close((plus + minus).double(), 2 * O.convolve_direct(xp, fe), 1e-5)


def test_model_logits_and_generate_match_reference(golden):
    g = golden("models")
    for name, r in g.items():
        dt = getattr(torch, r["dtype"])
        tol = 2e-5 if dt == torch.float32 else 2e-2
        logits = O.model_logits(r["ids"], r["sd"], r["cfg"])
        _close(logits, r["logits_full"], tol)
        T = r["T_short"]
        _close(O.model_logits(r["ids"][:, :T], r["sd"], r["cfg"]), r["logits_short"], tol)
        if dt == torch.float32:
            new = r["gen_greedy"].shape[1]
            gen = O.generate(r["gen_prompt"], r["sd"], r["cfg"], max_length=new, do_sample=False)
            assert torch.equal(gen, r["gen_greedy"]), name


def test_sampling_filters_match_reference(golden):
    for name, r in golden("models").items():
        if r["dtype"] != "float32":
            continue
        steps = r["filtered_probs"].shape[1]
        gen = r["gen_filtered"]
        T0 = r["gen_prompt"].shape[1]
        for s in range(steps):
            logits = O.model_logits(gen[:, : T0 + s], r["sd"], r["cfg"], last_only=True)
            z = O.filter_logits(logits, **r["filter_args"])
            p = torch.softmax(z, -1)
            assert torch.equal(p > 0, r["filtered_probs"][:, s] > 0)
            _close(p, r["filtered_probs"][:, s], 1e-4)


def test_block_matches_reference(golden):
    for name, r in golden("blocks").items():
        approx = name.startswith("approx")
        sd = {k[len("layer."):]: v for k, v in r["sd"].items() if k.startswith("layer.")}
        y = O.stu_layer(r["x"], sd, r["sd"]["phi"], r["n"], approx)
        _close(y, r["y"], 2e-5 if "float32" in name else 2e-2)


def test_mini_stu_matches_reference(golden):
    g = golden("mini_stu")
    r = g["spectral_fp32"]
    y = O.stu_forward(r["x"], r["phi"], r["params"], r["n"], use_approx=False)
    _close(y, r["y"], 1e-5)
    r = g["lds_fp64"]
    y = O.lds_forward(r["x"], r["A"], r["B_vec"], r["C"], r["h0"], r["M"])
    _close(y, r["y"], 1e-9)
    # impulse-response (convolution) form of the same features
    T = r["x"].shape[1]
    G = O.lds_impulse_response(r["A"], r["B_vec"], r["C"], T)
    u = r["x"].permute(0, 2, 1).reshape(-1, T)
    U = O.lds_features(u, r["A"], r["B_vec"], r["C"], r["h0"])
    Uc = torch.zeros_like(U)
    for j in range(T):
        Uc[:, j:] += u[:, : T - j, None] * G[j]
    _close(Uc, U, 1e-9)


def test_inference_variants_match_reference(golden):
    """STU layer with the MLP sandwich (full-length and shorter input), block-diagonal tiling of the approx operator
    and MiniSTU with the post-MLP."""
    g = golden("variants")
    for name in ("sandwich_approx_float32", "sandwich_approx_bfloat16"):
        r = g[name]
        sd = {k[len("layer."):]: v for k, v in r["sd"].items() if k.startswith("layer.")}
        tol = 2e-5 if "float32" in name else 2e-2
        _close(O.stu_layer_sandwich(r["x"], sd, r["sd"]["phi"], r["n"], True), r["y"], tol)
        T = r["T_short"]
        _close(O.stu_layer_sandwich(r["x"][:, :T], sd, r["sd"]["phi"], r["n"], True), r["y_short"], tol)
    for name in ("tiled16_approx_float32", "tiled20_approx_float32", "tiled16_approx_bfloat16", "tiled20_approx_bfloat16"):
        r = g[name]
        tile = min(r["tile"][0] or 48, r["tile"][1] or 48)
        _close(O.stu_forward_tiled(r["x"], r["phi"], r["params"], r["n"], tile), r["y"],
               2e-5 if "float32" in name else 2e-2)
    for name in ("mini_mlp_relu2", "mini_mlp_gelu3", "mini_mlp_tanh2", "mini_mlp_single"):
        r = g[name]
        n = O.fft_length(r["x"].shape[1])
        y = O.stu_forward(r["x"], r["phi"], r["sd"], n, use_approx=False)
        _close(O.post_mlp(y, r["sd"], r["kw"].get("mlp_activation", "relu")), r["y"], 1e-5)


def test_alibi_slopes_match_reference(golden):
    for H, s in golden("alibi_slopes").items():
        assert torch.allclose(O.alibi_slopes(H).double(), s.double(), rtol=1e-6, atol=0)


def test_lds_params_fixture(golden):
    p = golden("lds_params")
    assert p["A"].shape == (160,) and p["C"].shape == (160, 48) and p["B"].shape == (1, 160)
    assert float(p["A"].abs().max()) < 1.0


def test_full_size_12_layer_model_prompt_logits(golden):
    """The oracle on the full-size d=512 / 12-layer / vocabulary-50257 configuration: logits at the end of the
    128-token prompt and the first greedy token against the reference's run (fixture c1_full; synthetic weights
    rebuilt from the shared seeded generator)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "synth_weights", os.path.join(os.path.dirname(__file__), "golden", "synth_weights.py"))
    sw = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sw)
    r = golden("c1_full")
    sd = sw.fill_state_dict(r["shapes"], sw.C1_SEED)
    sd["phi"] = r["phi"]
    with torch.no_grad():
        last = O.model_logits(r["prompt"], sd, dict(sw.C1_CONFIG), last_only=True).float()
    assert O.rel_err(last[:, ::16], r["logits_prompt_end_sample"]) <= 1e-5
    top_v, top_i = r["logits_prompt_end_top"]
    assert torch.equal(last.argmax(-1), top_i[:, 0])
    assert torch.equal(last.argmax(-1), r["gen_greedy"][:, r["prompt"].shape[1]])
