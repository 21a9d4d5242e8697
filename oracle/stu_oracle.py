"""CPU oracle for the Flash STU token loop (prefill + cached decode).

TEST INFRASTRUCTURE ONLY.  This file restates, in plain torch-on-CPU code, the
arithmetic of the reference implementation (hazan-lab/flash-stu-2) for the one
path this repository accelerates.  It is imported by the test-suite, by the
smoke check and by the CPU-baseline leg of the benchmark, and by nothing in
the product package: the product path calls CUDA kernels only and raises when
they are missing.

Pinning: every function below is checked against outputs produced by the
reference's own modules (imported on CPU, see tests/golden/make_golden.py)
which are committed as fixtures under tests/golden/.  The attention function
has no CPU counterpart in the reference (its arithmetic lives in the
third-party flash-attn package, un-pinned by the reference); for it parity is
unpinned by any reference test and the restatement follows the documented
flash_attn_func contract plus the reference call site.

All citations are `path:line` inside the reference repository.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# --------------------------------------------------------------------------- numerics
def nearest_power_of_two(x: int, round_up: bool = False) -> int:
    """flash_stu/utils/numerics.py:3-6."""
    return 1 << (math.ceil(math.log2(x)) if round_up else math.floor(math.log2(x)))


def fft_length(seq_len: int) -> int:
    """FFT length the model uses for every STU layer, flash_stu/model.py:56."""
    return nearest_power_of_two(seq_len * 2 - 1, round_up=True)


# --------------------------------------------------------------------------- filters
def hankel(seq_len: int, use_hankel_L: bool = False) -> np.ndarray:
    """flash_stu/utils/stu_utils.py:18-31 (float64)."""
    e = np.arange(1, seq_len + 1, dtype=np.float64)
    s = e[:, None] + e[None, :]
    if use_hankel_L:
        sgn = (-1.0) ** (s - 2.0) + 1.0
        return sgn * (8.0 / ((s + 3.0) * (s - 1.0) * (s + 1.0)))
    return 2.0 / (s ** 3 - s)


def spectral_filters(seq_len: int, K: int, use_hankel_L: bool = False,
                     dtype: torch.dtype = torch.float32) -> Tensor:
    """Top-K Hankel eigenvectors scaled by sigma**0.25, flash_stu/utils/stu_utils.py:189-193."""
    sigma, phi = np.linalg.eigh(hankel(seq_len, use_hankel_L))
    sigma, phi = sigma[-K:], phi[:, -K:]
    phi = phi * sigma ** 0.25
    return torch.tensor(phi, dtype=dtype)


# --------------------------------------------------------------------------- S1 convolution
def convolve(u: Tensor, v: Tensor, n: int, use_approx: bool = True,
             return_both: bool = True) -> Tuple[Tensor, Optional[Tensor]]:
    """FFT causal convolution, flash_stu/utils/stu_utils.py:195-246.

    The sign vector is built at the *input* length (the `sgn is None` branch,
    stu_utils.py:204-206) so that inputs shorter than seq_len work; the reference
    module passes a cached seq_len-long buffer instead (modules/stu.py:30-33,95-98),
    which is the same vector when the input has full length.
    """
    bsz, seq_len, d_in = u.shape
    dt = u.dtype
    sgn = torch.ones(1, seq_len, 1, dtype=torch.int64)
    sgn[:, 1::2] *= -1
    if return_both:
        if use_approx:
            d_out = v.shape[1]
            v_fft = torch.fft.rfft(v.view(1, -1, d_out, 1).to(torch.float32), n=n, dim=1)
        else:
            sgn = sgn.unsqueeze(-1)
            K = v.shape[1]
            v_fft = torch.fft.rfft(v.view(1, -1, K, 1, 1).to(torch.float32), n=n, dim=1)
            u = u.view(bsz, -1, 1, d_in).expand(bsz, -1, K, d_in)
        U = torch.stack([u, u * sgn], dim=-1).to(torch.float32)
        U = torch.fft.rfft(U, n=n, dim=1)
        U_conv = torch.fft.irfft(v_fft * U, n=n, dim=1)[:, :seq_len]
        U_plus, U_minus = torch.unbind(U_conv, dim=-1)
        U_minus = U_minus * sgn
        return U_plus.to(dt), U_minus.to(dt)
    if use_approx:
        d_out = v.shape[1]
        v_fft = torch.fft.rfft(v.view(1, -1, d_out).to(torch.float32), n=n, dim=1)
    else:
        K = v.shape[1]
        v_fft = torch.fft.rfft(v.view(1, -1, K, 1).to(torch.float32), n=n, dim=1)
        u = u.view(bsz, -1, 1, d_in).expand(bsz, -1, K, d_in)
    U = torch.fft.rfft(u.to(torch.float32), n=n, dim=1)
    U_plus = torch.fft.irfft(v_fft * U, n=n, dim=1)[:, :seq_len]
    return U_plus.to(dt), None


def convolve_direct(u: Tensor, v: Tensor, minus: bool = False) -> Tensor:
    """Time-domain statement of the same sum in float64 (used to cross-check the FFT form):
    out[b,t,c] = sum_{j<=t} (+-1)^j v[j,c] u[b,t-j,c]."""
    B, T, d = u.shape
    vv = v[:T].double().clone()
    if minus:
        vv[1::2] *= -1
    out = torch.zeros(B, T, d, dtype=torch.float64)
    ud = u.double()
    for j in range(T):
        out[:, j:] += vv[j] * ud[:, : T - j]
    return out


# --------------------------------------------------------------------------- S2 / S2' STU
def stu_forward(x: Tensor, phi: Tensor, p: Dict[str, Tensor], n: int,
                use_approx: bool = True, use_hankel_L: bool = False) -> Tensor:
    """STU._forward_standard, flash_stu/modules/stu.py:81-120 (torch.fft branch).

    `p` holds M_inputs/M_filters (approx) or M_phi_plus[/M_phi_minus] (full).
    MiniSTU's spectral branch (mini_stu/stu.py:240-269) is the full variant of this.
    """
    return_both = not use_hankel_L
    if use_approx:
        x_proj = x @ p["M_inputs"]
        phi_proj = phi @ p["M_filters"]
        sp, sm = convolve(x_proj, phi_proj, n, True, return_both)
    else:
        U_plus, U_minus = convolve(x, phi, n, False, return_both)
        sp = torch.tensordot(U_plus, p["M_phi_plus"], dims=([2, 3], [0, 1]))
        sm = None
        if return_both:
            sm = torch.tensordot(U_minus, p["M_phi_minus"], dims=([2, 3], [0, 1]))
    return sp if use_hankel_L else sp + sm


def stu_forward_tiled(x: Tensor, phi: Tensor, p: Dict[str, Tensor], n: int, tile: int,
                      use_hankel_L: bool = False) -> Tensor:
    """STU._tile_diagonal_blocks, flash_stu/modules/stu.py:169-191: the approx operator on the diagonal
    tile x tile blocks of M_inputs, tile by tile, results concatenated."""
    outs = []
    d = x.shape[-1]
    for i in range(0, d, tile):
        e = min(i + tile, d)
        sub = {"M_inputs": p["M_inputs"][i:e, i:e], "M_filters": p["M_filters"][:, i:e]}
        outs.append(stu_forward(x[..., i:e], phi, sub, n, True, use_hankel_L))
    return torch.cat(outs, dim=-1)


# --------------------------------------------------------------------------- S9 / S4 pointwise blocks
RMS_EPS = float(torch.finfo(torch.float32).eps)


def rmsnorm(x: Tensor, w: Tensor, eps: float = RMS_EPS) -> Tensor:
    """torch.nn.RMSNorm(n_embd, dtype) as selected by the reference's fallback branch
    (flash_stu/layers/stu_layer.py:17-36): statistics, scale and weight in fp32, one
    rounding to the model dtype; eps=None resolves to finfo(float32).eps."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def mlp(x: Tensor, p: Dict[str, Tensor], prefix: str = "mlp.") -> Tensor:
    """Gated tanh-GELU MLP, flash_stu/modules/swiglu.py:22-29 (bias-free)."""
    gate = F.linear(x, p[prefix + "gate_proj.weight"])
    gate = F.gelu(gate, approximate="tanh")
    up = F.linear(x, p[prefix + "up_proj.weight"])
    gate = gate * up
    return F.linear(gate, p[prefix + "down_proj.weight"])


# --------------------------------------------------------------------------- S5 attention
def alibi_slopes(n_heads: int, interpolation_factor: float = 0.25) -> Tensor:
    """flash_stu/modules/attention.py:34-57."""
    def gen(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_heads).is_integer():
        s = gen(n_heads)
    else:
        n = nearest_power_of_two(n_heads, round_up=False)
        s = gen(n) + gen(2 * n)[0::2][: n_heads - n]
    return torch.tensor(s) * interpolation_factor


def attention(x: Tensor, p: Dict[str, Tensor], n_heads: int, window: int, softcap: float,
              past: Optional[Tuple[Tensor, Tensor]] = None, prefix: str = "attn."):
    """Attention.forward, flash_stu/modules/attention.py:59-105, with flash_attn_func(q,k,v,
    causal=True, window_size=(w,0), alibi_slopes, softcap) written out in fp32:
    score = softcap*tanh(q.k*scale/softcap) - slope_h*(i-j), keys j in [i-w, i].
    Returns (y, (k, v)) with k,v the concatenated caches as the reference keeps them."""
    B, T, d = x.shape
    H, hd = n_heads, d // n_heads
    qkv = F.linear(x, p[prefix + "c_attn.weight"])
    q, k, v = torch.chunk(qkv, 3, dim=2)
    q, k, v = (t.reshape(B, T, H, hd) for t in (q, k, v))
    if past is not None:
        k = torch.cat([past[0], k], dim=1)
        v = torch.cat([past[1], v], dim=1)
    Tk = k.shape[1]
    i = torch.arange(T)[:, None] + (Tk - T)
    j = torch.arange(Tk)[None, :]
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(hd)
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    s = s - alibi_slopes(H)[None, :, None, None] * (i - j).abs()[None, None].float()
    s = s.masked_fill(~((j <= i) & (j >= i - window))[None, None], float("-inf"))
    y = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v.float()).to(x.dtype)
    y = F.linear(y.reshape(B, T, d), p[prefix + "c_proj.weight"])
    return y, (k, v)


# --------------------------------------------------------------------------- S4 layers, S6 model
def _sub(sd: Dict[str, Tensor], prefix: str) -> Dict[str, Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def stu_layer(x: Tensor, p: Dict[str, Tensor], phi: Tensor, n: int, use_approx: bool,
              use_hankel_L: bool = False) -> Tensor:
    """STULayer._forward_impl, flash_stu/layers/stu_layer.py:78-97 (no sandwich)."""
    h = rmsnorm(x, p["stu_norm.weight"])
    h = stu_forward(h, phi, _sub(p, "stu."), n, use_approx, use_hankel_L)
    x = x + h
    return x + mlp(rmsnorm(x, p["mlp_norm.weight"]), p)


def stu_layer_sandwich(x: Tensor, p: Dict[str, Tensor], phi: Tensor, n: int, use_approx: bool) -> Tensor:
    """STULayer._forward_impl with stu_enable_mlp_sandwich, flash_stu/layers/stu_layer.py:39-63,83-88:
    up-projection, SiLU, the STU on the hidden width, down-projection; then the MLP half as in stu_layer."""
    h = rmsnorm(x, p["stu_norm.weight"])
    h = F.linear(h, p["stu_mlp_in_proj.weight"])
    h = F.silu(h)
    h = stu_forward(h, phi, _sub(p, "stu."), n, use_approx)
    h = F.linear(h, p["stu_mlp_out_proj.weight"])
    x = x + h
    return x + mlp(rmsnorm(x, p["mlp_norm.weight"]), p)


def post_mlp(y: Tensor, sd: Dict[str, Tensor], activation: str) -> Tensor:
    """The nn.Sequential post-MLP of MiniSTU(use_mlp=True), mini_stu/stu.py:171-211,267: Linear layers (with bias)
    at the indices present in the state dict, the activation after every layer but the last."""
    act = {"relu": F.relu, "gelu": F.gelu, "tanh": torch.tanh}[activation]
    idx = sorted({int(k.split(".")[1]) for k in sd if k.startswith("mlp.") and k.endswith(".weight")})
    for n_, i in enumerate(idx):
        y = F.linear(y, sd[f"mlp.{i}.weight"], sd[f"mlp.{i}.bias"])
        if n_ + 1 < len(idx):
            y = act(y)
    return y


def attention_layer(x: Tensor, p: Dict[str, Tensor], n_heads: int, window: int, softcap: float,
                    past=None):
    """AttentionLayer._forward_impl, flash_stu/layers/attention_layer.py:50-66."""
    a, present = attention(rmsnorm(x, p["attn_norm.weight"]), p, n_heads, window, softcap, past)
    x = x + a
    return x + mlp(rmsnorm(x, p["mlp_norm.weight"]), p), present


def layer_is_attention(idx: int, use_attn: bool) -> bool:
    """Even index -> STU, odd index -> attention when use_attn, flash_stu/model.py:77-87."""
    return (idx % 2 == 1) and use_attn


def model_hidden(ids: Tensor, sd: Dict[str, Tensor], cfg: dict) -> Tensor:
    """FlashSTU.forward up to the final norm, flash_stu/model.py:152-173 (no cache: the
    reference's STU layers hold none, so the full prefix is recomputed)."""
    n = fft_length(cfg["seq_len"])
    x = F.embedding(ids, sd["tok_emb.weight"])
    for i in range(cfg["n_layers"]):
        p = _sub(sd, f"layers.{i}.")
        if layer_is_attention(i, cfg.get("use_attn", True)):
            x, _ = attention_layer(x, p, cfg["n_heads"], cfg["window_size"], cfg.get("softcap", 50.0))
        else:
            x = stu_layer(x, p, sd["phi"], n, cfg.get("use_approx", True), cfg.get("use_hankel_L", False))
    return rmsnorm(x, sd["norm.weight"])


def model_logits(ids: Tensor, sd: Dict[str, Tensor], cfg: dict, last_only: bool = False) -> Tensor:
    """Logits [B,T,V] (or [B,V] for the last position), flash_stu/model.py:173-176."""
    h = model_hidden(ids, sd, cfg)
    if last_only:
        h = h[:, -1]
    return F.linear(h, sd["lm_head.weight"] if "lm_head.weight" in sd else sd["tok_emb.weight"])


# --------------------------------------------------------------------------- S7 sampling
def filter_logits(logits: Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                  top_p: Optional[float] = None) -> Tensor:
    """flash_stu/model.py:268-292: divide by temperature (in the logits dtype), clamp to
    +-1e4, top-k mask `z < kth largest` (ties kept), nucleus mask on the sorted cumulative
    softmax shifted right by one."""
    z = logits / temperature
    z = torch.clamp(z, min=-1e4, max=1e4)
    if top_k is not None:
        kth = torch.topk(z, top_k)[0][..., -1, None]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p is not None:
        sl, si = torch.sort(z, descending=True)
        cp = torch.cumsum(F.softmax(sl, dim=-1), dim=-1)
        rem = cp > top_p
        rem[..., 1:] = rem[..., :-1].clone()
        rem[..., 0] = 0
        z = z.masked_fill(rem.scatter(1, si, rem), float("-inf"))
    return z


def pick_token(z: Tensor, do_sample: bool, u: Optional[Tensor] = None) -> Tensor:
    """Greedy: argmax (lowest index among ties), flash_stu/model.py:299.  Sampling: the
    reference draws torch.multinomial(softmax(z)) (model.py:293-297), whose random stream is
    not reproducible across devices; both this oracle and the kernels instead take one
    uniform u in [0,1) per sequence and return the first vocabulary index whose running
    sum of exp(z - max) (fp32, vocabulary order) exceeds u * total."""
    if not do_sample:
        return torch.argmax(z, dim=-1, keepdim=True)
    zf = z.float()
    e = torch.exp(zf - zf.max(dim=-1, keepdim=True)[0])
    c = torch.cumsum(e, dim=-1)
    tgt = u.float().view(-1, 1) * c[:, -1:]
    idx = (c > tgt).float().argmax(dim=-1, keepdim=True)
    none = ~(c > tgt).any(dim=-1, keepdim=True)
    last = (e > 0).float().cumsum(-1).argmax(dim=-1, keepdim=True)
    return torch.where(none, last, idx)


def generate(ids: Tensor, sd: Dict[str, Tensor], cfg: dict, max_length: int,
             temperature: float = 1.0, top_k: Optional[int] = None, top_p: Optional[float] = None,
             do_sample: bool = False, uniforms: Optional[Tensor] = None,
             return_logits: bool = False):
    """FlashSTU.generate, flash_stu/model.py:207-304, as the no-cache loop: each new token is
    produced from a forward over the whole prefix (this is the only token loop the reference's
    STU layers can run, and the definition the cached decode must reproduce)."""
    gen = ids
    all_logits: List[Tensor] = []
    for step in range(max_length - ids.shape[1]):
        logits = model_logits(gen[:, -cfg["seq_len"]:], sd, cfg, last_only=True)
        all_logits.append(logits)
        z = filter_logits(logits, temperature, top_k, top_p)
        nxt = pick_token(z, do_sample, None if uniforms is None else uniforms[step])
        gen = torch.cat([gen, nxt], dim=-1)
    if return_logits:
        return gen, torch.stack(all_logits, dim=1)
    return gen


# --------------------------------------------------------------------------- S8 LDS variant
def lds_features(u: Tensor, A: Tensor, Bv: Tensor, C: Tensor, h0: Tensor) -> Tensor:
    """FixedDiagonalLDS.forward as the step recurrence it scans (mini_stu/stu_lds.py:279-338;
    recurrence form mini_stu/lds.py:95-101): h <- A*h + B*u_t ; out_t = h @ C.
    u: (N,T) -> (N,T,F), float64."""
    N, T = u.shape
    h = h0.double().view(1, -1).expand(N, -1).clone()
    A, Bv, C = A.double(), Bv.double(), C.double()
    out = torch.empty(N, T, C.shape[1], dtype=torch.float64)
    for t in range(T):
        h = h * A + u[:, t:t + 1].double() * Bv
        out[:, t] = h @ C
    return out


def lds_forward(x: Tensor, A: Tensor, Bv: Tensor, C: Tensor, h0: Tensor, M: Tensor) -> Tensor:
    """DistillSTUFast.forward, mini_stu/stu_lds.py:379-394, in float64 on the given inputs:
    y[b,t,o] = sum_{f,i} U[b,t,f,i] M[f,i,o], U = LDS features of channel i."""
    B, T, d_in = x.shape
    u = x.permute(0, 2, 1).reshape(-1, T)
    U = lds_features(u, A, Bv, C, h0)
    nf = U.shape[-1]
    U = U.reshape(B, d_in, T, nf).permute(0, 2, 3, 1)
    out = U.reshape(B * T, nf * d_in) @ M.double().reshape(nf * d_in, -1)
    return out.reshape(B, T, -1)


def lds_impulse_response(A: Tensor, Bv: Tensor, C: Tensor, T: int) -> Tensor:
    """G[j,f] = sum_n C[n,f] B[n] A_n^j: the LDS features are the causal convolution of the
    input with these T taps (h0 = 0)."""
    j = torch.arange(T, dtype=torch.float64)
    P = A.double()[None, :] ** j[:, None]
    return (P * Bv.double()[None, :]) @ C.double()


# --------------------------------------------------------------------------- helpers for tests
def rel_err(a: Tensor, b: Tensor) -> float:
    """max |a-b| / max |b| over the whole tensor."""
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def row_err(a: Tensor, b: Tensor, floor: float = 1e-3) -> float:
    """Worst row of max_row |a-b| / max_row |b|, a row being one vector along the last dimension (one token's
    channels, one sequence's logits).  Stricter than rel_err: a result that is wrong on every small-magnitude row
    passes rel_err (whose denominator is the largest value anywhere) and fails here.  Rows whose largest reference
    value is below `floor` times the tensor's largest are measured against that floor (an all-zero row has no
    relative error)."""
    a, b = a.double(), b.double()
    if a.dim() == 0:
        return rel_err(a, b)
    a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    den = b.abs().amax(dim=1).clamp_min(floor * float(b.abs().max()) + 1e-30)
    return float(((a - b).abs().amax(dim=1) / den).max())


def rms_err(a: Tensor, b: Tensor) -> float:
    """||a-b||_2 / ||b||_2 over the whole tensor."""
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
