"""MiniSTU (mini_stu/stu.py:12-275): the bare full-variant spectral transform with its own input and
output widths, same constructor signature and parameter names (M_phi_plus, M_phi_minus) as the reference.
The spectral backend runs on the kernels of the full STU variant.  The distilled-LDS backend
(mini_stu/stu_lds.py:213-394) prefills with a chunked scan (float64 recurrence, carry term in a balanced rotated
basis, one tensor-core GEMM per sequence for the features of all chunks) and decodes with a recurrent float64 state; forward() takes the optional
`past_key_value` / `use_cache` pair for that (the reference has no cached call).  The optional post-MLP is not
part of this implementation and raises."""
import os
from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .filters import get_spectral_filters, nearest_power_of_two
from .modules import STU, new_pos, host_pos

LDS_PARAMS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "lds_params.pt")


class FixedDiagonalLDS(nn.Module):
    """Buffers of the distilled diagonal LDS (mini_stu/stu_lds.py:213-252): A, B_vec, h0 float64, C model dtype."""

    def __init__(self, A, B_vec, C, h0):
        super().__init__()
        self.register_buffer("A", A.detach().clone())
        self.register_buffer("B_vec", B_vec.detach().clone())
        self.register_buffer("C", C.detach().clone())
        self.register_buffer("h0", h0.detach().clone())


class DistillSTUFast(nn.Module):
    """Holder of the learned contraction M [n_filters, d_in, d_out] (mini_stu/stu_lds.py:344-377)."""

    def __init__(self, lds, K, d_in, d_out, dtype):
        super().__init__()
        self.lds = lds
        self.K, self.d_in, self.d_out = K, d_in, d_out
        self.n_filters = 2 * K
        self.M = nn.Parameter(torch.randn(self.n_filters, d_in, d_out, dtype=dtype, device=lds.A.device)
                              / (self.n_filters * d_in) ** 0.5)


class MiniSTU(nn.Module):
    def __init__(
        self,
        seq_len: int,
        num_filters: int,
        input_dim: int,
        output_dim: int,
        use_hankel_L: bool = False,
        use_flash_fft: bool = True,
        use_mlp: bool = False,
        mlp_hidden_dim: Optional[int] = None,
        mlp_num_layers: int = 2,
        mlp_dropout: float = 0.0,
        mlp_activation: str = "relu",
        dtype: torch.dtype = torch.float32,
        device: Optional[torch.device] = None,
        precomputed_filters: Optional[torch.Tensor] = None,
        backend: str = "spectral",
    ):
        super().__init__()
        if backend not in ("spectral", "lds"):
            raise ValueError(f"unknown backend {backend!r}")
        if use_mlp and mlp_activation.lower() not in ("relu", "gelu", "tanh"):
            raise ValueError(f"Unsupported activation: {mlp_activation}")
        self.seq_len, self.num_filters = seq_len, num_filters
        self.input_dim, self.output_dim = input_dim, output_dim
        self.use_hankel_L, self.use_mlp, self.dtype, self.backend = use_hankel_L, use_mlp, dtype, backend
        self.device = device or torch.device("cpu")
        if backend == "lds":
            assert not use_hankel_L, "LDS backend requires use_hankel_L=False"
            assert num_filters == 24, "LDS backend requires num_filters=24"
            raw = torch.load(os.environ.get("STU_B200_LDS_PARAMS", LDS_PARAMS), map_location="cpu", weights_only=False)
            raw = raw.get("model_state_dict", raw)
            A = raw["A"].to(dtype=torch.float64, device=self.device)
            Bv = raw["B"].to(dtype=torch.float64, device=self.device).flatten()
            C = raw["C"].to(dtype=dtype, device=self.device)
            h0 = raw["h0"].to(dtype=torch.float64, device=self.device)
            self.lds_module = FixedDiagonalLDS(A, Bv, C, h0)
            self.distill_stu = DistillSTUFast(self.lds_module, num_filters, input_dim, output_dim, dtype)
            self.n = nearest_power_of_two(seq_len * 2 - 1, round_up=True)
            self.mlp = None
            self._lds_key = None
            object.__setattr__(self, "_op", None)
            return
        if precomputed_filters is not None:
            phi = precomputed_filters.to(self.device, dtype)
        else:
            phi = get_spectral_filters(seq_len, num_filters, use_hankel_L, self.device, dtype)
        self.register_buffer("phi", phi, persistent=False)
        self.n = nearest_power_of_two(seq_len * 2 - 1, round_up=True)
        scale = (num_filters * input_dim) ** -0.5
        self.M_phi_plus = nn.Parameter(torch.randn(num_filters, input_dim, output_dim, dtype=dtype, device=self.device) * scale)
        if not use_hankel_L:
            self.M_phi_minus = nn.Parameter(
                torch.randn(num_filters, input_dim, output_dim, dtype=dtype, device=self.device) * scale)
        # optional post-MLP on the operator's output (mini_stu/stu.py:171-211): the same nn.Sequential of Linear (with
        # bias), activation and dropout modules as the reference, so that state dicts carry over; only the Linear
        # parameters are read here, the layers run as stu_linear + stu_bias_act
        self.mlp = None
        self._mlp_plan = []
        if use_mlp:
            hid = mlp_hidden_dim if mlp_hidden_dim is not None else output_dim * 2
            act_code = {"relu": ops.ACT_RELU, "gelu": ops.ACT_GELU, "tanh": ops.ACT_TANH}[mlp_activation.lower()]
            act_mod = {"relu": nn.ReLU, "gelu": nn.GELU, "tanh": nn.Tanh}[mlp_activation.lower()]
            layers = []
            for i in range(mlp_num_layers):
                if mlp_num_layers == 1:
                    layers.append(nn.Linear(output_dim, output_dim, dtype=dtype, device=self.device))
                    self._mlp_plan.append((len(layers) - 1, ops.ACT_NONE))
                    break
                d_i = output_dim if i == 0 else hid
                d_o = output_dim if i == mlp_num_layers - 1 else hid
                layers.append(nn.Linear(d_i, d_o, dtype=dtype, device=self.device))
                last = i == mlp_num_layers - 1
                self._mlp_plan.append((len(layers) - 1, ops.ACT_NONE if last else act_code))
                if not last:
                    layers.append(act_mod())
                    if mlp_dropout > 0.0:
                        layers.append(nn.Dropout(mlp_dropout))   # inference: identity
            self.mlp = nn.Sequential(*layers)
        cfg = SimpleNamespace(num_eigh=num_filters, n_embd=input_dim, use_hankel_L=use_hankel_L, use_approx=False,
                              torch_dtype=dtype, d_in_tile=None, d_out_tile=None)
        inner = STU(cfg, phi, self.n)
        inner.d_out = output_dim
        # the operator shares this module's parameters; it is kept out of the module tree so that the
        # state dict has exactly the reference's keys
        del inner.M_phi_plus
        inner.M_phi_plus = self.M_phi_plus
        if not use_hankel_L:
            del inner.M_phi_minus
            inner.M_phi_minus = self.M_phi_minus
        object.__setattr__(self, "_op", inner)

    # ------------------------------------------------------------------ LDS backend
    def _lds_prepared(self):
        """Impulse responses G[j,f] = sum_n C[n,f] B[n] A[n]^j (float64 on the host, rounded once to the model
        dtype), wrapped as the filters of a single-branch full-variant operator whose M_phi is `distill_stu.M`."""
        lds, M = self.lds_module, self.distill_stu.M
        key = (lds.A._version, lds.B_vec._version, lds.C._version, lds.h0._version, M.data_ptr(), lds.C.data_ptr())
        if self._lds_key != key:
            if float(lds.h0.abs().max()) != 0.0:
                raise NotImplementedError("a non-zero initial LDS state h0 has no kernel here")
            A, Bv, C = lds.A.double().cpu(), lds.B_vec.double().cpu(), lds.C.double().cpu()
            j = torch.arange(self.seq_len, dtype=torch.float64)
            G = ((A[None, :] ** j[:, None]) * Bv[None, :]) @ C          # [L, F]
            F_ = C.shape[1]
            cfg = SimpleNamespace(num_eigh=F_, n_embd=self.input_dim, use_hankel_L=True, use_approx=False,
                                  torch_dtype=self.dtype, d_in_tile=None, d_out_tile=None)
            op = STU(cfg, G.to(device=M.device, dtype=self.dtype), self.n)
            op.d_out = self.output_dim
            del op.M_phi_plus
            op.M_phi_plus = M
            object.__setattr__(self, "_op", op)
            self._lds_f32 = (lds.A.to(M.device, torch.float64).contiguous(), lds.B_vec.to(M.device, torch.float64).contiguous(),
                             lds.C.to(M.device, self.dtype).contiguous())
            self._lds_unit_b = bool((Bv == 1.0).all())
            self._lds_scan = self._scan_operands(A, Bv, lds.C.to(self.dtype).double().cpu(), M.device)
            self._lds_key = key
        return self._op

    LDS_CHUNK = 128     # positions per chunk of the scan prefill
    LDS_RANK_CAP = 96   # at most this many balanced coordinates carry the state between chunks

    def _scan_operands(self, A, Bv, C, device):
        """Constant operands of the chunked-scan prefill (float64 on the host, once per parameter version).
        V, lambda: leading eigenpairs of the reachability Gramian P[n,m] = B_n B_m / (1 - A_n A_m); in the basis
        z = V^T h / sqrt(lambda) the carried state and the rotated output map are both O(1) and the carry term
        sum_n C[n,f] A_n^(tau+1) h[n] has no cancellation left (evaluated mode by mode it cancels to 1e-4 of its terms).
        Returns (Vs [D,R] float64, W [Ck*F, KZ] model dtype, R): W = [Q_hi | Q_hi | Q_lo | Toeplitz(G)] for bf16 (hi/lo
        split of the carry operand, the scan kernel writes [z_hi | z_lo | z_hi | x]), [Q | Toeplitz(G)] for fp32."""
        D, F_ = C.shape
        Ck = self.LDS_CHUNK
        P = torch.outer(Bv, Bv) / (1.0 - torch.outer(A, A))
        lam, V = torch.linalg.eigh((P + P.T) * 0.5)
        lam, V = lam.flip(0), V.flip(1)
        R = int((lam > 1e-13 * lam[0]).sum())
        R = max(8, min((R + 7) // 8 * 8, self.LDS_RANK_CAP, D // 8 * 8))
        scale = lam[:R].clamp_min(1e-16 * float(lam[0])).sqrt()
        Vs = (V[:, :R] / scale).contiguous()
        tau = torch.arange(1, Ck + 1, dtype=torch.float64)
        Pw = A[None, :] ** tau[:, None]                                         # [Ck, D]  A^(tau+1)
        Q = torch.einsum("td,df,dk->tfk", Pw, C, V[:, :R] * scale)              # [Ck, F, R]
        G = ((A[None, :] ** torch.arange(Ck, dtype=torch.float64)[:, None]) * Bv[None, :]) @ C   # [Ck, F]
        lag = torch.arange(Ck)[:, None] - torch.arange(Ck)[None, :]             # tau - sigma
        T2 = torch.where((lag >= 0)[:, None, :], G[lag.clamp_min(0)].permute(0, 2, 1), torch.zeros((), dtype=torch.float64))
        if self.dtype == torch.bfloat16:
            Qh = Q.to(torch.bfloat16)
            Ql = (Q - Qh.double()).to(torch.bfloat16)
            W = torch.cat([Qh, Qh, Ql, T2.to(torch.bfloat16)], dim=2)
        else:
            W = torch.cat([Q, T2], dim=2).to(self.dtype)
        return Vs.to(device), W.reshape(Ck * F_, -1).contiguous().to(device), R

    def _forward_lds(self, x, past_key_value=None, use_cache=False):
        op = self._lds_prepared()
        A32, B32, Cm = self._lds_f32
        B, T, d = x.shape
        D, F_ = Cm.shape
        x = x.contiguous()
        if past_key_value is not None:
            if T != 1:
                raise NotImplementedError("the LDS backend continues a cache one token at a time")
            h, pos = past_key_value
            t = host_pos(pos)
            U = torch.empty(B, F_ * d, dtype=x.dtype, device=x.device)
            ops.lds_decode_features(x.view(B, d), h, A32, B32, Cm, U)
            _, Mcat = op.prepared_full()
            y = ops.linear(U, Mcat).view(B, 1, self.output_dim)
            pos[:, 0] += 1
            pos._host_t = t + 1
            return (y, (h, pos)) if use_cache else y
        y = torch.empty(B, T, self.output_dim, dtype=x.dtype, device=x.device)
        if not MiniSTU.chunked_scan_prefill:
            # the same outputs as one causal convolution per feature with the full-length impulse responses
            # (O(T^2) per channel; kept for comparison)
            if not use_cache:
                op.full_forward(x, None, y)
                return y
            hist, pos = op.new_cache(B, x.device)
            op.full_forward(x, None, y, (hist, pos), True)
            h = torch.empty(B, d, D, dtype=torch.float64, device=x.device)
            ops.lds_final_state(hist, h, A32, B32, T)
            return y, (h, pos)
        # chunked scan: float64 recurrence + rotated carry (one kernel), then per sequence one GEMM that produces the
        # features of all chunks in the layout of the contraction with M, and that contraction
        Vs, W, R = self._lds_scan
        Ck = self.LDS_CHUNK
        nch = (T + Ck - 1) // Ck
        Z = torch.empty(B, nch, d, W.shape[1], dtype=x.dtype, device=x.device)
        h = torch.empty(B, d, D, dtype=torch.float64, device=x.device)
        ops.lds_chunk_scan(x, A32, B32, Vs, Z, h, Ck, unit_b=self._lds_unit_b)
        _, Mcat = op.prepared_full()
        U2 = torch.empty(nch * Ck, F_ * d, dtype=x.dtype, device=x.device)
        for b in range(B):
            ops.lds_chunk_features(W, Z[b].view(nch * d, W.shape[1]), U2, d, Ck, F_)
            ops.linear(U2[:T], Mcat, out=y[b])
        if not use_cache:
            return y
        pos = new_pos(B, x.device)
        pos[:, 0] += T
        pos._host_t = T
        return y, (h, pos)

    chunked_scan_prefill = True   # class switch: False runs the prefill as full-length convolutions

    def forward(self, x: torch.Tensor, past_key_value=None, use_cache: bool = False) -> torch.Tensor:
        if x.dim() == 2:
            x = x.unsqueeze(0)
        assert x.dim() == 3, f"Expected x with shape [B, L, I] or [L, I]; got {tuple(x.shape)}"
        if self.backend == "lds":
            return self._forward_lds(x.to(self.dtype), past_key_value, use_cache)
        x = x.to(self.M_phi_plus.dtype)
        op = self._op
        if op.phi.device != self.phi.device:
            op.phi = self.phi
        y = op(x)
        if self.mlp is not None:
            B, T, _ = y.shape
            h = y.view(B * T, -1)
            for idx, act in self._mlp_plan:
                lin = self.mlp[idx]
                h = ops.linear(h, lin.weight)
                ops.bias_act(h, lin.bias, act)
            y = h.view(B, T, -1)
        return y

    def get_num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
