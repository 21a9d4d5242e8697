"""Tensor-parallel token loop for models too large (or too slow) for one GPU: one process per GPU, every rank
holds a 1/g slice of every layer and the full residual stream.

Sharding (g ranks, rank r), one exchange per sub-layer:
  * STU layer (approx variant, flash_stu/modules/stu.py:85-98): `M_inputs` and `M_filters` are split by output
    channel; the projected history, the taps and the causal convolution are per-channel and therefore local;
    the d/g output channels are all-gathered into the residual stream.
  * MLP (flash_stu/modules/swiglu.py:22-29): gate/up split by column of the hidden layer, down by the matching
    rows of its input; the partial d-wide outputs are all-reduced.
  * attention (flash_stu/modules/attention.py:72-101): heads split; `c_proj` split by the matching input columns;
    partial outputs all-reduced.  The KV ring of a rank holds its heads only.
  * LM head: vocabulary split; the logits shards are all-gathered (rank-major, padded rows cut off).
Prefill: the collectives are torch.distributed calls (NCCL over NVLink on GPUs) between the same CUDA kernels the
single-GPU path uses.  Token steps (bf16, all sequences at one position): each exchange after an STU, attention or
MLP sub-layer is ONE kernel of this package (peer.PeerExchange.exchange, one CTA per sequence): it stores this rank's
rows into every rank's inbox over NVLink (whole 16-byte vectors), raises a per-row flag, waits (bounded) for the
other ranks' rows, adds them to the residual stream and applies the next sub-layer's RMSNorm - in place of a
collective, an add and a norm kernel.  (A second mode, "push", stores from inside the producing kernels instead;
measured slower: 2-byte stores over NVLink and a system-scope fence per CTA.)  Only the logits all-gather of a step
stays a library collective.  Every rank ends a step with
identical logits and, given the same uniforms, identical tokens.
"""
from typing import Dict, Optional

import torch
import torch.distributed as dist

from . import ops
from .modules import _round_up, host_pos, new_pos


def _rng(n: int, world: int, rank: int):
    if n % world:
        raise ValueError(f"dimension {n} does not divide over {world} ranks")
    w = n // world
    return rank * w, (rank + 1) * w


def shard_state_dict(sd: Dict[str, torch.Tensor], cfg: dict, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """The tensors rank `rank` of `world` keeps, cut out of a full FlashSTU state dict (keys as in
    flash_stu/model.py).  Replicated: embeddings' consumer side (tok_emb), all norm weights, phi.
      layers.i.stu.M_inputs [d, d/g], layers.i.stu.M_filters [K, d/g]           output channels
      layers.i.mlp.gate_proj/up_proj.weight [inter/g, d], down_proj.weight [d, inter/g]
      layers.i.attn.c_attn.weight [3*d/g, d] (q|k|v of the rank's heads), c_proj.weight [d, d/g]
      lm_head.weight [ceil(V/g), d] (rows past the vocabulary are zero)"""
    d, H = cfg["n_embd"], cfg["n_heads"]
    hd = d // H
    out = {}
    for k, v in sd.items():
        if k.endswith("stu.M_inputs") or k.endswith("stu.M_filters"):
            lo, hi = _rng(d, world, rank)
            out[k] = v[:, lo:hi].contiguous()
        elif k.endswith("stu.M_phi_plus") or k.endswith("stu.M_phi_minus"):
            raise NotImplementedError("tensor parallelism covers the approx STU variant")
        elif k.endswith("gate_proj.weight") or k.endswith("up_proj.weight"):
            lo, hi = _rng(v.shape[0], world, rank)
            out[k] = v[lo:hi].contiguous()
        elif k.endswith("down_proj.weight"):
            lo, hi = _rng(v.shape[1], world, rank)
            out[k] = v[:, lo:hi].contiguous()
        elif k.endswith("c_attn.weight"):
            lo, hi = _rng(H, world, rank)
            out[k] = v.view(3, H, hd, d)[:, lo:hi].reshape(3 * (hi - lo) * hd, d).contiguous()
        elif k.endswith("c_proj.weight"):
            lo, hi = _rng(H, world, rank)
            out[k] = v[:, lo * hd:hi * hd].contiguous()
        elif k == "lm_head.weight":
            V = v.shape[0]
            vl = -(-V // world)
            w = torch.zeros(vl, v.shape[1], dtype=v.dtype, device=v.device)
            rows = v[rank * vl:min(V, (rank + 1) * vl)]
            w[:rows.shape[0]] = rows
            out[k] = w
        else:
            out[k] = v
    return out


def random_shards(config, phi: torch.Tensor, rank: int, world: int, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init weights of rank `rank`, generated on `device` shard by shard (no full model is ever built: a 4.5 B
    parameter model would take 9 GB of host memory and minutes of initialisation per rank).  Replicated tensors
    (embedding, norms, filters) come from the same seeded generator on every rank, sharded ones from a per-rank
    seed; distributions as flash_stu/model.py:428-452 (normal with std d^-0.5 for the linears, Xavier for the STU and
    attention projections)."""
    d, H, K, V = config.n_embd, config.n_heads, config.num_eigh, config.vocab_size
    inter, dt = d * config.mlp_scale, config.torch_dtype
    dl, hd = d // world, d // H
    shared = torch.Generator(device=device).manual_seed(seed)
    own = torch.Generator(device=device).manual_seed(seed + 1000 * (rank + 1))

    def normal(gen, shape, std):
        return (torch.randn(*shape, device=device, dtype=torch.float32, generator=gen) * std).to(dt)

    sd = {"phi": phi.to(device), "tok_emb.weight": normal(shared, (V, d), d ** -0.5),
          "norm.weight": torch.ones(d, device=device, dtype=dt)}
    vl = -(-V // world)
    head = torch.zeros(vl, d, device=device, dtype=dt)
    rows = sd["tok_emb.weight"][rank * vl:min(V, (rank + 1) * vl)]
    head[:rows.shape[0]] = rows
    sd["lm_head.weight"] = head
    for i in range(config.n_layers):
        p = f"layers.{i}."
        if (i % 2 == 1) and config.use_attn:
            sd[p + "attn_norm.weight"] = torch.ones(d, device=device, dtype=dt)
            sd[p + "attn.c_attn.weight"] = normal(own, (3 * dl, d), (2.0 / (4 * d)) ** 0.5)
            sd[p + "attn.c_proj.weight"] = normal(own, (d, dl), (2.0 / (2 * d)) ** 0.5)
        else:
            sd[p + "stu_norm.weight"] = torch.ones(d, device=device, dtype=dt)
            sd[p + "stu.M_inputs"] = normal(own, (d, dl), (2.0 / (2 * d)) ** 0.5)
            sd[p + "stu.M_filters"] = normal(own, (K, dl), (2.0 / (K + d)) ** 0.5)
        sd[p + "mlp_norm.weight"] = torch.ones(d, device=device, dtype=dt)
        sd[p + "mlp.gate_proj.weight"] = normal(own, (inter // world, d), d ** -0.5)
        sd[p + "mlp.up_proj.weight"] = normal(own, (inter // world, d), d ** -0.5)
        sd[p + "mlp.down_proj.weight"] = normal(own, (d, inter // world), d ** -0.5 * (2 * config.n_layers) ** -0.5)
    return sd


class TensorParallelFlashSTU:
    """FlashSTU (approx STU layers, optional sliding-window attention layers) over the ranks of a process group.
    `state_dict` is the full model's; each rank cuts out its share.  Call from every rank with identical inputs."""

    def __init__(self, config, state_dict: Dict[str, torch.Tensor], device, group=None, presharded: bool = False):
        """`state_dict`: the full model's tensors (each rank cuts out its share), or, with presharded=True, this
        rank's share already in the shapes shard_state_dict documents (see random_shards)."""
        self.cfg = config
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        if not config.use_approx:
            raise NotImplementedError("tensor parallelism covers the approx STU variant")
        c = dict(n_embd=config.n_embd, n_heads=config.n_heads)
        if presharded:
            self.sd = {k: v.to(self.device) for k, v in state_dict.items()}
        else:
            self.sd = {k: v.to(self.device) for k, v in shard_state_dict(state_dict, c, self.rank, self.world).items()}
        if "tok_emb.weight" not in self.sd:
            raise ValueError("state_dict lacks tok_emb.weight")
        self.d, self.H = config.n_embd, config.n_heads
        self.hd = self.d // self.H
        self.dl = self.d // self.world
        self.Hl = self.H // self.world
        self.V = config.vocab_size if presharded else (
            state_dict["lm_head.weight"].shape[0] if "lm_head.weight" in state_dict else state_dict["tok_emb.weight"].shape[0])
        if "lm_head.weight" not in self.sd:   # tied head stored once
            self.sd["lm_head.weight"] = shard_state_dict({"lm_head.weight": state_dict["tok_emb.weight"]}, c, self.rank,
                                                         self.world)["lm_head.weight"].to(self.device)
        self.dtype = self.sd["tok_emb.weight"].dtype
        self.capacity = min(config.seq_len, getattr(config, "cache_len", None) or config.seq_len)
        self.Lh = _round_up((self.capacity + 1) // 2, 8)
        ws = config.window_size
        self.window = int(ws[0] if isinstance(ws, (tuple, list)) else ws)
        self.eps = ops.RMS_EPS
        self.fused_decode = True
        # token steps: "exchange" = one kernel per sub-layer exchange pushes this rank's rows to the other ranks over
        # peer memory, waits for theirs and folds them (and the next RMSNorm) into the residual stream; "push" = the
        # producing kernels store into the inboxes themselves and a combine kernel waits; False = NCCL collectives
        # Default by group size, from measurements on B200s (3B shapes, B = 64, ms per token step, exchange kernels
        # against NCCL): 2 GPUs 10.67 / 11.13, 4 GPUs 6.80 / 6.72, 8 GPUs 6.15 / 5.76 (NCCL with in-switch reduction):
        # every rank sends its full rows to every other rank, which is the cheapest pattern while latency dominates and
        # loses to a reduce-scatter + all-gather once eight ranks' rows cross every link.  "force" keeps the exchange
        # kernels at any group size.
        self.fused_exchange = "exchange" if self.world <= 4 else False
        self._exchange = None
        self._derived = {}
        from .modules import Attention
        self.slopes = Attention._get_alibi_slopes(Attention, self.H)[self.rank * self.Hl:(self.rank + 1) * self.Hl] \
            .to(self.device).contiguous()

    # ------------------------------------------------------------------ helpers
    def _is_attn(self, i: int) -> bool:
        return (i % 2 == 1) and bool(self.cfg.use_attn)

    def _stu_weights(self, i: int):
        """(MinT [d/g, d], taps [d/g, Lh], taps8 or None) of layer i, derived once."""
        if i not in self._derived:
            p = f"layers.{i}.stu."
            MinT = self.sd[p + "M_inputs"].t().contiguous()
            fp = ops.linear(self.sd["phi"][:self.capacity].to(self.dtype).contiguous(), self.sd[p + "M_filters"],
                            transposed_weight=True,
                            backend=ops.BACKEND_SIMT)
            taps = ops.taps_even(fp, self.Lh)
            taps8 = ops.taps_rev8(taps) if (self.dtype == torch.bfloat16 and self.dl % 8 == 0) else None
            self._derived[i] = (MinT, taps, taps8)
        return self._derived[i]

    def new_cache(self, B: int):
        cache = []
        for i in range(self.cfg.n_layers):
            if self._is_attn(i):
                W = self.window + 1
                cache.append((torch.zeros(B, W, self.dl, dtype=self.dtype, device=self.device),
                              torch.zeros(B, W, self.dl, dtype=self.dtype, device=self.device), new_pos(B, self.device)))
            else:
                cache.append((torch.zeros(B, self.dl, 2, self.Lh, dtype=self.dtype, device=self.device),
                              new_pos(B, self.device)))
        return cache

    def _all_reduce_add(self, x2: torch.Tensor, part: torch.Tensor):
        dist.all_reduce(part, group=self.group)
        x2.add_(part)

    def _mlp(self, x2: torch.Tensor, i: int):
        p = f"layers.{i}."
        xn = ops.rmsnorm(x2, self.sd[p + "mlp_norm.weight"], self.eps)
        h = ops.linear(xn, self.sd[p + "mlp.gate_proj.weight"], W2=self.sd[p + "mlp.up_proj.weight"],
                       epilogue=ops.EPI_GELU_MUL)
        self._all_reduce_add(x2, ops.linear(h, self.sd[p + "mlp.down_proj.weight"]))

    # ------------------------------------------------------------------ forward
    def hidden(self, ids: torch.Tensor, cache):
        """Residual stream [B,T,d] after all layers for the T new tokens; the cache is updated in place."""
        B, T = ids.shape
        d, dl = self.d, self.dl
        x = ops.embed(ids, self.sd["tok_emb.weight"])
        x2 = x.view(B * T, d)
        for i in range(self.cfg.n_layers):
            p = f"layers.{i}."
            if self._is_attn(i):
                k_ring, v_ring, pos = cache[i]
                t0 = host_pos(pos)
                xn = ops.rmsnorm(x2, self.sd[p + "attn_norm.weight"], self.eps)
                qkv = ops.linear(xn, self.sd[p + "attn.c_attn.weight"]).view(B, T, 3 * dl)
                attend = ops.swa_prefill_tc5 if ops.swa_prefill_tc5_supported(qkv, self.Hl, t0) else ops.swa_forward
                y = attend(qkv, k_ring, v_ring, pos, self.slopes, self.Hl, self.window, self.cfg.softcap,
                           update_cache=True)
                pos._host_t = t0 + T
                self._all_reduce_add(x2, ops.linear(y.view(B * T, dl), self.sd[p + "attn.c_proj.weight"]))
            else:
                hist, pos = cache[i]
                t0 = host_pos(pos)
                if t0 + T > self.capacity:
                    raise ValueError(f"sequence position {t0 + T} exceeds the capacity {self.capacity}")
                MinT, taps, taps8 = self._stu_weights(i)
                if T == 1 and taps8 is not None and self.fused_decode:
                    # one token: the fused kernel on this rank's channels (norm, projection, cache append, taps;
                    # position read on the device, so the step can be replayed from a graph)
                    y_loc = torch.empty(B, 1, dl, dtype=self.dtype, device=self.device)
                    ops.decode_approx_shard(x2, self.sd[p + "stu_norm.weight"], MinT, hist, taps8, pos, y_loc.view(B, dl),
                                            self.eps)
                else:
                    xn = ops.rmsnorm(x2, self.sd[p + "stu_norm.weight"], self.eps)
                    ops.linear(xn, MinT, out=hist, epilogue=ops.EPI_HIST, hist_T=T, hist_t0=t0, hist_Lh=self.Lh)
                    y_loc = torch.zeros(B, T, dl, dtype=self.dtype, device=self.device)
                    yT = torch.empty(B, dl, 2, _round_up((t0 + T + 1) // 2, 8), dtype=self.dtype, device=self.device)
                    if taps8 is not None and ops.conv_prefill_tc5_supported(hist, y_loc):
                        ops.conv_prefill_approx_tc5(hist, taps8, yT, y_loc, t0, t0 + T)
                    else:
                        ops.conv_prefill_approx(hist, taps, yT, y_loc, t0, t0 + T,
                                                use_tensor_cores=(self.dtype == torch.bfloat16 and dl % 8 == 0))
                    pos[:, 0] += T
                pos._host_t = t0 + T
                gathered = torch.empty(self.world, B, T, dl, dtype=self.dtype, device=self.device)
                dist.all_gather_into_tensor(gathered, y_loc, group=self.group)
                x.add_(gathered.permute(1, 2, 0, 3).reshape(B, T, d))
            self._mlp(x2, i)
        return x

    # ------------------------------------------------------------------ token step with fused exchanges
    def _exchange_for(self, B: int):
        """The peer buffers for token steps of B sequences (collective on first use; every rank makes the same calls)."""
        ok = (self.fused_exchange and self.world > 1 and self.device.type == "cuda" and self.dtype == torch.bfloat16
              and self.fused_decode and self.dl % 8 == 0 and B <= 64 and self.world <= 8)
        # the default ("exchange") also follows the message size: above 256 KB per exchange (64 sequences of d=3072:
        # 393 KB) NCCL between the kernels measured faster on two GPUs (8.90 against 9.26 ms per step), below it the
        # exchange kernel does (32 sequences of d=1536, 98 KB: 2.16 against 2.39 ms)
        if ok and self.fused_exchange == "exchange" and B * self.d * 2 > 256 * 1024:
            ok = False
        if not ok:
            return None
        if self._exchange is None or self._exchange.rows != B:
            from .peer import GATHER, REDUCE, PeerExchange
            if self._exchange is not None:
                torch.cuda.synchronize(self.device)
                self._exchange.close()
            kinds = []
            for i in range(self.cfg.n_layers):
                kinds += [REDUCE if self._is_attn(i) else GATHER, REDUCE]
            self._exchange = PeerExchange.connect(kinds, B, self.d, group=self.group)
            self._xn = [torch.empty(B, self.d, dtype=self.dtype, device=self.device) for _ in range(2)]
        return self._exchange

    def _token_step_fused(self, ids: torch.Tensor, cache, ex):
        """One new token per sequence: (residual stream [B,1,d], final-norm rows [B,d]).  Per layer the kernels are
        [STU shard decode | c_attn, attention, c_proj], exchange (+ MLP norm), gate/up, down, exchange (+ the next
        explicit norm); in "push" mode the producing kernels store into the inboxes and a combine kernel waits."""
        B = ids.shape[0]
        d, dl, n_layers = self.d, self.dl, self.cfg.n_layers
        x = ops.embed(ids, self.sd["tok_emb.weight"])
        x2 = x.view(B, d)
        xa, xb = self._xn
        push = self.fused_exchange == "push"
        have_norm = False      # xa holds the attention norm of the current layer's input
        e = 0
        for i in range(n_layers):
            p = f"layers.{i}."
            if self._is_attn(i):
                k_ring, v_ring, pos = cache[i]
                t0 = host_pos(pos)
                if not have_norm:
                    ops.rmsnorm(x2, self.sd[p + "attn_norm.weight"], self.eps, out=xa)
                qkv = ops.linear(xa, self.sd[p + "attn.c_attn.weight"]).view(B, 1, 3 * dl)
                y = ops.swa_forward(qkv, k_ring, v_ring, pos, self.slopes, self.Hl, self.window, self.cfg.softcap,
                                    update_cache=True)
                pos._host_t = t0 + 1
                if push:
                    ops.linear_push(y.view(B, dl), self.sd[p + "attn.c_proj.weight"], ex.dest(e), d)
                else:
                    src = ops.linear(y.view(B, dl), self.sd[p + "attn.c_proj.weight"])
            else:
                hist, pos = cache[i]
                t0 = host_pos(pos)
                if t0 + 1 > self.capacity:
                    raise ValueError(f"sequence position {t0 + 1} exceeds the capacity {self.capacity}")
                MinT, _, taps8 = self._stu_weights(i)
                if push:
                    ops.decode_approx_push(x2, self.sd[p + "stu_norm.weight"], MinT, hist, taps8, pos, ex.dest(e), d,
                                           self.eps)
                else:
                    src = torch.empty(B, dl, dtype=self.dtype, device=self.device)
                    ops.decode_approx_shard(x2, self.sd[p + "stu_norm.weight"], MinT, hist, taps8, pos, src, self.eps)
                pos._host_t = t0 + 1
            if push:
                ex.combine(e, x2, norm_w=self.sd[p + "mlp_norm.weight"], xn=xb, eps=self.eps)
            else:
                ex.exchange(e, x2, src, norm_w=self.sd[p + "mlp_norm.weight"], xn=xb, eps=self.eps)
            e += 1
            h = ops.linear(xb, self.sd[p + "mlp.gate_proj.weight"], W2=self.sd[p + "mlp.up_proj.weight"],
                           epilogue=ops.EPI_GELU_MUL)
            if i + 1 == n_layers:
                nw = self.sd["norm.weight"]
            elif self._is_attn(i + 1):
                nw = self.sd[f"layers.{i + 1}.attn_norm.weight"]
            else:
                nw = None      # the STU shard kernel normalises its input itself
            if push:
                ops.linear_push(h, self.sd[p + "mlp.down_proj.weight"], ex.dest(e), d)
                ex.combine(e, x2, norm_w=nw, xn=xa if nw is not None else None, eps=self.eps)
            else:
                ex.exchange(e, x2, ops.linear(h, self.sd[p + "mlp.down_proj.weight"]), norm_w=nw,
                            xn=xa if nw is not None else None, eps=self.eps)
            have_norm = nw is not None
            e += 1
        return x, xa

    def last_logits(self, ids: torch.Tensor, cache):
        ex = self._exchange_for(ids.shape[0]) if ids.shape[1] == 1 else None
        if ex is not None:
            x, last = self._token_step_fused(ids, cache, ex)
        else:
            x = self.hidden(ids, cache)
            last = ops.rmsnorm(x[:, -1].contiguous(), self.sd["norm.weight"], self.eps)
        loc = ops.linear(last, self.sd["lm_head.weight"])                     # [B, ceil(V/g)]
        allv = torch.empty(self.world, *loc.shape, dtype=loc.dtype, device=loc.device)
        dist.all_gather_into_tensor(allv, loc.contiguous(), group=self.group)
        return allv.permute(1, 0, 2).reshape(loc.shape[0], -1)[:, :self.V].contiguous()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_length: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, do_sample: bool = False,
                 uniforms: Optional[torch.Tensor] = None, return_logits: bool = False, cuda_graph: bool = True,
                 fence=None, fence_every: int = 16, timings: Optional[dict] = None):
        """Cached token loop; `uniforms` [steps, B] must be the same on every rank when sampling.
        `fence` (parallel.StepFence): every `fence_every` steps the ranks meet on the host between steps; a rank that
        is gone makes the others raise parallel.RankLost instead of entering a collective that would never finish."""
        B, T0 = input_ids.shape
        steps = max_length - T0
        if do_sample and uniforms is None:
            raise ValueError("sampling under tensor parallelism needs the same uniforms on every rank")
        gen = torch.empty(B, max_length, dtype=torch.int64, device=self.device)
        gen[:, :T0] = input_ids
        cache = self.new_cache(B)
        logs = []
        # as in FlashSTU.generate: cached steps after the first are replayed from one captured CUDA graph (the NCCL
        # collectives are captured with the kernels; every rank captures and replays in lock step)
        # (the unfused one-token path passes its position to the kernels as an argument and cannot be replayed)
        use_graph = cuda_graph and steps > 3 and max_length - 1 <= self.capacity and self.fused_decode and \
            self.dtype == torch.bfloat16 and self.dl % 8 == 0
        graph = None
        for step in range(steps):
            cur = T0 + step
            if fence is not None and step % fence_every == 0:
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)   # nothing of this rank is in flight while it waits
                fence.arrive(step)
            u = uniforms[step].to(self.device, torch.float32).contiguous() if do_sample else None
            if use_graph and step >= 2:
                if graph is None:
                    tok_in = torch.empty(B, 1, dtype=torch.int64, device=self.device)
                    tok_out = torch.empty(B, 1, dtype=torch.int64, device=self.device)
                    u_buf = torch.zeros(B, dtype=torch.float32, device=self.device)
                    host_t = [getattr(e[-1], "_host_t", None) for e in cache]
                    torch.cuda.synchronize(self.device)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        logits_g = self.last_logits(tok_in, cache)
                        ops.sample(logits_g, temperature, top_k, top_p, do_sample, u_buf if do_sample else None, tok_out,
                                   out_stride=1)
                    for e, t in zip(cache, host_t):
                        e[-1]._host_t = t
                if timings is not None and "_first" not in timings:
                    timings["_first"] = torch.cuda.Event(enable_timing=True)
                    timings["_first"].record()
                    timings["replayed_steps"] = 0
                tok_in.copy_(gen[:, cur - 1:cur])
                if do_sample:
                    u_buf.copy_(u)
                graph.replay()
                if timings is not None:
                    timings["replayed_steps"] += 1
                for e in cache:
                    e[-1]._host_t += 1
                gen[:, cur:cur + 1].copy_(tok_out)
                if return_logits:
                    logs.append(logits_g.clone())
                continue
            inp = gen[:, :cur] if step == 0 else gen[:, cur - 1:cur]
            logits = self.last_logits(inp.contiguous(), cache)
            if return_logits:
                logs.append(logits)
            ops.sample(logits, temperature, top_k, top_p, do_sample, u, gen[:, cur:], out_stride=max_length)
        if timings is not None and "_first" in timings:   # device time of the graph-replayed token steps
            last = torch.cuda.Event(enable_timing=True)
            last.record()
            last.synchronize()
            timings["replay_ms"] = timings.pop("_first").elapsed_time(last)
        return (gen, torch.stack(logs, 1)) if return_logits else gen
