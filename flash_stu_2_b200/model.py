"""FlashSTU language model and its token loop (flash_stu/model.py:26-304) on the CUDA kernels.

Same constructor, forward() and generate() signatures as the reference.  Differences that a caller
can observe, all forced by the reference's own gaps:
  * STU layers keep a decode cache (the reference's return None, so its cached generate() feeds a
    length-1 sequence to the convolution); one cached step here equals the full-prefix forward row;
  * inside generate() only the last position goes through the LM head;
  * sampling draws by inverse CDF from one uniform per sequence (optionally passed as
    `uniforms=[steps,B]` or drawn from `generator=`) instead of torch.multinomial.
"""
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import transformers
from transformers import PreTrainedModel
from transformers.modeling_outputs import CausalLMOutputWithPast

from . import ops
from .config import FlashSTUConfig
from .filters import get_spectral_filters, nearest_power_of_two
from .layers import AttentionLayer, STULayer
from .modules import STU, Attention, RMSNorm


class FlashSTU(PreTrainedModel):
    config_class = FlashSTUConfig
    # lm_head.weight is tok_emb.weight (flash_stu/model.py:50,99-102); transformers >= 5 wants the tie as a
    # {tied: source} mapping, older versions as a list of tied keys
    _tied_weights_keys = ({"lm_head.weight": "tok_emb.weight"} if int(transformers.__version__.split(".")[0]) >= 5
                          else ["lm_head.weight"])

    def __init__(self, config: FlashSTUConfig) -> None:
        super().__init__(config)
        self.config = config
        self.n_layers = config.n_layers
        self.n = nearest_power_of_two(config.seq_len * 2 - 1, round_up=True)
        self.use_approx = config.use_approx
        self.use_hankel_L = config.use_hankel_L
        phi = get_spectral_filters(config.seq_len, config.num_eigh, use_hankel_L=config.use_hankel_L,
                                   dtype=config.torch_dtype, load_from=config.filter_path)
        self.register_buffer("phi", phi, persistent=True)
        self.tok_emb = nn.Embedding(config.vocab_size, config.n_embd, dtype=config.torch_dtype)
        self.dropout = nn.Dropout(config.dropout)
        self.layers = nn.ModuleList()
        for idx in range(self.n_layers):
            if idx % 2 == 1 and config.use_attn:
                self.layers.append(AttentionLayer(config))
            else:
                self.layers.append(STULayer(config, self.phi, self.n))
        self.norm = RMSNorm(config.n_embd, dtype=config.torch_dtype)
        if config.bias:
            raise NotImplementedError("bias=True has no kernel here (the reference default is bias=False)")
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False, dtype=config.torch_dtype)
        self.tok_emb.weight = self.lm_head.weight
        self.std = config.n_embd ** -0.5
        # registers the tie and the other bookkeeping transformers keeps per model, then applies _init_weights to
        # every module (what the reference does with self.apply, flash_stu/model.py:104-105)
        self.post_init()

    # ------------------------------------------------------------------ checkpoints
    def _restore_derived_buffers(self):
        """Non-persistent buffers are not in a checkpoint: the STU layers' view of the filters (the reference registers
        it with persistent=False, flash_stu/modules/stu.py:36-41) and the ALiBi slopes (attention.py:34).  A loader
        that builds the module tree on the meta device and then materialises it leaves them uninitialised, so after
        loading they are re-derived from what the checkpoint does hold: `phi` and the configuration."""
        for layer in self.layers:
            if isinstance(layer, STULayer):
                layer.stu.phi = self.phi
                layer.stu._prep_key = None
            else:
                attn = layer.attn
                attn.alibi_slopes = attn._get_alibi_slopes(attn.n_heads).to(self.phi.device)

    @classmethod
    def from_pretrained(cls, *args, **kwargs):
        model = super().from_pretrained(*args, **kwargs)
        model._restore_derived_buffers()
        return model

    # ------------------------------------------------------------------ embeddings (resize_token_embeddings)
    def get_input_embeddings(self):
        return self.tok_emb

    def set_input_embeddings(self, value):
        self.tok_emb = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, value):
        self.lm_head = value

    # ------------------------------------------------------------------ backbone
    def _backbone(self, input_ids, past_key_values, use_cache: bool, collect_hidden: bool = False):
        if not input_ids.is_cuda:
            raise RuntimeError("flash_stu_2_b200 has no CPU path: move the model and input_ids to a CUDA device")
        if self.training and self.config.dropout > 0:
            raise NotImplementedError("dropout > 0 in training mode has no kernel here (inference path only)")
        x = ops.embed(input_ids, self.tok_emb.weight)
        hidden = (x.clone(),) if collect_hidden else None
        cache = () if use_cache else None
        for idx, layer in enumerate(self.layers):
            past = past_key_values[idx] if past_key_values is not None else None
            if use_cache:
                x, present = layer(x, past_key_value=past, use_cache=True)
                cache = cache + (present,)
            else:
                x = layer(x, past_key_value=past, use_cache=False)
            if collect_hidden:
                hidden = hidden + (x.clone(),)
        return x, cache, hidden

    def forward(
        self,
        input_ids: Optional[torch.LongTensor] = None,
        attention_mask: Optional[torch.Tensor] = None,
        past_key_values: Optional[Tuple[Tuple[torch.Tensor]]] = None,
        labels: Optional[torch.LongTensor] = None,
        use_cache: Optional[bool] = None,
        output_hidden_states: Optional[bool] = None,
        return_dict: Optional[bool] = None,
        **kwargs,
    ):
        if input_ids is None:
            raise ValueError("input_ids must be provided")
        if labels is not None:
            raise NotImplementedError("the loss/labels path is training code and is not part of this implementation")
        return_dict = True if return_dict is None else return_dict
        use_cache = use_cache if use_cache is not None else bool(getattr(self.config, "use_cache", False))
        x, cache, hidden = self._backbone(input_ids, past_key_values, use_cache, bool(output_hidden_states))
        B, T, d = x.shape
        xn = ops.rmsnorm(x, self.norm.weight, self.norm.eps)
        logits = ops.linear(xn.view(B * T, d), self.lm_head.weight).view(B, T, -1)
        if not return_dict:
            out = (logits,)
            if use_cache:
                out = out + (cache,)
            if output_hidden_states:
                out = out + (hidden,)
            return out
        return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=cache,
                                      hidden_states=hidden if output_hidden_states else None)

    def last_logits(self, input_ids, past_key_values=None, use_cache: bool = True):
        """Logits of the last position only, [B,V], plus the cache (what the token loop needs)."""
        x, cache, _ = self._backbone(input_ids, past_key_values, use_cache)
        last = x[:, -1]
        V = self.lm_head.weight.shape[0]
        B = last.shape[0]
        # logits rows padded to a multiple of 8 elements: the tensor-core GEMM needs 16-byte aligned output rows
        # and the vocabulary (50257) is odd
        Vp = (V + 7) // 8 * 8
        logits = torch.empty(B, Vp, dtype=last.dtype, device=last.device)[:, :V]
        if ops.can_fuse_norm(B, V, last.shape[1], ops.EPI_STORE, last.dtype) and last.stride(1) == 1:
            ops.linear(last, self.lm_head.weight, out=logits, norm_w=self.norm.weight, eps=self.norm.eps)
        else:
            ops.linear(ops.rmsnorm(last.contiguous(), self.norm.weight, self.norm.eps), self.lm_head.weight, out=logits)
        return logits, cache

    # ------------------------------------------------------------------ token loop
    @torch.no_grad()
    def generate(
        self,
        input_ids: torch.LongTensor,
        max_length: int = 100,
        temperature: float = 1.0,
        top_k: Optional[int] = None,
        top_p: Optional[float] = None,
        do_sample: bool = True,
        use_cache: bool = True,
        **kwargs,
    ) -> torch.LongTensor:
        """The reference's token loop (flash_stu/model.py:207-304) with a cache in every layer.

        Differences from the reference a caller can observe: (1) a sampled token is drawn by inverse CDF from ONE
        uniform number per sequence and step (`uniforms` [steps, B], else `generator`), walking the kept entries in
        vocabulary order, where the reference calls torch.multinomial: same distribution, other random stream;
        (2) the nucleus cut sums probability mass in 40-bit fixed point, so an entry whose cumulative mass lies
        within 2^-40 of top_p may fall on the other side of the cut; (3) a row with a NaN logit gets the token
        floor(u * vocab_size) from its uniform (the reference draws a uniformly random token there);
        (4) prompts may be shorter than seq_len and steps read cached state (the reference recomputes the prefix);
        (5) nucleus filtering without top_k, and top_k above 1024, need the vocabulary row in shared memory (at
        most 51712 entries; status 5 / 4 otherwise).  kwargs: uniforms, generator, return_logits, cuda_graph (replay
        the cached steps from one captured graph, default True), timings (dict filled with the device time of the
        replayed steps)."""
        uniforms = kwargs.get("uniforms")
        generator = kwargs.get("generator")
        return_logits = kwargs.get("return_logits", False)
        timings = kwargs.get("timings")   # optional dict: filled with the device time of the graph-replayed steps
        ev_first = ev_last = None
        replayed = 0
        B, T0 = input_ids.shape
        steps = max_length - T0
        if steps <= 0:
            return input_ids
        dev = input_ids.device
        generated = torch.empty(B, max_length, dtype=torch.int64, device=dev)
        generated[:, :T0] = input_ids
        all_logits = []
        past = None
        # Cached token steps after the first are replayed from one captured CUDA graph (every kernel reads its
        # position from device memory): the step is ~100 small launches for a 24-layer model, which the interpreter
        # cannot issue as fast as the GPU retires them.  cuda_graph=False keeps the eager loop.
        capacity = min(self.config.seq_len, getattr(self.config, "cache_len", None) or self.config.seq_len)
        use_graph = bool(kwargs.get("cuda_graph", True)) and use_cache and steps > 3 and max_length - 1 <= capacity
        # a sandwich layer's token step reads its position on the device only in the bf16 approx form
        for layer in self.layers:
            if getattr(layer, "stu_mlp_enabled", False) and not (
                    layer.stu.use_approx and self.config.torch_dtype == torch.bfloat16
                    and layer.stu_mlp_hidden_size % 8 == 0):
                use_graph = False
            if hasattr(layer, "stu") and layer.stu.use_approx and layer.stu.use_hankel_L:
                use_graph = False   # the single-branch token step is a one-position prefill (host position)
        graph = None
        for step in range(steps):
            cur = T0 + step
            u = None
            if do_sample:
                u = uniforms[step].to(device=dev, dtype=torch.float32).contiguous() if uniforms is not None else \
                    torch.rand(B, device=dev, generator=generator)
            if use_graph and past is not None and step >= 2:
                if graph is None:
                    tok_in = torch.empty(B, 1, dtype=torch.int64, device=dev)
                    tok_out = torch.empty(B, 1, dtype=torch.int64, device=dev)
                    u_buf = torch.zeros(B, dtype=torch.float32, device=dev)
                    host_t = [getattr(e[-1], "_host_t", None) if e is not None else None for e in past]
                    torch.cuda.synchronize(dev)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        logits_g, _ = self.last_logits(tok_in, past, True)
                        ops.sample(logits_g, temperature, top_k, top_p, do_sample, u_buf if do_sample else None, tok_out,
                                   out_stride=1)
                    for e, t in zip(past, host_t):   # capturing ran the host bookkeeping, not the kernels
                        if e is not None and t is not None:
                            e[-1]._host_t = t
                if timings is not None and ev_first is None:
                    ev_first = torch.cuda.Event(enable_timing=True)
                    ev_first.record()
                tok_in.copy_(generated[:, cur - 1:cur])
                if do_sample:
                    u_buf.copy_(u)
                graph.replay()
                replayed += 1
                for e in past:
                    if e is not None and getattr(e[-1], "_host_t", None) is not None:
                        e[-1]._host_t += 1
                generated[:, cur:cur + 1].copy_(tok_out)
                if return_logits:
                    all_logits.append(logits_g.clone())
                continue
            if use_cache and past is not None:
                inp = generated[:, cur - 1:cur]
            else:
                inp = generated[:, max(0, cur - self.config.seq_len):cur]
                past = None
            logits, past = self.last_logits(inp, past, use_cache)
            if return_logits:
                all_logits.append(logits)
            ops.sample(logits, temperature, top_k, top_p, do_sample, u, generated[:, cur:], out_stride=max_length)
        if timings is not None and ev_first is not None:
            ev_last = torch.cuda.Event(enable_timing=True)
            ev_last.record()
            ev_last.synchronize()
            timings["replayed_steps"] = replayed
            timings["replay_ms"] = ev_first.elapsed_time(ev_last)
        if return_logits:
            return generated, torch.stack(all_logits, dim=1)
        return generated

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, use_cache=None,
                                      **kwargs) -> Dict[str, Any]:
        if past_key_values is not None:
            input_ids = input_ids[:, -1:]
        return {"input_ids": input_ids, "past_key_values": past_key_values, "use_cache": use_cache,
                "attention_mask": attention_mask}

    @staticmethod
    def _reorder_cache(past_key_values, beam_idx: torch.Tensor):
        out = ()
        for layer_past in past_key_values:
            if layer_past is None:
                out += (None,)
            else:
                out += (tuple(t.index_select(0, beam_idx.to(t.device)) for t in layer_past),)
        return out

    def get_num_params(self, non_embedding: bool = False) -> int:
        n = sum(p.numel() for p in self.parameters())
        if non_embedding:
            n -= self.tok_emb.weight.numel()
        return n

    def _get_num_params(self):
        return self.get_num_params(non_embedding=False)

    def _init_weights(self, module):
        # same initialisers and the same running `std` rescale on SCALE_INIT modules as
        # flash_stu/model.py:428-452
        if isinstance(module, nn.Linear):
            if hasattr(module, "SCALE_INIT"):
                self.std *= (2 * self.n_layers) ** -0.5
            torch.nn.init.normal_(module.weight, mean=0.0, std=self.std)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=self.std)
        elif isinstance(module, STU):
            if module.use_approx:
                torch.nn.init.xavier_normal_(module.M_inputs)
                torch.nn.init.xavier_normal_(module.M_filters)
            else:
                torch.nn.init.xavier_normal_(module.M_phi_plus)
                if not module.use_hankel_L:
                    torch.nn.init.xavier_normal_(module.M_phi_minus)
        elif isinstance(module, Attention):
            torch.nn.init.xavier_normal_(module.c_attn.weight)
            torch.nn.init.xavier_normal_(module.c_proj.weight)
