"""Tensor-parallel sharding on CPU (gloo, world_size 2): the shards cut by tensor_parallel.shard_state_dict,
pushed through the reference arithmetic (oracle) with one all-gather per STU layer, one all-reduce per attention
and per MLP block and an all-gather of the vocabulary shards, reproduce the reference's logits."""
import math
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as Fn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tp_logits(ids, full_sd, cfg, rank, world):
    from oracle import stu_oracle as O
    from flash_stu_2_b200.tensor_parallel import shard_state_dict
    d, H, V = cfg["n_embd"], cfg["n_heads"], cfg["vocab_size"]
    hd, Hl = d // H, H // world
    sd = shard_state_dict(full_sd, dict(n_embd=d, n_heads=H), rank, world)
    n = O.fft_length(cfg["seq_len"])
    x = Fn.embedding(ids, sd["tok_emb.weight"])
    B, T = ids.shape
    for i in range(cfg["n_layers"]):
        p = {k[len(f"layers.{i}."):]: v for k, v in sd.items() if k.startswith(f"layers.{i}.")}
        if O.layer_is_attention(i, cfg["use_attn"]):
            xn = O.rmsnorm(x, p["attn_norm.weight"])
            q, k, v = torch.chunk(Fn.linear(xn, p["attn.c_attn.weight"]), 3, dim=2)
            q, k, v = (t.reshape(B, T, Hl, hd) for t in (q, k, v))
            ii, jj = torch.arange(T)[:, None], torch.arange(T)[None, :]
            s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(hd)
            s = cfg["softcap"] * torch.tanh(s / cfg["softcap"])
            slopes = O.alibi_slopes(H)[rank * Hl:(rank + 1) * Hl]
            s = s - slopes[None, :, None, None] * (ii - jj).abs()[None, None].float()
            s = s.masked_fill(~((jj <= ii) & (jj >= ii - cfg["window_size"]))[None, None], float("-inf"))
            y = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float()).to(x.dtype).reshape(B, T, Hl * hd)
            part = Fn.linear(y, p["attn.c_proj.weight"])
            dist.all_reduce(part)
            x = x + part
        else:
            xn = O.rmsnorm(x, p["stu_norm.weight"])
            y_loc = O.stu_forward(xn, sd["phi"], {"M_inputs": p["stu.M_inputs"], "M_filters": p["stu.M_filters"]}, n, True)
            parts = [torch.empty_like(y_loc) for _ in range(world)]
            dist.all_gather(parts, y_loc.contiguous())
            x = x + torch.cat(parts, dim=2)
        xn = O.rmsnorm(x, p["mlp_norm.weight"])
        h = Fn.gelu(Fn.linear(xn, p["mlp.gate_proj.weight"]), approximate="tanh") * Fn.linear(xn, p["mlp.up_proj.weight"])
        part = Fn.linear(h, p["mlp.down_proj.weight"])
        dist.all_reduce(part)
        x = x + part
    loc = Fn.linear(O.rmsnorm(x, sd["norm.weight"])[:, -1], sd["lm_head.weight"])
    parts = [torch.empty_like(loc) for _ in range(world)]
    dist.all_gather(parts, loc.contiguous())
    return torch.cat(parts, dim=1)[:, :V]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import sys
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    r = torch.load(os.path.join(ROOT, "tests", "golden", "models.pt"), map_location="cpu", weights_only=False)["hybrid_approx_fp32"]
    with torch.no_grad():
        got = _tp_logits(r["ids"], r["sd"], r["cfg"], rank, world)
    want = r["logits_full"][:, -1]
    err = float((got.double() - want.double()).norm() / want.double().norm())
    q.put((rank, err, got[:, :5].tolist()))
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_algebra_matches_reference(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] <= 1e-4 for r in res), res
    assert all(r[2] == res[0][2] for r in res)          # every rank ends with the same logits


def test_shards_tile_the_full_weights():
    from flash_stu_2_b200.tensor_parallel import shard_state_dict
    d, H, K, inter, V = 32, 4, 8, 128, 97
    torch.manual_seed(0)
    sd = {"layers.0.stu.M_inputs": torch.randn(d, d), "layers.0.stu.M_filters": torch.randn(K, d),
          "layers.0.mlp.gate_proj.weight": torch.randn(inter, d), "layers.0.mlp.up_proj.weight": torch.randn(inter, d),
          "layers.0.mlp.down_proj.weight": torch.randn(d, inter), "layers.1.attn.c_attn.weight": torch.randn(3 * d, d),
          "layers.1.attn.c_proj.weight": torch.randn(d, d), "lm_head.weight": torch.randn(V, d),
          "norm.weight": torch.ones(d)}
    for world in (2, 4):
        sh = [shard_state_dict(sd, dict(n_embd=d, n_heads=H), r, world) for r in range(world)]
        assert torch.equal(torch.cat([s["layers.0.stu.M_inputs"] for s in sh], 1), sd["layers.0.stu.M_inputs"])
        assert torch.equal(torch.cat([s["layers.0.mlp.gate_proj.weight"] for s in sh], 0), sd["layers.0.mlp.gate_proj.weight"])
        assert torch.equal(torch.cat([s["layers.0.mlp.down_proj.weight"] for s in sh], 1), sd["layers.0.mlp.down_proj.weight"])
        assert torch.equal(torch.cat([s["layers.1.attn.c_proj.weight"] for s in sh], 1), sd["layers.1.attn.c_proj.weight"])
        qkv = torch.cat([s["layers.1.attn.c_attn.weight"].view(3, H // world, d // H, d) for s in sh], 1)
        assert torch.equal(qkv.reshape(3 * d, d), sd["layers.1.attn.c_attn.weight"])
        assert torch.equal(torch.cat([s["lm_head.weight"] for s in sh], 0)[:V], sd["lm_head.weight"])
        assert all(s["norm.weight"] is sd["norm.weight"] for s in sh)
