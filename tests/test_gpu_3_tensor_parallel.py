"""Tensor-parallel token loop on two GPUs (NCCL): every rank cuts its shard out of the fixture's full state dict,
prefill logits are checked against the reference's (tests/golden/models.pt), a cached step against the
reference's shorter-prefix logits, and both ranks must generate the same tokens as the single-GPU model.  In bf16 the
cached steps run with the sub-layer exchanges fused into the kernels (stores into the other ranks' inboxes over
NVLink); the same steps through the NCCL collectives must give the same logits and tokens."""
import os
import socket

import pytest
import torch

from parity import close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, name, q):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flash_stu_2_b200 as F
        from flash_stu_2_b200 import ops
        from flash_stu_2_b200.tensor_parallel import TensorParallelFlashSTU
        r = torch.load(os.path.join(ROOT, "tests", "golden", "models.pt"), map_location="cpu", weights_only=False)[name]
        dt = getattr(torch, r["dtype"])
        cfg = F.FlashSTUConfig(torch_dtype=dt, **r["cfg"])
        tp = TensorParallelFlashSTU(cfg, r["sd"], dev)
        ids = r["ids"].to(dev)
        with torch.no_grad():
            full = tp.last_logits(ids, tp.new_cache(ids.shape[0])).float().cpu()
            T = r["T_short"]
            cache = tp.new_cache(ids.shape[0])
            tp.last_logits(ids[:, :T - 1].contiguous(), cache)
            short = tp.last_logits(ids[:, T - 1:T].contiguous(), cache).float().cpu()     # one cached step
            gen = tp.generate(ids[:, :9].contiguous(), max_length=21, do_sample=False).cpu()
            fused = tp._exchange is not None
            tp.fused_exchange = False                     # the same cached step and token loop through NCCL
            cache = tp.new_cache(ids.shape[0])
            tp.last_logits(ids[:, :T - 1].contiguous(), cache)
            short_nccl = tp.last_logits(ids[:, T - 1:T].contiguous(), cache).float().cpu()
            gen_nccl = tp.generate(ids[:, :9].contiguous(), max_length=21, do_sample=False).cpu()
        ops.check_status()
        single = None
        if rank == 0:   # the unsharded model on this GPU
            fp = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"phi_tp_{os.getpid()}.pt")
            F.save_spectral_filters(r["sd"]["phi"].float(), fp)
            m = F.FlashSTU(F.FlashSTUConfig(filter_path=fp, torch_dtype=dt, **r["cfg"]))
            m.load_state_dict(r["sd"])
            m = m.to(dev).eval()
            single = m.generate(ids[:, :9].contiguous(), max_length=21, do_sample=False).cpu()
            os.remove(fp)
        q.put((rank, full, short, gen, single, fused, short_nccl, gen_nccl))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("name", ["hybrid_approx_fp32", "hybrid_approx_bf16"])
def test_two_gpu_tensor_parallel_model(name, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    import torch.multiprocessing as mp
    from oracle import stu_oracle as O
    r = torch.load(os.path.join(ROOT, "tests", "golden", "models.pt"), map_location="cpu", weights_only=False)[name]
    tol = 1e-3 if r["dtype"] == "float32" else 2e-2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(rk, world, port, name, q)) for rk in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=300) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, full, short, gen, single, fused, short_nccl, gen_nccl in res:
        close(full, r["logits_full"][:, -1].float(), tol)
        close(short, r["logits_short"][:, -1].float(), tol)
        close(short_nccl, r["logits_short"][:, -1].float(), tol)
        assert fused == (r["dtype"] == "bfloat16")           # bf16 token steps took the fused exchanges
        if fused:
            close(short, short_nccl, 1e-2, what="fused exchange vs NCCL")
            # the same greedy tokens wherever the two largest logits are not within rounding of each other
            assert (gen == gen_nccl).float().mean() > 0.9
    assert all(torch.equal(res[0][3], rr[3]) for rr in res[1:])   # every rank generates the same tokens
    if r["dtype"] == "float32":
        assert torch.equal(res[0][3], res[0][4])             # and, in fp32, the single-GPU model's
