"""Benchmark of the Flash STU token loop on B200: standalone FlashSTUBlock (approx variant), bf16,
B=8 sequences per GPU, L=8192, d_model=1024, K=24 -- the 8K-context block configuration.

One step = one pass of the hot path over one batch of synthetic input:
  prefill  the block forward over all L positions (fills the decode cache), then
  decode   `--decode-steps` (512) cached single-token steps at positions L-512 .. L-1, teacher-forced from
           the same inputs (so every decode row is checkable against the prefill rows).
`value` is decode tokens/s summed over GPUs with inputs resident in HBM (CUDA events, max over ranks);
`prefill` holds the prefill tokens/s of the same steps; `e2e` repeats the step through the public
module API from pinned host buffers with the host<->device copies inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
Launch with torch.distributed.run for N > 1 (one rank per GPU, weak scaling: B=8 per GPU, no collective
on the data path; NCCL only carries the max-over-ranks of the timings).
`--impl reference` times the CPU restatement of the reference's path (oracle/) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D_MODEL, NUM_FILTERS = 1024, 24
# dram__bytes_read.sum + dram__bytes_write.sum of one stu_decode_rows8_kernel launch at B=8, L=8192, t~7690, from one ncu
# capture of this command (algorithmic bytes there: 73.0 MB)
DECODE_KERNEL_DRAM_BYTES = 79.8e6
# the same two counters for one stu_block_step_kernel launch (the whole token step) at B=8, L=8192 (None until captured)
STEP_KERNEL_DRAM_BYTES = 106.0e6


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU (default: the benchmark's 8)")
    ap.add_argument("--seq-len", type=int, default=8192, help="context length (default: the benchmark's 8192)")
    ap.add_argument("--decode-steps", type=int, default=512)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--variant", choices=["approx", "full"], default="approx",
                    help="STU variant of the block: approx (M_inputs/M_filters, the headline) or full (M_phi_plus/minus)")
    ap.add_argument("--model", choices=["c1", "c3", "c4", "c5"], default=None,
                    help="instead of the headline block workload, time FlashSTU.generate() on a whole model: "
                         "c1 = d512/12 layers/fp32/B=2/prompt 128/+128 greedy; "
                         "c3 = d1536/24 layers/bf16/B=32/prompt 2048/+512, top_k=40, T=0.8; "
                         "c5 = d3072/32 layers/bf16/B=64/prompt 8192/+1024 greedy, seq_len 32768 (cache laid out for "
                         "9216 positions); "
                         "c4 = 12 stacked MiniSTU(backend='lds', 1024->1024), bf16, B=16, prefill 15360 + 1024 steps")
    ap.add_argument("--tp", action="store_true",
                    help="with --model c1|c3 under torchrun: shard the model over the ranks (tensor parallelism) "
                         "instead of running it on one GPU")
    ap.add_argument("--new-tokens", type=int, default=None, help="with --model: tokens to generate (default: the config's)")
    ap.add_argument("--kernel-split", action="store_true",
                    help="also time every kernel of the token step in a graph of its own (adds `decode_split`)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="plain stream-ordered launches for the decode kernels (no programmatic dependent launch)")
    ap.add_argument("--no-graph", action="store_true", help="launch decode steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--early-decode", type=int, default=1, choices=[0, 1],
                    help="1: the STU decode kernel starts while the down projection before it still runs (only its "
                         "projection waits for it); 0: it starts after it")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the extra objects of the default line (`generate`: the 24-layer model through "
                         "FlashSTU.generate(); `tp`, N > 1 only: the 3B shapes tensor-parallel over the N ranks)")
    ap.add_argument("--cache-len", type=int, default=None,
                    help="with --model: positions the layer caches hold (default: the config's seq_len)")
    ap.add_argument("--extra-new-tokens", type=int, default=64, help="tokens generated for the `generate` object")
    ap.add_argument("--tp-new-tokens", type=int, default=32, help="tokens generated for the `tp` object")
    ap.add_argument("--conv-timeline", action="store_true",
                    help="adds `conv_timeline`: %%globaltimer stamps of CTA 0 inside one launch of the tcgen05 prefill "
                         "convolution (first 8 units and phases, microseconds after the first stage became free)")
    ap.add_argument("--step-timeline", action="store_true",
                    help="adds `step_timeline`: %%globaltimer stamps of CTA 0 inside three launches of the fused token-step "
                         "kernel (us after kernel entry)")
    ap.add_argument("--lds-layers", type=int, default=12, help="with --model c4: number of stacked layers")
    ap.add_argument("--lds-batch", type=int, default=16, help="with --model c4: sequences")
    ap.add_argument("--fused-step", type=int, default=1, choices=[0, 1],
                    help="1: a token step of the block is one persistent kernel (STU sub-layer + MLP + the next position's "
                         "history stream); 0: three kernels per step")
    ap.add_argument("--decode-kernel", choices=["pipe", "rows8"], default="pipe",
                    help="fused decode kernel: the persistent bulk-copy pipeline (default) or the 8x8 register-streaming one")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def workload_name(a):
    return (f"FlashSTUBlock(use_attention=False, {a.variant}) bf16 B={a.batch}/GPU L={a.seq_len} d_model={D_MODEL} "
            f"K={NUM_FILTERS} mlp_scale=4: prefill over L positions + {a.decode_steps} cached decode steps")


def filter_file(L):
    p = os.path.join(ROOT, "flash_stu_2_b200", "data", f"phi_{L}_{NUM_FILTERS}.pt")
    return p if os.path.exists(p) else None


def make_state(L, seed=1, approx=True):
    """Random-init block parameters (seed 1, xavier for the STU projections, default Linear init)."""
    import flash_stu_2_b200 as F
    torch.manual_seed(seed)
    fp = filter_file(L)
    cfg = F.FlashSTUConfig(n_embd=D_MODEL, seq_len=L, num_eigh=NUM_FILTERS, use_attn=False, use_approx=approx,
                           mlp_scale=4, torch_dtype=torch.bfloat16, n_layers=1, vocab_size=1, n_heads=D_MODEL // 64,
                           filter_path=fp)
    phi = None
    if fp is not None:
        phi = F.load_spectral_filters(fp, device="cpu", dtype=torch.bfloat16, verify_shape=(L, NUM_FILTERS))
    blk = F.FlashSTUBlock(config=cfg, phi=phi)
    for name, p in blk.named_parameters():
        if ".stu.M_" in name:
            torch.nn.init.xavier_normal_(p)
    return blk


# ----------------------------------------------------------------------------------------------- CPU arm
def cpu_forward_seconds(blk_sd, n, x1, T):
    from oracle import stu_oracle as O
    lsd = {k[len("layer."):]: v for k, v in blk_sd.items() if k.startswith("layer.")}
    t = time.perf_counter()
    with torch.no_grad():
        O.stu_layer(x1[:, :T], lsd, blk_sd["phi"], n, "layer.stu.M_inputs" in blk_sd)
    return time.perf_counter() - t


def cpu_baseline(a, blk, x_host):
    """The reference's arithmetic for this block on the host cores (oracle port).  The reference has no
    incremental STU decode, so one decode token costs a forward over the whole prefix."""
    from oracle import stu_oracle as O
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    sd = {k: v.detach().clone() for k, v in blk.state_dict().items()}
    n = O.fft_length(a.seq_len)
    x1 = x_host[:1].clone()
    t_dec = cpu_forward_seconds(sd, n, x1, a.seq_len - a.decode_steps // 2)
    t_pre = cpu_forward_seconds(sd, n, x1, a.seq_len)
    return {"value": 1.0 / t_dec, "unit": "decode tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "prefill_tokens_per_s": a.seq_len / t_pre,
            "sample": f"1 of {a.batch} sequences: one decode position by full-prefix recompute "
                      f"(T={a.seq_len - a.decode_steps // 2}) and one {a.seq_len}-token prefill forward, fp32 FFT path"}


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import stu_oracle as O
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the host arm uses every core this process may run on
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    blk = make_state(a.seq_len, approx=(a.variant == "approx"))
    sd = {k: v.detach().clone() for k, v in blk.state_dict().items()}
    n = O.fft_length(a.seq_len)
    torch.manual_seed(1)
    x1 = torch.randn(1, a.seq_len, D_MODEL).bfloat16()
    first = a.seq_len - a.decode_steps
    for i in range(a.warmup):
        cpu_forward_seconds(sd, n, x1, first + i + 1)
    t0 = time.perf_counter()
    for i in range(a.steps):
        cpu_forward_seconds(sd, n, x1, first + i + 1)   # one decode token of one sequence = one prefix forward
    dt = time.perf_counter() - t0
    val = a.steps / dt
    cores = torch.get_num_threads()
    sample = (f"each step = one decode token of one sequence at position {first}+i by full-prefix recompute "
              f"(the reference keeps no STU cache), torch.fft fp32 path, {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/s (aggregate over GPUs)", "value": val, "unit": "tokens/s",
        "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": dt / a.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(a), "l2": "n/a (host run)"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# ----------------------------------------------------------------------------------------------- GPU arm
def run_b200(a):
    import torch.distributed as dist
    from flash_stu_2_b200 import ops, parallel
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl b200 needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, L, d, S = a.batch, a.seq_len, D_MODEL, a.decode_steps
    from flash_stu_2_b200.modules import STU
    if a.no_overlap:
        ops.overlap_decode = False
    ops.early_decode = bool(a.early_decode)
    ops.fused_step = bool(a.fused_step)
    STU.pipelined_decode = (a.decode_kernel == "pipe")
    approx = a.variant == "approx"
    blk = make_state(L, approx=approx).to(dev).eval()
    torch.manual_seed(1 + rank)
    x_host = torch.randn(B, L, d).bfloat16().pin_memory()
    x_dev = x_host.to(dev)
    first = L - S
    ev = lambda: torch.cuda.Event(enable_timing=True)

    x_work = torch.empty_like(x_dev)
    x_step = torch.empty(B, 1, d, dtype=torch.bfloat16, device=dev)       # token buffer of the end-to-end loop
    x_steps = torch.zeros(S, B, 1, d, dtype=torch.bfloat16, device=dev)   # teacher-forced inputs, overwritten in
    state = {"cache": None, "graph": None, "graph_launches": 0}   # place by the block's outputs

    def prefill():
        # the cache buffers are allocated once and reused (a captured decode graph holds their addresses):
        # rewinding the position to 0 makes the call a prefill from the start of the sequence
        x_work.copy_(x_dev)
        if state["cache"] is not None:
            pos = state["cache"][1]
            pos[:, 0] = 0
            pos._host_t = 0
        _, state["cache"] = blk(x_work, past_key_value=state["cache"], use_cache=True)

    def rewind():
        pos = state["cache"][1]
        pos[:, 0] = first
        pos._host_t = first

    def eager_step(buf):
        _, state["cache"] = blk(buf, past_key_value=state["cache"], use_cache=True)

    def eager_steps():
        for i in range(S):
            eager_step(x_steps[i])

    def decode():
        # the block works in place (as the reference's layers do), so the S input rows are laid out token-major
        # once per pass; every token step then reads its row and leaves its output there
        x_steps.copy_(x_dev[:, first:].transpose(0, 1).unsqueeze(2))
        if state["graph"] is not None:
            state["graph"].replay()
        else:
            eager_steps()
        state["cache"][1]._host_t = first + S

    def capture(fn):
        rewind()
        g = torch.cuda.CUDAGraph()
        n0 = ops.launch_count
        with torch.cuda.graph(g):
            fn()
        return g, ops.launch_count - n0

    with torch.no_grad():
        # first pass: eager, builds derived weights / scratch / status word before any capture
        prefill(); rewind(); eager_step(x_steps[0]); eager_step(x_step)
        torch.cuda.synchronize()
        if not a.no_graph:
            # all S token steps in one graph (positions are read from device memory, so the same graph serves every pass)
            state["graph"], state["graph_launches"] = capture(eager_steps)
        for _ in range(a.warmup):
            prefill(); rewind(); decode()
        torch.cuda.synchronize()
        ops.check_status()

        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t_pre = t_dec = 0.0
        n_launch0 = ops.launch_count
        wall0 = time.perf_counter()
        for _ in range(a.steps):
            e0, e1, e2 = ev(), ev(), ev()
            e0.record(); prefill(); e1.record(); rewind(); decode(); e2.record()
            torch.cuda.synchronize()
            t_pre += e0.elapsed_time(e1)
            t_dec += e1.elapsed_time(e2)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        launches = ops.launch_count - n_launch0
        if state["graph"] is not None:
            launches += a.steps * state["graph_launches"]
        clocks = sampler.stop() if rank == 0 else None
        ops.check_status()
        t_pre, t_dec = parallel.max_over_ranks([t_pre, t_dec], device=dev)   # ms, summed over steps

        # ---- dominant kernel alone (fused decode kernel), CUDA events on the launching stream
        layer = blk.layer
        kern_ms, kern_bytes = None, None
        if approx:
            hist, pos = state["cache"]
            MinT, taps, taps8 = layer.stu.prepared()
            x2 = x_step.view(B, d)
            out2 = torch.empty_like(x2)
            reps = min(256, S)

            def kernel_only():
                if STU.pipelined_decode:
                    ops.decode_approx_pipelined(x2, layer.stu_norm.weight, MinT, hist, taps8, pos, out2)
                else:
                    ops.decode_approx(x2, layer.stu_norm.weight, MinT, hist, taps, pos, out2, taps8=taps8,
                                      flags=ops.FLAG_UNIFORM_POS)

            rewind()
            for _ in range(3):
                kernel_only()
            # the launches are replayed from a graph: issued one by one from Python they would be paced by the host
            # (the kernel is shorter than a ctypes call), and the figure would be the interpreter's, not the GPU's
            kg = None
            if not a.no_graph:
                kg, _ = capture(lambda: [kernel_only() for _ in range(reps)])
            rewind()
            torch.cuda.synchronize()
            k0, k1 = ev(), ev()
            k0.record()
            if kg is not None:
                kg.replay()
            else:
                for _ in range(reps):
                    kernel_only()
            k1.record()
            torch.cuda.synchronize()
            kern_ms = k0.elapsed_time(k1) / reps
            t_mid = first + reps / 2.0
            # algorithmic bytes of one launch at position t: half the history (one parity) of every sequence,
            # the even taps of every channel, M_inputs, and the token's row in and out
            kern_bytes = B * d * (t_mid / 2) * 2 + d * (t_mid / 2 + 1) * 2 + d * d * 2 + 3 * B * d * 2

        # ---- optional: timeline of the fused token-step kernel (stamps of CTA 0, written to its workspace)
        timeline = None
        if a.step_timeline and approx and B <= 8:
            ws = ops.block_step_workspace(d, layer.mlp.intermediate_size, dev)
            xs = x_step.view(B, d)
            mlp = layer.mlp
            targs = (xs, layer.stu_norm.weight, MinT, hist, taps8, pos, layer.mlp_norm.weight, mlp.gate_proj.weight,
                     mlp.up_proj.weight, mlp.down_proj.weight, xs, ws)
            rewind()
            ops.block_decode_step(*targs, mode=1)
            names = ["kernel entry", "positions read", "projection + combine done", "past grid barrier 1", "gate|up done",
                     "past grid barrier 2", "down + residual done", "history stream done"]
            timeline = []
            for _ in range(3):
                ops.block_decode_step(*targs, mode=0 | 0x10)
                torch.cuda.synchronize()
                tl = ws[128:128 + 8 * 8].view(torch.int64).cpu().tolist()
                timeline.append({n: (v - tl[0]) / 1e3 for n, v in zip(names, tl)})
            rewind()

        # ---- optional: timeline of the tcgen05 prefill convolution (stamps of CTA 0)
        conv_timeline = None
        if a.conv_timeline and approx:
            words = torch.zeros(128, dtype=torch.int64, device=dev)
            prefill()
            torch.cuda.synchronize()
            ops.conv_prefill_timeline(words)
            prefill()
            torch.cuda.synchronize()
            ops.conv_prefill_timeline(None)
            tw = words.cpu().view(8, 16)
            t_first = int(tw[0, 5])
            unit_names = ["accumulator free", "first operands ready", "last MMA issued", "accumulator complete",
                          "epilogue done"]
            phase_names = ["stage free", "history chunk landed", "stage ready"]
            conv_timeline = {
                "units": [{n: (int(tw[u, k]) - t_first) / 1e3 for k, n in enumerate(unit_names)} for u in range(8)],
                "phases": [{n: (int(tw[u, 5 + k]) - t_first) / 1e3 for k, n in enumerate(phase_names)} for u in range(8)]}
            rewind()

        # ---- optional: every kernel of the token step in a graph of its own (64 launches each)
        split = None
        if a.kernel_split and not a.no_graph and approx:
            mlp = layer.mlp
            mid = torch.empty_like(x2)
            hbuf = torch.empty(B, mlp.intermediate_size, dtype=torch.bfloat16, device=dev)

            def graph_us(fn, n=64):
                rewind()
                for _ in range(2):
                    fn()
                g, _ = capture(lambda: [fn() for _ in range(n)])
                best = float("inf")
                for _ in range(3):
                    rewind()
                    torch.cuda.synchronize()
                    g0, g1 = ev(), ev()
                    g0.record(); g.replay(); g1.record()
                    torch.cuda.synchronize()
                    best = min(best, g0.elapsed_time(g1) / n * 1e3)
                return best

            def dec(flags):
                ops.decode_approx(x2, layer.stu_norm.weight, MinT, hist, taps, pos, mid, taps8=taps8, flags=flags)

            def decp(flags=0):
                ops.decode_approx_pipelined(x2, layer.stu_norm.weight, MinT, hist, taps8, pos, mid, flags=flags)

            def gate_up(f=0):
                ops.linear(mid, mlp.gate_proj.weight, W2=mlp.up_proj.weight, out=hbuf, epilogue=ops.EPI_GELU_MUL | f,
                           norm_w=layer.mlp_norm.weight, eps=layer.mlp_norm.eps)

            def down(f=0):
                ops.linear(hbuf, mlp.down_proj.weight, resid=mid, out=out2, epilogue=ops.EPI_RESID | f)

            UN, OV, EA = ops.FLAG_UNIFORM_POS, ops.FLAG_OVERLAP, ops.FLAG_EARLY_TRIGGER
            split = {"unit": "us per launch, 64 launches replayed from one graph",
                     "stu_decode_pipe_kernel": graph_us(decp),
                     "stu_decode_rows8_kernel": graph_us(lambda: dec(UN)),
                     "stu_decode_diag_kernel": graph_us(lambda: dec(0)),
                     "skinny gate/up (norm fused)": graph_us(gate_up),
                     "skinny down (+residual)": graph_us(down),
                     "step, plain launches": graph_us(lambda: (dec(UN), gate_up(), down())),
                     "step, MLP kernels overlapped": graph_us(lambda: (dec(UN | EA), gate_up(OV), down(OV))),
                     "step (pipe), plain launches": graph_us(lambda: (decp(), gate_up(), down())),
                     "step (pipe), MLP kernels overlapped": graph_us(lambda: (decp(EA), gate_up(OV), down(OV))),
                     "step (pipe), MLP overlapped + decode started early":
                         graph_us(lambda: (decp(EA | OV), gate_up(OV), down(OV | EA)))}

        # ---- end to end through the module API from pinned host memory
        # token steps: the S teacher-forced input rows come from pinned host memory in one copy per pass (they do not
        # depend on the outputs), the S output rows go back to pinned host memory in one copy; the copies and the
        # graph replay between them are in the timed region, one synchronise per pass
        x_tok_host = x_host[:, first:].transpose(0, 1).contiguous().unsqueeze(2).pin_memory()     # [S, B, 1, d]
        y_tok_host = torch.empty(S, B, 1, d, dtype=torch.bfloat16).pin_memory()
        yp_host = torch.empty(B, L, d, dtype=torch.bfloat16).pin_memory()
        e2e_steps = max(1, min(a.steps, 3))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        dec_s = 0.0
        for _ in range(e2e_steps):
            x_work.copy_(x_host, non_blocking=True)
            pos = state["cache"][1]
            pos[:, 0] = 0
            pos._host_t = 0
            _, state["cache"] = blk(x_work, past_key_value=state["cache"], use_cache=True)
            yp_host.copy_(x_work, non_blocking=True)
            torch.cuda.synchronize()
            rewind()
            d0 = time.perf_counter()
            x_steps.copy_(x_tok_host, non_blocking=True)
            if state["graph"] is not None:
                state["graph"].replay()
            else:
                eager_steps()
            y_tok_host.copy_(x_steps, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            state["cache"][1]._host_t = first + S
            dec_s += time.perf_counter() - d0
        e2e_wall = time.perf_counter() - w0
        dec_s, e2e_wall = parallel.max_over_ranks([dec_s, e2e_wall], device=dev)

    # ---- extra objects (same line, headline unchanged): the whole-model token loop, and for N > 1 the tensor-parallel split
    extra = {}
    if not a.no_extra and approx:
        with torch.no_grad():
            extra["generate"] = generate_object(a, dev, world)
            if world > 1:
                extra["tp"] = tp_object(a, dev, world, rank)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    dec_tokens = world * B * S * a.steps
    pre_tokens = world * B * L * a.steps
    value = dec_tokens / (t_dec / 1e3)
    step_us = t_dec / a.steps / S * 1e3
    t_mid_step = first + S / 2.0
    fused = approx and ops.fused_step and B <= 8 and STU.pipelined_decode
    alone = None
    if approx:
        alone = {"kernel": "stu_decode_pipe_kernel" if STU.pipelined_decode else "stu_decode_rows8_kernel",
                 "what": "the STU decode kernel of the unfused path, 256 launches replayed from one graph",
                 "bytes_per_launch": kern_bytes, "us_per_launch": kern_ms * 1e3,
                 "achieved": kern_bytes / (kern_ms / 1e3) / 1e9}
    if fused:
        # the timed region launches ONE kernel per token step (stu_block_step_kernel: STU sub-layer + MLP + the next
        # position's history stream): its launch duration is the step time measured over the timed region, its
        # algorithmic bytes the step's (one parity run of the history, taps, M_inputs, the token rows, the MLP weights)
        kern_bytes = (B * d * (t_mid_step / 2) * 2 + d * (t_mid_step / 2 + 1) * 2 + d * d * 2 + 3 * B * d * 2
                      + 12 * d * d * 2)
        kern_ms = step_us / 1e3
        achieved = kern_bytes / (kern_ms / 1e3) / 1e9
        roof_kernel = "stu_block_step_kernel"
    elif approx:
        achieved = kern_bytes / (kern_ms / 1e3) / 1e9
        roof_kernel = "stu_decode_pipe_kernel" if STU.pipelined_decode else "stu_decode_rows8_kernel"
    else:
        # full variant: no single dominant kernel; the roofline object describes the whole token step: the history of
        # every sequence (both parities), the 2K d x d matrices M_phi_plus/minus, the MLP weights
        kern_bytes = B * d * t_mid_step * 2 + 2 * NUM_FILTERS * d * d * 2 + 12 * d * d * 2 + 3 * B * d * 2
        kern_ms = step_us / 1e3
        achieved = kern_bytes / (kern_ms / 1e3) / 1e9
        roof_kernel = "whole token step (prepare, history x filters GEMM, combine, contraction, MLP)"
    # prefill FLOPs per token: dense 2*(P + 3*4*d^2) with P = d^2 (approx) or 2K d^2 (full), plus the FFT-as-GEMM form of
    # the convolutions: one per channel (approx) or (2K+1)/2 per channel (full)
    n_fft = 1 << (2 * L - 2).bit_length()          # 2^ceil(log2(2L-1))
    n1 = 1 << ((n_fft.bit_length() - 1) // 2)      # two-factor split n_fft = n1 * n2
    n2 = n_fft // n1
    conv_mult = 1.0 if approx else (2 * NUM_FILTERS + 1) / 2.0
    p_stu = d * d if approx else 2 * NUM_FILTERS * d * d
    flops_tok = 2 * (p_stu + 12 * d * d) + conv_mult * d * 16 * n_fft * (n1 + n2) / L
    pre_tflops = flops_tok * B * L / (t_pre / a.steps / 1e3) / 1e12
    ws_mb = (B * d * L * 2 + d * L + 13 * d * d * 2) / 1e6
    line = {
        "metric": "decode tokens/s (aggregate over GPUs)", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": (t_pre + t_dec) / a.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": f"dp{world} (independent sequences, no collective)",
                   "l2": f"inputs larger than L2: decode working set {ws_mb:.0f} MB (history+taps+weights) and "
                         f"prefill input {B * L * d * 2 / 1e6:.0f} MB vs 126 MB L2; no explicit flush",
                   "decode_launch": (f"one CUDA graph of all {S} token steps (device-resident positions)"
                                     if state["graph"] is not None else "eager launches") +
                                    ("; one fused kernel per token step" if fused else "")},
        "decode_ms_per_token_step": t_dec / a.steps / S,
        "prefill": {"value": pre_tokens / (t_pre / 1e3), "unit": "tokens/s", "ms": t_pre / a.steps,
                    "tflops_algorithmic": pre_tflops,
                    "frac_of_tensor_peak": pre_tflops / pk["bf16_tflops_sustained"],
                    "peak_tflops": pk["bf16_tflops_sustained"], "peak_source": pk["source"] + " (sustained)"},
        "roofline": {"bound": "hbm", "kernel": roof_kernel, "achieved": achieved, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"],
                     "bytes_per_launch": kern_bytes, "us_per_launch": kern_ms * 1e3, "traffic": None},
        "e2e": {"value": world * B * S * e2e_steps / dec_s, "unit": "tokens/s",
                "h2d_bytes_per_step": B * L * d * 2 + S * B * d * 2, "d2h_bytes_per_step": B * L * d * 2 + S * B * d * 2,
                "wall_s_per_step": e2e_wall / e2e_steps,
                "note": "decode tokens/s, wall clock: per pass the 512 teacher-forced input rows are copied in from pinned "
                        "host memory (one copy), the token steps are replayed from one CUDA graph, the 512 output rows are "
                        "copied back to pinned host memory (one copy), then one synchronise; the prefill of each pass also "
                        "copies its 134 MB input in and its output back"},
        "gpu_launches": launches, "wall_s_timed_region": wall, "clocks": clocks,
    }
    if (B, L, d) == (8, 8192, 1024) and approx:
        line["roofline"]["traffic"] = STEP_KERNEL_DRAM_BYTES if fused else (
            None if STU.pipelined_decode else DECODE_KERNEL_DRAM_BYTES)
    if alone is not None:
        alone["frac"] = alone["achieved"] / pk["hbm_gbs"]
        line["stu_kernel_alone"] = alone
    if approx:
        # the whole token step of the block: the decode kernel's bytes plus the MLP weights (gate, up, down)
        step_bytes = (B * d * (t_mid_step / 2) * 2 + d * (t_mid_step / 2 + 1) * 2 + d * d * 2 + 3 * B * d * 2
                      + 12 * d * d * 2)
        line["roofline_step"] = {"bound": "hbm", "what": "whole token step (STU decode kernel + gate/up + down)",
                                 "bytes_per_step": step_bytes, "us_per_step": step_us,
                                 "achieved": step_bytes / (step_us * 1e-6) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                                 "frac": step_bytes / (step_us * 1e-6) / 1e9 / pk["hbm_gbs"]}
    if split is not None:
        line["decode_split"] = split
    if conv_timeline is not None:
        line["conv_timeline"] = {"unit": "us after the first stage became free, CTA 0", **conv_timeline}
    if timeline is not None:
        line["step_timeline"] = {"unit": "us after kernel entry, CTA 0, three consecutive launches", "launches": timeline}
    if extra.get("generate") is not None:
        line["generate"] = extra["generate"]
    if extra.get("tp") is not None:
        line["tp"] = extra["tp"]
    if world == 1 and not a.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(a, make_state(L, approx=approx), x_host)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------- extra objects
def _decode_bytes_per_step(cfg, b, t, e=2):
    """Algorithmic HBM bytes of one cached token step of a FlashSTU model at position t for b resident sequences:
    every weight once (tied LM head included), per STU layer one parity run of the projected history of every sequence
    plus the even taps, per attention layer the keys and values inside the window plus the new pair."""
    d, n_layers, K, V, s_, w = cfg["n_embd"], cfg["n_layers"], cfg["num_eigh"], cfg["vocab_size"], cfg["mlp_scale"], cfg["window_size"]
    n_attn = n_layers // 2 if cfg.get("use_attn", True) else 0
    n_stu = n_layers - n_attn
    weights = n_stu * (d * d + 3 * s_ * d * d + 2 * d) + n_attn * (4 * d * d + 3 * s_ * d * d + 2 * d) + V * d + d
    taps = n_stu * d * (t // 2 + 1)
    stu_state = n_stu * b * (d * (t // 2) + d)
    kv_state = n_attn * b * (2 * min(t, w + 1) * d + 2 * d)
    return e * (weights + taps + stu_state + kv_state)


def generate_object(a, dev, world):
    """The 24-layer d=1536 bf16 model (B=32 per GPU, prompt 2048, top_k=40, T=0.8) through FlashSTU.generate() with
    random-init weights built on the GPU: decode tokens/s per GPU (time of a full generate minus the time of one that
    stops after the first new token, CUDA events, max over ranks), prefill tokens/s, kernels launched per token step
    and the fraction of the HBM roofline of a step."""
    import tempfile
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops, parallel
    spec = MODEL_CONFIGS["c3"]
    cfg = dict(spec["cfg"])
    L, K = cfg["seq_len"], cfg["num_eigh"]
    B, T0, new = spec["B"], spec["prompt"], a.extra_new_tokens
    with tempfile.TemporaryDirectory() as tmp:
        fp = filter_file(L)
        if fp is None:
            fp = os.path.join(tmp, "phi.pt")
            F.save_spectral_filters(F.get_spectral_filters(L, K, device=dev, dtype=torch.float32), fp)
        torch.manual_seed(0)
        with torch.device(dev):
            model = F.FlashSTU(F.FlashSTUConfig(filter_path=fp, torch_dtype=torch.bfloat16, cache_len=T0 + new + 8,
                                                **cfg))
        model = model.to(dev).eval()
    ids = torch.randint(0, cfg["vocab_size"], (B, T0), device=dev)
    gen = torch.Generator(device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(max_length, graph=True, timings=None):
        gen.manual_seed(0)
        e0, e1 = ev(), ev()
        torch.cuda.synchronize()
        e0.record()
        out = model.generate(ids, max_length=max_length, generator=gen, cuda_graph=graph, timings=timings,
                             **spec["sampling"])
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    timed(T0 + 6)                                              # warm-up: derived weights, scratch, graph capture path
    c0 = ops.launch_count
    timed(T0 + 1, graph=False)
    c1 = ops.launch_count
    timed(T0 + 5, graph=False)
    c2 = ops.launch_count
    per_step = ((c2 - c1) - (c1 - c0)) / 4.0
    t_first = min(timed(T0 + 1)[0] for _ in range(2))
    # the token step is timed on the device over the graph-replayed steps alone (CUDA events inside generate()): the
    # two eager steps and the capture of the step graph before them are host work that varies by tens of milliseconds
    tm = {}
    timed(T0 + new, timings=tm)
    ops.check_status()
    t_first, replay_ms = parallel.max_over_ranks([t_first, tm["replay_ms"]], device=dev)
    dec_ms = replay_ms / tm["replayed_steps"]
    pk = peaks()
    nbytes = _decode_bytes_per_step(cfg, B, T0 + new // 2)
    n_param = sum(p.numel() for p in model.parameters())
    del model
    torch.cuda.empty_cache()
    return {"workload": f"FlashSTU.generate: 24 layers d=1536 H=12 window 1024 K=24 V=50257 bf16, {n_param / 1e6:.0f} M "
                        f"parameters, B={B}/GPU, prompt {T0}, +{new} tokens top_k=40 T=0.8 (random-init weights)",
            "decode_tokens_per_s_per_gpu": B / (dec_ms * 1e-3), "decode_ms_per_token_step": dec_ms,
            "prefill_tokens_per_s_per_gpu": B * T0 / (t_first * 1e-3), "prefill_ms": t_first,
            "launches_per_token_step": per_step,
            "roofline": {"bound": "hbm", "bytes_per_step": nbytes, "achieved": nbytes / (dec_ms * 1e-3) / 1e9,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": nbytes / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "accounting": "one parity run of the STU history per step (parity-split cache), keys and values "
                                       "inside the window, every weight once"},
            "decode_launch": "one CUDA graph per token step", "n_gpus": world,
            "parallelism": f"dp{world}: every rank generates for its own {B} sequences"}


def _err_figures(a, b):
    a, b = a.double(), b.double()
    rel = float((a - b).abs().max() / b.abs().max())
    a2, b2 = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    den = b2.abs().amax(1).clamp_min(1e-3 * float(b2.abs().max()))
    return {"rel": rel, "row": float(((a2 - b2).abs().amax(1) / den).max())}


def tp_object(a, dev, world, rank):
    """N > 1: the 3B configuration's shapes (32 layers, d=3072, 24 heads, window 2048, K=32 filters of 32768 positions,
    B=64, prompt 8192, greedy) tensor-parallel over the N ranks, weights generated shard by shard on the GPUs; plus the
    parity of the sharded path against the reference's logits on the small hybrid fixtures (2 or 4 ranks)."""
    import torch.distributed as dist
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops, parallel
    from flash_stu_2_b200.tensor_parallel import TensorParallelFlashSTU, random_shards
    spec = MODEL_CONFIGS["c5"]
    cfg = dict(spec["cfg"])
    B, T0, new = spec["B"], spec["prompt"], a.tp_new_tokens
    cfg["cache_len"] = T0 + new + 8
    config = F.FlashSTUConfig(torch_dtype=torch.bfloat16, **cfg)
    phi = F.get_spectral_filters(cfg["seq_len"], cfg["num_eigh"], device=dev, dtype=torch.float32).to(torch.bfloat16)
    # every rank must hold the same filters: take rank 0's
    dist.broadcast(phi, src=0)
    tp = TensorParallelFlashSTU(config, random_shards(config, phi, rank, world, dev, seed=0), dev, presharded=True)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg["vocab_size"], (B, T0), generator=g).to(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(prompt, max_length, timings=None):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        out = tp.generate(prompt, max_length=max_length, do_sample=False, timings=timings)
        e1.record()
        torch.cuda.synchronize()
        return parallel.max_over_ranks([e0.elapsed_time(e1)], device=dev)[0], out

    timed(ids[:, :256].contiguous(), 256 + 6)                 # warm-up on a short prompt (derived weights, graph path)
    t_first, _ = timed(ids, T0 + 1)
    tm = {}
    _, out = timed(ids, T0 + new, timings=tm)      # token steps: device time of the graph-replayed steps alone
    ops.check_status()
    same = parallel.gather_token_ids(out[:1, T0:].contiguous(), world)
    dec_ms = parallel.max_over_ranks([tm["replay_ms"]], device=dev)[0] / tm["replayed_steps"]
    fused = tp._exchange is not None      # what the group-size default picked for the figure above
    default_mode = tp.fused_exchange
    # the same token steps with the other way of exchanging: NCCL collectives between the kernels / exchange kernels
    tp.fused_exchange = False if fused else "force"
    tm2 = {}
    _, out2 = timed(ids, T0 + new, timings=tm2)
    ops.check_status()
    tp.fused_exchange = default_mode
    other_ms = parallel.max_over_ranks([tm2["replay_ms"]], device=dev)[0] / tm2["replayed_steps"]
    dec_ms_nccl, dec_ms_xchg = (other_ms, dec_ms) if fused else (dec_ms, other_ms)
    pk = peaks()
    nbytes = _decode_bytes_per_step(cfg, B, T0 + new // 2) / world
    res = {"workload": f"FlashSTU.generate, 3B shapes: 32 layers d=3072 H=24 window 2048 K=32 L=32768 V=50257 bf16 "
                       f"B={B} prompt {T0} +{new} greedy, tensor-parallel over {world} GPUs (random-init shards)",
           "decode_ms_per_token_step": dec_ms, "decode_tokens_per_s_per_gpu": B / (dec_ms * 1e-3) / world,
           "decode_tokens_per_s": B / (dec_ms * 1e-3),
           "prefill_ms": t_first, "prefill_tokens_per_s": B * T0 / (t_first * 1e-3),
           "ranks_agree": bool((same == same[0]).all()),
           "roofline": {"bound": "hbm", "bytes_per_step_per_gpu": nbytes, "achieved": nbytes / (dec_ms * 1e-3) / 1e9,
                        "peak": pk["hbm_gbs"], "unit": "GB/s per GPU", "frac": nbytes / (dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"]},
           "decode_ms_per_token_step_nccl": dec_ms_nccl, "decode_ms_per_token_step_exchange_kernels": dec_ms_xchg,
           "tokens_equal_to_nccl_path": float((out[:, T0:] == out2[:, T0:]).float().mean()),
           "collectives": ("token steps: the all-gather after every STU shard and the all-reduce after every attention / "
                           "MLP block are one exchange kernel each (rows stored into the other ranks' inboxes over "
                           "NVLink peer memory, bounded wait, sum + residual + RMSNorm); logits all-gather and "
                           "prefill: NCCL; `decode_ms_per_token_step_nccl` = the same steps with NCCL collectives "
                           "between the kernels"
                           if fused else
                           "NCCL all-gather per STU layer, all-reduce per attention / MLP block, captured in the step "
                           "graph (the default above 4 ranks or above 256 KB per exchange); "
                           "`decode_ms_per_token_step_exchange_kernels` = the same steps with the peer-memory "
                           "exchange kernels")}
    del tp
    torch.cuda.empty_cache()
    # ---- parity of the sharded path on the reference's small hybrid fixtures (needs n_heads % ranks == 0)
    par = {}
    gold = os.path.join(ROOT, "tests", "golden", "models.pt")
    sub = 4 if world >= 4 else 2
    group = dist.new_group(ranks=list(range(sub)))
    if os.path.exists(gold) and rank < sub:
        fixtures = torch.load(gold, map_location="cpu", weights_only=False)
        for name in ("hybrid_approx_fp32", "hybrid_approx_bf16"):
            r = fixtures[name]
            c = F.FlashSTUConfig(torch_dtype=getattr(torch, r["dtype"]), **r["cfg"])
            m = TensorParallelFlashSTU(c, r["sd"], dev, group=group)
            with torch.no_grad():
                logits = m.last_logits(r["ids"].to(dev), m.new_cache(r["ids"].shape[0])).float().cpu()
            ops.check_status()
            par[name] = dict(_err_figures(logits, r["logits_full"][:, -1].float()), ranks=sub,
                             tolerance=1e-3 if r["dtype"] == "float32" else 2e-2)
    res["parity_vs_reference_logits"] = par if par else "fixture file missing"
    return res


# ----------------------------------------------------------------------------------------------- whole models
MODEL_CONFIGS = {
    "c1": dict(cfg=dict(n_embd=512, n_layers=12, n_heads=8, seq_len=2048, window_size=512, vocab_size=50257,
                        mlp_scale=12, num_eigh=24, use_attn=True, use_approx=True), dtype="float32", B=2, prompt=128,
               new=128, sampling=dict(do_sample=False)),
    "c3": dict(cfg=dict(n_embd=1536, n_layers=24, n_heads=12, seq_len=8192, window_size=1024, vocab_size=50257,
                        mlp_scale=4, num_eigh=24, use_attn=True, use_approx=True), dtype="bfloat16", B=32, prompt=2048,
               new=512, sampling=dict(do_sample=True, temperature=0.8, top_k=40)),
    "c5": dict(cfg=dict(n_embd=3072, n_layers=32, n_heads=24, seq_len=32768, window_size=2048, vocab_size=50257,
                        mlp_scale=4, num_eigh=32, use_attn=True, use_approx=True, cache_len=9216), dtype="bfloat16",
               B=64, prompt=8192, new=1024, sampling=dict(do_sample=False)),
}


def run_lds_stack(a):
    """12 x MiniSTU(backend='lds') applied one after the other (no norm or residual between them): chunked-scan
    prefill of 16 x 15360 positions, then 1024 recurrent steps replayed from one CUDA graph."""
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --model needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device("cuda:0")
    B, L, d, n_layers = a.lds_batch, 16384, 1024, a.lds_layers
    new = a.new_tokens or 1024
    T0 = L - 1024
    torch.manual_seed(0)
    layers = [F.MiniSTU(seq_len=L, num_filters=24, input_dim=d, output_dim=d, backend="lds", dtype=torch.bfloat16,
                        device=dev) for _ in range(n_layers)]
    x = (torch.randn(B, L, d, device=dev) * 0.5).bfloat16()
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def prefill():
        h, caches = x[:, :T0].contiguous(), []
        for m in layers:
            h, c = m(h, use_cache=True)
            caches.append(c)
        return caches

    def step(tok, caches):
        h = tok
        for i, m in enumerate(layers):
            h, caches[i] = m(h, past_key_value=caches[i], use_cache=True)
        return h

    with torch.no_grad():
        caches = prefill()                        # warm-up (impulse responses, scratch)
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record(); caches = prefill(); e1.record()
        torch.cuda.synchronize()
        pre_ms = e0.elapsed_time(e1)
        tok = x[:, T0:T0 + 1].contiguous()
        step(tok, caches)                         # eager warm-up of the decode path
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = step(tok, caches)
        e0, e1 = ev(), ev()
        e0.record()
        for i in range(new):
            tok.copy_(x[:, T0 + (i % 1024):T0 + (i % 1024) + 1])
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        dec_ms = e0.elapsed_time(e1)
    ops.check_status()
    split = None
    if a.kernel_split:   # the three pieces of one layer's prefill, each alone (CUDA events, 3 repetitions)
        m = layers[0]
        op = m._lds_prepared()
        A64, B64, Cm = m._lds_f32
        Vs, W, R = m._lds_scan
        Ck = m.LDS_CHUNK
        nch = (T0 + Ck - 1) // Ck
        xin = x[:, :T0].contiguous()
        with torch.no_grad():
            Z = torch.empty(B, nch, d, W.shape[1], dtype=x.dtype, device=dev)
            hfin = torch.empty(B, d, Cm.shape[0], dtype=torch.float64, device=dev)
            U2 = torch.empty(nch * Ck, Cm.shape[1] * d, dtype=x.dtype, device=dev)
            yb = torch.empty(T0, d, dtype=x.dtype, device=dev)
            _, Mcat = op.prepared_full()

            def t3(fn):
                fn()
                torch.cuda.synchronize()
                e0, e1 = ev(), ev()
                e0.record()
                for _ in range(3):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) / 3

            split = {"unit": "ms per layer", "batch": B, "positions": T0,
                     "lds_chunk_scan_kernel (all sequences)": t3(lambda: ops.lds_chunk_scan(xin, A64, B64, Vs, Z, hfin, Ck,
                                                                                          unit_b=m._lds_unit_b)),
                     "features GEMM, per sequence": t3(lambda: ops.lds_chunk_features(W, Z[0].view(nch * d, W.shape[1]), U2,
                                                                                      d, Ck, Cm.shape[1])),
                     "contraction with M, per sequence": t3(lambda: ops.linear(U2[:T0], Mcat, out=yb))}
    D_, F_ = 160, 48
    pre_flops = B * T0 * n_layers * (2 * F_ * d * d + 2 * D_ * F_ * d + 2 * D_ * d)
    step_bytes = n_layers * (F_ * d * d * 2 + B * d * D_ * 16 + D_ * F_ * 2)
    pk = peaks()
    print(json.dumps({
        "metric": "decode tokens/s (aggregate over GPUs)", "value": B * new / (dec_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "higher_is_better": True, "dtype": "bf16 (LDS state float64)", "data": "synthetic",
        "config": {"workload": f"{n_layers} x MiniSTU(backend='lds', 1024->1024) L={L} B={B}: prefill {T0} + {new} recurrent steps",
                   "decode_launch": "one CUDA graph per token step"},
        "decode_ms_per_token_step": dec_ms / new,
        "roofline": {"bound": "hbm", "kernel": "whole token step", "achieved": step_bytes / (dec_ms / new * 1e-3) / 1e9,
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": step_bytes / (dec_ms / new * 1e-3) / 1e9 / pk["hbm_gbs"],
                     "bytes_per_launch": step_bytes},
        "prefill": {"value": B * T0 / (pre_ms * 1e-3), "unit": "tokens/s", "ms": pre_ms,
                    "tflops_algorithmic": pre_flops / (pre_ms * 1e-3) / 1e12,
                    "frac_of_tensor_peak": pre_flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
                    "peak_tflops": pk["bf16_tflops_sustained"],
                    "note": "chunked scan: float64 recurrence + rotated carry per chunk of 128 positions (one kernel), one "
                            "tensor-core GEMM per sequence for the features of all chunks, one for the contraction with M; "
                            "FLOPs counted per token and layer as 2*48*d^2 + 2*160*48*d + 2*160*d (recurrent form)"},
        **({"prefill_split": split} if split is not None else {}),
    }))


def run_model_tp(a):
    """The --model workload with the model sharded over the ranks of the job (one process per GPU, NCCL).  Every
    rank builds the same random-init model on the host and keeps its shard; times are the max over ranks."""
    import tempfile
    import torch.distributed as dist
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops, parallel
    from flash_stu_2_b200.tensor_parallel import TensorParallelFlashSTU
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --model --tp needs CUDA devices: the kernels have no CPU fallback")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    spec = MODEL_CONFIGS[a.model]
    cfg, dt = dict(spec["cfg"]), getattr(torch, spec["dtype"])
    L, K = cfg["seq_len"], cfg["num_eigh"]
    with tempfile.TemporaryDirectory() as tmp:
        fp = filter_file(L)
        if fp is None:
            fp = os.path.join(tmp, "phi.pt")
            F.save_spectral_filters(F.get_spectral_filters(L, K, device=dev, dtype=torch.float32), fp)
        torch.manual_seed(0)
        config = F.FlashSTUConfig(filter_path=fp, torch_dtype=dt, **cfg)
        full = F.FlashSTU(config)
        sd = {k: v.detach().cpu() for k, v in full.state_dict().items()}
        del full
    tp = TensorParallelFlashSTU(config, sd, dev)
    del sd
    B, T0, new = spec["B"], spec["prompt"], (a.new_tokens or spec["new"])
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg["vocab_size"], (B, T0), generator=g).to(dev)
    uniforms = torch.rand(new, B, generator=g)
    samp = dict(spec["sampling"])
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(max_length, timings=None):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        out = tp.generate(ids, max_length=max_length, uniforms=uniforms if samp.get("do_sample") else None,
                          timings=timings, **samp)
        e1.record()
        torch.cuda.synchronize()
        return parallel.max_over_ranks([e0.elapsed_time(e1)], device=dev)[0], out

    timed(T0 + min(6, new))
    t_first = min(timed(T0 + 1)[0] for _ in range(2))
    tm = {}
    t_full, out = timed(T0 + new, tm)
    ops.check_status()
    fused = tp._exchange is not None
    step_ms = parallel.max_over_ranks([tm["replay_ms"]], device=dev)[0] / tm["replayed_steps"]
    tp.fused_exchange = False          # the same token steps with NCCL collectives between the kernels
    timed(T0 + min(6, new))
    tm2 = {}
    timed(T0 + new, tm2)
    ops.check_status()
    step_ms_nccl = parallel.max_over_ranks([tm2["replay_ms"]], device=dev)[0] / tm2["replayed_steps"]
    same = parallel.gather_token_ids(out[:1].contiguous(), world)
    if rank == 0:
        dec_ms = t_full - t_first
        print(json.dumps({
            "token_step_ms": {"graph replays, device time": step_ms, "same with NCCL collectives": step_ms_nccl,
                              "exchanges_in_kernels": fused},
            "metric": "decode tokens/s (aggregate over GPUs)", "value": B * (new - 1) / (dec_ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "higher_is_better": True, "scaling": "strong", "dtype": spec["dtype"],
            "data": "synthetic",
            "config": {"workload": f"FlashSTU.generate {a.model}, tensor parallel over {world} GPUs: {cfg['n_layers']} layers "
                                   f"d={cfg['n_embd']} B={B} prompt {T0} +{new} tokens",
                       "parallelism": f"tp{world} (all-gather per STU layer, all-reduce per attention / MLP block: in token "
                                      "steps one exchange kernel each over peer memory, in the prefill NCCL)",
                       "decode_launch": "one CUDA graph per token step, fused STU step on the rank's channels"},
            "decode_ms_per_token_step": dec_ms / (new - 1),
            "prefill": {"value": B * T0 / (t_first * 1e-3), "unit": "tokens/s", "ms": t_first},
            "ranks_agree": bool((same == same[0]).all()),
        }))
    dist.destroy_process_group()


def run_model(a):
    """FlashSTU.generate() on a whole model with random-init weights (secondary workloads; the headline is the
    block).  Decode tokens/s = B / (device time per graph-replayed token step, CUDA events inside generate), one GPU;
    the eager loop's figure is the difference of two whole-run times."""
    import tempfile
    import flash_stu_2_b200 as F
    from flash_stu_2_b200 import ops
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --model needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device("cuda:0")
    spec = MODEL_CONFIGS[a.model]
    cfg, dt = dict(spec["cfg"]), getattr(torch, spec["dtype"])
    L, K = cfg["seq_len"], cfg["num_eigh"]
    with tempfile.TemporaryDirectory() as tmp:
        fp = filter_file(L) if K == NUM_FILTERS else None
        if fp is None:
            fp = os.path.join(tmp, "phi.pt")
            F.save_spectral_filters(F.get_spectral_filters(L, K, device=dev, dtype=torch.float32), fp)
        torch.manual_seed(0)
        extra = {"cache_len": a.cache_len} if a.cache_len else {}
        model = F.FlashSTU(F.FlashSTUConfig(filter_path=fp, torch_dtype=dt, **extra, **cfg)).to(dev).eval()
    B, T0, new = spec["B"], spec["prompt"], (a.new_tokens or spec["new"])
    ids = torch.randint(0, cfg["vocab_size"], (B, T0), device=dev)
    gen = torch.Generator(device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(max_length, graph, timings=None):
        gen.manual_seed(0)
        e0, e1 = ev(), ev()
        torch.cuda.synchronize()
        e0.record()
        out = model.generate(ids, max_length=max_length, generator=gen, cuda_graph=graph, timings=timings,
                             **spec["sampling"])
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    res = {}
    tm = {}
    for graph in (True, False):
        timed(T0 + min(8, new), graph)                          # warm-up (derived weights, scratch)
        t_first = min(timed(T0 + 1, graph)[0] for _ in range(2))
        t_full, out = timed(T0 + new, graph, tm if graph else None)
        res[graph] = (t_first, t_full, out)
    ops.check_status()
    t_first, t_full, out = res[True]
    # token steps: device time of the graph-replayed steps alone (the two eager steps and the capture before them are
    # host work that varies by milliseconds from run to run, which makes differences of whole-run times useless)
    dec_ms = tm["replay_ms"] / tm["replayed_steps"] * (new - 1) if tm.get("replayed_steps") else t_full - t_first
    n_param = sum(p.numel() for p in model.parameters())
    print(json.dumps({
        "metric": "decode tokens/s (aggregate over GPUs)", "value": B * (new - 1) / (dec_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "higher_is_better": True, "dtype": spec["dtype"], "data": "synthetic",
        "config": {"workload": f"FlashSTU.generate {a.model}: {cfg['n_layers']} layers d={cfg['n_embd']} "
                               f"V={cfg['vocab_size']} L={L} B={B} prompt {T0} +{new} tokens, {n_param / 1e6:.0f} M parameters",
                   "sampling": spec["sampling"], "decode_launch": "one CUDA graph per token step"},
        "decode_ms_per_token_step": dec_ms / (new - 1),
        "prefill": {"value": B * T0 / (t_first * 1e-3), "unit": "tokens/s", "ms": t_first},
        "eager_loop": {"decode_tokens_per_s": B * (new - 1) / ((res[False][1] - res[False][0]) * 1e-3),
                       "same_tokens_as_graph": bool(torch.equal(out, res[False][2]))},
    }))


if __name__ == "__main__":
    # stdout carries the one JSON line: Python's prints keep the original stream, while whatever native libraries write
    # to file descriptor 1 (NCCL's version banner) is sent to stderr
    sys.stdout.flush()
    sys.stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    args = parse()
    if args.impl != "reference":
        from flash_stu_2_b200 import ops as _ops
        from flash_stu_2_b200.modules import STU as _STU
        _ops.early_decode = bool(args.early_decode)
        _ops.fused_step = bool(args.fused_step)
        _STU.pipelined_decode = (args.decode_kernel == "pipe")
        if args.no_overlap:
            _ops.overlap_decode = False
    if args.impl == "reference":
        run_reference(args)
    elif args.model == "c4":
        run_lds_stack(args)
    elif args.model and args.tp:
        run_model_tp(args)
    elif args.model:
        run_model(args)
    else:
        run_b200(args)
