"""Times the token-step linear layers (17..64 activation rows, bf16) the way a token step meets them: weights rotated
through more matrices than L2 holds, launches replayed from a CUDA graph, CUDA events around the replay.

    python -m flash_stu_2_b200.linear_bench [M N K epilogue ...]

Without arguments: the four shapes of the 24-layer d=1536 model at 32 sequences (down, c_proj / M_inputs, c_attn,
gate/up).  Environment switches of the library select the kernel (STU_B200_DISABLE_UMMA_SKINNY=1: mma.sync
weight-streaming kernels; STU_B200_UMMA_KS / STU_B200_UMMA_STAGES: K split and ring depth of the tcgen05 kernel)."""
import math
import sys

import torch

from . import ops


def time_linear(M: int, N: int, K: int, epi: int, dev="cuda") -> float:
    """Microseconds per launch of y = epilogue(x[M,K] @ W[N,K]^T) (epi 0 store, 1 residual, 2 GELU(gate)*up)."""
    per = N * K * 2 * (2 if epi == 2 else 1)
    n_w = max(4, int(math.ceil(300e6 / per)))          # > 126 MB of L2 between two uses of a matrix
    x = torch.randn(M, K, device=dev).bfloat16()
    Ws = [(torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16() for _ in range(n_w)]
    W2s = [(torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16() for _ in range(n_w)] if epi == 2 else Ws
    resid = torch.randn(M, N, device=dev).bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

    def run():
        for W, W2 in zip(Ws, W2s):
            ops.linear(x, W, W2=W2 if epi == 2 else None, resid=resid if epi == 1 else None, out=out, epilogue=epi)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(4):
            run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g.replay()
    torch.cuda.synchronize()
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    return e0.elapsed_time(e1) * 1e3 / (4 * n_w)


def main(argv):
    if not torch.cuda.is_available():
        raise RuntimeError("needs a CUDA device: the kernels have no CPU fallback")
    vals = [int(v) for v in argv]
    shapes = [tuple(vals[i:i + 4]) for i in range(0, len(vals), 4)] or [
        (32, 1536, 6144, 1), (32, 1536, 1536, 1), (32, 4608, 1536, 0), (32, 6144, 1536, 2)]
    for (M, N, K, epi) in shapes:
        us = time_linear(M, N, K, epi)
        gbs = N * K * 2 * (2 if epi == 2 else 1) / us / 1e3
        print(f"M={M} N={N} K={K} epilogue={epi}: {us:.1f} us per launch, {gbs:.0f} GB/s of weights", flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
