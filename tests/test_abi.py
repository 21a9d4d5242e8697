"""The C-ABI library builds, loads without a GPU and exports every symbol include/stu_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "stu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|long long)\s+(stu_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "stu_linear" in names and "stu_decode_approx" in names and len(names) >= 10


def test_library_exports_every_declared_symbol():
    from flash_stu_2_b200 import _lib
    lib = _lib.load()
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} declared in include/stu_b200.h but not exported"
    # the Python binding covers exactly the declared set
    assert sorted(_lib.exported_symbols()) == declared_symbols()
    assert lib.stu_b200_version() >= 100


def test_argument_errors_are_reported_without_a_gpu():
    from flash_stu_2_b200 import _lib
    lib = _lib.load()
    # null pointers / bad shapes are rejected on the host before any CUDA call
    assert lib.stu_rmsnorm(None, None, None, 1, 8, 8, 8, 1e-6, 1, None) == -5
    assert lib.stu_linear_can_fuse_norm(8, 4096, 1024, 2, 1) == 1
    assert lib.stu_linear_can_fuse_norm(8, 4096, 1024, 2, 0) == 0
    assert lib.stu_linear_can_fuse_norm(128, 4096, 1024, 2, 1) == 0
    # the prefill convolution reads its scratch in 16-byte vectors: a row pitch that is not a multiple of 8 bf16
    # (4 fp32) elements, or a misaligned scratch base, is refused with -3 and nothing is launched
    a = 0x10000   # stands for an aligned device address; the checks return before anything dereferences it
    assert lib.stu_conv_prefill_approx(a, a, a, a, 333 * 8, 8, 1, 8, 168, 167, 0, 333, 1, 1, None) == -3
    assert lib.stu_conv_prefill_approx(a, a, a, a, 333 * 8, 8, 1, 8, 168, 166, 0, 332, 0, 0, None) == -3
    assert lib.stu_conv_prefill_approx(a, a, a + 2, a, 333 * 8, 8, 1, 8, 168, 168, 0, 333, 1, 1, None) == -3
    # the tcgen05 convolution: misaligned scratch -3, a history that is not tiled in 128-position blocks -4, fp32 -1
    assert lib.stu_conv_prefill_approx_tc5(a, a, a + 2, a, 333 * 8, 8, 1, 8, 256, 168, 0, 333, None, 1, None) == -3
    assert lib.stu_conv_prefill_approx_tc5(a, a, a, a, 333 * 8, 8, 1, 8, 168, 168, 0, 333, None, 1, None) == -4
    assert lib.stu_conv_prefill_approx_tc5(a, a, a, a, 333 * 8, 8, 1, 8, 256, 168, 0, 333, None, 0, None) == -1


def test_programmatic_launch_switch_round_trips_without_a_gpu():
    """stu_set_programmatic_launch returns the previous setting; the token-step kernels read it at launch time."""
    from flash_stu_2_b200 import ops
    prev = ops.set_programmatic_launch(False)
    try:
        assert ops.set_programmatic_launch(True) is False
        assert ops.set_programmatic_launch(True) is True
    finally:
        ops.set_programmatic_launch(prev)


def test_linear_bench_module_imports_without_a_gpu():
    import torch
    import flash_stu_2_b200.linear_bench as lb
    if torch.cuda.is_available():
        pytest.skip("with a GPU the module would run its measurement")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        lb.main([])


def test_ops_refuse_cpu_tensors():
    import torch
    from flash_stu_2_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.rmsnorm(torch.randn(2, 8), torch.ones(8))
