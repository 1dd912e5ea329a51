"""The allocation-free Q4_K product (gufo_cuda_matmul_q4k_static_device), for callers that may
not call cudaMalloc while they run (capture regions, hosts that own the whole device through an
arena). It stages x in a 64 KiB buffer built into the library instead of the context's
growable one. Checked here against the ordinary entry point and the CPU oracle on the same
inputs, over calls in a row that widen and narrow the staged image (the buffer is shared and
keeps the previous call's contents), at the largest shape it accepts, and for leaving the
device's free memory untouched.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from gufo_npu_b200 import quantize as Q
from gufo_npu_b200._capi import GufoCudaError
from gufo_npu_b200.backend import Context

pytestmark = pytest.mark.gpu


def test_static_buffer_product_matches_the_ordinary_one(oracle):
    dev = torch.device("cuda:0")
    ctx = Context(0)
    rows, cols = 1000, 2048
    raw = Q.quantize_q4_k(torch.randn(rows, cols, generator=torch.Generator().manual_seed(3)) * 0.02)
    raw_host = raw.numpy()
    raw = raw.to(dev)
    m = ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), rows, cols)
    parts = Context._parts([(m, 0, rows)])
    gen = torch.Generator(device=dev).manual_seed(4)

    def static(x, tokens, out):
        ctx._check(ctx.lib.gufo_cuda_matmul_q4k_static_device(
            ctx.handle, C.c_void_p(raw.data_ptr()), rows, cols, C.c_void_p(x.data_ptr()), tokens,
            C.c_void_p(out.data_ptr())))

    # Calls in a row: narrow, wider, the widest shape the buffer takes at this width (8 tokens,
    # 52736 bytes), then narrow again: stale planes, column factors and sums of a wider layout
    # must not leak into a narrower product.
    for call, tokens in enumerate((1, 3, 8, 1, 2)):
        x = torch.randn(tokens, cols, device=dev, generator=gen)
        want = torch.empty(tokens, rows, device=dev)
        got = torch.full((tokens, rows), float("nan"), device=dev)
        ctx.matmul_device(parts, 1, x, tokens, want)
        ctx.synchronize()
        free_before = torch.cuda.mem_get_info(0)[0]
        static(x, tokens, got)
        ctx.synchronize()
        free_after = torch.cuda.mem_get_info(0)[0]
        if call > 0:
            # After the first call (whose set-up looks the buffer's address up), a call leaves
            # the device's free memory as it found it: nothing was allocated or freed. The
            # kernels' code is already loaded: the ordinary product above runs the same ones.
            assert free_after == free_before, (call, free_before, free_after)
        err = float(torch.linalg.norm(got - want) / torch.linalg.norm(want))
        assert err <= 1e-6, (call, err)              # same kernels, same arithmetic
        ref = oracle.matmul([(raw_host, Q.GGML_Q4_K, 0, rows)], cols, x.cpu().numpy())
        err = float(np.linalg.norm(got.cpu().numpy().astype(np.float64) - ref) / np.linalg.norm(ref))
        assert err <= 1e-3, (call, err)
    # Beyond the built-in buffer: refused with a clear message, nothing launched.
    big = torch.zeros(8, 4096, device=dev)
    wide = torch.zeros(16 * Q.row_bytes(Q.GGML_Q4_K, 4096), dtype=torch.uint8, device=dev)
    before = ctx.launch_count()
    with pytest.raises(GufoCudaError) as e:
        ctx._check(ctx.lib.gufo_cuda_matmul_q4k_static_device(
            ctx.handle, C.c_void_p(wide.data_ptr()), 16, 4096, C.c_void_p(big.data_ptr()), 8,
            C.c_void_p(torch.empty(8, 16, device=dev).data_ptr())))
    assert e.value.status == 7 and "built-in buffer" in str(e.value)
    # A width no buffer of this size could hold, far past the range of an int: refused as well.
    with pytest.raises(GufoCudaError) as e:
        ctx._check(ctx.lib.gufo_cuda_matmul_q4k_static_device(
            ctx.handle, C.c_void_p(wide.data_ptr()), 16, 256 * (1 << 32), C.c_void_p(big.data_ptr()), 1,
            C.c_void_p(torch.empty(8, 16, device=dev).data_ptr())))
    assert e.value.status == 7
    assert ctx.launch_count() == before
    ctx.close()
