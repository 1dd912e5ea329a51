"""The allocation-free Q4_K product (gufo_cuda_matmul_q4k_static_device), for callers that may
not call cudaMalloc while they run (capture regions, hosts that own the whole device through an
arena). It stages x in a 64 KiB buffer built into the library instead of the context's
growable one. Checked here against the ordinary entry point on the same inputs, twice in a row
(the buffer is shared and keeps the previous call's contents), and at its size limit.

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


def test_static_buffer_product_matches_the_ordinary_one():
    dev = torch.device("cuda:0")
    ctx = Context(0)
    rows, cols = 1000, 2048
    raw = Q.quantize_q4_k(torch.randn(rows, cols, generator=torch.Generator().manual_seed(3)) * 0.02).to(dev)
    m = ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), rows, cols)
    parts = Context._parts([(m, 0, rows)])
    gen = torch.Generator(device=dev).manual_seed(4)
    for call, tokens in enumerate((1, 3)):          # two calls in a row, the second wider
        x = torch.randn(tokens, cols, device=dev, generator=gen)
        want = torch.empty(tokens, rows, device=dev)
        got = torch.full((tokens, rows), float("nan"), device=dev)
        torch.cuda.synchronize()
        ctx.matmul_device(parts, 1, x, tokens, want)
        ctx._check(ctx.lib.gufo_cuda_matmul_q4k_static_device(
            ctx.handle, C.c_void_p(raw.data_ptr()), rows, cols, C.c_void_p(x.data_ptr()), tokens,
            C.c_void_p(got.data_ptr())))
        ctx.synchronize()
        err = float(torch.linalg.norm(got - want) / torch.linalg.norm(want))
        assert err <= 1e-6, (call, err)              # same kernels, same arithmetic
    # Beyond the built-in buffer: refused with a clear message, nothing launched.
    big = torch.zeros(8, 4096, device=dev)
    wide = torch.zeros(16 * Q.row_bytes(Q.GGML_Q4_K, 4096), dtype=torch.uint8, device=dev)
    before = ctx.launch_count()
    with pytest.raises(GufoCudaError) as e:
        ctx._check(ctx.lib.gufo_cuda_matmul_q4k_static_device(
            ctx.handle, C.c_void_p(wide.data_ptr()), 16, 4096, C.c_void_p(big.data_ptr()), 8,
            C.c_void_p(torch.empty(8, 16, device=dev).data_ptr())))
    assert e.value.status == 7 and "built-in buffer" in str(e.value)
    assert ctx.launch_count() == before
    ctx.close()
