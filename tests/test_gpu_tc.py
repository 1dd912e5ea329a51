"""GPU parity of the tcgen05 small-M GEMM (16 or more token rows per weight read) against the
CPU oracle's fused row dots. Weights and activations are rounded to fp16 on this path, so the
bound is the 1e-3 relative L2 of the GEMM outputs, with the measured error asserted tighter."""
import numpy as np
import pytest
import torch

from gufo_npu_b200 import quantize as Q
from gufo_npu_b200.backend import Context
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-3


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture(scope="module")
def ctx():
    """Every product of 16 or more token rows goes to the tcgen05 GEMM here (option value 2);
    by default the dispatcher keeps small batches on the 8-token passes where those are faster."""
    c = Context(0)
    c.set_option("tc_gemm", 2)
    yield c
    c.close()


def _weights(seed, rows, cols, ggml_type=Q.GGML_Q4_K):
    raw = Q.quantize(ggml_type, torch.from_numpy(G.normal(seed, rows, cols) * 0.02)).numpy()
    return raw.reshape(rows, -1)


@pytest.mark.parametrize("ggml_type", [Q.GGML_Q4_K, Q.GGML_Q6_K])
@pytest.mark.parametrize("rows,cols", [(256, 512), (130, 256), (1000, 2560), (2560, 9728)])
@pytest.mark.parametrize("tokens", [16, 17, 33, 128, 131])
def test_gemm_matches_oracle(ctx, oracle, ggml_type, rows, cols, tokens):
    """One Q4_K or Q6_K part: row counts off the 256-row tile, K split over thread blocks
    (2560 x 9728), block counts that leave a partial slab in the Q6_K device arrangement (10, 38),
    token counts off the tile granule and past one pass."""
    if rows * cols * tokens > 1.5e9:
        tokens = min(tokens, 33)
    raw = _weights(40 + rows % 7, rows, cols, ggml_type)
    x = G.normal(50 + tokens, tokens, cols)
    m = ctx.matrix_upload(ggml_type, raw, rows, cols)
    got = ctx.matmul([(m, 0, rows)], x, tokens, rows)
    ctx.synchronize()
    want = oracle.matmul([(raw, ggml_type, 0, rows)], cols, x)
    err = rel_l2(got, want)
    assert err <= GEMM_TOL, err
    assert err <= 5e-4, err
    # Per token too: no row of the batch may hide behind the others.
    for t in range(tokens):
        assert rel_l2(got[t], want[t]) <= GEMM_TOL, t
    ctx.matrix_free(m)


def test_gemm_agrees_with_the_eight_token_passes(ctx):
    """The same product with the tensor-memory path switched off (int8 tensor-core passes of 8
    tokens) differs only by the fp16 rounding of this path."""
    rows, cols, tokens = 384, 1024, 40
    raw = _weights(61, rows, cols)
    x = G.normal(62, tokens, cols)
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, rows, cols)
    got = ctx.matmul([(m, 0, rows)], x, tokens, rows)
    ctx.set_option("tc_gemm", 0)
    try:
        ref = ctx.matmul([(m, 0, rows)], x, tokens, rows)
    finally:
        ctx.set_option("tc_gemm", 2)
    assert not np.array_equal(got, ref)
    assert rel_l2(got, ref) <= 5e-4
    ctx.matrix_free(m)


def test_gemm_stacked_parts_and_row_ranges(ctx, oracle):
    """Gate and up stacked (one Q4_K, one Q6_K: two launches), a row range inside a matrix, an
    F32 part beside them (it takes the other kernels), every output column in its place."""
    cols, tokens = 768, 24
    gate, up = _weights(63, 300, cols), _weights(64, 300, cols, Q.GGML_Q6_K)
    extra = G.normal(65, 5, cols)
    mg = ctx.matrix_upload(Q.GGML_Q4_K, gate, 300, cols)
    mu = ctx.matrix_upload(Q.GGML_Q6_K, up, 300, cols)
    mf = ctx.matrix_upload(Q.GGML_F32, extra.view(np.uint8), 5, cols)
    x = G.normal(66, tokens, cols)
    got = ctx.matmul([(mg, 0, 300), (mf, 0, 5), (mu, 17, 200)], x, tokens, 505)
    want = oracle.matmul([(gate, Q.GGML_Q4_K, 0, 300), (extra.view(np.uint8).reshape(5, -1), Q.GGML_F32, 0, 5),
                          (up, Q.GGML_Q6_K, 17, 200)], cols, x)
    assert rel_l2(got[:, :300], want[:, :300]) <= 5e-4
    assert rel_l2(got[:, 300:305], want[:, 300:305]) <= 1e-5
    assert rel_l2(got[:, 305:], want[:, 305:]) <= 5e-4
    for m in (mg, mu, mf):
        ctx.matrix_free(m)


def test_gemm_ragged_verify_batch(ctx, oracle):
    """Config-5 packing at reduced width: 32 sequences of 1 to 4 draft tokens (seeded) packed into
    M rows with offsets[33]; each sequence's rows equal the same rows multiplied alone."""
    rng = np.random.default_rng(77)
    lengths = rng.integers(1, 5, size=32)
    offsets = np.concatenate([[0], np.cumsum(lengths)])
    m_rows = int(offsets[-1])
    rows, cols = 512, 1280
    raw = _weights(67, rows, cols)
    x = G.normal(68, m_rows, cols)
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, rows, cols)
    got = ctx.matmul([(m, 0, rows)], x, m_rows, rows)
    want = oracle.matmul([(raw, Q.GGML_Q4_K, 0, rows)], cols, x)
    for s in range(32):
        lo, hi = int(offsets[s]), int(offsets[s + 1])
        assert rel_l2(got[lo:hi], want[lo:hi]) <= GEMM_TOL, s
    ctx.matrix_free(m)


def test_gemm_activation_range(ctx, oracle):
    """Rows of very different magnitude in one batch: each row is scaled on its own, so a huge
    row does not flush a tiny one and neither overflows fp16. A zero row stays zero."""
    rows, cols, tokens = 256, 512, 16
    raw = _weights(69, rows, cols)
    x = G.normal(70, tokens, cols)
    x[1] *= 1e30
    x[2] *= 1e-30
    x[3] = 0.0
    x[4] *= 65504.0 * 4
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, rows, cols)
    got = ctx.matmul([(m, 0, rows)], x, tokens, rows)
    want = oracle.matmul([(raw, Q.GGML_Q4_K, 0, rows)], cols, x)
    assert np.isfinite(got).all()
    assert np.all(got[3] == 0.0)
    for t in range(tokens):
        if t != 3:
            assert rel_l2(got[t], want[t]) <= GEMM_TOL, t
    ctx.matrix_free(m)
