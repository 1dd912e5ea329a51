"""The one-token decode step as one persistent kernel (context option "step_kernel" = 1):
same logits as the launch chain and as the reference, and a wait that runs out is reported
without losing the context."""
import numpy as np
import pytest
import torch

from gufo_npu_b200 import _capi
from gufo_npu_b200 import synth
from gufo_npu_b200._capi import GufoCudaError
from gufo_npu_b200.backend import Context, CudaDecoder, CudaProjections
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

STEP_TOL = 2e-3      # logits relative L2 (the reference's own decoder bound, decoder_test.cpp:30-31)


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture()
def ctx():
    c = Context(0)
    c.set_option("step_kernel", 1)
    yield c
    c.close()


def test_step_kernel_matches_reference_logits(ctx, golden):
    """The dense test model: the 8 committed tokens, then 1100 positions against the reference's
    logits (attention slices of many positions), all through the persistent kernel."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=G.LONG_STEPS, use_graph=True)
    g = golden("decoder")
    for i, tok in enumerate(int(t) for t in g["decoder_dense_tokens"]):
        logits = dec.Step(tok)
        want = g["decoder_dense_logits"][i]
        assert rel_l2(logits, want) <= 1e-4, (i, rel_l2(logits, want))
        assert int(np.argmax(logits)) == int(np.argmax(want))
    profile = dec.step_profile()
    assert len(profile) > 0 and profile[0]["stage"] == "embed" and profile[-1]["stage"] == "lm_head"
    assert all(p["us"] > 0 for p in profile)
    dec.Reset()
    long = golden("decoder_long")
    keep = {int(p): i for i, p in enumerate(long["positions"])}
    for pos, tok in enumerate(G.long_tokens(cfg.vocab)):
        if pos in keep:
            got = dec.Step(int(tok))
            want = long["logits"][keep[pos]]
            assert rel_l2(got, want) <= 5e-4, (pos, rel_l2(got, want))
            assert int(np.argmax(got)) == int(np.argmax(want)), pos
        else:
            dec.step_device(int(tok))
    dec.status()
    dec.close()


@pytest.mark.parametrize("shape", [dict(hidden=512, ffn=2560, vocab=1000), dict(hidden=2304, ffn=768, vocab=777),
                                   dict(hidden=256, ffn=512, vocab=512, linear_head_dim=64, linear_key_heads=2,
                                        linear_value_heads=4)])
def test_step_kernel_matches_the_launch_chain(shape):
    """Shapes that split a product over K (ffn 2560: two slabs, partial rows added by the next
    stage), that accumulate several slabs per row tile (hidden 2304), a 64-wide DeltaNet head
    and a vocabulary off the tile size: the persistent kernel against the launch chain on the
    same tokens, with and without logits, and the states afterwards."""
    kwargs = dict(G.DENSE)
    kwargs.update(shape)
    cfg = synth.ModelConfig(**kwargs)
    tensors = synth.build_model(cfg, 21)
    tokens = [int(t) for t in np.random.default_rng(3).integers(0, cfg.vocab, size=10)]
    outs, states = [], []
    for kernel in (0, 1):
        c = Context(0)
        c.set_option("step_kernel", kernel)
        dec = CudaDecoder(CudaProjections(c, cfg, tensors), tensors, max_positions=32, use_graph=True)
        rows = []
        for i, tok in enumerate(tokens):
            if i == 4:
                assert dec.StepTokens([tok], logits=False) is None    # a step without the LM head
                rows.append(dec.hidden(0))
            else:
                rows.append(dec.Step(tok))
        if kernel:
            assert len(dec.step_profile()) > 0, "the model was expected to run on the persistent kernel"
        outs.append(rows)
        states.append(dec.linear_state(0))
        dec.close()
        c.close()
    for i, (a, b) in enumerate(zip(*outs)):
        assert rel_l2(b, a) <= 1e-4, (i, rel_l2(b, a))   # summation orders differ; the step bound is 2e-3
    assert rel_l2(states[1][0], states[0][0]) <= 1e-5
    assert rel_l2(states[1][1], states[0][1]) <= 1e-5


def test_step_kernel_wait_that_runs_out_is_reported(ctx, golden):
    """Block 0 stays away from one grid barrier (a test hook): the other blocks' waits run out
    after the two milliseconds set here, the kernel ends by itself, the step reports
    GUFO_CUDA_TIMEOUT once, and after a reset the same decoder computes the right logits."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=16, use_graph=True)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_dense_tokens"]]
    assert rel_l2(dec.Step(tokens[0]), g["decoder_dense_logits"][0]) <= 1e-4
    ctx.set_option("step_wait_us", 2000)
    ctx.set_option("step_skip_arrival", 3)
    with pytest.raises(GufoCudaError) as e:
        dec.Step(tokens[1])
    assert e.value.status == _capi.STATUS_TIMEOUT
    ctx.set_option("step_skip_arrival", -1)
    ctx.set_option("step_wait_us", 2000000)
    dec.status()                       # the failure was reported once and cleared
    dec.Reset()
    for i, tok in enumerate(tokens[:3]):
        assert rel_l2(dec.Step(tok), g["decoder_dense_logits"][i]) <= 1e-4, i
    # A failure in a step that leaves its logits on the device surfaces at the next status call.
    ctx.set_option("step_wait_us", 2000)
    ctx.set_option("step_skip_arrival", 0)
    dec.step_device(tokens[3])
    with pytest.raises(GufoCudaError) as e:
        dec.status()
    assert e.value.status == _capi.STATUS_TIMEOUT
    ctx.set_option("step_skip_arrival", -1)
    ctx.set_option("step_wait_us", 2000000)
    dec.Reset()
    assert rel_l2(dec.Step(tokens[0]), g["decoder_dense_logits"][0]) <= 1e-4
    dec.close()
