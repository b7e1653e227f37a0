"""The reference's model-level golden on the GPU decoder.

tests/golden/parity-tiny (the reference's tests/fixtures/parity-tiny) is read with the
model-directory reader and served by the device decoder in float32, one teacher-forced
token at a time over one KV cache; the logits must stay within the reference's own budget
(1e-2, crates/quantibbler-server/tests/parity_tiny.rs:26) of the HF goldens and within
float32 rounding of the NumPy restatement of the forward.  The model has per-head q/k norms
and head_dim 32.

The file name sorts after every other test file, so a run that stops at the first failure
has already run the rest.
"""

import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import decoder_np
from quantibbler_b200 import model_dir
from quantibbler_b200.decoder import Decoder

pytestmark = pytest.mark.gpu

FIXTURE = os.path.join(GOLDEN, "parity-tiny")


@pytest.fixture(autouse=True)
def _restore_stream(gpu_ctx):
    yield
    gpu_ctx.set_stream(None)


@pytest.mark.parametrize("kv_dtype,tol", [("float32", 5e-4), ("bfloat16", 5e-3)])
def test_parity_tiny_logits_on_the_device_decoder(gpu_ctx, kv_dtype, tol):
    md = model_dir.load(FIXTURE)
    cfg, weights = model_dir.decoder_inputs(md, max_seq=16, max_batch=1)
    cfg.kv_dtype = kv_dtype
    with open(os.path.join(FIXTURE, "goldens.json")) as f:
        g = json.load(f)
    dec = Decoder(gpu_ctx, cfg, weights)
    assert dec.has_qk_norm
    session = decoder_np.Session(cfg, weights,
                                 kv_round=decoder_np._bf16 if kv_dtype == "bfloat16" else None)
    worst_golden = worst_oracle = 0.0
    for pos, tok in enumerate(g["input_ids"]):
        dec.start([tok], [pos])          # the cache keeps the earlier positions
        dec.step()
        gpu_ctx.synchronize()
        got = dec.logits.cpu().numpy()[0]
        _, want = session.step(tok)
        worst_oracle = max(worst_oracle, float(np.abs(got - want).max()))
        worst_golden = max(worst_golden,
                           float(np.abs(got - np.asarray(g["logits"][pos], np.float32)).max()))
    assert worst_golden <= 1e-2
    assert worst_oracle <= tol


def test_batched_decode_with_qk_norms_matches_the_restatement(gpu_ctx):
    # three sequences at once, greedy, through the q/k-norm path
    md = model_dir.load(FIXTURE)
    cfg, weights = model_dir.decoder_inputs(md, max_seq=16, max_batch=3)
    first = [5, 17, 99]
    dec = Decoder(gpu_ctx, cfg, weights)
    dec.start(first, [0, 0, 0])
    sessions = [decoder_np.Session(cfg, weights) for _ in first]
    toks = list(first)
    for _ in range(5):
        dec.step()
        gpu_ctx.synchronize()
        got = dec.logits.cpu().numpy()
        want = []
        for b, s in enumerate(sessions):
            toks[b], lg = s.step(toks[b])
            want.append(lg)
        want = np.array(want)
        assert np.abs(got - want).max() <= 1e-3 * max(1.0, float(np.abs(want).max()))
        dec.advance()
        # follow the device's greedy choice only where it is not a rounding tie
        dev_toks = dec.token_ids.cpu().numpy()
        for b in range(len(first)):
            top2 = np.sort(want[b])[-2:]
            if top2[1] - top2[0] > 1e-3:
                assert dev_toks[b] == toks[b]
        toks = [int(t) for t in dev_toks]   # the restatement is fed what the device chose


def test_generate_follows_the_engine_control_flow(gpu_ctx):
    # engine/mod.rs:1377-1500: prefill position by position, first token from the last prompt
    # position, EOS ends the run and is not returned, max_tokens ends it with "length"
    md = model_dir.load(FIXTURE)
    cfg, weights = model_dir.decoder_inputs(md, max_seq=64, max_batch=1)
    dec = Decoder(gpu_ctx, cfg, weights)
    for prompt in ([5, 17, 3], [1], [99, 42, 7, 0, 64]):
        want, finish = decoder_np.generate(cfg, weights, prompt, 12, eos_token_id=md.eos_token_id)
        got = dec.generate(prompt, 12, eos_token_id=md.eos_token_id)
        assert got["completion_tokens"] == want and got["finish"] == finish
        assert got["prompt_tokens"] == len(prompt) and got["prompt_ms"] >= 1
    # a token the model does produce, declared as EOS: the run stops before it
    want, finish = decoder_np.generate(cfg, weights, [5, 17, 3], 12, eos_token_id=29)
    assert finish == "stop" and want == [73, 34, 38]
    got = dec.generate([5, 17, 3], 12, eos_token_id=29)
    assert (got["completion_tokens"], got["finish"]) == (want, "stop")
    got = dec.generate([5, 17, 3], 0)
    assert (got["completion_tokens"], got["finish"]) == ([73], "length")
    with pytest.raises(ValueError, match="prompt tokenized to zero tokens"):
        dec.generate([], 4)
    with pytest.raises(ValueError, match="does not fit the KV cache"):
        dec.generate([1] * 60, 8)


def test_bf16_blob_is_served_in_bfloat16_on_the_device(gpu_ctx):
    # the reference's writer packed parity-tiny at bf16; a blob is served at its declared
    # dtype (model/mod.rs:725-734): bfloat16 linears, norms (incl. q/k norms) and head
    from quantibbler_b200 import blob
    md = blob.load_any(os.path.join(GOLDEN, "parity-tiny-bf16.qpk"))
    cfg, weights = model_dir.decoder_inputs(md, max_seq=16, max_batch=1)
    assert cfg.serving == "bfloat16"
    with open(os.path.join(FIXTURE, "goldens.json")) as f:
        g = json.load(f)
    dec = Decoder(gpu_ctx, cfg, weights)
    session = decoder_np.Session(cfg, weights)
    worst_golden = worst_oracle = 0.0
    for pos, tok in enumerate(g["input_ids"]):
        dec.start([tok], [pos])
        dec.step()
        gpu_ctx.synchronize()
        got = dec.logits.cpu().numpy()[0]
        _, want = session.step(tok)
        worst_oracle = max(worst_oracle, float(np.abs(got - want).max()))
        worst_golden = max(worst_golden,
                           float(np.abs(got - np.asarray(g["logits"][pos], np.float32)).max()))
    assert worst_golden <= 1e-2          # the reference's budget, parity_tiny.rs:26
    assert worst_oracle <= 1e-2          # bfloat16 roundings land on different ties
