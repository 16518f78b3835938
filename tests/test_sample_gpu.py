"""GPU sampler (csrc/sample.cu, nt_model_sample) against the host sampler on the same logits, settings and mt19937 stream.

Green on hardware; the sampler is the default of Engine::generate since.  Its logic is also verified on the
CPU emulator against the reference's own sampler (tests/test_sample_sim.py).  On hardware the only expected
difference is exp(): double-precision exp rounded to float vs glibc expf — identical draws except when r falls within an ulp
of a CDF step, hence the >= 97 % bar below instead of equality."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = [pytest.mark.gpu]

from ntransformer_b200._lib import lib  # noqa: E402
from ntransformer_b200.engine import Model  # noqa: E402
from ntransformer_b200.model_spec import LlamaConfig  # noqa: E402


def test_gpu_draws_match_the_host_sampler():
    cfg = LlamaConfig(vocab_size=32000, hidden_size=512, intermediate_size=1024, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64,
                      max_seq_len=64, bos_token_id=1, eos_token_id=2)
    m = Model.synthetic(cfg, "Q8_0", seed=5)
    rng = np.random.default_rng(3)
    same = total = 0
    pos = 0
    for trial in range(60):
        logits = m.forward([int(rng.integers(3, cfg.vocab_size))], pos).copy()
        pos = (pos + 1) % (cfg.max_seq_len - 1)
        temperature = float(rng.choice([0.5, 0.7, 1.0, 1.3]))
        top_k = int(rng.choice([1, 8, 40, 200, 1024]))
        top_p = float(rng.choice([0.5, 0.9, 1.0]))
        penalty = float(rng.choice([1.0, 1.1, 1.3]))
        window = int(rng.choice([0, 16, 64]))
        recent = rng.integers(0, cfg.vocab_size, size=int(rng.integers(0, 80))).astype(np.int32)
        seed = int(rng.integers(0, 2**31))
        host = lib().nt_sample_token(logits.ctypes.data_as(C.c_void_p), cfg.vocab_size, temperature, top_k, top_p, penalty, window,
                                     recent.ctypes.data_as(C.c_void_p) if len(recent) else None, len(recent), seed)
        w = min(len(recent), window) if penalty > 1.0 else 0
        win = np.ascontiguousarray(recent[len(recent) - w:])
        r = lib().nt_sampler_uniform(seed, 0)
        gpu = lib().nt_model_sample(m._h, temperature, top_k, top_p, penalty, win.ctypes.data_as(C.c_void_p) if w else None, w, r)
        assert 0 <= gpu < cfg.vocab_size
        total += 1
        same += int(gpu == host)
    m.close()
    assert same >= 0.97 * total, (same, total)


def test_uncovered_settings_return_minus_one():
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, n_layers=1, n_heads=8, n_kv_heads=2, head_dim=64,
                      max_seq_len=32, bos_token_id=1, eos_token_id=2)
    m = Model.synthetic(cfg, "Q8_0", seed=5)
    m.forward([1], 0)
    for temperature, top_k in ((0.0, 40), (0.7, 0), (0.7, 512), (0.7, 5000)):
        assert lib().nt_model_sample(m._h, temperature, top_k, 0.9, 1.0, None, 0, 0.5) == -1
    m.close()
