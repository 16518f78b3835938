"""CPU tests of the Savidra family: the oracle's own invariants, and the engine's reading of a model folder (what it accepts, what it
refuses and why).  Nothing here needs a GPU: nt_model_dir_describe parses config.json and the safetensors header only."""
import ctypes as C

import numpy as np
import pytest

import savidra_oracle as O
from zelunex_util import write_model_dir

from ntransformer_b200._lib import lib


def describe(path):
    buf = C.create_string_buffer(1 << 16)
    rc = lib().nt_model_dir_describe(str(path).encode(), buf, len(buf))
    return rc, buf.value.decode()


def test_oracle_is_causal_and_cut_free():
    rng = np.random.default_rng(0)
    cfg, W = O.random_model(rng)
    toks = rng.integers(0, cfg["vocab"], 40)
    full = O.forward(cfg, W, toks)
    np.testing.assert_allclose(O.forward(cfg, W, toks[:17]), full[:17], rtol=1e-9, atol=1e-9)      # a prefix does not see what follows
    other = toks.copy(); other[30] = (other[30] + 1) % cfg["vocab"]
    np.testing.assert_allclose(O.forward(cfg, W, other)[:30], full[:30], rtol=1e-9, atol=1e-9)


def test_oracle_conventions():
    u = np.arange(1.0, 6.0)[:, None]
    np.testing.assert_allclose(O.causal_conv(u, np.array([[0.0, 0.0, 1.0]]))[:, 0], u[:, 0])        # the last tap is the current token's
    np.testing.assert_allclose(O.causal_conv(u, np.array([[1.0, 0.0, 0.0]]))[:, 0], [0, 0, 1, 2, 3])
    v = np.array([[[1.0, 0.0, 0.0, 0.0, 7.0]]])                                                      # dims 4: channel 0 pairs with channel 2; channel 4 passes
    np.testing.assert_allclose(O.rotate_half(v, [1], 4, 100.0)[0, 0], [np.cos(1.0), 0.0, np.sin(1.0), 0.0, 7.0], atol=1e-12)
    np.testing.assert_allclose(O.rotate_half(v, [8], 4, 100.0, divide=8.0)[0, 0], [np.cos(1.0), 0.0, np.sin(1.0), 0.0, 7.0], atol=1e-12)
    np.testing.assert_allclose(O.token_shift(np.array([[2.0], [4.0]]), np.array([0.25])), [[1.5], [3.5]])
    # the sink counts once, unscaled, and has no value: two equal keys and a sink of the same height share the weight in thirds
    w = O.causal_weights(np.zeros((2, 1, 3)), np.zeros((2, 1, 3)), 5.0, 1, sink=np.zeros(1))
    np.testing.assert_allclose(w[0], [[0.5, 0.0], [1 / 3, 1 / 3]])
    # the delta rule's read-out sees the current token's write: one step from an empty state gives beta * <q, k> * v
    o = O.delta_rule(np.array([[[0.5, 0.0]]]), np.array([[[1.0, 0.0]]]), np.array([[[3.0]]]), np.array([[0.5]]), np.array([[[0.1, 0.1]]]))
    np.testing.assert_allclose(o, [[[0.75]]])


def test_model_folder_is_read_as_configured(tmp_path):
    rng = np.random.default_rng(1)
    cfg, W = O.random_model(rng)
    for L in cfg["layers"]:
        if L["type"] == "parallel":
            del L["mixer"]["right"]["decay_rank"], L["mixer"]["right"]["gate_rank"]                  # read from the tensors' shapes
    rc, text = describe(write_model_dir(tmp_path / "ok", cfg, W))
    assert rc == 0, text
    assert "architecture=Savidra" in text and "layers=4" in text
    assert "delta(heads=4 kv=2 dim=10 vdim=6 conv=2 ranks=5/7)" in text
    assert "attention(heads=4 kv=2 dim=12 vdim=10 rot=8 divide=4.000000 conv=3 bias=1 temp=1 talking=1 sink=0 v_first=-1)" in text
    assert "attention(heads=4 kv=2 dim=8 vdim=12 rot=4 divide=1.000000 conv=0 bias=0 temp=0 talking=0 sink=1 v_first=1)" in text
    assert "tensors=%d" % len(W) in text


@pytest.mark.parametrize("what", ["missing_tensor", "wrong_shape", "odd_rot", "rot_over_dim", "heads_not_in_groups", "unknown_mixer", "unknown_ff", "blend_width_differs",
                                  "missing_key", "missing_alpha", "rank_tensor_missing", "conv_too_long", "zero_scaling"])
def test_bad_model_folders_are_refused(tmp_path, what):
    rng = np.random.default_rng(2)
    cfg, W = O.random_model(rng)
    L = cfg["layers"]
    if what == "missing_tensor":
        del W["l0.mix.left.talk"]
    elif what == "wrong_shape":
        W["l0.mix.right.k.conv"] = W["l0.mix.right.k.conv"][:, :1]
    elif what == "odd_rot":
        L[1]["mixer"]["rot"]["dims"] = 3
    elif what == "rot_over_dim":
        L[0]["mixer"]["left"]["rot"]["dims"] = 14
    elif what == "heads_not_in_groups":
        L[0]["mixer"]["right"]["kv_heads"] = 3
    elif what == "unknown_mixer":
        L[2]["type"] = "convolution"
    elif what == "unknown_ff":
        L[2]["mlp"]["kind"] = "moe"
    elif what == "blend_width_differs":
        L[3]["mixer"]["vdim"] = 6
    elif what == "missing_key":
        del L[1]["mixer"]["scale"]
    elif what == "missing_alpha":
        del cfg["postln_alpha"]
    elif what == "rank_tensor_missing":
        del L[0]["mixer"]["right"]["decay_rank"]
        del W["l0.mix.right.a1"]
    elif what == "conv_too_long":
        L[0]["mixer"]["left"]["conv"] = 17
    elif what == "zero_scaling":
        L[0]["mixer"]["left"]["rot"]["scaling"]["factor"] = 0.0
    rc, text = describe(write_model_dir(tmp_path / what, cfg, W))
    assert rc != 0, text
