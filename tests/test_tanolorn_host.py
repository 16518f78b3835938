"""CPU tests of the Tanolorn family: the oracle's own invariants, and the engine's reading of a model folder (what it accepts, what it
refuses and why).  Nothing here needs a GPU: nt_model_dir_describe parses config.json and the safetensors header only."""
import ctypes as C

import numpy as np
import pytest

import tanolorn_oracle as O
from zelunex_util import write_model_dir

from ntransformer_b200._lib import lib


def describe(path):
    buf = C.create_string_buffer(1 << 16)
    rc = lib().nt_model_dir_describe(str(path).encode(), buf, len(buf))
    return rc, buf.value.decode()


def test_oracle_is_causal_and_cut_free():
    rng = np.random.default_rng(0)
    cfg, W = O.random_model(rng, kv_from={3: 1})
    toks = rng.integers(0, cfg["vocab"], 40)
    full = O.forward(cfg, W, toks)
    np.testing.assert_allclose(O.forward(cfg, W, toks[:17]), full[:17], rtol=1e-9, atol=1e-9)      # a prefix does not see what follows
    other = toks.copy(); other[30] = (other[30] + 1) % cfg["vocab"]
    np.testing.assert_allclose(O.forward(cfg, W, other)[:30], full[:30], rtol=1e-9, atol=1e-9)


def test_oracle_router_groups_and_negative_choice_scores():
    P = {"mlp.router": np.eye(6), "mlp.correction": np.array([0.0, 0.0, 0.0, 0.0, -5.0, -5.0])}
    mlp = {"router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}}
    h = np.array([[0.0, 0.0, 4.0, 0.0, 9.0, 9.0]])            # the last group has the largest plain scores, but its correction sinks it
    sel, wt = O.route(h, P, "", mlp)
    assert sel.tolist() == [[2, 3]]                            # group (2, 3) wins and both choices come from inside it
    P["mlp.correction"] = np.full(6, -3.0)                     # every choice score negative: an excluded group must not return as 0
    sel, wt = O.route(h, P, "", mlp)
    assert set(sel[0].tolist()) == {4, 5} and np.allclose(wt, 1 / (1 + np.exp(-9.0)))


def test_oracle_conv_and_rotation_conventions():
    u = np.arange(1.0, 6.0)[:, None]
    w = np.array([[0.0, 0.0, 1.0]])                            # the last tap is the current token's
    np.testing.assert_allclose(O.causal_conv(u, w, np.zeros(1))[:, 0], u[:, 0])
    w = np.array([[1.0, 0.0, 0.0]])
    np.testing.assert_allclose(O.causal_conv(u, w, np.zeros(1))[:, 0], [0, 0, 1, 2, 3])
    v = np.array([[1.0, 0.0, 0.0, 0.0, 7.0]])                  # dims 4: channel 0 pairs with channel 2; channel 4 passes
    r = O.rotate_half(v, [1], 4, 100.0)
    np.testing.assert_allclose(r[0], [np.cos(1.0), 0.0, np.sin(1.0), 0.0, 7.0], atol=1e-12)


def test_model_folder_is_read_as_configured(tmp_path):
    rng = np.random.default_rng(1)
    cfg, W = O.random_model(rng, kv_from={3: 1})
    rc, text = describe(write_model_dir(tmp_path / "ok", cfg, W))
    assert rc == 0, text
    assert "architecture=Tanolorn" in text and "layers=4" in text
    assert "mixer=scan state=12 groups=2 conv=4 norm_groups=2 ff_kind=dense" in text
    assert "mixer=latent q_rank=12 kv_rank=20 rot_dim=6 rot=6 kv_from=-1 ff_kind=moe experts=6 top=2 route_groups=3/2 side=5" in text
    assert "kv_from=1 ff_kind=none" in text
    assert "tensors=%d" % len(W) in text


@pytest.mark.parametrize("what", ["missing_tensor", "wrong_shape", "kv_from_forward", "kv_from_scan", "kv_from_chain", "kv_rank_differs", "odd_rot", "top_over_experts",
                                  "groups_uneven", "kept_groups_too_small", "unknown_mixer", "unknown_ff", "heads_not_in_groups", "norm_groups_uneven", "missing_key"])
def test_bad_model_folders_are_refused(tmp_path, what):
    rng = np.random.default_rng(2)
    cfg, W = O.random_model(rng, kv_from={3: 1})
    L = cfg["layers"]
    if what == "missing_tensor":
        del W["l2.mlp.correction"]
    elif what == "wrong_shape":
        W["l0.mix.conv"] = W["l0.mix.conv"][:, :3]
    elif what == "kv_from_forward":
        L[1]["mixer"]["kv_from"] = 3
    elif what == "kv_from_scan":
        L[3]["mixer"]["kv_from"] = 0
    elif what == "kv_from_chain":
        cfg, W = O.random_model(rng, pattern=("latent", "latent", "latent"), kv_from={1: 0, 2: 1})
    elif what == "kv_rank_differs":
        L[3]["mixer"]["kv_rank"] = 24
    elif what == "odd_rot":
        L[1]["mixer"]["rot"]["dims"] = 5
    elif what == "top_over_experts":
        L[1]["mlp"]["router"]["top"] = 7
    elif what == "groups_uneven":
        L[1]["mlp"]["router"]["groups"]["count"] = 4
    elif what == "kept_groups_too_small":
        L[1]["mlp"]["router"]["groups"] = {"count": 6, "keep": 1}
    elif what == "unknown_mixer":
        L[0]["type"] = "attention"
    elif what == "unknown_ff":
        L[0]["mlp"]["kind"] = "glu"
    elif what == "heads_not_in_groups":
        L[0]["mixer"]["groups"] = 3
    elif what == "norm_groups_uneven":
        L[0]["mixer"]["norm_groups"] = 5
    elif what == "missing_key":
        del L[0]["mixer"]["state"]
    rc, text = describe(write_model_dir(tmp_path / what, cfg, W))
    assert rc != 0, text
