"""Ligirax without a GPU: the configuration reader, the model's description, the rotary tables, and the plain
implementation's own invariants."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_ligirax as plain
import tiny_ligirax
from rust_deeplearning_b200.config.base import ConfigError, architecture_for
from rust_deeplearning_b200.parts.position import Rotary, rotary_frequencies


def test_configuration_becomes_parts():
    cfg, _ = tiny_ligirax.config("LA")
    arch = architecture_for(cfg)
    assert arch.name == "Ligirax"
    spec = arch.build_spec(arch.parse_config(cfg))
    assert [e.reads_cache_of for e in spec.schedule] == [None, 0, None]
    assert spec.layers[2].feed_forward is None and "pre_feed_forward" not in spec.layers[2].norms
    assert spec.layers[0].mixer.params["cache_window"] == 12      # the reader's window is the wider one
    assert spec.layers[0].mixer.params["window"] == 8 and spec.layers[2].mixer.params["cache_window"] is None
    names = spec.tensor_specs()
    assert "l1.mix.dkv" not in names and "l0.mix.dkv.norm" in names and "l2.norm2" not in names
    assert names["l0.mlp.router"].shape == (7, 64) and names["l1.mlp.e3.down"].shape == (64, 40)
    assert spec.layers[0].norms["post_mixer"].params["scale"] == 0.5 and spec.head.params["scale"] == 2.0


def test_configuration_errors_are_listed_together():
    cfg, _ = tiny_ligirax.config("LA")
    bad = copy.deepcopy(cfg)
    del bad["width"]
    bad["layers"][0]["mixer"]["rot"]["dims"] = 7
    bad["layers"][1]["mixer"]["kv_from"] = 1
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError) as e:
        architecture_for(bad).parse_config(bad)
    text = str(e.value)
    assert "width" in text and "dims" in text and "top" in text
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match="kv_from"):
        architecture_for(bad).parse_config(bad)
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["mixer"]["kv_rank"] = 32
    with pytest.raises(ConfigError, match="kv_rank"):
        architecture_for(bad).parse_config(bad)


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0},
                                     {"factor": 1.5, "original": 4096, "fast": 32.0, "slow": 1.0}])
def test_rotary_tables_against_the_plain_rotation(scaling):
    rot = {"base": 700.0, "dims": 12, **({"scaling": scaling} if scaling else {})}
    f, mag = plain.rotary_frequencies(rot)
    inv, m2 = rotary_frequencies(rot["base"], rot["dims"], dict(scaling, kind="yarn") if scaling else None)
    assert np.allclose(inv.numpy(), f, rtol=1e-14) and math.isclose(mag, m2)
    part = Rotary(rot["base"], 16, 12, 50, "cpu", pairing="interleaved", scaling=dict(scaling, kind="yarn") if scaling else None)
    v = np.random.default_rng(0).normal(size=16)
    for p in (0, 1, 17, 49):
        want = plain.rotate(v, p, rot)
        c, s = part.cos[p].double().numpy(), part.sin[p].double().numpy()
        got = v.copy()
        got[0:12:2], got[1:12:2] = v[0:12:2] * c - v[1:12:2] * s, v[1:12:2] * c + v[0:12:2] * s
        assert np.allclose(got, want, atol=1e-6)
        assert np.array_equal(want[12:], v[12:])


def test_plain_model_invariants(tmp_path):
    """What the plain implementation must satisfy by construction: a token's logits do not depend on later tokens, nor
    on tokens before every window; the absorbed form of latent attention equals the expanded one."""
    from rust_deeplearning_b200 import write_random_model
    cfg, seed = tiny_ligirax.config("LB")
    write_random_model(str(tmp_path), cfg, seed, "bfloat16")
    pcfg, w = plain.load_folder(str(tmp_path))
    ids = [int(v) for v in np.random.default_rng(1).integers(0, cfg["vocab"], size=30)]
    full = plain.forward(pcfg, w, ids)
    assert np.allclose(plain.forward(pcfg, w, ids[:12]), full[:12], atol=1e-12)
    # absorbed: q' = [W_uk^T q_un | q_rot] over rows [c | kr], then W_uv on the latent part of the result
    m = pcfg["layers"][0]["mixer"]
    h = np.random.default_rng(2).normal(size=(9, cfg["width"]))
    c, kr = plain.latent_rows(h, w, "l0.mix.", m, 1e-4)
    want = plain.latent_attention(h, w, "l0.mix.", m, 1e-4, (c, kr))
    H, d, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w["l0.mix.q"].T).reshape(9, H, d + rd)
    uk, uv = w["l0.mix.uk"].reshape(H, d, r), w["l0.mix.uv"].reshape(H, vd, r)
    gate = 1 / (1 + np.exp(-(h @ w["l0.mix.g"].T)))
    out = np.zeros((9, H, vd))
    for i in range(9):
        lo = max(0, i - m["mask"]["size"] + 1)
        for hh in range(H):
            qa = np.concatenate([uk[hh].T @ q[i, hh, :d], plain.rotate(q[i, hh, d:], i, m["rot"])])
            s = np.array([qa @ np.concatenate([c[j], kr[j]]) * m["scale"] for j in range(lo, i + 1)])
            p = np.exp(s - s.max()); p /= p.sum()
            out[i, hh] = uv[hh] @ (p[:, None] * c[lo:i + 1]).sum(axis=0) * gate[i, hh]
    assert np.allclose(out.reshape(9, -1) @ w["l0.mix.o"].T, want, atol=1e-10)


def test_random_weights_have_their_means():
    from rust_deeplearning_b200.parts.spec import TensorSpec
    from rust_deeplearning_b200.weights.loader import random_tensor
    x = random_tensor(TensorSpec("n", (4000,), "vector", init_std=0.1, init_mean=1.0), 3, torch.float32)
    assert abs(float(x.mean()) - 1.0) < 0.01 and abs(float(x.std()) - 0.1) < 0.01
