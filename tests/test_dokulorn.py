"""Dokulorn without a GPU: the configuration reader, the model's description as parts, and the plain implementation's
own invariants (the chunked form of the recurrence, what a sink does, what the far past contributes)."""
import copy

import numpy as np
import pytest

import plain_dokulorn as plain
import tiny_dokulorn
from rust_deeplearning_b200.cache.cache import Cache, StateRequirement
from rust_deeplearning_b200.config.base import ConfigError, architecture_for
from rust_deeplearning_b200.parts.spec import PartSpec


def _spec(name):
    cfg, _ = tiny_dokulorn.config(name)
    arch = architecture_for(cfg)
    assert arch.name == "Dokulorn"
    return cfg, arch.build_spec(arch.parse_config(cfg))


def test_configuration_becomes_parts():
    cfg, spec = _spec("DA")
    assert [l.block for l in spec.layers] == ["postnorm"] * 3 and all(l.params["alpha"] == 1.7 for l in spec.layers)
    pair, ret = spec.layers[0].mixer, spec.layers[1].mixer
    assert pair.kind == "mixer_pair" and pair.params["factor"] == 0.5
    left, right = pair.params["left"], pair.params["right"]
    assert isinstance(left, PartSpec) and left.kind == "attention" and right.kind == "decay_attention"
    assert left.params["n_kv_heads"] == 2 and left.params["qk_norm_eps"] == 1e-5 and left.params["gate"] == "sigmoid"
    assert left.params["position"].params["rotary_dim"] == 16 and left.params["window"] is None
    assert right.params["activation"] == "silu" and right.params["out_norm"] == "all_heads" and right.params["position"] is None
    assert ret.kind == "decay_attention" and ret.params["out_norm"] == "per_head" and ret.params["gate"] == "silu"
    assert ret.params["k_scale"] == 32 ** -0.5 and ret.params["decay"] == (0.95, 1.0)
    assert spec.layers[1].feed_forward is None and "post_feed_forward" not in spec.layers[1].norms
    assert spec.layers[0].norms["post_mixer"].params["offset"] == 1.0
    names = spec.tensor_specs()       # the tensors of both halves of a pair are found through the pair
    assert names["l0.mix.left.sink"].shape == (4,) and names["l0.mix.right.norm"].shape == (96,)
    assert names["l0.mix.left.k"].shape == (64, 64) and names["l0.mix.right.out"].shape == (64,)
    assert names["l1.mix.g"].shape == (128, 64) and "l1.norm2" not in names and "l1.mlp.gate" not in names
    assert spec.embedding.params["scale"] == 3.0 and spec.head.tensors["weight"].name == "embed" and spec.head.params["scale"] == 1.0


def test_configuration_errors_are_listed_together():
    cfg, _ = tiny_dokulorn.config("DB")
    bad = copy.deepcopy(cfg)
    del bad["postln_alpha"]
    bad["layers"][0]["mixer"]["decay"] = [0.5, 0.9]
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 2
    bad["layers"][2]["mixer"]["right"]["decay"][1] = 1.5
    bad["layers"][2]["mlp"]["kind"] = "sparse"
    with pytest.raises(ConfigError) as e:
        architecture_for(bad).parse_config(bad)
    text = str(e.value)
    assert "postln_alpha" in text and "2 numbers for 5 heads" in text and "3 heads cannot share 2" in text
    assert "[0, 1]" in text and "sparse" in text
    bad = copy.deepcopy(cfg)
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="convolution"):
        architecture_for(bad).parse_config(bad)
    bad = copy.deepcopy(cfg)
    bad["layers"][0]["mixer"]["rot"]["dims"] = 14
    with pytest.raises(ConfigError, match="dims"):
        architecture_for(bad).parse_config(bad)


def test_cache_needs_keys_for_the_pairs_and_state_for_every_layer():
    """What the cache is asked for, from the descriptions alone (no device): a pair needs keys and values (the softmax
    half, at the padded head size) and state (the lightning half); a retention layer needs state only."""
    from rust_deeplearning_b200.cache.cache import KVRequirement, RunNeeds
    cfg, spec = _spec("DB")
    needs = []
    for layer in spec.layers:
        m = layer.mixer
        if m.kind == "mixer_pair":
            l, r = m.params["left"].params, m.params["right"].params
            d = max(l["head_dim"], l["value_dim"])
            needs.append(RunNeeds(KVRequirement(l["n_kv_heads"], d, None), StateRequirement((r["n_heads"], r["dim"], r["vdim"]))))
        else:
            needs.append(RunNeeds(None, StateRequirement((m.params["n_heads"], m.params["dim"], m.params["vdim"]))))
    cache = Cache(needs, max_tokens=64, max_seqs=2, page_size=16, device="cpu", allocate=False)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 3
    assert cache.kv_groups[0].requirement.head_dim == 40           # keys of 24 and values of 40 share rows of 40
    a = cache.alloc_slot()
    cache.reserve([a], [20]); cache.advance([a], [20])
    assert all(len(g.pages[a]) == 2 for g in cache.kv_groups)
    cache.free_slot(a)
    assert all(g.pool.n_free == g.pool.n_pages for g in cache.kv_groups)


def test_the_recurrence_in_chunks_equals_the_recurrence_token_by_token():
    """o_i = sum_{j<=i} d^(i-j) (q_i . k_j) v_j + d^(i+1) S^T q_i and S' = d^L S + sum_j d^(L-1-j) k_j v_j^T over chunks of
    any length reproduce the token-by-token recurrence (the identity the tensor-core kernel rests on), also for d = 0, 1."""
    rng = np.random.default_rng(3)
    T, d, e = 75, 6, 5
    q, k, v = rng.normal(size=(T, d)), rng.normal(size=(T, d)), rng.normal(size=(T, e))
    for decay in (0.0, 0.6, 0.999, 1.0):
        want = plain.decay_recurrence(q, k, v, decay)
        for chunk in (1, 2, 16, 64, 100):
            S, got = np.zeros((d, e)), np.zeros((T, e))
            for t0 in range(0, T, chunk):
                L = min(chunk, T - t0)
                for i in range(L):
                    acc = decay ** (i + 1) * (S.T @ q[t0 + i])
                    for j in range(i + 1):
                        acc = acc + decay ** (i - j) * float(q[t0 + i] @ k[t0 + j]) * v[t0 + j]
                    got[t0 + i] = acc
                S = decay ** L * S + sum(decay ** (L - 1 - j) * np.outer(k[t0 + j], v[t0 + j]) for j in range(L))
            assert np.allclose(got, want, rtol=1e-10, atol=1e-10), (decay, chunk)


def test_the_oracle_shows_a_sink_a_far_token_and_the_order_of_layers():
    """The tiny models are sensitive to what the tests are meant to catch: dropping the sinks, forgetting the first
    token (a head that never decays carries it to the end) and the place of a rotation all move the logits by far
    more than any tolerance in use."""
    import dokulorn_helpers as dh
    cfg, w = dh.plain_model("DA")
    ids = dh.prompt("DA", 5, 90)
    want = plain.forward(cfg, w, ids)
    no_sink = dict(w)
    no_sink["l0.mix.left.sink"] = np.full_like(w["l0.mix.left.sink"], -50.0)
    assert np.abs(plain.forward(cfg, no_sink, ids) - want).max() > 0.05
    other_first = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    assert np.abs(plain.forward(cfg, w, other_first)[-1] - want[-1]).max() > 0.02
    moved = copy.deepcopy(cfg)
    moved["layers"][0]["mixer"]["left"]["rot"]["dims"] = 32
    assert np.abs(plain.forward(moved, w, ids) - want).max() > 0.05
    # a sequence's logits do not depend on what follows (causal everywhere)
    assert np.allclose(plain.forward(cfg, w, ids[:40]), want[:40], rtol=1e-9, atol=1e-9)
