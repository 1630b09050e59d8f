"""Shared by the Dokulorn tests: tiny model folders, engines on them, the plain logits."""
import functools
import os

import model_helpers as mh
import plain_dokulorn as plain
import tiny_dokulorn

assert_logits = mh.assert_logits


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from rust_deeplearning_b200 import write_random_model
    cfg, seed = tiny_dokulorn.config(name)
    folder = os.path.join(mh.tmp_root(), f"tiny_{name}")
    write_random_model(folder, cfg, seed, "bfloat16")
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return plain.load_folder(model_folder(name))


@functools.lru_cache(maxsize=None)
def loaded_model(name: str, dtype: str):
    from rust_deeplearning_b200 import load_model
    return load_model(model_folder(name), dtype, "cuda:0")


def engine(name: str, dtype: str, **kw):
    from rust_deeplearning_b200 import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine(loaded_model(name, dtype), **kw)


def vocab(name):
    return tiny_dokulorn.config(name)[0]["vocab"]


def prompt(name, seed, n):
    return mh.prompt(seed, n, vocab(name))


_LOGITS = {}


def plain_logits(name: str, ids):
    key = (name, tuple(ids))
    if key not in _LOGITS:
        cfg, w = plain_model(name)
        _LOGITS[key] = plain.forward(cfg, w, list(ids))
    return _LOGITS[key]
