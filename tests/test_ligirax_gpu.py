"""Ligirax on a GPU against the plain implementation, in 32-bit and in bfloat16: each mechanism's kernels alone,
whole prompts, single tokens through the cache, portions, unequal batches on reused slots and pages, window
edges under a sharp softmax, long decoding, greedy generation and the trace replay."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import ligirax_helpers as lh
import plain_ligirax as plain
import tiny_ligirax

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["LA", "LB", "LC"]
DEV = "cuda:0"


def _t(a, dtype):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(DEV).to(getattr(torch, dtype))


def _close(got, want, dtype, what):
    got = got.detach().float().cpu().double().numpy()
    tol = (1e-5 if dtype == "float32" else 2e-2) * max(1.0, float(np.abs(want).max()))
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.abs(got - want).max() <= tol, f"{what}: {np.abs(got - want).max():.3e} > {tol:.3e}"


# ---- each mechanism alone ----

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("sizes", [(3, 5, 12, 20, 2), (3, 8, 16, 24, 8)])
def test_latent_prepare_norms_rotates_and_writes(dtype, interleaved, sizes):
    """The kernel between projection and attention against the plain norm and rotation, with rot.dims below rot_dim,
    queries written elsewhere, and the cache write read back through the page list; sizes that are no whole number of
    16-byte chunks, and sizes that are (the kernel's chunked form)."""
    from rust_deeplearning_b200.kernels import ops
    from rust_deeplearning_b200.parts.position import Rotary
    rng = np.random.default_rng(1)
    H, d, rd, r, extra = sizes
    T, page = 9, 4
    rot = {"base": 50.0, "dims": 8, "scaling": {"factor": 3.0, "original": 8, "fast": 4.0, "slow": 0.5}}
    width = H * (d + rd) + r + rd + extra
    rows = rng.normal(size=(T, width))
    w = rng.normal(size=r) + 1.0
    pos = np.array([3, 4, 5, 6, 7, 8, 9, 10, 11], dtype=np.int32)
    part = Rotary(rot["base"], rd, rot["dims"], 64, DEV, pairing="interleaved" if interleaved else "half",
                  scaling=dict(rot["scaling"], kind="yarn"))
    x = _t(rows, dtype)
    rows = x.float().cpu().double().numpy()
    wt = _t(w, dtype)
    w = wt.float().cpu().double().numpy()
    cache = torch.zeros((5, 1, page, r + rd), dtype=x.dtype, device=DEV)
    tables = torch.tensor([[4, 2, 0, 1, 3]], dtype=torch.int32, device=DEV)
    pages = ops.KVPages(cache, cache, tables, page, 5)
    ti = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    qp = torch.zeros((T, H * (r + rd)), dtype=x.dtype, device=DEV)
    lat = ops.latent_prepare(x, q_col=0, n_heads=H, dim=d, rot_dim=rd, latent_col=H * (d + rd), kv_rank=r,
                             norm=ops.NormParams(wt, 1e-3, 0.0), cos=part.cos, sin=part.sin, rot_n=rot["dims"], interleaved=interleaved,
                             tok_seq=ti([0] * T), tok_pos=ti(pos), q_rot_out=qp, q_rot_col=r, q_rot_head=r + rd, pages=pages,
                             seq_end=ti([12]))

    def turn(v, p):
        if interleaved:
            return plain.rotate(v, p, rot)
        # half-split pairing of the same angles: (i, i + n/2)
        n = rot["dims"]
        il = np.concatenate([np.stack([v[:n // 2], v[n // 2:n]], axis=1).reshape(-1), v[n:]])
        o = plain.rotate(il, p, rot)
        return np.concatenate([o[:n:2], o[1:n:2], o[n:]])

    for t in range(T):
        c = plain.rms_norm(rows[t, H * (d + rd):H * (d + rd) + r], w, 1e-3)
        kr = turn(rows[t, H * (d + rd) + r:H * (d + rd) + r + rd], int(pos[t]))
        _close(lat[t], np.concatenate([c, kr]), dtype, f"latent row {t}")
        for h in range(H):
            _close(qp[t, h * (r + rd) + r:(h + 1) * (r + rd)], turn(rows[t, h * (d + rd) + d:(h + 1) * (d + rd)], int(pos[t])), dtype, "q_rot")
    # the cache rows, read back through the page list by the plain attention kernel: with a window of one key every
    # token sees only its own row, which comes out as the value
    ab = ops.AttentionBatch(T, 1, ti([0] * T), ti(pos), ti([0, T]), ti([3]), ti([12]))
    got = ops.attention(lat, ab, pages, n_heads=1, n_kv_heads=1, head_dim=r + rd, score_scale=0.0, softcap=None, window=1, kind="plain")
    assert torch.equal(got, lat)


@pytest.mark.parametrize("dtype", DTYPES)
def test_products_per_head_gate_and_packing(dtype):
    from rust_deeplearning_b200.kernels import ops
    rng = np.random.default_rng(2)
    T, H, k, n = 11, 3, 7, 5
    x, w, g = rng.normal(size=(T, 2 + H * 9)), rng.normal(size=(H, n, k)), rng.normal(size=(T, H))
    xt, wt, gt = _t(x, dtype), _t(w, dtype), _t(g, dtype)
    x, w, g = (a.float().cpu().double().numpy() for a in (xt, wt, gt))
    want = np.stack([np.stack([w[h] @ x[t, 2 + h * 9:2 + h * 9 + k] for h in range(H)]) for t in range(T)])
    _close(ops.heads_linear(xt, 2, 9, wt), want.reshape(T, H * n), dtype, "heads_linear")
    gated = want / (1 + np.exp(-g))[:, :, None]
    _close(ops.heads_linear(xt, 2, 9, wt, gate=gt), gated.reshape(T, H * n), dtype, "heads_linear with gate")
    out = torch.zeros((T, 40), dtype=xt.dtype, device=DEV)
    ops.heads_linear(xt, 2, 9, wt, out=out, out_col=3, out_head=12)
    for h in range(H):
        _close(out[:, 3 + 12 * h:3 + 12 * h + n], want[:, h], dtype, "heads_linear into wider rows")
    _close(ops.gate_heads(xt, 9, gt, H, 4), (x[:, :27].reshape(T, H, 9)[:, :, :4] / (1 + np.exp(-g))[:, :, None]).reshape(T, H * 4), dtype, "gate_heads")
    d, rd, vd, r, pad = 3, 4, 5, 6, 16
    rows, kv, lat = rng.normal(size=(T, 1 + H * (d + rd))), rng.normal(size=(T, H * (d + vd))), rng.normal(size=(T, r + rd))
    rt, kt, lt = _t(rows, dtype), _t(kv, dtype), _t(lat, dtype)
    rows, kv, lat = (a.float().cpu().double().numpy() for a in (rt, kt, lt))
    packed = ops.latent_assemble(rt, 1, kt, lt, n_heads=H, dim=d, rot_dim=rd, vdim=vd, kv_rank=r, pad=pad).float().cpu().numpy().reshape(T, 3, H, pad)
    for h in range(H):
        assert np.array_equal(packed[:, 0, h, :d + rd], rows[:, 1 + h * (d + rd):1 + (h + 1) * (d + rd)].astype(np.float32))
        assert np.array_equal(packed[:, 1, h, :d], kv[:, h * d:(h + 1) * d].astype(np.float32))
        assert np.array_equal(packed[:, 1, h, d:d + rd], lat[:, r:].astype(np.float32))
        assert np.array_equal(packed[:, 2, h, :vd], kv[:, H * d + h * vd:H * d + (h + 1) * vd].astype(np.float32))
    assert not packed[:, 0, :, d + rd:].any() and not packed[:, 1, :, d + rd:].any() and not packed[:, 2, :, vd:].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 200])
@pytest.mark.parametrize("shape", [(5, 2, 3), (3, 0, 1), (40, 3, 6), (0, 2, 2)])
def test_router_and_experts(dtype, rows, shape):
    """Router and experts against the plain ones: identity experts, one expert of several, every expert, none real."""
    from rust_deeplearning_b200.kernels import ops
    n_real, n_id, top = shape
    rng = np.random.default_rng(3)
    W, ff, limit = 48, 24, 0.8
    f = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": n_real, "identity": n_id, "top": top}}
    w = {"router": rng.normal(size=(n_real + n_id, W)) * 0.5, "correction": rng.normal(size=n_real + n_id) * 0.2}
    for e in range(n_real):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (rng.normal(size=s) * 0.3 for s in ((ff, W), (ff, W), (W, ff)))
    wt = {k: _t(v, dtype) for k, v in w.items()}
    w = {k: v.float().cpu().double().numpy() for k, v in wt.items()}
    x = rng.normal(size=(rows, W))
    xt = _t(x, dtype)
    x = xt.float().cpu().double().numpy()
    chosen, weight, margin = plain.router(x, w, "", f)
    sel, sel_w = ops.moe_route(xt, wt["router"].float(), wt["correction"].float(), top)
    safe = margin > 1e-6
    assert np.array_equal(np.sort(sel.cpu().numpy()[safe], axis=1), np.sort(chosen[safe], axis=1))
    order = np.argsort(sel.cpu().numpy(), axis=1)
    _close(torch.gather(sel_w, 1, torch.tensor(order, device=DEV)), np.take_along_axis(weight, np.argsort(chosen, axis=1), axis=1), "float32", "weights")
    gu = torch.stack([torch.cat([wt[f"e{e}.gate"], wt[f"e{e}.up"]]) for e in range(n_real)]) if n_real else None
    dn = torch.stack([wt[f"e{e}.down"] for e in range(n_real)]) if n_real else None
    got = ops.moe_experts(xt, sel, sel_w, gu, dn, n_real, "swish_limit", limit)
    want = plain.routed_experts(x, w, "", f)
    _close(got[torch.tensor(safe, device=DEV)], want[safe], dtype, "routed experts")


@pytest.mark.parametrize("case", [
    # heads, kv_rank, rot_dim, page, window, splits
    (6, 32, 16, 16, 9, 1), (6, 32, 16, 16, 9, 3), (16, 96, 32, 64, 72, None), (20, 48, 16, 8, None, 2), (3, 448, 64, 64, 200, None),
    (2, 512, 64, 64, 300, 4),
    (17, 256, 64, 32, None, 5), (1, 16, 16, 16, 64, 1)])
def test_latent_decode_kernel_against_the_plain_kernel(case):
    """The tensor-core decode kernel of the absorbed form against the float kernel: pages in random order, sequences of
    unequal lengths, a padding row, one split and several.  In every sequence one key is made to dominate: the first key
    the window keeps, the key just outside it, the newest key, a key at a page's edge, in turn."""
    from rust_deeplearning_b200.kernels import ops
    H, r, rd, page, window, splits = case
    width = r + rd
    rng = np.random.default_rng(sum(case[:4]))
    lens = [1, 5, page, page + 1, 150, 333, 64, 65]
    T = len(lens) + 1
    n_pages = sum(-(-n // page) for n in lens) + 2
    cache = torch.tensor(rng.normal(size=(n_pages, 1, page, width)) * 0.5, dtype=torch.float32).to(DEV).to(torch.bfloat16)
    order = rng.permutation(n_pages)
    tw = max(-(-n // page) for n in lens)
    tables = np.zeros((T, tw), dtype=np.int32)
    at = 0
    for i, n in enumerate(lens):
        k = -(-n // page)
        tables[i, :k] = order[at:at + k]
        at += k
    q = torch.tensor(rng.normal(size=(T, H * width)) * 0.5, dtype=torch.float32).to(DEV).to(torch.bfloat16)
    # the dominating key: a cached row that equals a multiple of head 0's query
    for i, n in enumerate(lens):
        p = n - 1
        lo = max(0, p - window + 1) if window else 0
        target = [lo, lo - 1, p, (p // page) * page, max(lo, (p // page) * page - 1)][i % 5]
        if 0 <= target <= p:
            row = q[i, :width].float() * 6.0
            pg, rr = tables[i, target // page], target % page
            sw = torch.empty(width, dtype=torch.float32, device=DEV)
            for c in range(width // 8):      # the stored row has its 16-byte chunks swizzled by its place in the page
                cc = (c ^ (rr & 7)) if (c | 7) < width // 8 else c
                sw[cc * 8:cc * 8 + 8] = row[c * 8:c * 8 + 8]
            cache[pg, 0, rr] = sw.to(torch.bfloat16)
    ti = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    pos = [n - 1 for n in lens] + [-1]
    ab = ops.AttentionBatch(T, T, ti(list(range(T))), ti(pos), ti(list(range(T + 1))), ti(pos[:-1] + [0]), ti(lens + [0]),
                            max_keys=min(max(lens), window or max(lens)))
    pages = ops.KVPages(cache, cache, ti(tables), page, tw)
    want = ops.attention(q, ab, pages, n_heads=H, n_kv_heads=1, head_dim=width, score_scale=0.3, softcap=None, window=window, kind="plain")
    got = ops.latent_decode(q, ab, pages, n_heads=H, kv_rank=r, score_scale=0.3, window=window, n_splits=splits)
    w = want.float().view(T, H, width)[:-1, :, :r]
    g = got.float().view(T, H, width)[:-1, :, :r]
    assert torch.isfinite(g).all()
    assert (g - w).abs().max().item() <= 0.02 * max(1.0, w.abs().max().item()), (g - w).abs().max().item()


# ---- the model ----

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(name, dtype):
    eng = lh.engine(name, dtype, page_size=16)
    for seed, n in ((1, 1), (2, 2), (3, 37), (4, 70)):
        ids = lh.prompt(name, seed, n, dtype)
        slot = eng.new_sequence()
        lh.assert_logits(eng.step([slot], [ids], "all"), lh.plain_logits(name, ids), dtype, f"{name} whole n={n}")
        eng.release(slot)
    ids = lh.prompt(name, 5, 6, dtype)
    slot = eng.new_sequence()
    for t in range(6):      # positions 0, 1, 2, ... each as a step of its own
        lh.assert_logits(eng.step([slot], [[ids[t]]], "all"), lh.plain_logits(name, ids)[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype):
    """The last 40 tokens one by one: in LA and LB the windows (8, 12, 5, 3 keys) pass wholly over decoded tokens, pages
    of 16 positions are crossed and the rings wrap; bit-equal to a second run on other slots and pages in 32-bit."""
    eng = lh.engine(name, dtype, page_size=16)
    ids = lh.prompt(name, 6, 75, dtype)
    want = lh.plain_logits(name, ids)
    other = eng.new_sequence()
    eng.step([other], [ids[:20]], [[]])          # shifts which pages the next sequence gets
    slot = eng.new_sequence()
    lh.assert_logits(eng.step([slot], [ids[:35]], "all"), want[:35], dtype, "prefix")
    for t in range(35, 75):
        lh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype):
    """A prompt cut into portions of 2 to 19 tokens on a cached prefix (pages of 8: rings wrap inside a portion)."""
    eng = lh.engine(name, dtype, page_size=8)
    ids = lh.prompt(name, 7, 66, dtype)
    want = lh.plain_logits(name, ids)
    slot = eng.new_sequence()
    at = 0
    for n in (5, 2, 19, 2, 3, 16, 11, 8):
        lh.assert_logits(eng.step([slot], [ids[at:at + n]], "all"), want[at:at + n], dtype, f"{name} portion at {at}")
        at += n
    assert at == 66


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Batches one after another on a cache with 4 slots and few pages: prompts of unequal lengths in one step, then one
    token each; shorter requests end earlier; later batches land on what earlier ones gave back.  Each request's logits
    equal those it gives alone (the plain implementation runs it alone)."""
    eng = lh.engine(name, dtype, max_tokens=10 * 16, max_seqs=4, page_size=16)
    shapes = [([5, 11, 17], [8, 8, 8]), ([1, 9, 23, 30], [12, 3, 7, 1]), ([40, 2, 20], [2, 22, 5])]
    for b, (lens, extra) in enumerate(shapes):
        seqs = [lh.prompt(name, 100 + 10 * b + i, n + e, dtype) for i, (n, e) in enumerate(zip(lens, extra))]
        want = [lh.plain_logits(name, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        lh.assert_logits(got, np.concatenate([w[:n] for w, n in zip(want, lens)]), dtype, f"batch {b} prompts")
        pos, live = list(lens), list(range(len(seqs)))
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            lh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), dtype, f"batch {b} decode at {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert eng.cache.n_free_slots == 4
    if dtype == "bfloat16":
        assert eng.graph_replays > 0


def test_window_edges_under_a_sharp_softmax():
    """With scores multiplied by 40 nearly all weight lies on one key per query and head; over 90 positions that key
    is often the first or the last one the window keeps, or would be the one just outside it.  32-bit, whole and
    token by token, pages of 16, windows of 8 and 12 keys and none."""
    from rust_deeplearning_b200 import Engine, load_model, write_random_model
    cfg, seed = tiny_ligirax.config("LA")
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] *= 40.0
    folder = os.path.join(lh.mh.tmp_root(), "tiny_LA_sharp")
    write_random_model(folder, cfg, seed, "bfloat16")
    pcfg, w = plain.load_folder(folder)
    ids = [int(v) for v in np.random.default_rng(9).integers(0, cfg["vocab"], size=90)]
    margins = []
    want = plain.forward(pcfg, w, ids, margins)
    safe = np.minimum.reduce(margins) > 1e-4
    assert safe.sum() > 60
    first_unsafe = int(np.argmin(safe)) if not safe.all() else len(ids)      # logits after a close call are another computation
    # one key more or one key less changes the plain logits by far more than the tolerance: the test can see an edge
    moved = json.loads(json.dumps(pcfg))
    moved["layers"][0]["mixer"]["mask"]["size"] += 1
    assert np.abs(plain.forward(moved, w, ids)[:first_unsafe] - want[:first_unsafe]).max() > 1e-2
    eng = Engine(load_model(folder, "float32", DEV), max_tokens=1024, page_size=16)
    slot = eng.new_sequence()
    lh.assert_logits(eng.step([slot], [ids[:first_unsafe]], "all"), want[:first_unsafe], "float32", "whole")
    slot = eng.new_sequence()
    n0 = min(30, first_unsafe)
    lh.assert_logits(eng.step([slot], [ids[:n0]], "all"), want[:n0], "float32", "prefix")
    for t in range(n0, first_unsafe):
        lh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], "float32", f"position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """300 single-token steps with every expert chosen: crosses pages, wraps the window's ring several times."""
    name = "LD"
    eng = lh.engine(name, dtype)
    ids = lh.mh.prompt(11, 300, lh.vocab(name))
    want = lh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:3]], [[]])
    for t in range(3, 300):
        got = eng.step([slot], [[ids[t]]], "last")
        if t % 7 == 0 or t > 280:
            lh.assert_logits(got, want[t:t + 1], dtype, f"position {t}")


def test_greedy_generation_through_the_entry_point():
    from rust_deeplearning_b200 import Generator
    name = "LC"
    cfg, w = lh.plain_model(name)
    prompts = [lh.prompt(name, 300 + i, n, "float32") for i, n in enumerate((1, 9, 23))]
    gen = Generator(lh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    got = gen.generate_batch(prompts, 10)
    for p, g in zip(prompts, got):
        assert g[:len(p)] == p
        # the plain loop, as long as its own margin between the best and the second best token is not a close call
        ids = list(p)
        for tok in g[len(p):]:
            row = np.sort(plain.forward(cfg, w, ids)[-1])
            if row[-1] - row[-2] < 1e-3 or plain.min_margin(cfg, w, ids) < 1e-4:
                break
            assert tok == int(np.argmax(plain.forward(cfg, w, ids)[-1]))
            ids.append(tok)
        assert gen.generate(p, 10) == g


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype, tmp_path):
    """bin/trace_run on a Ligirax folder: two requests as one batch, then one token each, the shorter one ending first."""
    name = "LA"
    a, b = lh.prompt(name, 40, 30, dtype), lh.prompt(name, 41, 21, dtype)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:26], "want": [0, 25]}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[26]], "want": [0]}, {"id": "b", "tokens": [b[19]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[27]], "want": [0]}, {"id": "b", "tokens": [b[20]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[28]], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[29]], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", lh.model_folder(name), "--dtype", dtype,
                             "--out", str(tmp_path), "--max-tokens", "128"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    wa, wb = lh.plain_logits(name, a), lh.plain_logits(name, b)
    V = lh.vocab(name)
    read = lambda n: torch.tensor(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
    lh.assert_logits(read(0), np.stack([wa[0], wa[25], wb[18]]), dtype, "step 0")
    lh.assert_logits(read(1), wa[26:27], dtype, "step 1")
    lh.assert_logits(read(2), np.stack([wa[27], wb[20]]), dtype, "step 2")
    lh.assert_logits(read(3), wa[28:29], dtype, "step 3")
    lh.assert_logits(read(4), wa[29:30], dtype, "step 4")


def test_command_line_generates_with_a_ligirax_folder(capsys):
    """The command line picks the architecture by config.json; its greedy tokens are the entry point's."""
    import io
    from rust_deeplearning_b200 import Generator, cli
    name = "LC"
    p = lh.prompt(name, 50, 12, "float32")
    out = io.StringIO()
    code = cli.main([lh.model_folder(name), "--prompt-ids", " ".join(map(str, p)), "--max-tokens", "6", "--temperature", "0",
                     "--dtype", "float32", "--max-context", "64"], stdout=out)
    assert code == 0
    assert "arch=Ligirax" in capsys.readouterr().err
    gen = Generator(lh.loaded_model(name, "float32"), max_batch=1, max_context=64).with_temperature(0.0)
    assert [int(t) for t in out.getvalue().split()] == gen.generate(p, 6)[len(p):]
