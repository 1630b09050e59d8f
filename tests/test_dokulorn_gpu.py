"""Dokulorn on the GPU: each new kernel alone against plain numpy / float64 torch, then the engine against the plain
implementation (`plain_dokulorn.py`): whole prompts, token by token, portions, unequal batches on reused slots and
pages, long decoding, generation, the command line and the trace replay."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dokulorn_helpers as dh
import kernel_refs as ref
import plain_dokulorn as plain
import tiny_dokulorn
from rust_deeplearning_b200.kernels import ops
from test_kernels_gpu import Case, assert_close, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["DA", "DB", "DC"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def _rms64(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 64), (5, 72), (130, 1000), (3, 4608)])
def test_norm_after_the_sum_pair_norm_and_gates(dtype, rows, width):
    res = rnd((rows, width), torch.float32, 1)
    branch = rnd((rows, width), dtype, 2)
    w = rnd((width,), dtype, 3, 0.1)
    want = _rms64(1.7 * res.to(F64) + branch.to(F64), 1e-5) * (w.to(F64) + 1.0)
    got_res = res.clone()
    y = ops.postnorm_(got_res, branch, ops.NormParams(w, 1e-5, 1.0), 1.7, dtype)
    assert_close(got_res, want.float(), torch.float32, what="stream")
    assert_close(y, want.to(dtype), dtype, what="rows for the next part")
    assert ops.postnorm_(res.clone(), branch, ops.NormParams(w, 1e-5, 1.0), 1.7, None) is None
    # the sum of squares of a row is formed the same way whatever the row count (bit-equal rows)
    one = res[:1].clone()
    ops.postnorm_(one, branch[:1].contiguous(), ops.NormParams(w, 1e-5, 1.0), 1.7, None)
    assert torch.equal(one, got_res[:1])

    a, b = rnd((rows, width), dtype, 4), rnd((rows, width), dtype, 5, 3.0)
    wa, wb = rnd((width,), dtype, 6), rnd((width,), dtype, 7)
    want = 0.5 * (_rms64(a.to(F64), 1e-6) * wa.to(F64) + _rms64(b.to(F64), 1e-6) * wb.to(F64))
    assert_close(ops.norm_pair(a, b, wa, wb, 1e-6, 0.5), want.float(), torch.float32, what="norm_pair")

    wide = rnd((rows, 3 * width + 8), dtype, 8)
    x, g = wide[:, 8:8 + width], wide[:, 8 + width:8 + 2 * width]        # column slices of wider rows
    for kind, fn in (("sigmoid", torch.sigmoid), ("silu", torch.nn.functional.silu)):
        assert_close(ops.gate_mul(x, g, kind), (x.to(F64) * fn(g.to(F64))).to(dtype), dtype, what=f"gate_mul {kind}")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,groups,group", [(1, 1, 16), (7, 5, 20), (70, 2, 128), (3, 1, 2304)])
def test_group_norm_and_gate(out_dtype, rows, groups, group):
    x = rnd((rows, groups * group), torch.float32, 11, 4.0)
    gate = rnd((rows, groups * group + 5), out_dtype, 12)[:, 5:]
    w = rnd((groups * group,), out_dtype, 13)
    n = _rms64(x.to(F64).view(rows, groups, group), 1e-5).view(rows, -1)
    assert_close(ops.group_norm_gate(x, groups, eps=1e-5, out_dtype=out_dtype), n.to(out_dtype), out_dtype, what="norm only")
    want = n * w.to(F64) * torch.sigmoid(gate.to(F64))
    assert_close(ops.group_norm_gate(x, groups, eps=1e-5, weight=w, gate=gate, gate_kind="sigmoid", out_dtype=out_dtype),
                 want.to(out_dtype), out_dtype, what="weight and sigmoid gate")
    want = n * torch.nn.functional.silu(gate.to(F64))
    assert_close(ops.group_norm_gate(x, groups, eps=1e-5, gate=gate, gate_kind="silu", out_dtype=out_dtype),
                 want.to(out_dtype), out_dtype, what="silu gate")


def _sink_attention_ref(c, b, sinks, new_kv, scale, softcap):
    """Key by key in float64, from the cache (through the page lists, rows unswizzled) or the step's packed rows."""
    hd, group = c.head_dim, c.n_heads // c.n_kv_heads
    out = torch.zeros((c.T, c.n_heads * hd), dtype=F64)
    q = c.qkv.cpu().to(F64)
    k_all, v_all = c.pages.k.cpu(), c.pages.v.cpu()
    tables = c.pages.tables.cpu()
    for t in range(c.T):
        p, seq = int(b.tok_pos[t]), int(b.tok_seq[t])
        cached, row0 = int(b.seq_cached[seq]), int(b.seq_start[seq]) - int(b.seq_past[seq])
        for h in range(c.n_heads):
            g = h // group
            s, vs = [], []
            for j in range(p + 1):
                if j < cached:
                    page, r = ref._cache_index(tables[seq], j, c.page_size, c.ring_pages)
                    kr, vr = ref.cache_load(k_all[page, g, r], r).to(F64), ref.cache_load(v_all[page, g, r], r).to(F64)
                else:
                    rows, k_col, v_col = new_kv
                    kr = rows[row0 + j, k_col + g * hd:k_col + (g + 1) * hd].cpu().to(F64)
                    vr = rows[row0 + j, v_col + g * hd:v_col + (g + 1) * hd].cpu().to(F64)
                z = float(q[t, h * hd:(h + 1) * hd] @ kr) * scale
                s.append(softcap * math.tanh(z / softcap) if softcap else z)
                vs.append(vr)
            s = torch.tensor(s, dtype=F64)
            sink = float(sinks[h])
            top = max(float(s.max()), sink)
            e = torch.exp(s - top)
            out[t, h * hd:(h + 1) * hd] = (e / (e.sum() + math.exp(sink - top))) @ torch.stack(vs)
    return out


@pytest.mark.parametrize("kind,dtype,head_dim", [("plain", torch.float32, 24), ("plain", torch.bfloat16, 40), ("prefill", torch.bfloat16, 32),
                                                 ("prefill", torch.bfloat16, 96), ("prefill_tc", torch.bfloat16, 64), ("decode", torch.bfloat16, 64),
                                                 ("decode", torch.bfloat16, 96)])
def test_attention_with_sinks(kind, dtype, head_dim):
    """Every attention kernel with a logit per head in the denominator: sinks from far below every score (no effect) to
    far above (the output all but vanishes), with and without a soft-cap, keys from cache pages in shuffled order and
    from the step's rows, several key splits in the decode kernel."""
    decode = kind == "decode"
    past = [130, 0, 67] if decode else ([0, 0, 0] if kind == "prefill_tc" else [70, 0, 5])
    new = [1, 1, 1] if decode else [9, 140, 66]
    if decode:
        past[1] = 63
    c = Case(past=past, new=new, n_heads=6, n_kv_heads=2, head_dim=head_dim, page_size=16 if kind != "decode" else 64, window=None,
             dtype=dtype, seed=41)
    sinks = torch.tensor([-30.0, -1.0, 0.0, 0.7, 3.0, 12.0], dtype=torch.float32, device=DEV)
    b = c.batch("all" if decode else "past")
    # one key far back (position 2 of the longest sequence) is made to stand out for that sequence's last query: random
    # keys would hide a kernel that loses the oldest page or the first key tile
    s_far = int(np.argmax([p + n for p, n in zip(past, new)]))
    last_row = int(c.seq_start[s_far + 1]) - 1
    for g in range(2):
        qv = c.qkv[last_row, g * 3 * head_dim:(g * 3 + 1) * head_dim].float()
        kv = (qv / qv.norm() * 12.0).to(dtype)
        if past[s_far] > 2:
            page, r = ref._cache_index(c.pages.tables[s_far].cpu(), 2, c.page_size, c.ring_pages)
            ref.cache_store(c.pages.k[page, g, r], kv, r)
        else:
            row = int(c.seq_start[s_far]) + 2
            c.qkv[row, (6 + g) * head_dim:(7 + g) * head_dim] = kv
    if decode:       # the step's own rows are in the cache already
        ref.rope_cache(c.qkv, 6, 2, head_dim, tok_seq=c.tok_seq, tok_pos=c.tok_pos, pages=c.pages, seq_end=c.seq_end)
    for softcap in (None, 4.0):
        kw = c.kw(softcap=softcap)
        extra = dict(keys_per_split=64) if decode else dict(new_kv=c.new_kv())
        got = ops.attention(c.qkv, b, c.pages, kind=kind, sinks=sinks, **extra, **kw)
        want = _sink_attention_ref(c, b, sinks.cpu(), None if decode else c.new_kv(), kw["score_scale"], softcap)
        assert_close(got, want.to(dtype).to(DEV), dtype, rel=8.0, what=f"{kind} softcap={softcap}")
        none = ops.attention(c.qkv, b, c.pages, kind=kind, **extra, **kw)
        h5 = slice(5 * head_dim, 6 * head_dim)          # the head whose sink outweighs every key
        assert float(got[:, h5].float().abs().max()) < 0.05 * float(none[:, h5].float().abs().max())
        h0 = slice(0, head_dim)                          # the head whose sink weighs nothing
        assert_close(got[:, h0], none[:, h0], dtype, rel=2.0, what="a sink far below the scores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 1, 24, 10, 24), (4, 2, 40, 16, 24), (2, 2, 64, 32, 64)])
def test_rotation_head_norm_and_cache_write(dtype, sizes):
    """rope_norm_cache on rows wider than their heads (a gate's logits follow): queries and keys against the plain
    rotation and norm (heads zero-padded beyond norm_dim), the cache through plain attention over it, which must equal
    attention over the step's rows."""
    H, G, hd, rot, norm_dim = sizes
    c = Case(past=[0, 0], new=[37, 5], n_heads=H, n_kv_heads=G, head_dim=hd, page_size=8, window=None, dtype=dtype, seed=50)
    width = (H + 2 * G) * hd
    rows = torch.cat([c.qkv, rnd((c.T, 24), dtype, 51)], dim=1).contiguous()
    view = rows.view(c.T, -1)
    for head in range(H + G):                                  # padding of the query and key heads
        view[:, head * hd + norm_dim:(head + 1) * hd] = 0
    before = rows.clone()
    rotd = {"base": 300.0, "dims": rot}
    ang = torch.arange(64, dtype=F64)[:, None] * torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64)[None]
    cos, sin = torch.cos(ang).float().to(DEV).contiguous(), torch.sin(ang).float().to(DEV).contiguous()
    ops.rope_norm_cache(rows, H, G, hd, tok_seq=c.tok_seq, tok_pos=c.tok_pos, cos=cos, sin=sin, rotary_dim=rot, norm_eps=1e-5,
                        norm_dim=norm_dim, pages=c.pages, seq_end=c.seq_end)
    want = before.clone().cpu().to(F64)
    pos = c.tok_pos.cpu().tolist()
    for t in range(c.T):
        for head in range(H + G):
            v = plain.turn(want[t, head * hd:head * hd + norm_dim].numpy(), pos[t], rotd)
            want[t, head * hd:head * hd + norm_dim] = torch.from_numpy(plain.unit_rms(v, 1e-5))
    assert_close(rows, want.to(dtype).to(DEV), dtype, what="rotated and normed rows; values and the gate untouched")
    kw = dict(n_heads=H, n_kv_heads=G, head_dim=hd, score_scale=0.8, softcap=None, window=None, kind="plain")
    over_rows = ops.attention(rows, c.batch("past"), c.pages, new_kv=(rows, H * hd, (H + G) * hd), **kw)
    over_cache = ops.attention(rows, c.batch("all"), c.pages, **kw)
    assert torch.equal(over_rows, over_cache)
    assert width + 24 == rows.shape[1] and torch.equal(rows[:, width:], before[:, width:])


def _decay_case(H, dim, vdim, lens, past, rot_n, silu, k_scale, decays, dtype, seed):
    n, T = len(lens), sum(lens)
    width = 2 * H * dim + H * vdim + 8
    rows = rnd((T, width), dtype, seed, 0.8)
    pos = np.concatenate([np.arange(p, p + L) for p, L in zip(past, lens)]).astype(np.int32)
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    slots = np.arange(n, dtype=np.int32)[::-1].copy() + 1
    state = rnd((n + 2, H, dim, vdim), torch.float32, seed + 1, 0.5)
    for i, p in enumerate(past):
        if p == 0:
            state[int(slots[i])] = 0
    rot = {"base": 1000.0, "dims": rot_n}
    cos = sin = None
    if rot_n:
        ang = torch.arange(int(pos.max()) + 1, dtype=F64)[:, None] * torch.tensor([1000.0 ** (-2.0 * i / rot_n) for i in range(rot_n // 2)], dtype=F64)[None]
        cos, sin = torch.cos(ang).float().to(DEV).contiguous(), torch.sin(ang).float().to(DEV).contiguous()
    # the plain recurrence, from the given state
    r64 = rows.cpu().to(F64).numpy()
    want = np.zeros((T, H * vdim))
    want_state = state.cpu().to(F64).numpy().copy()
    for s in range(n):
        for h in range(H):
            S = want_state[int(slots[s]), h]
            for t in range(starts[s], starts[s + 1]):
                q, k = r64[t, 4 + h * dim:4 + (h + 1) * dim], r64[t, 4 + (H + h) * dim:4 + (H + h + 1) * dim]
                v = r64[t, 4 + 2 * H * dim + h * vdim:4 + 2 * H * dim + (h + 1) * vdim]
                if rot_n:
                    q, k = plain.turn(q, int(pos[t]), rot), plain.turn(k, int(pos[t]), rot)
                if silu:
                    q, k, v = plain.silu(q), plain.silu(k), plain.silu(v)
                S = decays[h] * S + np.outer(k * k_scale, v)
                want[t, h * vdim:(h + 1) * vdim] = S.T @ q
            want_state[int(slots[s]), h] = S
    dev = lambda a: torch.from_numpy(a).to(DEV)
    kw = dict(q_col=4, k_col=4 + H * dim, v_col=4 + 2 * H * dim, n_heads=H, dim=dim, vdim=vdim,
              decay=torch.tensor(decays, dtype=torch.float32, device=DEV), tok_pos=dev(pos), seq_start=dev(starts), slots=dev(slots),
              n_seqs=n, silu=silu, k_scale=k_scale, cos=cos, sin=sin, rot_n=rot_n)
    return rows, state, kw, want, want_state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(H=2, dim=12, vdim=20, lens=[33, 1, 2], past=[0, 7, 0], rot_n=6, silu=False, k_scale=0.3, decays=[0.5, 1.0]),
    dict(H=3, dim=64, vdim=48, lens=[5, 70], past=[3, 0], rot_n=0, silu=True, k_scale=1.0, decays=[0.0, 0.9, 0.999]),
    dict(H=1, dim=300, vdim=33, lens=[9], past=[0], rot_n=300, silu=False, k_scale=0.05, decays=[0.97]),
])
def test_decay_attention_token_by_token(dtype, case):
    """The scan kernel against the plain recurrence in float64: carried state on slots in another order than the
    sequences, sizes that are no multiples of anything, decays 0 and 1; and the same bits when the tokens come one by one."""
    rows, state, kw, want, want_state = _decay_case(dtype=dtype, seed=60, **case)
    st = state.clone()
    got = ops.decay_attention(rows, state=st, kind="scan", **kw)
    tol = 2e-5 if dtype is torch.float32 else 2e-5      # the rows are given in `dtype`; the arithmetic is float either way
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(got.cpu().double().numpy() - want).max() <= tol * scale
    touched = kw["slots"].cpu().long()
    assert np.abs(st.cpu().double().numpy() - want_state).max() <= tol * max(1.0, float(np.abs(want_state).max()))
    untouched = [i for i in range(state.shape[0]) if i not in touched.tolist()]
    assert torch.equal(st[untouched], state[untouched])
    # one token a step, one sequence after the other: the same bits
    st2 = state.clone()
    starts = kw["seq_start"].cpu().tolist()
    for s in range(len(case["lens"])):
        for t in range(starts[s], starts[s + 1]):
            one = dict(kw, tok_pos=kw["tok_pos"][t:t + 1].contiguous(), seq_start=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                       slots=kw["slots"][s:s + 1].contiguous(), n_seqs=1)
            o = ops.decay_attention(rows[t:t + 1], state=st2, kind="scan", **one)
            assert torch.equal(o[0], got[t])
    assert torch.equal(st2, st)


@pytest.mark.parametrize("case", [
    dict(H=2, dim=64, vdim=64, lens=[64], past=[0], rot_n=64, silu=False, k_scale=0.125, decays=[0.98, 0.999]),
    dict(H=2, dim=32, vdim=96, lens=[200, 1, 65, 63], past=[0, 9, 0, 130], rot_n=16, silu=True, k_scale=1.0, decays=[0.6, 1.0]),
    dict(H=3, dim=128, vdim=128, lens=[130, 2], past=[0, 0], rot_n=0, silu=True, k_scale=1.0, decays=[0.0, 0.95, 0.9999]),
    dict(H=1, dim=16, vdim=16, lens=[300], past=[0], rot_n=6, silu=False, k_scale=0.5, decays=[0.99]),
    dict(H=5, dim=96, vdim=48, lens=[100, 129], past=[4, 0], rot_n=48, silu=False, k_scale=0.1, decays=[0.9995, 0.99, 0.98, 0.9, 0.5]),
])
def test_decay_attention_in_chunks_on_tensor_cores(case):
    """The chunked kernel against the plain recurrence: chunk edges at 64, partial chunks, one-token sequences in the
    same call, carried state, two column blocks of a state, decays 0 and 1.  Its operands are bfloat16 (q, k, v as they
    enter the recurrence; P), its sums and the state float: errors of a few bfloat16 roundings of the largest output."""
    rows, state, kw, want, want_state = _decay_case(dtype=torch.bfloat16, seed=70, **case)
    st = state.clone()
    got = ops.decay_attention(rows, state=st, kind="chunked", **kw)
    assert torch.isfinite(got).all()
    err = np.abs(got.cpu().double().numpy() - want)
    assert err.max() <= 6e-3 * np.abs(want).max(), (err.max(), np.abs(want).max())
    serr = np.abs(st.cpu().double().numpy() - want_state)
    assert serr.max() <= 6e-3 * np.abs(want_state).max()
    # the error of a token does not grow with its distance from the sequence's start (the state stays float)
    first = kw["seq_start"].cpu().tolist()[0]
    n0 = case["lens"][0]
    if n0 >= 128:
        head, tail = err[first:first + 64].max(), err[first + n0 - 64:first + n0].max()
        assert tail <= 4 * head + 1e-3 * np.abs(want).max()


# ------------------------------------------------------------------------------------------
# the model through the engine
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(name, dtype):
    eng = dh.engine(name, dtype)
    for seed, n in ((1, 1), (2, 2), (3, 63), (4, 64), (5, 65), (6, 200)):
        ids = dh.prompt(name, seed, n)
        slot = eng.new_sequence()
        dh.assert_logits(eng.step([slot], [ids], "all"), dh.plain_logits(name, ids), dtype, f"{name} whole {n}")
        eng.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_and_after_a_prompt(name, dtype):
    """From position 0 one token a step; and a prompt of 100 tokens, then 40 single tokens past page and chunk edges
    (pages of 16), another sequence alive meanwhile on other pages and another state row."""
    eng = dh.engine(name, dtype, page_size=16)
    ids = dh.prompt(name, 7, 140)
    want = dh.plain_logits(name, ids)
    slot = eng.new_sequence()
    for t in range(20):
        dh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")
    other = eng.new_sequence()
    eng.step([other], [ids[:20]], [[]])
    slot2 = eng.new_sequence()
    dh.assert_logits(eng.step([slot2], [ids[:100]], "all"), want[:100], dtype, "prefix")
    for t in range(100, 140):
        dh.assert_logits(eng.step([slot2], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype):
    """A prompt in portions of 2 to 70 tokens on what earlier portions left in cache and state (pages of 8)."""
    eng = dh.engine(name, dtype, page_size=8)
    ids = dh.prompt(name, 8, 170)
    want = dh.plain_logits(name, ids)
    slot, at = eng.new_sequence(), 0
    for n in (5, 2, 70, 2, 3, 64, 16, 8):
        dh.assert_logits(eng.step([slot], [ids[at:at + n]], "all"), want[at:at + n], dtype, f"{name} portion at {at}")
        at += n
    assert at == 170


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Batches one after another on a cache with 4 slots and few pages: prompts of unequal lengths in one step, then one
    token each; shorter requests end earlier; later batches land on the slots, pages and state rows earlier ones gave
    back (a state row must start from zero again).  Each request's logits equal those it gives alone."""
    eng = dh.engine(name, dtype, max_tokens=14 * 16, max_seqs=4, page_size=16)
    shapes = [([5, 11, 17], [8, 8, 8]), ([1, 9, 70, 30], [12, 3, 7, 1]), ([90, 2, 20], [2, 22, 5])]
    for b, (lens, extra) in enumerate(shapes):
        seqs = [dh.prompt(name, 100 + 10 * b + i, n + e) for i, (n, e) in enumerate(zip(lens, extra))]
        want = [dh.plain_logits(name, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        dh.assert_logits(got, np.concatenate([w[:n] for w, n in zip(want, lens)]), dtype, f"batch {b} prompts")
        pos, live = list(lens), list(range(len(seqs)))
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            dh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), dtype, f"batch {b} decode at {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert eng.cache.n_free_slots == 4
    if dtype == "bfloat16":
        assert eng.graph_replays > 0


def test_float32_logits_do_not_depend_on_the_cut():
    """In 32-bit the same bits whole, in portions and token by token, alone and in a batch."""
    name = "DB"
    ids, other = dh.prompt(name, 9, 90), dh.prompt(name, 10, 33)
    eng = dh.engine(name, "float32", page_size=16)
    a = eng.new_sequence()
    whole = eng.step([a], [ids], "all").clone()
    b, c = eng.new_sequence(), eng.new_sequence()
    first = eng.step([c, b], [other, ids[:50]], "all")[33:].clone()
    rest = torch.cat([eng.step([b, c], [[ids[t]], [other[0]]], "all")[:1].clone() for t in range(50, 70)]
                     + [eng.step([b], [ids[70:]], "all").clone()])
    assert torch.equal(torch.cat([first, rest]), whole)


def test_a_token_far_back_and_the_sinks_show_in_long_prompts():
    """A head that never decays carries the first token to the end of a long prompt, through chunks and through
    single-token steps; with the first token changed the logits at the end differ, and the engine follows the plain
    implementation in both.  bfloat16, 330 tokens, the last 10 one by one."""
    name = "DA"
    eng = dh.engine(name, "bfloat16")
    ids = dh.prompt(name, 12, 330)
    changed = [(ids[0] + 7) % dh.vocab(name)] + ids[1:]
    want, want_changed = dh.plain_logits(name, ids), dh.plain_logits(name, changed)
    assert np.abs(want[-10:] - want_changed[-10:]).max() > 0.02
    for seq, w in ((ids, want), (changed, want_changed)):
        slot = eng.new_sequence()
        dh.assert_logits(eng.step([slot], [seq[:320]], [[300, 319]]), w[[300, 319]], "bfloat16", "prompt", bf16_fraction=0.01)
        for t in range(320, 330):
            dh.assert_logits(eng.step([slot], [[seq[t]]], "last"), w[t:t + 1], "bfloat16", f"position {t}", bf16_fraction=0.01)
        eng.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """400 single-token steps: crosses pages, and the state is updated 400 times in place."""
    name = "DC"
    eng = dh.engine(name, dtype)
    ids = dh.prompt(name, 11, 400)
    want = dh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:3]], [[]])
    for t in range(3, 400):
        got = eng.step([slot], [[ids[t]]], "last")
        if t % 9 == 0 or t > 385:
            dh.assert_logits(got, want[t:t + 1], dtype, f"position {t}")


def test_greedy_generation_through_the_entry_point():
    from rust_deeplearning_b200 import Generator
    name = "DA"
    cfg, w = dh.plain_model(name)
    prompts = [dh.prompt(name, 300 + i, n) for i, n in enumerate((1, 9, 70))]
    gen = Generator(dh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    got = gen.generate_batch(prompts, 10)
    for p, g in zip(prompts, got):
        assert g[:len(p)] == p and len(g) == len(p) + 10
        ids = list(p)
        for tok in g[len(p):]:      # the plain loop, while its own margin between the best two tokens is no close call
            row = np.sort(plain.forward(cfg, w, ids)[-1])
            if row[-1] - row[-2] < 1e-3:
                break
            assert tok == int(np.argmax(plain.forward(cfg, w, ids)[-1]))
            ids.append(tok)
        assert gen.generate(p, 10) == g
    # bfloat16 through the same entry point, with sampling: it runs, and the same seed gives the same tokens
    gen16 = Generator(dh.loaded_model(name, "bfloat16"), max_batch=4, max_context=128).with_temperature(0.8).with_top_k(20).with_seed(5)
    assert gen16.generate_batch(prompts, 8) == gen16.generate_batch(prompts, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype, tmp_path):
    """bin/trace_run on a Dokulorn folder: two requests as one batch, then one token each, the shorter one ending first."""
    name = "DB"
    a, b = dh.prompt(name, 40, 30), dh.prompt(name, 41, 21)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:26], "want": [0, 25]}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[26]], "want": [0]}, {"id": "b", "tokens": [b[19]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[27]], "want": [0]}, {"id": "b", "tokens": [b[20]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[28]], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[29]], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dh.model_folder(name), "--dtype", dtype,
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
    wa, wb = dh.plain_logits(name, a), dh.plain_logits(name, b)
    V = dh.vocab(name)
    read = lambda n: torch.tensor(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
    dh.assert_logits(read(0), np.stack([wa[0], wa[25], wb[18]]), dtype, "step 0")
    dh.assert_logits(read(1), wa[26:27], dtype, "step 1")
    dh.assert_logits(read(2), np.stack([wa[27], wb[20]]), dtype, "step 2")
    dh.assert_logits(read(3), wa[28:29], dtype, "step 3")
    dh.assert_logits(read(4), wa[29:30], dtype, "step 4")


def test_command_line_generates_with_a_dokulorn_folder(capsys):
    """The command line picks the architecture by config.json; its greedy tokens are the entry point's."""
    import io
    from rust_deeplearning_b200 import Generator, cli
    name = "DC"
    p = dh.prompt(name, 50, 12)
    out = io.StringIO()
    code = cli.main([dh.model_folder(name), "--prompt-ids", " ".join(map(str, p)), "--max-tokens", "6", "--temperature", "0",
                     "--dtype", "float32", "--max-context", "64"], stdout=out)
    assert code == 0
    assert "arch=Dokulorn" in capsys.readouterr().err
    gen = Generator(dh.loaded_model(name, "float32"), max_batch=1, max_context=64).with_temperature(0.0)
    assert [int(t) for t in out.getvalue().split()] == gen.generate(p, 6)[len(p):]
