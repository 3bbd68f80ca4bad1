"""The Tinevik family through the engine (GPU) against the plain restatement in oracle/tinevik_oracle.py.

Every test builds its own small configuration and random weights.  The engine runs in fp32 (tight bars: a lost key, a window
one token off, a state that was not carried, a stale page or slot shows far above fp32 rounding) and in bf16 (loose bars).
Covered: each mechanism alone (single-layer models); every layer's residual stream; whole prompts against token-by-token
decoding; prompt portions down to two tokens; unequal requests in one batch against each alone; pages and sequence slots
freed and used again (matrix states included); keys far back, at page borders and just inside / outside the window, in
prompts and in decoding, with weights sharpened so that one key decides; the first tokens of a sequence; a long run of
decode steps; layers that run with another layer's tensors; sizes that differ per layer and values a model may make equal
or one; the registry and the checkpoint loader (integer table included) from a model directory; greedy generation through
the engine's own entry points and through b2serve's scheduler.
"""
import http.client
import importlib
import json
import os
import re
import subprocess
import time

import numpy as np
import pytest
import torch

from _util import pkg
from oracle.tinevik_oracle import forward, greedy, random_weights

pytestmark = pytest.mark.gpu


def gla(heads, dim, vdim, tau, rank=4):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def att(heads, kv, dim, vdim, scale, rot=None, cap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if cap is not None:
        m["softcap"] = cap
    if rot is not None:   # (base, dims, factor or None)
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if rot[2] is not None:
            m["rot"]["scaling"] = {"factor": rot[2]}
    return {"type": "attention", "mixer": m}


def lat(heads, dim, vdim, kv_rank, q_rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def dense(n):
    return {"kind": "dense", "ff": n}


def moe(experts, top, n, limit=1.5):
    return {"kind": "moe", "expert": {"ff": n, "limit": limit}, "router": {"experts": experts, "top": top}}


def model(layers, vocab=203, width=88, escale=9.0, eps=1e-5, lscale=1.5):
    out = []
    for entry in layers:
        m, f = entry[0], entry[1]
        d = dict(m, mlp=f)
        if len(entry) > 2:
            d["weights_of"] = entry[2]
        out.append(d)
    return {"architecture": "Tinevik", "vocab": vocab, "width": width, "embedding": {"scale": escale}, "norm": {"eps": eps},
            "logit_scale": lscale, "layers": out}


def cfg_a():
    """Odd sizes, none a multiple of a tile; three query heads per key/value head; a window shorter than a page; partly rotated heads with
    stretched angles; a dense layer behind the first mixer only; two layers that run with an earlier layer's tensors."""
    g, a, l = gla(3, 10, 12, 7.0), att(6, 2, 10, 12, 0.3, rot=(5000.0, 6, 2.0), cap=12.0), lat(3, 6, 10, 20, 14, 0.4, window=11)
    return model([(g, dense(36)), (a, moe(5, 2, 14)), (l, moe(4, 3, 10)), (g, dense(36), 0), (a, moe(5, 2, 14), 1), (l, None)])


def cfg_b():
    """Values a model may make equal or one: one head everywhere, as many key/value heads as heads, fully rotated heads without stretching,
    no cap, no rotation at all, a window of one key, no mask, one expert that is always chosen, every expert chosen, tau 1, equal latent
    widths, no embedding scale, no logit scale, a layer without a feed-forward."""
    return model([(gla(1, 8, 8, 1.0, rank=1), moe(1, 1, 8)),
                  (att(1, 1, 8, 8, 0.35, rot=(100.0, 8, None)), moe(3, 3, 6)),
                  (att(2, 2, 6, 4, 0.4), None),
                  (lat(1, 8, 8, 8, 8, 0.5, window=1), dense(8)),
                  (lat(2, 4, 6, 12, 5, 0.5), dense(16))], vocab=97, width=64, escale=1.0, eps=1e-6, lscale=1.0)


def cfg_c():
    """Sizes the tensor-core products take: inner dimensions in multiples of 64, more than 64 tokens per call."""
    return model([(gla(2, 32, 64, 16.0, rank=16), dense(192)),
                  (att(4, 2, 32, 32, 0.18, rot=(10000.0, 16, 4.0), cap=30.0), moe(6, 2, 64)),
                  (lat(4, 32, 32, 64, 64, 0.18, window=70), moe(4, 1, 128)),
                  (att(4, 2, 32, 32, 0.18, rot=(10000.0, 16, 4.0), cap=30.0), moe(6, 2, 64), 1)], vocab=300, width=128)


def engine(cfg, w, f32=True, **rt):
    P = pkg()
    rt = {"max_model_len": 1024, "num_blocks": 80, "max_seqs": 4, "max_batch_tokens": 1024, **rt}
    e = P.Engine(P.EngineConfig.tinevik(cfg, compute_f32=f32, **rt))
    e.load_state_dict({k: (v if v.dtype == torch.int64 else v.to(torch.bfloat16)) for k, v in w.items()})
    return e


def tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def ref_logits(cfg, w, toks):
    return forward(cfg, w, toks)[0].numpy()


def err(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-9))


F32_BAR, BF16_BAR = 3e-5, 6e-2


def run_schedule(e, cfg, toks, ref, bar, cuts, decode_from):
    """One request: portions of the given sizes up to `decode_from`, the rest token by token; every position is compared."""
    sid = e.seq_create(len(toks))
    at = 0
    for c in cuts:
        c = min(c, decode_from - at)
        if c <= 0:
            break
        lg, _ = e.prefill_logits([sid], [toks[at:at + c]], list(range(c)))
        assert err(lg, ref[at:at + c]) < bar, "portion at %d of %d tokens" % (at, c)
        at += c
    assert at == decode_from, (at, decode_from)
    for p in range(at, len(toks)):
        e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
        assert err(e.get_logits(1)[0], ref[p]) < bar, "decoded position %d" % p
    e.seq_free(sid)


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_every_layer_fp32(make):
    cfg = make()
    w = random_weights(cfg, seed=1)
    toks = tokens(cfg, 37, 2)
    logits, streams = forward(cfg, w, toks)
    assert streams.shape[0] == len(cfg["layers"])
    with engine(cfg, w) as e:
        e.set_debug(hidden=True)
        sid = e.seq_create(64)
        got, _ = e.prefill_logits([sid], [toks], list(range(len(toks))))
        for r in range(streams.shape[0]):
            assert err(e.get_hidden_f32(r, len(toks)), streams[r].numpy()) < F32_BAR, "residual stream after layer %d" % r
        assert err(got, logits.numpy()) < F32_BAR


SINGLE = {
    "gla, three heads": [(gla(3, 10, 7, 4.0), None)],
    "gla, value columns beyond one tile": [(gla(2, 12, 80, 8.0), None)],
    "gla, keys beyond a warp, tau 1": [(gla(1, 72, 8, 1.0, rank=2), None)],
    "attention, three query heads per group, cap, stretched angles": [(att(6, 2, 10, 6, 0.5, rot=(300.0, 4, 3.0), cap=5.0), None)],
    "attention, every entry rotated": [(att(2, 1, 8, 8, 0.35, rot=(50.0, 8, None)), None)],
    "attention, nothing rotated, no cap": [(att(3, 3, 9, 5, 0.4), None)],
    "attention, wide heads and odd widths": [(att(2, 2, 70, 34, 0.12, rot=(1000.0, 70, 1.5), cap=20.0), None)],
    "attention, more heads than a score tile is wide": [(att(40, 8, 4, 4, 0.5, rot=(10.0, 2, None), cap=3.0), None)],
    "latent attention, window": [(lat(3, 6, 10, 20, 14, 0.4, window=9), None)],
    "latent attention, no mask": [(lat(2, 8, 8, 12, 6, 0.35), None)],
    "latent attention, a window of one key": [(lat(2, 9, 5, 7, 3, 0.4, window=1), None)],
    "latent attention, a window of a page and one": [(lat(1, 8, 8, 16, 16, 0.3, window=17), None)],
    "dense feed-forward": [(gla(1, 8, 8, 2.0), dense(33))],
    "experts, one choice": [(gla(1, 8, 8, 2.0), moe(7, 1, 12))],
    "experts, three choices, a tight clamp": [(gla(1, 8, 8, 2.0), moe(5, 3, 9, limit=0.3))],
    "more experts than a warp": [(gla(1, 8, 8, 2.0), moe(40, 2, 6))],
    "a layer run three times with one layer's tensors": [(att(2, 1, 8, 8, 0.4, rot=(100.0, 4, None)), dense(12)), (att(2, 1, 8, 8, 0.4, rot=(100.0, 4, None)), dense(12), 0),
                                                         (att(2, 1, 8, 8, 0.4, rot=(100.0, 4, None)), dense(12), 0)],
    "tensors of a later layer, and of a layer that borrows its own": [(lat(2, 8, 6, 10, 7, 0.4, window=5), moe(4, 2, 6), 1), (lat(2, 8, 6, 10, 7, 0.4, window=5), moe(4, 2, 6)),
                                                                      (lat(2, 8, 6, 10, 7, 0.4, window=5), moe(4, 2, 6), 0)],
}


@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name):
    cfg = model(SINGLE[name], vocab=131, width=48)
    w = random_weights(cfg, seed=3)
    toks = tokens(cfg, 75, 4)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        run_schedule(e, cfg, toks, ref, F32_BAR, [75], 75)                      # the whole prompt
        run_schedule(e, cfg, toks, ref, F32_BAR, [2, 31, 3, 16, 2], 54)         # portions, then 21 decode steps


@pytest.mark.parametrize("make", [cfg_a, cfg_b, cfg_c])
def test_bf16_close_to_the_restatement(make):
    cfg = make()
    w = random_weights(cfg, seed=5)
    toks = tokens(cfg, 150, 6)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w, f32=False) as e:
        sid = e.seq_create(200)
        lg, _ = e.prefill_logits([sid], [toks[:140]], list(range(140)))
        rel = np.abs(lg - ref[:140]).max(axis=1) / np.abs(ref).max()
        assert np.median(rel) < BF16_BAR / 3 and rel.max() < 3 * BF16_BAR, (np.median(rel), rel.max())
        for p in range(140, 150):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            assert err(e.get_logits(1)[0], ref[p]) < 3 * BF16_BAR, "decoded position %d" % p


@pytest.mark.parametrize("heads,kv,dim,vdim", [(12, 4, 48, 64), (20, 20, 16, 32), (16, 8, 64, 128), (3, 1, 32, 16)])
def test_bf16_head_mixed_attention_on_tensor_cores(heads, kv, dim, vdim):
    """bf16 prompt portions of head sizes in multiples of 16 take the tensor-core form of the head-mixed attention, decode steps the form that
    splits the keys: several head counts (above and below a register tile of heads, one key/value head, as many as heads), with sharpened scores,
    whole prompts against portions that start and end inside key tiles, and decoding behind them.  A mixing matrix applied the wrong way round,
    a key tile that is lost or a value turned by the wrong position moves the logits far beyond bf16 rounding."""
    cfg = model([(att(heads, kv, dim, vdim, dim ** -0.5, rot=(3000.0, dim // 2, 2.0), cap=25.0), dense(64)),
                 (att(heads, kv, dim, vdim, dim ** -0.5, rot=(3000.0, dim // 2, 2.0), cap=25.0), dense(64), 0)], vocab=211, width=96)
    w = sharpen(cfg, random_weights(cfg, seed=23), factor=3.0)
    toks = tokens(cfg, 230, 24)
    ref = ref_logits(cfg, w, toks)
    swapped = dict(w)
    swapped["l0.mix.talk"] = w["l0.mix.talk"].t().contiguous()
    assert err(ref_logits(cfg, swapped, toks)[100:], ref[100:]) > 3 * BF16_BAR     # the test would see the matrix transposed
    with engine(cfg, w, f32=False) as e:
        for cuts, decode_from in ([230], 230), ([70, 33, 2, 47, 17, 40], 209):
            sid = e.seq_create(len(toks))
            at, rel = 0, []
            for c in cuts:
                lg, _ = e.prefill_logits([sid], [toks[at:at + c]], list(range(c)))
                rel += list(np.abs(lg - ref[at:at + c]).max(axis=1) / np.abs(ref).max())
                at += c
            for p_ in range(at, len(toks)):
                e.decode_step([sid], in_tokens=[toks[p_]], want_output=False)
                rel.append(np.abs(e.get_logits(1)[0] - ref[p_]).max() / np.abs(ref).max())
            e.seq_free(sid)
            assert at == decode_from and np.median(rel) < BF16_BAR / 3 and max(rel) < 3 * BF16_BAR, (cuts, np.median(rel), max(rel))


def test_bf16_long_step_runs_the_experts_one_by_one():
    """A step with at least 2048 (token, choice) pairs takes the per-expert tensor-core products; short portions of the same prompt take
    the ragged ones: both agree with the restatement."""
    cfg = cfg_c()
    w = random_weights(cfg, seed=7)
    toks = tokens(cfg, 1100, 8)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w, f32=False, max_model_len=1280, num_blocks=200, max_batch_tokens=1280) as e:
        sid = e.seq_create(1100)
        rows = list(range(0, 1100, 7))
        lg, _ = e.prefill_logits([sid], [toks], rows)
        rel = np.abs(lg - ref[rows]).max(axis=1) / np.abs(ref).max()
        assert np.median(rel) < BF16_BAR / 3 and rel.max() < 3 * BF16_BAR, (np.median(rel), rel.max())
        sid2 = e.seq_create(1100)
        at = 0
        for c in [100, 40, 2, 70]:
            l2, _ = e.prefill_logits([sid2], [toks[at:at + c]], [c - 1])
            assert err(l2[0], ref[at + c - 1]) < 3 * BF16_BAR
            at += c


def test_prefill_against_token_by_token_decoding():
    cfg = cfg_a()
    w = random_weights(cfg, seed=9)
    toks = tokens(cfg, 70, 10)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        run_schedule(e, cfg, toks, ref, F32_BAR, [70], 70)
        run_schedule(e, cfg, toks, ref, F32_BAR, [1], 1)       # the first token as a one-token prompt, everything after it as decode steps
        run_schedule(e, cfg, toks, ref, F32_BAR, [2], 2)


@pytest.mark.parametrize("cuts", [[2, 2, 2, 64, 3, 17, 2, 31], [16, 16, 32, 1, 1, 57], [63, 2, 58], [1, 1, 1, 2, 1, 3, 100]])
def test_portions_of_a_prompt(cuts):
    cfg = cfg_a()
    w = random_weights(cfg, seed=11)
    n = sum(cuts)
    toks = tokens(cfg, n, 12)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        run_schedule(e, cfg, toks, ref, F32_BAR, cuts, n)


def test_mixed_batch_equals_each_alone():
    cfg = cfg_a()
    w = random_weights(cfg, seed=13)
    lens = [140, 5, 60, 1]
    prompts = [tokens(cfg, n, 20 + i) for i, n in enumerate(lens)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    with engine(cfg, w) as e:
        sids = [e.seq_create(160) for _ in prompts]
        done = [0, 0, 0, 0]
        # unequal portions beside single tokens, several steps; request 3 is one token long and joins late
        plan = [[(0, 64), (1, 3)], [(0, 2), (1, 1), (2, 40)], [(0, 60), (1, 1), (2, 1), (3, 1)], [(0, 4), (2, 6)]]
        for step in plan:
            chunks, rows, base = [], [], 0
            for r, c in step:
                chunks.append(prompts[r][done[r]:done[r] + c])
                rows += list(range(base, base + c))
                base += c
            lg, _ = e.prefill_logits([sids[r] for r, _ in step], chunks, rows)
            base = 0
            for r, c in step:
                assert err(lg[base:base + c], refs[r][done[r]:done[r] + c]) < F32_BAR, "request %d at %d" % (r, done[r])
                base += c
                done[r] += c
        # pure decode batches of unequal lengths (the captured step) in two orders, against the same references
        for live in ([0, 2], [2, 0], [0]):
            e.decode_step([sids[r] for r in live], in_tokens=[prompts[r][done[r]] for r in live], want_output=False)
            lg = e.get_logits(len(live))
            for k, r in enumerate(live):
                assert err(lg[k], refs[r][done[r]]) < F32_BAR, "decode batch %r, request %d" % (live, r)
                done[r] += 1


def test_pages_and_slots_are_used_again():
    """Eight usable pages, two sequence slots: every round frees its request, the next one gets the same slot (and with it the matrix
    states the last request left) and the same pages in another order."""
    cfg = cfg_a()
    w = random_weights(cfg, seed=15)
    with engine(cfg, w, num_blocks=9, max_seqs=2, max_model_len=128, max_batch_tokens=128) as e:
        for rnd in range(5):
            na, nb = 30 + 13 * rnd, 70 - 11 * rnd
            a, b = tokens(cfg, na, 100 + rnd), tokens(cfg, nb, 200 + rnd)
            ra, rb = ref_logits(cfg, w, a), ref_logits(cfg, w, b)
            sa, sb = (e.seq_create(na), e.seq_create(nb)) if rnd % 2 else tuple(reversed((e.seq_create(nb), e.seq_create(na))))
            cut = 9 + rnd
            l1, _ = e.prefill_logits([sa, sb], [a[:cut], b[:nb - 3]], list(range(cut)) + [cut + nb - 4])
            assert err(l1[:cut], ra[:cut]) < F32_BAR and err(l1[cut], rb[nb - 4]) < F32_BAR, "round %d, first step" % rnd
            l2, _ = e.prefill_logits([sb, sa], [b[nb - 3:nb - 1], a[cut:]], [1, 2 + na - cut - 1])
            assert err(l2[0], rb[nb - 2]) < F32_BAR and err(l2[1], ra[na - 1]) < F32_BAR, "round %d, second step" % rnd
            e.decode_step([sb], in_tokens=[b[nb - 1]], want_output=False)
            assert err(e.get_logits(1)[0], rb[nb - 1]) < F32_BAR, "round %d, decode" % rnd
            e.seq_free(sa)
            e.seq_free(sb)
        assert e.info()["free_blocks"] == 8


def sharpen(cfg, w, factor=6.0):
    """Scores that decide: queries of the softmax mixers scaled up so that one key takes nearly all the weight, and states that forget
    slowly, so that a key far back, one across a page border or one a window should hide changes the logits by far more than rounding."""
    w = dict(w)
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p = "l%d.mix." % i
        if L["type"] == "attention":
            w[p + "q.norm"] = (w[p + "q.norm"] * factor).to(torch.bfloat16).float()
        elif L["type"] == "latent_attention":
            w[p + "uq"] = (w[p + "uq"] * factor).to(torch.bfloat16).float()
        else:
            w[p + "a2.b"] = (w[p + "a2.b"] + 4.0).to(torch.bfloat16).float()
    return w


def test_window_edges_page_borders_and_far_keys():
    cfg = model([(att(4, 2, 12, 8, 0.3, rot=(2000.0, 8, 2.0), cap=40.0), None), (lat(2, 8, 8, 16, 10, 0.35, window=33), None),
                 (gla(2, 8, 8, 64.0), None), (lat(2, 8, 8, 16, 10, 0.35, window=16), dense(24))], vocab=151, width=56)
    w = sharpen(cfg, random_weights(cfg, seed=17))
    toks = tokens(cfg, 400, 18)
    ref = ref_logits(cfg, w, toks)
    # the sharpened model must really depend on far keys and on the window: hiding one more key moves the logits visibly
    moved = dict(cfg, layers=[dict(L, mixer=dict(L["mixer"], mask={"size": L["mixer"]["mask"]["size"] - 1})) if L["mixer"].get("mask") else L
                              for L in cfg["layers"]])
    assert err(ref_logits(moved, w, toks)[300:], ref[300:]) > 100 * F32_BAR
    with engine(cfg, w) as e:
        run_schedule(e, cfg, toks, ref, F32_BAR, [400], 400)
        # portions that end and start at page borders, at window edges and one token off them; decoding across a page border
        run_schedule(e, cfg, toks, ref, F32_BAR, [16, 1, 15, 33, 31, 2, 62, 17, 47, 100], 324)


def test_long_decoding():
    cfg = cfg_a()
    w = sharpen(cfg, random_weights(cfg, seed=19), factor=3.0)
    toks = tokens(cfg, 260, 20)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        run_schedule(e, cfg, toks, ref, F32_BAR, [20], 20)


@pytest.mark.parametrize("nseq", [1, 3, 4])
def test_bf16_decode_batches(nseq):
    cfg = cfg_c()
    w = random_weights(cfg, seed=21)
    prompts = [tokens(cfg, 90 + 37 * i, 300 + i) for i in range(nseq)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    with engine(cfg, w, f32=False) as e:
        sids = [e.seq_create(len(p)) for p in prompts]
        e.prefill_logits(sids, [p[:-6] for p in prompts], [])
        for k in range(6, 0, -1):
            e.decode_step(sids, in_tokens=[p[len(p) - k] for p in prompts], want_output=False)
            lg = e.get_logits(nseq)
            for i in range(nseq):
                assert err(lg[i], refs[i][len(prompts[i]) - k]) < 3 * BF16_BAR


def test_a_missing_tensor_is_named():
    cfg = cfg_b()
    w = random_weights(cfg, seed=23)
    del w["l1.mlp.table"]
    P = pkg()
    with pytest.raises(P.B2Error, match="l1.mlp.table"):
        engine(cfg, w)


def test_a_table_entry_outside_the_experts_is_refused():
    cfg = cfg_b()
    w = random_weights(cfg, seed=23)
    w["l1.mlp.table"][5, 0] = 3
    P = pkg()
    with pytest.raises(P.B2Error, match="expert"):
        engine(cfg, w)


def write_dir(cfg, w, path):
    weights = importlib.import_module("aws-k8s-ansible-provisioner_b200.weights")
    clean = json.loads(json.dumps(cfg))
    for L in clean["layers"]:
        L["mixer"].pop("rank", None)
    weights.write_model_dir(clean, {k: (v.to(torch.int32) if v.dtype == torch.int64 else v.to(torch.bfloat16)) for k, v in w.items()}, str(path))
    return str(path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_from_a_model_directory(tmp_path, dtype):
    """The registry reads config.json, the loader model.safetensors (bf16 tensors and the int32 table)."""
    cfg = cfg_a()
    w = random_weights(cfg, seed=25)
    toks = tokens(cfg, 50, 26)
    ref = ref_logits(cfg, w, toks)
    P = pkg()
    with P.Engine.from_model_dir(write_dir(cfg, w, tmp_path), dtype=dtype, max_model_len=128, num_blocks=20, max_seqs=2, max_batch_tokens=128) as e:
        sid = e.seq_create(50)
        lg, _ = e.prefill_logits([sid], [toks], list(range(50)))
        assert err(lg, ref) < (F32_BAR if dtype == "float32" else 3 * BF16_BAR)


def test_greedy_generation_through_the_engine():
    cfg = cfg_a()
    w = random_weights(cfg, seed=27)
    prompts = [tokens(cfg, 33, 40), tokens(cfg, 9, 41)]
    refs = [greedy(cfg, w, p, 12) for p in prompts]
    with engine(cfg, w) as e:
        sids = [e.seq_create(64) for _ in prompts]
        out = [e.prefill(sids, prompts)]
        for _ in range(11):
            out.append(e.decode_step(sids))          # the token feedback stays on the device
        got = np.stack(out, axis=1)
        for i in range(2):
            assert got[i].tolist() == refs[i], (got[i].tolist(), refs[i])


def test_greedy_generation_through_the_server(tmp_path):
    """b2serve picks the family from config.json, loads model.safetensors, and its scheduler (chunked prefill, then decode
    steps over the running requests) generates what the restatement generates."""
    P = pkg()
    exe = os.path.join(os.path.dirname(P.LIB_PATH), "b2serve")
    assert os.path.exists(exe), "b2serve not built"
    cfg = cfg_a()
    cfg["vocab"] = 1000         # the byte tokenizer renders ids >= 256 as <|id|>: those are read back from the reply's text
    w = random_weights(cfg, seed=29)
    write_dir(cfg, w, tmp_path)
    proc = subprocess.Popen([exe, str(tmp_path), "--served-model-name", "tinevik-test", "--port", "0", "--host", "127.0.0.1", "--max-model-len", "256",
                             "--max-num-seqs", "4", "--num-gpu-blocks-override", "64", "--max-num-batched-tokens", "32", "--eos-token-id", "-1",
                             "--dtype", "float32"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        port, t0 = None, time.time()
        while time.time() - t0 < 120:
            line = proc.stdout.readline()
            if line.startswith("READY"):
                port = int(line.split()[1])
                break
            if proc.poll() is not None:
                break
        assert port is not None, "b2serve did not start: " + proc.stderr.read()
        prompt = tokens(cfg, 70, 30)   # longer than --max-num-batched-tokens: prefilled in three portions
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
        c.request("POST", "/v1/completions", body=json.dumps({"model": "tinevik-test", "prompt": prompt, "max_tokens": 10, "temperature": 0,
                                                              "ignore_eos": True}), headers={"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read().decode())
        assert r.status == 200, body
        ref = greedy(cfg, w, prompt, 10)
        got_big = [int(x) for x in re.findall(r"<\|(\d+)\|>", body["choices"][0]["text"])]
        ref_big = [t for t in ref if t >= 256]
        assert body["usage"]["completion_tokens"] == 10
        assert len(ref_big) >= 5 and got_big == ref_big, (body["choices"][0]["text"], ref)
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except Exception:
            proc.kill()


def random_model(seed):
    """A random layer list: every mixer and feed-forward kind in a random order, sizes drawn per layer, some layers running with an earlier
    layer's tensors."""
    rng = np.random.RandomState(seed)
    pick = lambda xs: xs[rng.randint(len(xs))]
    layers = []
    for i in range(int(rng.randint(3, 7))):
        if i >= 2 and rng.rand() < 0.3:
            j = int(rng.randint(0, i))
            while len(layers[j]) > 2:
                j = layers[j][2]
            layers.append((layers[j][0], layers[j][1], j))
            continue
        kind = pick(["gla", "attention", "latent"])
        if kind == "gla":
            m = gla(pick([1, 2, 3]), pick([6, 8, 20]), pick([4, 10, 36]), pick([1.0, 4.0, 16.0]), rank=pick([1, 3, 5]))
        elif kind == "attention":
            kv = pick([1, 2, 3])
            d, dv = pick([6, 8, 16, 22]), pick([4, 8, 16, 18])
            rot = pick([None, (pick([100.0, 1e4, 2.5e5]), pick([2, d - d % 2, 4]), pick([None, 2.0, 8.0]))])
            m = att(kv * pick([1, 2, 4]), kv, d, dv, pick([0.2, 0.35]), rot=rot, cap=pick([None, 6.0, 30.0]))
        else:
            m = lat(pick([1, 2, 5]), pick([4, 8, 12]), pick([4, 8, 14]), pick([6, 16, 24]), pick([5, 8, 16]), pick([0.3, 0.5]), window=pick([None, 1, 7, 16, 33]))
        f = pick([None, dense(pick([8, 24, 50])), moe(pick([1, 3, 8]), 1, pick([6, 16])), moe(pick([4, 6]), pick([2, 4]), pick([6, 10]))])
        layers.append((m, f))
    return model(layers, vocab=int(pick([53, 160, 301])), width=int(pick([24, 40, 56, 72])), escale=float(pick([1.0, 4.0, 16.0])),
                 eps=float(pick([1e-6, 1e-5])), lscale=float(pick([1.0, 2.0])))


@pytest.mark.parametrize("seed", range(8))
def test_random_models_and_schedules(seed):
    """Up to four live requests over a pool that holds only what is live: portions of some beside single tokens of others, requests that end
    and give their pages and slots to the next, in fp32 and (even seeds) in bf16."""
    cfg = random_model(seed)
    w = random_weights(cfg, seed=50 + seed)
    rng = np.random.RandomState(1000 + seed)
    f32 = seed % 2 == 1
    bar = F32_BAR if f32 else 4 * BF16_BAR
    lens = [int(rng.randint(1, 130)) for _ in range(7)]
    prompts = [tokens(cfg, n, 2000 + 10 * seed + i) for i, n in enumerate(lens)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    with engine(cfg, w, f32=f32, num_blocks=4 * 9 + 1, max_seqs=4, max_model_len=144, max_batch_tokens=576) as e:
        live, done, nxt, sid = [], {}, 0, {}
        worst = []
        while nxt < len(prompts) or live:
            while len(live) < 4 and nxt < len(prompts) and (not live or rng.rand() < 0.6):
                sid[nxt] = e.seq_create(1)
                done[nxt] = 0
                live.append(nxt)
                nxt += 1
            step = [r for r in live if rng.rand() < 0.8] or live[:1]
            sizes = {r: min(len(prompts[r]) - done[r], int(pick_size(rng))) for r in step}
            for r in step:
                e.seq_reserve(sid[r], done[r] + sizes[r])
            if all(sizes[r] == 1 and done[r] >= 1 for r in step):
                e.decode_step([sid[r] for r in step], in_tokens=[prompts[r][done[r]] for r in step], want_output=False)
                lg = e.get_logits(len(step))
                got = {r: lg[k:k + 1] for k, r in enumerate(step)}
            else:
                chunks = [prompts[r][done[r]:done[r] + sizes[r]] for r in step]
                lg, _ = e.prefill_logits([sid[r] for r in step], chunks, list(range(sum(sizes.values()))))
                got, base = {}, 0
                for r in step:
                    got[r] = lg[base:base + sizes[r]]
                    base += sizes[r]
            for r in step:
                worst.append(err(got[r], refs[r][done[r]:done[r] + sizes[r]]))
                done[r] += sizes[r]
                if done[r] == len(prompts[r]):
                    e.seq_free(sid[r])
                    live.remove(r)
        worst = np.array(worst)
        if f32:
            assert worst.max() < bar, (cfg, worst.max())
        else:    # a bf16 product rounds its operands: the bulk is barred tightly, the worst loosely
            assert np.median(worst) < BF16_BAR and worst.max() < bar, (cfg, np.median(worst), worst.max())


def pick_size(rng):
    return [1, 1, 1, 2, 2, 3, 16, 17, 40, 64, 100][rng.randint(11)]


def test_a_trace_replayed_through_the_command_line(tmp_path):
    """bin/trace_run: steps on standard input, the logits asked for as files, a pool sized for the live tokens only."""
    cfg = cfg_a()
    w = random_weights(cfg, seed=31)
    a, b = tokens(cfg, 90, 32), tokens(cfg, 21, 33)
    ra, rb = ref_logits(cfg, w, a), ref_logits(cfg, w, b)
    mdir, out = write_dir(cfg, w, tmp_path / "m"), tmp_path / "out"
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:72], "want": []}, {"id": "b", "tokens": b[:20], "want": [19]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[72:73], "want": [0]}, {"id": "b", "tokens": b[20:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[73:], "want": [16]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [20]}], "end": ["c"]}]
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([exe, "--model", mdir, "--dtype", "float32", "--out", str(out), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == ["done %d" % i for i in range(5)]
    rd = lambda i: np.fromfile(str(out / ("%d.f32" % i)), dtype="<f4").reshape(-1, cfg["vocab"])
    assert err(rd(0), ra[[0, 69]]) < F32_BAR and err(rd(1), rb[[19]]) < F32_BAR
    assert err(rd(2), np.stack([ra[72], rb[20]])) < F32_BAR and err(rd(3), ra[[89]]) < F32_BAR and err(rd(4), rb[[20]]) < F32_BAR
