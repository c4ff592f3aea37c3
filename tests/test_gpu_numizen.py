"""Numizen through the serving path (ServingEngine -> SequenceEngine -> tha_hyb_step) against the plain float64
statement of the design in tests/numizen_oracle.py.

Every test builds its own small configuration with random weights.  float32 runs are compared tightly (they differ from
float64 by rounding only), bfloat16 runs loosely.  Where random weights would hide a fault (one far key among hundreds,
a key at a border of the block table, an expert outside the kept groups) the weights are made sharp: keys equal queries
and the score scale is large, so that a query puts nearly all its weight on the earlier occurrence of its own token;
corrections push the router towards experts it must not take.
"""
import copy
import os
import subprocess

import numpy as np
import pytest

import numizen_oracle as O
from pkgload import load_pkg

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 6e-2


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / (np.sqrt((want ** 2).mean()) + 1e-12))


# ---- configurations ---------------------------------------------------------------------------------------------------
def moe(experts=6, top=2, ff=40, shared=24, groups=(3, 2)):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def latent(mlp, heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, rot_dims=None, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if rot_dims != 0:
        m["rot"] = {"base": base, "dims": rot_dims or rot_dim}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def gla(mlp, heads=2, dim=24, vdim=16, tau=8.0):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def model(layers, width=64, vocab=130, loop=None, max_positions=1024):
    c = {"architecture": "Numizen", "layers": layers, "norm": {"eps": 1e-5}, "vocab": vocab, "width": width, "max_positions": max_positions}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


class Built:
    """A model folder, its oracle view, and engines on demand."""

    def __init__(self, tmp, cfg, seed=0, tweak=None, gla_rank=6):
        self.serving = load_pkg("serving")
        self.cfg = cfg
        self.w = O.random_weights(cfg, seed, gla_rank=gla_rank)
        if tweak:
            tweak(self.w)
            for k in self.w:
                self.w[k] = O.bf16_round(self.w[k]).astype(np.float64)
        self.folder = str(tmp)
        self.serving.save_model_folder(self.folder, cfg, {k: np.asarray(v, np.float32) for k, v in self.w.items()})
        self._ref = {}

    def engine(self, dtype="float32", max_tokens=1024, max_seqs=4):
        return self.serving.ServingEngine(self.folder, dtype, max_tokens, max_seqs)

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            taps = []
            z = O.forward(self.cfg, self.w, list(tokens), taps)
            self._ref[key] = (z, np.stack(taps))
        return self._ref[key]


def general_layers():
    # heads, ranks, rotated share and value sizes differ between the layers; one layer without a feed-forward, one dense
    return [latent(dense()), gla(moe()), latent(moe(experts=8, top=3, ff=24, shared=0, groups=(4, 3)), heads=2, dim=24, rot_dim=12, vdim=8,
                                                 q_rank=24, kv_rank=48, rot_dims=8),
            gla(None, heads=3, dim=40, vdim=10, tau=3.0), latent(moe(experts=4, top=2, groups=None), heads=4, dim=8, rot_dim=16, vdim=16, q_rank=56,
                                                                  kv_rank=16, base=500.0)]


@pytest.fixture(scope="module")
def general(tmp_path_factory):
    return Built(tmp_path_factory.mktemp("general"), model(general_layers(), loop=(1, 3, 3)), seed=1)


def tokens_for(built, n, seed):
    return np.random.default_rng(seed).integers(0, built.cfg["vocab"], n).tolist()


def feed(e, rid, toks, cuts, want_all=True):
    """the tokens in portions of the given sizes (the last size repeats); logits of every position"""
    out, at, i = [], 0, 0
    while at < len(toks):
        c = min(cuts[min(i, len(cuts) - 1)], len(toks) - at)
        r = e.step([(rid, toks[at:at + c], list(range(c)) if want_all else [])])
        if want_all:
            out.append(r)
        at += c
        i += 1
    return np.concatenate(out, 0) if want_all else None


# ---- whole prompts, every layer run -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompt_every_layer_run(general, dtype, tol):
    toks = tokens_for(general, 97, 3)
    z, layers = general.ref(toks)
    assert len(layers) == 1 + 2 * 3 + 2                      # the looped pair counts every time
    e = general.engine(dtype)
    logits, taps = e.step([("a", toks, list(range(len(toks))))], taps=True)
    assert taps.shape == layers.shape
    for i in range(len(layers)):
        assert rel_err(taps[i], layers[i]) < tol, f"residual stream after layer run {i}"
    assert rel_err(logits, z) < tol
    for p in range(4):                                        # the first tokens of a sequence, one by one
        assert rel_err(logits[p], z[p]) < tol * 3, f"position {p}"


# ---- each mechanism alone ---------------------------------------------------------------------------------------------
def one_layer(tmp, layer, width=48, seed=2, tweak=None, **kw):
    return Built(tmp, model([layer], width=width, **kw), seed, tweak)


def check_all_positions(b, n=70, dtype="float32", tol=F32_TOL, cuts=None):
    toks = tokens_for(b, n, 1)
    z, layers = b.ref(toks)
    e = b.engine(dtype)
    if cuts is None:
        logits, taps = e.step([("a", toks, list(range(n)))], taps=True)
        assert rel_err(taps[-1], layers[-1]) < tol
    else:
        logits = feed(e, "a", toks, cuts)
    assert rel_err(logits, z) < tol
    return toks, z


def test_latent_attention_alone(tmp_path):
    b = one_layer(tmp_path, latent(None, heads=5, dim=12, rot_dim=6, vdim=20, q_rank=28, kv_rank=36))
    toks, z = check_all_positions(b)
    # the mixer does carry the layer: with its scale at zero the logits move
    other = copy.deepcopy(b.w)
    other["l0.ls1"][...] = 0.0
    assert rel_err(O.forward(b.cfg, other, toks), z) > 0.05


def test_latent_attention_rotates_part_of_the_shared_key_only(tmp_path):
    b = one_layer(tmp_path, latent(None, heads=2, dim=8, rot_dim=12, vdim=8, q_rank=16, kv_rank=24, rot_dims=4, base=50.0))
    check_all_positions(b)
    b2 = one_layer(tmp_path / "norot", latent(None, heads=2, dim=8, rot_dim=12, vdim=8, q_rank=16, kv_rank=24, rot_dims=0))
    check_all_positions(b2)


def test_gated_linear_attention_alone(tmp_path):
    b = one_layer(tmp_path, gla(None, heads=3, dim=20, vdim=12, tau=4.0))
    toks, z = check_all_positions(b, n=90)
    check_all_positions(b, n=90, cuts=[31, 2, 1])
    other = copy.deepcopy(b.w)
    other["l0.ls1"][...] = 0.0
    assert rel_err(O.forward(b.cfg, other, toks), z) > 0.05


def test_gated_linear_attention_decay_extremes(tmp_path):
    """biases that close the decay gate (the state is forgotten at once) or open it (nothing is forgotten), tau of 1 and
    a large tau"""
    for i, (bias, tau) in enumerate([(-12.0, 1.0), (12.0, 1.0), (0.0, 64.0)]):
        def tweak(w, bias=bias):
            w["l0.mix.a2.b"][...] = bias
        b = one_layer(tmp_path / str(i), gla(None, heads=2, dim=16, vdim=8, tau=tau), tweak=tweak)
        check_all_positions(b, n=50, cuts=[20, 1])


def test_dense_feed_forward_alone(tmp_path):
    def tweak(w):
        w["l0.ls1"][...] = 0.0
    b = one_layer(tmp_path, latent(dense(72)), tweak=tweak)
    toks, z = check_all_positions(b)
    other = copy.deepcopy(b.w)
    other["l0.ls2"][...] = 0.0
    assert rel_err(O.forward(b.cfg, other, toks), z) > 0.05


def test_mixture_of_experts_alone(tmp_path):
    def tweak(w):
        w["l0.ls1"][...] = 0.0
    b = one_layer(tmp_path, gla(moe(experts=12, top=3, ff=20, shared=16, groups=(4, 2))), tweak=tweak)
    check_all_positions(b)
    check_all_positions(b, dtype="bfloat16", tol=BF16_TOL)


def test_router_keeps_to_the_best_groups_and_weighs_without_the_correction(tmp_path):
    """Corrections far below zero for two groups (their choice scores are negative: minus infinity, not zero, is what keeps
    an expert of a dropped group from being taken) and a large one for a single expert of another group, which wins its
    group a place although its experts' scores are small; the weights must not contain the correction."""
    def tweak(w):
        w["l0.ls1"][...] = 0.0
        w["l0.mlp.correction"][...] = np.array([-3.0, -3.0, -2.0, -2.0, 4.0, -5.0, 0.0, 0.0])
    b = one_layer(tmp_path, gla(moe(experts=8, top=4, ff=16, shared=0, groups=(4, 2))), tweak=tweak)
    toks = tokens_for(b, 40, 4)
    h = O.dyt(O.embed(b.cfg, b.w, toks), b.w, "l0.norm2")
    picked, weights = O.route(h, b.cfg["layers"][0]["mlp"], b.w, "l0.mlp.")
    # the kept groups are {4, 5} and {6, 7}; expert 5 is taken last, with a choice score far below zero, and an expert of a
    # dropped group whose score counted as zero would have beaten it
    assert (np.sort(picked, axis=1) == np.array([4, 5, 6, 7])).all() and (picked[:, 0] == 4).all() and (picked[:, 3] == 5).all()
    assert np.allclose(weights.sum(-1), 1.0) and (weights > 0).all()
    check_all_positions(b, n=40)


# ---- prompts in portions, decoding, long decoding ------------------------------------------------------------------
@pytest.mark.parametrize("cuts", [[1], [2], [3, 5, 2, 7, 1, 16, 2], [40, 1], [64, 2, 2, 33]])
def test_portions_equal_the_whole_prompt(general, cuts):
    toks = tokens_for(general, 150, 7)
    z, _ = general.ref(toks)
    got = feed(general.engine(), "a", toks, cuts)
    assert rel_err(got, z) < F32_TOL
    assert max(rel_err(got[p], z[p]) for p in range(len(toks))) < 5 * F32_TOL


def test_prefill_equals_token_by_token_decoding(general):
    toks = tokens_for(general, 80, 5)
    e1, e2 = general.engine(), general.engine()
    whole = e1.step([("a", toks, list(range(80)))])
    single = feed(e2, "a", toks, [1])
    assert rel_err(single, whole) < F32_TOL
    st = O.Stepper(general.cfg, general.w)                    # the plain statement's own decoding through caches and states
    ref = np.concatenate([st.feed([t]) for t in toks], 0)
    assert rel_err(single, ref) < F32_TOL


def test_portions_bfloat16(general):
    toks = tokens_for(general, 120, 8)
    z, _ = general.ref(toks)
    got = feed(general.engine("bfloat16"), "a", toks, [50, 2, 1, 1, 1, 9, 1])
    assert rel_err(got, z) < BF16_TOL


def test_long_decoding(general):
    toks = tokens_for(general, 330, 9)
    z, _ = general.ref(toks)
    got = feed(general.engine(), "a", toks, [30, 1])
    assert rel_err(got[30:], z[30:]) < F32_TOL
    assert rel_err(got[-1], z[-1]) < 5 * F32_TOL


# ---- batches of unequal requests, slots and blocks used again ------------------------------------------------------
def test_mixed_batches_equal_each_request_alone(general):
    rng = np.random.default_rng(11)
    lens = {"a": 140, "b": 37, "c": 75, "d": 9, "e": 58, "f": 101}
    toks = {k: tokens_for(general, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    e = general.engine(max_tokens=448, max_seqs=4)      # not enough for all six at once: blocks and slots come back
    total_blocks = e.free_blocks()
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    waiting, live, slots_seen = list(lens), [], {}
    while waiting or live:
        while waiting and len(live) < 4 and sum(-(-lens[k] // 64) * 64 for k in live + [waiting[0]]) <= 448:
            live.append(waiting.pop(0))
        entries = []
        for k in list(live):
            if rng.random() < 0.25 and len(live) > 1:
                continue                                     # left out of this step, goes on later
            n = int(min(rng.choice([1, 1, 2, 3, 17, 64]), lens[k] - fed[k]))
            entries.append((k, toks[k][fed[k]:fed[k] + n], list(range(n))))
        if not entries:
            continue
        out = e.step(entries)
        at = 0
        for k, t, w in entries:
            got[k].append(out[at:at + len(w)])
            at += len(w)
            fed[k] += len(t)
            slots_seen.setdefault(e.slot(k), []).append(k)
            if fed[k] == lens[k]:
                e.finish(k)
                live.remove(k)
    assert e.free_blocks() == total_blocks
    assert any(len(set(v)) > 1 for v in slots_seen.values()), "no slot was used by two requests"
    for k in lens:
        z, _ = general.ref(toks[k])
        assert rel_err(np.concatenate(got[k], 0), z) < F32_TOL, k


def test_a_reused_slot_starts_from_zero_state_and_reused_blocks_hold_nothing(general):
    e = general.engine(max_tokens=128, max_seqs=1)
    a, b = tokens_for(general, 100, 31), tokens_for(general, 90, 32)
    feed(e, "first", a, [64, 1], want_all=False)
    e.finish("first")
    got = feed(e, "second", b, [7, 64, 1])
    assert e.slot("second") == 0
    assert rel_err(got, general.ref(b)[0]) < F32_TOL


def test_pool_exhaustion_and_the_end_of_the_position_table_are_errors_not_faults(general, tmp_path):
    serving = load_pkg("serving")
    e = general.engine(max_tokens=64, max_seqs=2)
    e.step([("a", tokens_for(general, 60, 1), [])])
    with pytest.raises(serving.ServingError):
        e.step([("b", tokens_for(general, 30, 2), [])])
    short = Built(tmp_path, model([gla(None)], width=32, max_positions=20), 3)
    e = short.engine(max_tokens=64)
    e.step([("a", tokens_for(short, 20, 1), [19])])
    with pytest.raises(serving.ServingError) as err:
        e.step([("a", [1], [0])])
    assert "position" in str(err.value)


# ---- sharp attention: far keys, borders of the block table --------------------------------------------------------------
def sharp_model(tmp, vocab=1024, rot_dim=4):
    """The query latent reads the upper half of the layer's input, the key/value latent the lower half, through the same
    matrix; the query expansion is the key expansion; the score scale is large and the position vectors are small.  The
    upper half of the embedding of the QUERY probe is the lower half of the embedding of the KEY probe, so the query probe
    puts nearly all its weight on the key probe wherever that is -- a different token with a different value, so losing
    that key (or seeing another in its place) moves the output at the query a lot."""
    cfg = model([latent(None, heads=2, dim=16, rot_dim=rot_dim, vdim=16, q_rank=24, kv_rank=24, scale=2.5),
                 latent(moe(), heads=2)], width=64, vocab=vocab)

    def tweak(w):
        w["pos"][...] *= 0.02
        w["embed"][vocab - 2, 32:] = w["embed"][vocab - 1, :32]
        for n in ("l0.norm1", "l0.norm1.b"):
            w[n][32:] = w[n][:32]
        w["l0.mix.dkv"][:24, 32:] = 0.0
        w["l0.mix.dq"][:, :32] = 0.0
        w["l0.mix.dq"][:, 32:] = w["l0.mix.dkv"][:24, :32]
        w["l0.mix.dq.norm"][...] = w["l0.mix.dkv.norm"]
        uq = w["l0.mix.uq"].reshape(2, 16 + rot_dim, 24)
        uq[:, :16] = w["l0.mix.uk"].reshape(2, 16, 24)
        uq[:, 16:] *= 0.05
        w["l0.ls1"][...] = 1.5
    return Built(tmp, cfg, 12, tweak)


def distinct_tokens(n, vocab, seed):
    return np.random.default_rng(seed).permutation(vocab - 2)[:n].tolist()   # the last two tokens are the probes


def with_probes(b, n, key_pos, query_pos, seed):
    """distinct tokens with the key probe and the query probe in place; and the same without the key probe"""
    toks = distinct_tokens(n + 1, b.cfg["vocab"], seed)
    spare = toks.pop()
    toks[key_pos], toks[query_pos] = b.cfg["vocab"] - 1, b.cfg["vocab"] - 2
    other = list(toks)
    other[key_pos] = spare
    return toks, other


@pytest.mark.parametrize("key_pos,query_pos", [(0, 1), (0, 149), (63, 64), (64, 65), (63, 127), (64, 128), (127, 128), (1, 63)])
def test_keys_at_the_borders_of_the_block_table(tmp_path, key_pos, query_pos):
    b = sharp_model(tmp_path)
    toks, other = with_probes(b, 150, key_pos, query_pos, key_pos * 7 + query_pos)
    z, _ = b.ref(toks)
    assert rel_err(b.ref(other)[0][query_pos], z[query_pos]) > 0.1       # the probe's key does carry the weight
    for cuts in ([150], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 1]):
        cuts = [c for c in cuts if c > 0] or [1]
        got = feed(b.engine(), "a", toks, cuts)
        assert rel_err(got[query_pos], z[query_pos]) < 10 * F32_TOL, cuts
        assert rel_err(got, z) < F32_TOL, cuts


@pytest.mark.parametrize("dtype,decoded", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_one_far_key_among_hundreds(tmp_path, dtype, decoded):
    b = sharp_model(tmp_path)
    toks, other = with_probes(b, 700, 3, 690, 5)
    z, _ = b.ref(toks)
    moved = rel_err(b.ref(other)[0][690], z[690])
    assert moved > 0.1
    got = feed(b.engine(dtype), "a", toks, [670, 1] if decoded else [300, 400])
    if dtype == "float32":
        assert rel_err(got[690], z[690]) < 10 * F32_TOL
        assert rel_err(got, z) < F32_TOL
    else:
        assert rel_err(got[690], z[690]) < min(BF16_TOL, moved / 2)


@pytest.mark.parametrize("cuts", [[300], [150, 86, 2, 1], [64, 1]])
def test_wide_latent_bfloat16_every_position(tmp_path, cuts):
    """A cached row of more than 128 channels takes, in bfloat16, the attention form in which a block of warps shares the
    query rows and the output (whole prompts: 64 pairs per block; single tokens: 16; few rows at a long context: cut along
    the keys and merged).  Peaked scores and a check of EVERY position by itself: a key too many or too few, or a tile of
    keys lost, is an error of tens of percent there."""
    cfg = model([latent(None, heads=4, dim=24, rot_dim=32, vdim=16, q_rank=48, kv_rank=160, scale=0.5)], width=64, vocab=200)
    b = Built(tmp_path, cfg, 41)
    n = 300
    toks = tokens_for(b, n, 3)
    _, layers = b.ref(toks)
    base = O.embed(b.cfg, b.w, toks)
    mix = layers[0] - base
    e = b.engine("bfloat16")
    at, got, i = 0, [], 0
    while at < n:
        c = min(cuts[min(i, len(cuts) - 1)], n - at)
        got.append(e.step([("a", toks[at:at + c], [])], taps=True)[1][0])
        at += c
        i += 1
    got = np.concatenate(got, 0) - base
    worst = max(rel_err(got[p], mix[p]) for p in range(n))
    assert worst < 6e-2, worst
    assert rel_err(got, mix) < 2e-2


# ---- other sizes: values that are often equal, or 1 ------------------------------------------------------------------
@pytest.mark.parametrize("case", ["single", "wide_heads", "everything_small", "loop_all_twice", "loop_nothing", "odd_sizes", "no_loop_key"])
def test_other_sizes(tmp_path, case):
    width, loop, rank = 32, None, 6
    if case == "single":
        layers = [latent(moe(experts=2, top=1, ff=8, shared=8, groups=(1, 1)), heads=1, dim=8, rot_dim=2, vdim=40, q_rank=8, kv_rank=8),
                  gla(moe(experts=4, top=4, ff=16, shared=0, groups=(4, 4)), heads=1, dim=40, vdim=8, tau=1.0)]
        width, rank = 24, 1
    elif case == "wide_heads":
        layers = [gla(dense(40), heads=1, dim=72, vdim=70, tau=16.0), latent(None, heads=2, dim=72, rot_dim=24, vdim=72, q_rank=16, kv_rank=104),
                  gla(None, heads=2, dim=136, vdim=6)]
        width = 40
    elif case == "everything_small":
        layers = [latent(moe(experts=1, top=1, ff=1, shared=1, groups=None), heads=1, dim=1, rot_dim=2, vdim=1, q_rank=1, kv_rank=1),
                  gla(dense(1), heads=1, dim=1, vdim=1)]
        width, rank = 8, 2
    elif case == "loop_all_twice":
        layers, loop = [gla(dense()), latent(moe())], (0, 2, 2)
    elif case == "loop_nothing":
        layers, loop = [gla(dense()), latent(moe()), gla(None)], (1, 1, 5)
    elif case == "odd_sizes":
        layers = [latent(moe(experts=9, top=2, ff=11, shared=7, groups=(3, 1)), heads=3, dim=7, rot_dim=6, vdim=5, q_rank=13, kv_rank=19, rot_dims=2),
                  gla(moe(experts=5, top=5, ff=9, shared=3, groups=(5, 5)), heads=3, dim=11, vdim=7, tau=2.5)]
        width, loop, rank = 27, (0, 1, 3), 3
    else:
        layers = [latent(dense(24)), gla(None)]
    b = Built(tmp_path, model(layers, width=width, vocab=61, loop=loop), 5, gla_rank=rank)
    toks = tokens_for(b, 75, 2)
    z, layers_ref = b.ref(toks)
    e = b.engine()
    logits, taps = e.step([("a", toks, list(range(75)))], taps=True)
    for i in range(len(layers_ref)):
        assert rel_err(taps[i], layers_ref[i]) < F32_TOL, f"layer run {i}"
    assert rel_err(logits, z) < F32_TOL
    assert rel_err(feed(b.engine(), "a", toks, [9, 2, 1]), z) < F32_TOL
    assert rel_err(feed(b.engine("bfloat16"), "a", toks, [40, 1]), z) < 2 * BF16_TOL


# ---- generation through the scheduler ---------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler(general):
    prompts = [tokens_for(general, n, 40 + n) for n in (5, 23, 70, 12, 3, 41)]
    new = [6, 9, 4, 12, 8, 5]
    e = general.engine(max_tokens=384, max_seqs=3)      # fewer slots than requests
    got = e.generate(prompts, new, temperature=0.0, portion=32)
    assert e.free_blocks() > 0 and e.steps_run() > max(new)
    for p, n, g in zip(prompts, new, got):
        assert len(g) == n
        st = O.Stepper(general.cfg, general.w)
        z = st.feed(p)[-1]
        for tok in g:
            best = int(np.argmax(z))
            if tok != best:                                # only a near tie may differ
                assert z[best] - z[tok] < 1e-3 * max(1.0, float(np.abs(z).max()))
            z = st.feed([tok])[-1]


def test_sampled_generation_is_reproducible_and_independent_of_the_batch(general):
    prompts = [tokens_for(general, n, 60 + n) for n in (9, 30)]
    a = general.engine(max_seqs=2).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7)
    b = general.engine(max_seqs=1).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7, portion=4)
    assert a == b


def test_the_app_serves_a_model_folder(general, tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    app = os.path.join(root, "build", "apps", "llama")
    if not os.path.exists(app):
        pytest.skip("the app is not built")
    prompts = [tokens_for(general, n, 80 + n) for n in (4, 19, 33)]
    (tmp_path / "in.txt").write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([app, general.folder, "-m", "test", "-f", str(tmp_path / "in.txt"), "-o", str(tmp_path / "out.txt"), "-n", "7", "-b", "2",
                        "-d", "f32", "-j", "16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in line.split()] for line in (tmp_path / "out.txt").read_text().splitlines()]
    want = general.engine(max_seqs=2).generate(prompts, [7, 7, 7], temperature=0.0, portion=16)
    assert got == want


def test_the_trace_replayer_answers_every_step(general, tmp_path):
    """bin/trace_run on a model folder: steps in, logits files out, requests ended and their slot used again"""
    import json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "build", "apps", "trace_run")
    if not os.path.exists(exe):
        pytest.skip("the program is not built")
    a, b = tokens_for(general, 70, 1), tokens_for(general, 20, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[64:], "want": [5]}, {"id": "b", "tokens": b[:18], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b[18:], "want": [0, 1]}], "end": ["b"]}]
    out = tmp_path / "out"
    out.mkdir()
    r = subprocess.run([exe, "--model", general.folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128", "--max-seqs", "2"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    za, zb = general.ref(a)[0], general.ref(b)[0]
    V = general.cfg["vocab"]
    assert rel_err(np.fromfile(out / "0.f32", np.float32).reshape(-1, V), za[[0, 63]]) < F32_TOL
    assert rel_err(np.fromfile(out / "1.f32", np.float32).reshape(-1, V), za[[69]]) < F32_TOL
    assert rel_err(np.fromfile(out / "2.f32", np.float32).reshape(-1, V), zb[[18, 19]]) < F32_TOL
