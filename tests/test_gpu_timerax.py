"""Timerax through the serving path (ServingEngine -> SequenceEngine -> tha_hyb_step) against the plain float64
statement of the design in tests/timerax_oracle.py.

Every test builds its own small configuration with random weights.  float32 runs are compared tightly (they differ from
float64 by rounding only), bfloat16 runs loosely.  Where random weights would hide a fault (a key at the edge of a block
of positions, one far key among hundreds) the weights are made sharp: keys equal queries, a large score scale and only
a few rotated dimensions, so that a query puts nearly all its weight on the earlier occurrence of its own token.
"""
import copy

import numpy as np
import pytest

import timerax_oracle as O
from pkgload import load_pkg

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 6e-2


def rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / (np.sqrt((want ** 2).mean()) + 1e-12))


def moe_cfg(experts=6, top=2, ff=40, shared=24):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": 2.0}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": 1.25}
    return m


def parallel_cfg(mlp, heads=4, kv_heads=2, dim=24, vdim=16, chunk=40, rot_dims=16, scale=0.3, mheads=3, mdim=16, mvdim=24, yarn=True):
    rot = {"base": 10000.0, "dims": rot_dims}
    if yarn:
        rot["scaling"] = {"factor": 4.0, "fast": 32.0, "original": 64, "slow": 1.0}
    left = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "mask": {"size": chunk}, "rot": rot, "scale": scale}
    right = {"dim": mdim, "heads": mheads, "vdim": mvdim, "gate_cap": 10.0}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def delta_cfg(mlp, heads=4, kv_heads=2, dim=16, vdim=24, conv=3, rank=12):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "rank": rank},
            "mlp": mlp}


def model_cfg(layers, width=80, vocab=130, softcap=20.0):
    return {"architecture": "Timerax", "layers": layers, "logit_softcap": softcap, "norm": {"eps": 1e-5}, "vocab": vocab, "width": width}


class Built:
    """A model folder, its oracle view, and engines on demand."""

    def __init__(self, tmp, cfg, seed=0, tweak=None):
        self.serving = load_pkg("serving")
        self.cfg = cfg
        t = self.serving.random_timerax_tensors(cfg, seed)
        if tweak:
            tweak(t)
        self.folder = str(tmp)
        self.serving.save_model_folder(self.folder, cfg, t)
        self.ocfg, self.w = O.load_model(self.folder)
        self._ref = {}

    def engine(self, dtype="float32", max_tokens=1024, max_seqs=4):
        return self.serving.ServingEngine(self.folder, dtype, max_tokens, max_seqs)

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            layers = []
            z = O.forward(self.ocfg, self.w, list(tokens), layers)
            self._ref[key] = (z, np.stack(layers))
        return self._ref[key]


def general_layers():
    return [delta_cfg(moe_cfg()), parallel_cfg(moe_cfg(experts=5, top=1, ff=24, shared=0)), parallel_cfg(None, chunk=33, yarn=False),
            delta_cfg(None, heads=2, kv_heads=2, dim=8, vdim=40, conv=2, rank=5), parallel_cfg(moe_cfg(experts=3, top=3))]


@pytest.fixture(scope="module")
def general(tmp_path_factory):
    return Built(tmp_path_factory.mktemp("general"), model_cfg(general_layers()), seed=1)


def tokens_for(built, n, seed):
    return np.random.default_rng(seed).integers(0, built.cfg["vocab"], n).tolist()


# ---- whole prompts, every layer ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompt_every_layer(general, dtype, tol):
    toks = tokens_for(general, 97, 3)
    z, layers = general.ref(toks)
    e = general.engine(dtype)
    logits, taps = e.step([("a", toks, list(range(len(toks))))], taps=True)
    for i in range(len(layers)):
        assert rel_err(taps[i], layers[i]) < tol, f"residual stream after layer {i}"
    assert rel_err(logits, z) < tol
    # the first tokens of a sequence, one by one
    for p in range(4):
        assert rel_err(logits[p], z[p]) < tol, f"position {p}"


# ---- each mechanism alone: one layer, the other parts switched off through their weights ----------------------------
def _zero(names):
    def f(t):
        for n in names:
            t[n][...] = 0.0
    return f


def test_attention_side_alone(tmp_path):
    cfg = model_cfg([parallel_cfg(None, heads=6, kv_heads=2, dim=20, vdim=12, chunk=17, rot_dims=10)], width=48, softcap=0)
    b = Built(tmp_path, cfg, 2, _zero(["l0.mix.right.out"]))
    toks = tokens_for(b, 60, 1)
    h = O.layer_norm_weight(b.w["embed"][toks], b.w["l0.norm1"], 1e-5)
    left = O.attention_side(h, b.w, "l0.mix.left.", cfg["layers"][0]["mixer"]["left"], 1e-5)
    want = b.w["embed"][toks] + 0.5 * O.unit_rms(left, 1e-5) * b.w["l0.mix.left.out"]
    _, taps = b.engine().step([("a", toks, [])], taps=True)
    assert rel_err(taps[0], want) < F32_TOL


def test_matrix_memory_side_alone(tmp_path):
    cfg = model_cfg([parallel_cfg(None, mheads=2, mdim=12, mvdim=300)], width=48, softcap=0)   # more value channels than threads
    b = Built(tmp_path, cfg, 3, _zero(["l0.mix.left.out"]))
    toks = tokens_for(b, 50, 2)
    h = O.layer_norm_weight(b.w["embed"][toks], b.w["l0.norm1"], 1e-5)
    right = O.memory_side(h, b.w, "l0.mix.right.", cfg["layers"][0]["mixer"]["right"], 1e-5)
    want = b.w["embed"][toks] + 0.5 * O.unit_rms(right, 1e-5) * b.w["l0.mix.right.out"]
    _, taps = b.engine().step([("a", toks, [])], taps=True)
    assert rel_err(taps[0], want) < F32_TOL


def test_matrix_memory_small_input_gates_keep_the_floor(tmp_path):
    """With strongly negative input gates |n.q| stays below exp(-m) for many tokens: the running maximum starts at 0."""
    def tweak(t):
        t["l0.mix.left.out"][...] = 0.0
        t["l0.mix.right.i.b"][...] = -8.0
    cfg = model_cfg([parallel_cfg(None)], width=48, softcap=0)
    b = Built(tmp_path, cfg, 4, tweak)
    toks = tokens_for(b, 30, 5)
    _, layers = b.ref(toks)
    _, taps = b.engine().step([("a", toks, [])], taps=True)
    assert rel_err(taps[0], layers[0]) < F32_TOL


def test_delta_rule_alone(tmp_path):
    cfg = model_cfg([delta_cfg(None, heads=6, kv_heads=3, dim=12, vdim=20, conv=5, rank=7)], width=48, softcap=0)
    b = Built(tmp_path, cfg, 5)
    toks = tokens_for(b, 70, 3)
    h = O.layer_norm_weight(b.w["embed"][toks], b.w["l0.norm1"], 1e-5)
    want = b.w["embed"][toks] + O.delta_mixer(h, b.w, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5)
    _, taps = b.engine().step([("a", toks, [])], taps=True)
    assert rel_err(taps[0], want) < F32_TOL


def test_mixture_of_experts_alone(tmp_path):
    cfg = model_cfg([parallel_cfg(moe_cfg(experts=9, top=4, ff=36, shared=20))], width=48, softcap=0)
    b = Built(tmp_path, cfg, 6, _zero(["l0.mix.left.out", "l0.mix.right.out"]))
    toks = tokens_for(b, 90, 4)
    h = O.layer_norm_weight(b.w["embed"][toks], b.w["l0.norm1"], 1e-5)
    want = b.w["embed"][toks] + O.moe(h, b.w, "l0.mlp.", cfg["layers"][0]["mlp"])
    _, taps = b.engine().step([("a", toks, [])], taps=True)
    assert rel_err(taps[0], want) < F32_TOL


def test_router_picks_and_weights():
    z = np.array([[0.1, 2.0, -1.0, 2.0, 0.5]])
    idx, wt = O.route(z, 3)
    assert idx.tolist() == [[1, 3, 4]]     # equal logits: the lower index first
    assert abs(wt.sum() - 1.0) < 1e-12 and wt[0, 0] == wt[0, 1]


# ---- one sequence cut in different ways ----------------------------------------------------------------------------
def feed(engine, rid, toks, cuts, want_all=True):
    """Feed toks in portions of the given sizes (the last size repeats); returns logits of every position."""
    out, at, k = [], 0, 0
    while at < len(toks):
        n = min(cuts[min(k, len(cuts) - 1)], len(toks) - at)
        out.append(engine.step([(rid, toks[at:at + n], list(range(n)) if want_all else [])]))
        at += n
        k += 1
    return np.concatenate(out, 0)


@pytest.mark.parametrize("cuts", [[1], [2], [3, 5, 2, 7, 1, 16, 2], [40, 1], [64, 2, 2, 33]])
def test_portions_equal_the_whole_prompt(general, cuts):
    toks = tokens_for(general, 150, 7)
    z, _ = general.ref(toks)
    e = general.engine()
    got = feed(e, "a", toks, cuts)
    assert rel_err(got, z) < F32_TOL
    worst = max(rel_err(got[p], z[p]) for p in range(len(toks)))
    assert worst < 5 * F32_TOL


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


def test_a_reused_slot_starts_from_zero_state(general):
    e = general.engine(max_tokens=128, max_seqs=1)
    a, b = tokens_for(general, 100, 31), tokens_for(general, 90, 32)
    feed(e, "first", a, [64, 1], want_all=False)
    e.finish("first")
    got = feed(e, "second", b, [7, 64, 1])
    assert e.slot("second") == 0
    assert rel_err(got, general.ref(b)[0]) < F32_TOL


def test_pool_exhaustion_is_an_error_not_a_fault(general):
    e = general.engine(max_tokens=64, max_seqs=2)
    serving = load_pkg("serving")
    e.step([("a", tokens_for(general, 60, 1), [])])
    with pytest.raises(serving.ServingError):
        e.step([("b", tokens_for(general, 30, 2), [])])


# ---- sharp attention: edges of the blocks of positions, block-table borders, far keys -------------------------------
def sharp_model(tmp, chunk, vocab=1024):
    cfg = model_cfg([parallel_cfg(None, heads=2, kv_heads=2, dim=16, vdim=16, chunk=chunk, rot_dims=2, scale=3.0, yarn=False),
                     parallel_cfg(moe_cfg(), chunk=chunk)], width=64, vocab=vocab, softcap=0)

    def tweak(t):
        t["l0.mix.left.k"][...] = t["l0.mix.left.q"]      # a query matches the key of its own token
        t["l0.mix.right.out"][...] *= 0.05                 # the attention side carries the layer
    return Built(tmp, cfg, 12, tweak)


def distinct_tokens(n, vocab, seed):
    return np.random.default_rng(seed).permutation(vocab - 1)[:n].tolist()   # token vocab-1 is kept for the probe


@pytest.mark.parametrize("key_pos,query_pos", [(48, 95), (47, 95), (48, 49), (95, 96), (96, 143), (15, 40), (16, 40), (63, 64), (64, 65)])
def test_keys_at_the_edges(tmp_path, key_pos, query_pos):
    """Blocks of 48 positions: a key is seen exactly when it lies in the query's block (48 | 95: first and last of one;
    47 | 95 and 95 | 96: neighbours across an edge); 15 / 16 / 63 / 64 also sit on borders of the block table."""
    b = sharp_model(tmp_path, 48)
    probe = b.cfg["vocab"] - 1
    toks = distinct_tokens(150, b.cfg["vocab"], key_pos * 7 + query_pos)
    toks[key_pos] = probe
    toks[query_pos] = probe
    z, layers = b.ref(toks)
    # the probe's key does carry the weight when visible: without it the output at the query moves a lot
    other = list(toks)
    other[key_pos] = distinct_tokens(151, b.cfg["vocab"], 1)[150]
    z2, _ = b.ref(other)
    if key_pos // 48 == query_pos // 48:
        assert rel_err(z2[query_pos], z[query_pos]) > 0.02
    for cuts in ([150], [query_pos, 1], [key_pos, 2, 1], [key_pos + 1, 1]):
        got = feed(b.engine(), "a", toks, cuts)
        assert rel_err(got[query_pos], z[query_pos]) < 10 * F32_TOL, cuts
        assert rel_err(got, z) < F32_TOL, cuts


@pytest.mark.parametrize("decoded", [False, True])
def test_one_far_key_among_hundreds(tmp_path, decoded):
    b = sharp_model(tmp_path, 512)
    probe = b.cfg["vocab"] - 1
    toks = distinct_tokens(500, b.cfg["vocab"], 5)
    toks[3] = probe
    toks[490] = probe
    z, _ = b.ref(toks)
    other = list(toks)
    other[3] = distinct_tokens(501, b.cfg["vocab"], 1)[500]
    assert rel_err(b.ref(other)[0][490], z[490]) > 0.02
    got = feed(b.engine(), "a", toks, [470, 1] if decoded else [200, 300])
    assert rel_err(got[490], z[490]) < 10 * F32_TOL
    assert rel_err(got, z) < F32_TOL


# ---- other sizes: values that are often equal, or 1 ------------------------------------------------------------------
@pytest.mark.parametrize("case", ["single_heads", "wide_heads", "everything_one", "no_rotation_all_keys", "odd_sizes"])
def test_other_sizes(tmp_path, case):
    if case == "single_heads":
        layers = [parallel_cfg(moe_cfg(experts=2, top=1, ff=8, shared=8), heads=1, kv_heads=1, dim=8, vdim=40, chunk=5, rot_dims=8, mheads=1, mdim=40, mvdim=8),
                  delta_cfg(moe_cfg(experts=4, top=4, ff=16, shared=0), heads=1, kv_heads=1, dim=40, vdim=8, conv=1, rank=3)]
        width = 24
    elif case == "wide_heads":
        layers = [delta_cfg(None, heads=8, kv_heads=1, dim=72, vdim=136, conv=4, rank=16),
                  parallel_cfg(moe_cfg(experts=33, top=5, ff=72, shared=136), heads=8, kv_heads=1, dim=136, vdim=72, chunk=64, rot_dims=70, mheads=1, mdim=136, mvdim=72)]
        width = 200
    elif case == "odd_sizes":     # nothing a multiple of 4 or 8: every vector path falls back to its scalar form
        layers = [parallel_cfg(moe_cfg(experts=7, top=3, ff=13, shared=21), heads=3, kv_heads=1, dim=10, vdim=7, chunk=7, rot_dims=6, mheads=2, mdim=7, mvdim=11),
                  delta_cfg(moe_cfg(experts=3, top=2, ff=9, shared=0), heads=3, kv_heads=1, dim=11, vdim=5, conv=2, rank=3)]
        width = 53
    elif case == "everything_one":
        layers = [parallel_cfg(moe_cfg(experts=1, top=1, ff=1, shared=1), heads=1, kv_heads=1, dim=2, vdim=1, chunk=1, rot_dims=2, mheads=1, mdim=1, mvdim=1),
                  delta_cfg(None, heads=1, kv_heads=1, dim=1, vdim=1, conv=1, rank=1)]
        width = 8
    else:
        layers = [parallel_cfg(None, chunk=40)]
        del layers[0]["mixer"]["left"]["mask"]
        del layers[0]["mixer"]["left"]["rot"]
        width = 40
    b = Built(tmp_path, model_cfg(layers, width=width, vocab=70), 21)
    toks = tokens_for(b, 75, 6)
    z, layers_ref = b.ref(toks)
    e = b.engine()
    logits, taps = e.step([("w", toks, list(range(len(toks))))], taps=True)
    for i in range(len(layers_ref)):
        assert rel_err(taps[i], layers_ref[i]) < F32_TOL, f"layer {i}"
    assert rel_err(logits, z) < F32_TOL
    assert rel_err(feed(e, "p", toks, [9, 2, 1]), z) < F32_TOL
    assert rel_err(feed(b.engine("bfloat16"), "q", toks, [31, 1]), z) < 2 * BF16_TOL


# ---- generation through the scheduler ----------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler(general):
    prompts = [tokens_for(general, n, 40 + n) for n in (5, 23, 70, 12, 3, 41)]
    new = [6, 9, 4, 12, 8, 5]
    e = general.engine(max_tokens=384, max_seqs=3)      # fewer slots than requests
    got = e.generate(prompts, new, temperature=0.0, portion=32)
    assert e.free_blocks() > 0 and e.steps_run() > max(new)
    for p, n, g in zip(prompts, new, got):
        assert len(g) == n
        seq = list(p)
        for tok in g:                                      # the oracle's greedy loop, recomputed from the start every token
            z = O.forward(general.ocfg, general.w, seq)[-1]
            best = int(np.argmax(z))
            if tok != best:                                # only a near tie may differ
                assert z[best] - z[tok] < 1e-3 * max(1.0, float(np.abs(z).max()))
            seq.append(tok)


def test_sampled_generation_is_reproducible_and_independent_of_the_batch(general):
    prompts = [tokens_for(general, n, 60 + n) for n in (9, 30)]
    a = general.engine(max_seqs=2).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7)
    b = general.engine(max_seqs=1).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=7, portion=4)
    assert a == b
    c = general.engine(max_seqs=2).generate(prompts, [10, 10], temperature=1.0, topp=0.9, seed=8)
    assert a != c


def test_shared_memory_form_of_the_scans(general, monkeypatch):
    """Heads of more than 256 key channels take the scans that keep the state in shared memory; the switch forces that
    form at the test's sizes."""
    monkeypatch.setenv("THA_HYB_SCAN", "shared")
    toks = tokens_for(general, 90, 13)
    z, _ = general.ref(toks)
    assert rel_err(feed(general.engine(), "a", toks, [33, 2, 1]), z) < F32_TOL


def test_plain_products_everywhere(general, monkeypatch):
    """bfloat16 without the tensor-core products (the form odd sizes fall back to)."""
    monkeypatch.setenv("THA_HYB_TC", "0")
    # the switch is read once per process: only meaningful when this test runs first; otherwise it repeats the default
    toks = tokens_for(general, 60, 14)
    z, _ = general.ref(toks)
    assert rel_err(feed(general.engine("bfloat16"), "a", toks, [60]), z) < BF16_TOL


def test_the_app_serves_a_model_folder(general, tmp_path):
    """build/apps/llama on a folder: the registry picks the design, requests are lines of token ids."""
    import os
    import subprocess
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


def test_prompt_sized_step_runs_the_experts_one_matmul_each(tmp_path, monkeypatch):
    """From 1024 rows a bfloat16 step may gather the rows into expert order and give each expert to the tensor-core matmul
    (it does when experts get many rows each; the switch lowers that bar to the test's size)."""
    monkeypatch.setenv("THA_HYB_EXPERT_ROWS", "100")
    cfg = model_cfg([parallel_cfg(moe_cfg(experts=5, top=2, ff=64, shared=64), heads=2, kv_heads=1, dim=32, vdim=32, chunk=128, rot_dims=32,
                                  mheads=2, mdim=32, mvdim=32),
                     delta_cfg(moe_cfg(experts=3, top=1, ff=72, shared=0), heads=2, kv_heads=1, dim=32, vdim=32)], width=64, vocab=90)
    b = Built(tmp_path, cfg, 31)
    toks = tokens_for(b, 1100, 9)
    z, _ = b.ref(toks)
    e = b.engine("bfloat16", max_tokens=1152)
    got = e.step([("a", toks, list(range(0, 1100, 7)))])
    assert rel_err(got, z[::7]) < BF16_TOL
    small = b.engine("bfloat16", max_tokens=1152)          # the same prompt in small steps: the grouped kernel
    got2 = feed(small, "a", toks, [500])[::7]
    assert rel_err(got2, z[::7]) < BF16_TOL
    assert rel_err(got2, got) < BF16_TOL / 2


@pytest.mark.parametrize("chunk,cuts", [(48, [150]), (48, [47, 2, 1]), (512, [380, 1]), (512, [33, 200, 1])])
def test_tensor_core_attention_bfloat16(tmp_path, chunk, cuts):
    """bfloat16 with heads of 64 / 32 channels takes the tensor-core form of the attention (64 pairs per block, weights
    and values in bf16).  Peaked scores (a few keys carry a query's weight) and a check of EVERY position by itself: the
    first positions of a block of positions see one, two, three keys, so a key too many or too few there is an error of
    tens of percent, and a skipped tile of keys shows at the positions whose heavy keys lie in it."""
    cfg = model_cfg([parallel_cfg(None, heads=4, kv_heads=2, dim=64, vdim=32, chunk=chunk, rot_dims=32, scale=0.5)], width=64, vocab=200,
                    softcap=0)
    b = Built(tmp_path, cfg, 41, _zero(["l0.mix.right.out"]))
    n = 150 if chunk == 48 else 400
    toks = tokens_for(b, n, chunk)
    _, layers = b.ref(toks)
    mix = layers[0] - b.w["embed"][toks]                 # the attention side alone (normed, halved)
    e = b.engine("bfloat16")
    at, got = 0, []
    for c in cuts + [cuts[-1]] * n:
        c = min(c, n - at)
        if c <= 0:
            break
        got.append(e.step([("a", toks[at:at + c], [])], taps=True)[1][0])
        at += c
    got = np.concatenate(got, 0) - b.w["embed"][toks]
    worst = max(rel_err(got[p], mix[p]) for p in range(n))
    assert worst < 6e-2, worst
    assert rel_err(got, mix) < 2e-2
