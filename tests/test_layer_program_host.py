"""Host-side pieces of the layer-program path that need no GPU: exported symbols, the architecture registry and its
error texts, and self-checks of the plain statement of Timerax that the GPU tests compare against."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import timerax_oracle as O
from pkgload import load_pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "hip_llama.cpp_b200", "lib")
built = pytest.mark.skipif(not os.path.exists(os.path.join(LIB, "libthablas.so")), reason="libraries are not built")


def _declared(header, pattern):
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", header)).read(), flags=re.S)
    return sorted(set(re.findall(pattern, text)))


@built
def test_every_declared_entry_point_is_exported():
    cuda = C.CDLL(os.path.join(LIB, "libtha_b200.so"))
    for name in _declared("tha_hybrid.h", r"\b(tha_hyb_[a-z0-9_]+)\s*\("):
        assert hasattr(cuda, name), name
    host = C.CDLL(os.path.join(LIB, "libthablas.so"))
    names = _declared("tha_engine.h", r"\b(thaEngine[A-Za-z]+)\s*\(")
    assert "thaEngineStep" in names and "thaEngineGenerate" in names
    for name in names:
        assert hasattr(host, name), name


@built
def test_registry_names_what_it_knows(tmp_path):
    serving = load_pkg("serving")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "Nope" in str(e.value) and "Timerax" in str(e.value) and "llama2" in str(e.value)


@built
def test_a_config_without_a_needed_key_is_refused_by_name(tmp_path):
    serving = load_pkg("serving")
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Timerax", "vocab": 10, "norm": {"eps": 1e-5}, "layers": []}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "width" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Timerax", "vocab": 10, "width": 8, "norm": {"eps": 1e-5},
                                                       "layers": [{"type": "spiral", "mixer": {}}]}))
    with pytest.raises(serving.ServingError) as e:
        serving.ServingEngine(str(tmp_path), "float32", 64, 1)
    assert "spiral" in str(e.value)


def test_tensor_shapes_cover_a_config():
    serving = load_pkg("serving")
    cfg = {"architecture": "Timerax", "width": 16, "vocab": 20, "norm": {"eps": 1e-5}, "layers": [
        {"type": "channel_delta", "mixer": {"conv": 3, "dim": 4, "heads": 2, "kv_heads": 1, "vdim": 6, "rank": 5}, "mlp": None}]}
    t = serving.random_timerax_tensors(cfg, 0)
    assert t["l0.mix.q.conv"].shape == (4, 3) and t["l0.mix.a2"].shape == (8, 5) and t["l0.mix.norm"].shape == (6,)
    assert "l0.mlp.router" not in t


# ---- the plain statement checks itself: a recurrence cut in two equals the whole -------------------------------------
def test_plain_matrix_memory_carries_its_state():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((9, 5)), rng.standard_normal((9, 5)), rng.standard_normal((9, 3))
    ig, fg = rng.standard_normal(9), -np.abs(rng.standard_normal(9))
    whole, _ = O.matrix_memory(q, k, v, ig, fg)
    a, st = O.matrix_memory(q[:4], k[:4], v[:4], ig[:4], fg[:4])
    b, _ = O.matrix_memory(q[4:], k[4:], v[4:], ig[4:], fg[4:], st)
    assert np.allclose(np.concatenate([a, b]), whole, atol=1e-12)


def test_plain_delta_rule_carries_its_state_and_reads_its_own_write():
    rng = np.random.default_rng(1)
    q, k, v = rng.standard_normal((7, 4)), rng.standard_normal((7, 4)), rng.standard_normal((7, 2))
    beta, g = rng.random(7), rng.random((7, 4))
    whole, _ = O.delta_rule(q, k, v, beta, g)
    a, S = O.delta_rule(q[:3], k[:3], v[:3], beta[:3], g[:3])
    b, _ = O.delta_rule(q[3:], k[3:], v[3:], beta[3:], g[3:], S)
    assert np.allclose(np.concatenate([a, b]), whole, atol=1e-12)
    # one token from the zero state: S = k u^T with u = beta v, read out with q
    assert np.allclose(whole[0], beta[0] * v[0] * (k[0] @ q[0]))


def test_plain_convolution_and_rotation():
    x = np.arange(12.0).reshape(6, 2)
    taps = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])      # channel 0: the current token; channel 1: two tokens back
    y = O.causal_conv(x, taps)
    assert np.allclose(y[:, 0], x[:, 0]) and np.allclose(y[2:, 1], x[:-2, 1]) and np.allclose(y[:2, 1], 0.0)
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 32.0, "original": 8, "slow": 1.0}}
    cos, sin = O.rotary_tables(rot, [0, 3])
    mag = 0.1 * np.log(2.0) + 1.0
    assert np.allclose(cos[0], mag) and np.allclose(sin[0], 0.0) and np.allclose(cos[1] ** 2 + sin[1] ** 2, mag ** 2)
    v = np.random.default_rng(2).standard_normal((2, 1, 6))
    r = O.rotate_interleaved(v, cos, sin)
    assert np.allclose(r[..., 4:], v[..., 4:]) and np.allclose(r[0, 0, :4], v[0, 0, :4] * mag)


def test_plain_attention_sees_its_own_block_only():
    rng = np.random.default_rng(3)
    q, k, v = rng.standard_normal((10, 2, 4)), rng.standard_normal((10, 1, 4)), rng.standard_normal((10, 1, 3))
    o = O.chunked_attention(q, k, v, 0.5, 4)
    assert np.allclose(o[4], np.repeat(v[4], 2, 0)) and np.allclose(o[8], np.repeat(v[8], 2, 0))   # first of a block: itself only
    v2 = v.copy()
    v2[3] += 1.0                                                                                     # the last of block 0
    o2 = O.chunked_attention(q, k, v2, 0.5, 4)
    assert np.allclose(o2[4:], o[4:]) and not np.allclose(o2[3], o[3])
