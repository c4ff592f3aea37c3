// Numizen: config.json -> layer program.
// A decoder with learned position vectors and parallel blocks of two norms,
//     x <- x + s_mix * mixer(norm1 x) + s_ff * ff(norm2 x),
// where every norm over the width is a dynamic tanh (tanh(alpha x) w + b) and s_mix / s_ff are per-channel layer scales.
// Layer types:
//   "latent_attention"  causal softmax attention whose queries pass through a normed low-rank latent and whose keys and
//                       values are expanded per head from one cached normed latent, plus one rotated key part shared by
//                       the heads (interleaved rotary pairs); sigmoid output gate;
//   "gla"               gated linear attention with a decay per key channel from a low-rank projection,
//                       sigmoid(z)^(1/tau); per-head rms norm of the read-out, silu gate.
// Feed-forward: none, dense (gelu-tanh gated), or a mixture of squared-relu experts chosen by corrected softmax scores
// inside the best groups of neighbouring experts, plus a shared expert scaled by a per-token sigmoid.
// "loop" runs a segment of the layer list several times with the same weights; every run has its own cache or state.
// Every size and constant comes from the config; constants the design fixes live with the mechanisms.
#include <math.h>

#include "layer_model.hpp"

static void numizen_mixer(const JsonValue& L, const std::string& pre, LayerSpec* out) {
  LayerSpec& ls = *out;
  const std::string type = L.at("type").string();
  const JsonValue& m = L.at("mixer");
  const std::string p = pre + "mix.";
  if (type == "latent_attention") {
    ls.mixer = THA_MIX_LATENT;
    LatentSpec& a = ls.latent;
    a.heads = m.at("heads").integer();
    a.dim = m.at("dim").integer();
    a.rot_dim = m.at("rot_dim").integer();
    a.vdim = m.at("vdim").integer();
    a.q_rank = m.at("q_rank").integer();
    a.kv_rank = m.at("kv_rank").integer();
    a.scale = (float)m.number_or("scale", 1.0 / sqrt((double)(a.dim + a.rot_dim)));
    if (m.has("rot")) {
      const JsonValue& r = m.at("rot");
      a.rotary = true;
      a.rot.dims = r.at("dims").integer();
      a.rot.base = r.at("base").number();
    }
    a.dq = p + "dq"; a.dq_norm = p + "dq.norm"; a.uq = p + "uq";
    a.dkv = p + "dkv"; a.dkv_norm = p + "dkv.norm"; a.uk = p + "uk"; a.uv = p + "uv";
    a.g = p + "g"; a.o = p + "o";
  } else if (type == "gla") {
    ls.mixer = THA_MIX_GLA;
    GlaSpec& g = ls.gla;
    g.heads = m.at("heads").integer();
    g.dim = m.at("dim").integer();
    g.vdim = m.at("vdim").integer();
    g.tau = (float)m.at("tau").number();
    g.q = p + "q"; g.k = p + "k"; g.v = p + "v"; g.g = p + "g"; g.o = p + "o"; g.norm = p + "norm";
    g.a1 = p + "a1"; g.a2 = p + "a2"; g.a2_b = p + "a2.b";
  } else {
    throw std::runtime_error("config: unknown layer type '" + type + "'");
  }
}

static void numizen_ff(const JsonValue& L, const std::string& pre, LayerSpec* out) {
  LayerSpec& ls = *out;
  if (!L.has("mlp")) return;   // absent or null: the layer has no feed-forward
  const JsonValue& f = L.at("mlp");
  const std::string kind = f.at("kind").string();
  const std::string p = pre + "mlp.";
  ls.has_ff = true;
  if (kind == "dense") {
    ls.ff_kind = THA_FF_DENSE;
    ls.dense.ff = f.at("ff").integer();
    ls.dense.act = THA_ACT_GELU_TANH_GLU;
    ls.dense.gate = p + "gate"; ls.dense.up = p + "up"; ls.dense.down = p + "down";
  } else if (kind == "moe") {
    ls.ff_kind = THA_FF_MOE;
    MoeSpec& e = ls.moe;
    const JsonValue& r = f.at("router");
    e.experts = r.at("experts").integer();
    e.top = r.at("top").integer();
    e.ff = f.at("expert").at("ff").integer();
    e.act = THA_ACT_RELU2;
    e.route = THA_ROUTE_SOFTMAX_GROUPS;
    e.router = p + "router";
    e.correction = p + "correction";
    e.prefix = p;
    if (r.has("groups")) {
      e.groups = r.at("groups").at("count").integer();
      e.keep_groups = r.at("groups").at("keep").integer();
    }
    if (f.has("shared")) {
      e.shared_ff = f.at("shared").at("ff").integer();
      e.s_up = p + "shared.up"; e.s_down = p + "shared.down"; e.s_scale = p + "shared.sg";
    }
  } else {
    throw std::runtime_error("config: unknown feed-forward kind '" + kind + "'");
  }
}

static void numizen_translate(const JsonValue& c, LayerProgramSpec* out) {
  LayerProgramSpec& s = *out;
  s.width = c.at("width").integer();
  s.vocab = c.at("vocab").integer();
  s.eps = (float)c.at("norm").at("eps").number();
  s.norm_kind = THA_NORM_DYT;
  s.embed = "embed";
  s.pos_embed = "pos";
  s.max_positions = c.at("max_positions").integer();
  s.final_norm = "final.norm";
  s.head = "head";
  const JsonValue& layers = c.at("layers");
  if (layers.kind != JsonValue::Array) throw std::runtime_error("config: 'layers' must be a list");
  const int n = (int)layers.arr.size();
  // the order of execution: the looped segment repeated in place
  int start = 0, stop = 0, times = 1;
  if (c.has("loop")) {
    const JsonValue& lp = c.at("loop");
    start = lp.at("start").integer();
    stop = lp.at("stop").integer();
    times = lp.at("times").integer();
    if (start < 0 || stop < start || stop > n || times < 0) throw std::runtime_error("config: 'loop' does not fit the layer list");
  }
  std::vector<int> first_run(n, -1);
  auto run = [&](int i) {
    LayerSpec ls;
    const JsonValue& L = layers.arr[i];
    const std::string pre = "l" + std::to_string(i) + ".";
    ls.norm1 = pre + "norm1";
    ls.norm2 = pre + "norm2";
    ls.scale_mix = pre + "ls1";
    ls.scale_ff = pre + "ls2";
    numizen_mixer(L, pre, &ls);
    numizen_ff(L, pre, &ls);
    if (first_run[i] >= 0) ls.same_weights_as = first_run[i];
    else first_run[i] = (int)s.layers.size();
    s.layers.push_back(ls);
  };
  for (int i = 0; i < start; i++) run(i);
  for (int t = 0; t < times; t++)
    for (int i = start; i < stop; i++) run(i);
  for (int i = stop; i < n; i++) run(i);
}

void register_numizen() { register_architecture({"Numizen", ModelFamily::LayerProgram, numizen_translate}); }
