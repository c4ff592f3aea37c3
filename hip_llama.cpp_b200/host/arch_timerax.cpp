// Timerax: config.json -> layer program.
// A decoder of parallel blocks x <- x + mixer(norm(x)) + ff(norm(x)), one norm per layer.  Layer types:
//   "parallel"       chunk-masked softmax attention (YaRN-scaled interleaved rotary positions on part of each head, q and
//                    k divided by their root mean square) beside a matrix memory with soft-capped log gates; each side's
//                    output is normed over the width with its own weight and the two are averaged;
//   "channel_delta"  gated delta rule with a decay per head and key channel from a low-rank projection, short causal
//                    convolutions on q, k and v, low-rank output gate.
// Feed-forward: top-k mixture of experts with clamped gated units plus a shared expert.  Every size and constant comes
// from the config; the fixed ones (1.702 in the gated unit, the stabilisers of the norms) live with the mechanisms.
#include <stdio.h>

#include "layer_model.hpp"

static void timerax_translate(const JsonValue& c, LayerProgramSpec* out) {
  LayerProgramSpec& s = *out;
  s.width = c.at("width").integer();
  s.vocab = c.at("vocab").integer();
  s.eps = (float)c.at("norm").at("eps").number();
  s.logit_softcap = (float)c.number_or("logit_softcap", 0.0);
  s.embed = "embed";
  s.final_norm = "final.norm";
  s.head = "head";
  const JsonValue& layers = c.at("layers");
  if (layers.kind != JsonValue::Array) throw std::runtime_error("config: 'layers' must be a list");
  for (size_t i = 0; i < layers.arr.size(); i++) {
    const JsonValue& L = layers.arr[i];
    const std::string pre = "l" + std::to_string(i) + ".";
    const std::string type = L.at("type").string();
    const JsonValue& m = L.at("mixer");
    LayerSpec ls;
    ls.norm1 = pre + "norm1";
    if (type == "parallel") {
      ls.mixer = THA_MIX_PARALLEL;
      const JsonValue& a = m.at("left");
      const std::string lp = pre + "mix.left.";
      ls.attn.heads = a.at("heads").integer();
      ls.attn.kv_heads = a.at("kv_heads").integer();
      ls.attn.dim = a.at("dim").integer();
      ls.attn.vdim = a.at("vdim").integer();
      ls.attn.scale = (float)a.at("scale").number();
      ls.attn.chunk = a.has("mask") ? a.at("mask").at("size").integer() : 0;
      ls.attn.unit_rms = true;
      if (a.has("rot")) {
        const JsonValue& r = a.at("rot");
        ls.attn.rotary = true;
        ls.attn.rot.dims = r.at("dims").integer();
        ls.attn.rot.base = r.at("base").number();
        if (r.has("scaling")) {
          const JsonValue& y = r.at("scaling");
          ls.attn.rot.yarn = true;
          ls.attn.rot.factor = y.at("factor").number();
          ls.attn.rot.original = y.at("original").number();
          ls.attn.rot.fast = y.at("fast").number();
          ls.attn.rot.slow = y.at("slow").number();
        }
      }
      ls.attn.q = lp + "q"; ls.attn.k = lp + "k"; ls.attn.v = lp + "v"; ls.attn.o = lp + "o";
      const JsonValue& r = m.at("right");
      const std::string rp = pre + "mix.right.";
      ls.mem.heads = r.at("heads").integer();
      ls.mem.dim = r.at("dim").integer();
      ls.mem.vdim = r.at("vdim").integer();
      ls.mem.gate_cap = (float)r.at("gate_cap").number();
      ls.mem.q = rp + "q"; ls.mem.k = rp + "k"; ls.mem.v = rp + "v"; ls.mem.g = rp + "g"; ls.mem.o = rp + "o";
      ls.mem.norm = rp + "norm"; ls.mem.i = rp + "i"; ls.mem.i_b = rp + "i.b"; ls.mem.f = rp + "f"; ls.mem.f_b = rp + "f.b";
      ls.left_out = pre + "mix.left.out";
      ls.right_out = pre + "mix.right.out";
    } else if (type == "channel_delta") {
      ls.mixer = THA_MIX_DELTA;
      const std::string p = pre + "mix.";
      DeltaSpec& d = ls.delta;
      d.heads = m.at("heads").integer();
      d.kv_heads = m.at("kv_heads").integer();
      d.dim = m.at("dim").integer();
      d.vdim = m.at("vdim").integer();
      d.taps = m.at("conv").integer();
      d.q = p + "q"; d.k = p + "k"; d.v = p + "v";
      d.q_conv = p + "q.conv"; d.k_conv = p + "k.conv"; d.v_conv = p + "v.conv";
      d.b = p + "b"; d.a_log = p + "A_log"; d.norm = p + "norm"; d.a1 = p + "a1"; d.a2 = p + "a2"; d.dt_bias = p + "dt_bias";
      d.g1 = p + "g1"; d.g2 = p + "g2"; d.o = p + "o";
    } else {
      throw std::runtime_error("config: unknown layer type '" + type + "'");
    }
    if (L.has("mlp")) {
      const JsonValue& f = L.at("mlp");
      const std::string kind = f.has("kind") ? f.at("kind").string() : "moe";
      if (kind != "moe") throw std::runtime_error("config: unknown feed-forward kind '" + kind + "'");
      ls.has_ff = true;
      MoeSpec& e = ls.moe;
      e.experts = f.at("router").at("experts").integer();
      e.top = f.at("router").at("top").integer();
      e.ff = f.at("expert").at("ff").integer();
      e.limit = (float)f.at("expert").at("limit").number();
      e.alpha = 1.702f;
      e.router = pre + "mlp.router";
      e.prefix = pre + "mlp.";
      if (f.has("shared")) {
        e.shared_ff = f.at("shared").at("ff").integer();
        e.shared_limit = (float)f.at("shared").at("limit").number();
        e.s_gate = pre + "mlp.shared.gate"; e.s_up = pre + "mlp.shared.up"; e.s_down = pre + "mlp.shared.down";
      }
    }
    s.layers.push_back(ls);
  }
}

void register_timerax() { register_architecture({"Timerax", ModelFamily::LayerProgram, timerax_translate}); }
