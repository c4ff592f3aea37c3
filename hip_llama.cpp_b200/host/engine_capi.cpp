// C entry points over LayerModel + SequenceEngine (include/tha_engine.h).
#include "tha_engine.h"

#include <string>
#include <vector>

#include "sequence_engine.hpp"

struct tha_engine {
  LayerModel* model = nullptr;
  SequenceEngine* engine = nullptr;
  std::string err;
};
static thread_local std::string g_open_error;

extern "C" int thaEngineOpen(const char* model_dir, int dtype, int max_tokens, int max_seqs, tha_engine_t** out) {
  if (!model_dir || !out || (dtype != THA_DT_BF16 && dtype != THA_DT_F32)) { g_open_error = "bad argument"; return 2; }
  tha_engine* e = new tha_engine();
  e->model = LayerModel::load(model_dir, dtype, &g_open_error);
  if (!e->model) { delete e; return 2; }
  e->engine = new SequenceEngine(e->model, max_tokens, max_seqs);
  if (!e->engine->ok()) {
    g_open_error = e->engine->error();
    delete e->engine;
    delete e->model;
    delete e;
    return 5;
  }
  *out = e;
  return 0;
}
extern "C" const char* thaEngineOpenError(void) { return g_open_error.c_str(); }
extern "C" const char* thaEngineError(tha_engine_t* e) { return e ? e->engine->error().c_str() : ""; }
extern "C" void thaEngineClose(tha_engine_t* e) {
  if (!e) return;
  delete e->engine;
  delete e->model;
  delete e;
}
extern "C" int thaEngineVocab(tha_engine_t* e) { return e->model->vocab(); }
extern "C" int thaEngineWidth(tha_engine_t* e) { return e->model->device_model()->width; }
extern "C" int thaEngineLayers(tha_engine_t* e) { return e->model->device_model()->n_layers; }
extern "C" long long thaEngineFreeBlocks(tha_engine_t* e) { return (long long)e->engine->free_blocks(); }
extern "C" int thaEngineSlot(tha_engine_t* e, const char* id) { return e->engine->slot(id); }
extern "C" long long thaEngineSteps(tha_engine_t* e) { return e->engine->steps_run(); }

extern "C" int thaEngineStep(tha_engine_t* e, int n_entries, const char* const* ids, const int* counts, const int* tokens,
                             const int* want_counts, const int* wants, float* logits_out, float* taps_out) {
  std::vector<StepEntry> entries(n_entries);
  size_t t = 0, w = 0;
  for (int i = 0; i < n_entries; i++) {
    entries[i].id = ids[i];
    entries[i].tokens.assign(tokens + t, tokens + t + counts[i]);
    t += counts[i];
    const int nw = want_counts ? want_counts[i] : 0;
    entries[i].want.assign(wants + w, wants + w + nw);
    w += nw;
  }
  std::vector<float> taps;
  if (!e->engine->step_pinned(entries, taps_out ? &taps : nullptr)) return 5;
  if (logits_out) std::copy(e->engine->last_logits(), e->engine->last_logits() + e->engine->last_wanted() * (size_t)e->model->vocab(), logits_out);
  if (taps_out) std::copy(taps.begin(), taps.end(), taps_out);
  return 0;
}
extern "C" const float* thaEngineLogits(tha_engine_t* e) { return e->engine->last_logits(); }
extern "C" long long thaEngineWanted(tha_engine_t* e) { return (long long)e->engine->last_wanted(); }
extern "C" int thaEngineFinish(tha_engine_t* e, const char* id) { e->engine->finish(id); return 0; }

extern "C" int thaEngineGenerate(tha_engine_t* e, int n_requests, const int* prompt_lens, const int* prompts, const int* max_new,
                                 float temperature, float topp, unsigned long long seed, int portion, int* out_tokens) {
  std::vector<GenerationRequest> reqs(n_requests);
  size_t at = 0;
  for (int i = 0; i < n_requests; i++) {
    reqs[i].prompt.assign(prompts + at, prompts + at + prompt_lens[i]);
    at += prompt_lens[i];
    reqs[i].max_new = max_new[i];
  }
  SamplingOptions opt;
  opt.temperature = temperature;
  opt.topp = topp;
  opt.seed = seed;
  if (!e->engine->generate(&reqs, opt, portion)) return 5;
  size_t o = 0;
  for (auto& q : reqs)
    for (int tkn : q.output) out_tokens[o++] = tkn;
  return 0;
}
