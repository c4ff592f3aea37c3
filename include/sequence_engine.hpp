// sequence_engine.hpp -- continuous batching for layer-program models: admission, the per-step row batch, the step call,
// release, and a generation loop with the library's samplers.
//
// The llama2 driver (include/llama_driver.hpp) keeps one token per slot per step and ingests prompts in a separate
// call.  Here a step is a list of entries (request, next tokens): prompt portions of any length beside single decoded
// tokens, all rows of the step through tha_hyb_step together.  The BatchManager owns what a request holds between
// steps -- its slot, the cache blocks behind its block-table row, its recurrent state slot -- and takes it back when the
// request ends, so blocks and slots are used again by later requests.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "BatchManager.hpp"
#include "layer_model.hpp"

struct StepEntry {
  std::string id;            // request name; admitted at its first entry
  std::vector<int> tokens;   // its next tokens, in order
  std::vector<int> want;     // indices into `tokens` whose logits are asked for
};

struct GenerationRequest {
  std::vector<int> prompt;
  int max_new = 16;
  std::vector<int> output;   // filled by generate()
};

struct SamplingOptions {
  float temperature = 0.0f;  // 0: greedy (first maximum)
  float topp = 0.9f;
  unsigned long long seed = 1;
};

class SequenceEngine {
 public:
  // max_tokens: the most positions live requests hold together (the block pool is sized for this, each request rounded up
  // to whole blocks); max_seqs: state slots / block-table rows.
  SequenceEngine(LayerModel* model, int max_tokens, int max_seqs);
  ~SequenceEngine();
  bool ok() const { return ok_; }
  const std::string& error() const { return err_; }

  // One step.  logits: [sum of wants, vocab] in entry order (may be NULL when nothing is wanted); taps (optional):
  // the residual stream after every layer, [layers, rows, width].
  bool step(const std::vector<StepEntry>& entries, std::vector<float>* logits, std::vector<float>* taps = nullptr);
  // The same step with the wanted logits left in the engine's pinned host buffer (no second copy): last_logits() is
  // [last_wanted(), vocab] and stays valid until the next step.
  bool step_pinned(const std::vector<StepEntry>& entries, std::vector<float>* taps = nullptr);
  const float* last_logits() const { return logits_h_; }
  size_t last_wanted() const { return last_wanted_; }
  // the request is finished: its blocks and its slot go back
  void finish(const std::string& id);
  int live() const { return (int)slot_of_.size(); }
  int position(const std::string& id) const;   // tokens the request has been fed so far, -1 if unknown
  size_t free_blocks() const { return bm_.free_blocks(); }
  int slot(const std::string& id) const;       // -1 if not live

  // Greedy or sampled generation of many requests through step(): prompts enter in portions of at most `portion` tokens
  // beside the single tokens of the requests that are already decoding; at most max_seqs requests are live.
  bool generate(std::vector<GenerationRequest>* requests, const SamplingOptions& opt, int portion = 256);
  long long steps_run() const { return steps_; }

 private:
  bool fail(const std::string& why) { err_ = why; return false; }
  LayerModel* model_;
  BatchManager bm_;
  int max_seqs_;
  bool ok_ = false;
  std::string err_;
  void* stream_ = nullptr;
  std::map<std::string, int> slot_of_;
  std::vector<int> filled_;               // per slot: positions fed
  int next_request_id_ = 0;
  // staging: one pinned host block and one device block for the row arrays, regrown on demand
  int* stage_h_ = nullptr; int* stage_d_ = nullptr; size_t stage_cap_ = 0;
  bool run(const std::vector<StepEntry>& entries, bool to_host, std::vector<float>* taps);
  float* logits_d_ = nullptr; size_t logits_cap_ = 0;
  float* logits_h_ = nullptr; size_t logits_h_cap_ = 0; size_t last_wanted_ = 0;
  float* taps_d_ = nullptr; size_t taps_cap_ = 0;
  // samplers
  unsigned long long* rng_d_ = nullptr; int* next_d_ = nullptr; int* samp_pos_d_ = nullptr; unsigned long long* reseed_d_ = nullptr;
  long long steps_ = 0;
};
