// Continuous batching over tha_hyb_step (include/sequence_engine.hpp).
#include "sequence_engine.hpp"

#include <string.h>

#include <algorithm>
#include <set>

#include "tha_b200.h"

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

SequenceEngine::SequenceEngine(LayerModel* model, int max_tokens, int max_seqs)
    : model_(model),
      // table rows long enough for one request to hold the whole pool
      bm_(max_seqs, round_up(max_tokens < 1 ? 1 : max_tokens, 64), model->n_cache_layers() > 0 ? model->n_cache_layers() : 1, model->kv_dim()),
      max_seqs_(max_seqs) {
  if (max_tokens < 1 || max_seqs < 1) { err_ = "max_tokens and max_seqs must be positive"; return; }
  const size_t blocks = bm_.blocks_for(round_up(max_tokens, 64));
  if (!bm_.create_pool(blocks, model->separate_values())) { err_ = std::string("cannot allocate the cache pool: ") + tha_last_error(); return; }
  if (!bm_.create_state_slots((size_t)model->state_floats())) { err_ = std::string("cannot allocate the state slots: ") + tha_last_error(); return; }
  if (tha_stream_create(&stream_) != 0) { err_ = tha_last_error(); return; }
  filled_.assign(max_seqs, 0);
  ok_ = true;
}

SequenceEngine::~SequenceEngine() {
  if (stream_) { tha_stream_sync(stream_); tha_stream_destroy(stream_); }
  if (stage_h_) tha_host_free(stage_h_);
  if (logits_h_) tha_host_free(logits_h_);
  for (void* p : {(void*)stage_d_, (void*)logits_d_, (void*)taps_d_, (void*)rng_d_, (void*)next_d_, (void*)samp_pos_d_, (void*)reseed_d_})
    if (p) tha_free(p);
}

int SequenceEngine::slot(const std::string& id) const {
  auto it = slot_of_.find(id);
  return it == slot_of_.end() ? -1 : it->second;
}
int SequenceEngine::position(const std::string& id) const {
  const int s = slot(id);
  return s < 0 ? -1 : filled_[s];
}

void SequenceEngine::finish(const std::string& id) {
  auto it = slot_of_.find(id);
  if (it == slot_of_.end()) return;
  bm_.release_slot(it->second);
  filled_[it->second] = 0;
  slot_of_.erase(it);
}

bool SequenceEngine::step(const std::vector<StepEntry>& entries, std::vector<float>* logits, std::vector<float>* taps) {
  if (!run(entries, logits != nullptr, taps)) return false;
  if (logits) logits->assign(logits_h_, logits_h_ + last_wanted_ * (size_t)model_->vocab());
  return true;
}
bool SequenceEngine::step_pinned(const std::vector<StepEntry>& entries, std::vector<float>* taps) { return run(entries, true, taps); }

bool SequenceEngine::run(const std::vector<StepEntry>& entries, bool to_host, std::vector<float>* taps) {
  if (!ok_) return false;
  last_wanted_ = 0;
  const int vocab = model_->vocab();
  // ---- admission and blocks ---------------------------------------------------------------------------------------
  std::vector<const StepEntry*> live;
  std::set<std::string> seen;
  size_t R = 0, n_want = 0;
  bool admitted = false;
  for (const StepEntry& e : entries) {
    if (!seen.insert(e.id).second) return fail("request '" + e.id + "' appears twice in one step");
    int s = slot(e.id);
    if (s < 0) {
      s = bm_.acquire_slot(next_request_id_++);
      if (s < 0) return fail("no free slot for request '" + e.id + "'");
      slot_of_[e.id] = s;
      filled_[s] = 0;
      admitted = true;
    }
    if (e.tokens.empty()) continue;
    for (int t : e.tokens)
      if (t < 0 || t >= vocab) return fail("token out of range");
    for (int w : e.want)
      if (w < 0 || w >= (int)e.tokens.size()) return fail("wanted place out of range");
    const int last = filled_[s] + (int)e.tokens.size() - 1;
    if (last >= bm_.nrow_blocks * bm_.block_size) return fail("request '" + e.id + "' is longer than the cache can address");
    if (model_->max_positions() > 0 && last >= model_->max_positions()) return fail("request '" + e.id + "' is longer than the model's position table");
    if (!bm_.ensure_position(s, last)) return fail("cache pool exhausted");
    live.push_back(&e);
    R += e.tokens.size();
    n_want += e.want.size();
  }
  if (R == 0) return true;
  // a slot taken in this step was zeroed on the null stream; the engine's stream does not order itself behind that
  if (admitted) tha_stream_sync(nullptr);
  bm_.sync_table(stream_);
  // ---- row arrays: token | pos | row_seq | seq_first | seq_slot | want_rows ------------------------------------------
  const size_t S = live.size();
  const size_t n_int = 3 * R + (S + 1) + S + n_want;
  if (n_int > stage_cap_) {
    if (stage_h_) tha_host_free(stage_h_);
    if (stage_d_) tha_free(stage_d_);
    stage_cap_ = n_int * 2;
    if (tha_host_alloc((void**)&stage_h_, stage_cap_ * sizeof(int)) != 0 || tha_malloc((void**)&stage_d_, stage_cap_ * sizeof(int)) != 0)
      return fail(std::string("staging allocation failed: ") + tha_last_error());
  }
  int* token = stage_h_;
  int* pos = token + R;
  int* row_seq = pos + R;
  int* seq_first = row_seq + R;
  int* seq_slot = seq_first + S + 1;
  int* want_rows = seq_slot + S;
  size_t r = 0, w = 0;
  int max_rows = 0, max_pos = 0;
  for (size_t i = 0; i < S; i++) {
    const StepEntry& e = *live[i];
    const int s = slot_of_[e.id];
    seq_first[i] = (int)r;
    seq_slot[i] = s;
    for (int wv : e.want) want_rows[w++] = (int)r + wv;
    for (size_t k = 0; k < e.tokens.size(); k++, r++) {
      token[r] = e.tokens[k];
      pos[r] = filled_[s] + (int)k;
      row_seq[r] = (int)i;
    }
    max_rows = std::max(max_rows, (int)e.tokens.size());
    max_pos = std::max(max_pos, filled_[s] + (int)e.tokens.size() - 1);
  }
  seq_first[S] = (int)R;
  if (tha_memcpy_async(stage_d_, stage_h_, n_int * sizeof(int), stream_) != 0) return fail(tha_last_error());
  tha_rows_t rows;
  rows.n_rows = (int)R;
  rows.n_seqs = (int)S;
  rows.token = stage_d_;
  rows.pos = stage_d_ + R;
  rows.row_seq = stage_d_ + 2 * R;
  rows.seq_first = stage_d_ + 3 * R;
  rows.seq_slot = rows.seq_first + S + 1;
  rows.max_seq_rows = max_rows;
  rows.max_pos = max_pos;
  const int* want_d = rows.seq_slot + S;
  tha_kv_t kv;
  kv.k_pool = bm_.pool_k();
  kv.v_pool = bm_.pool_v();
  kv.table = bm_.device_table();
  kv.table_stride = bm_.nrow_blocks;
  kv.block_size = bm_.block_size;
  kv.n_cache_layers = bm_.n_layers;
  kv.kv_dim = bm_.kv_dim;
  tha_state_store_t st;
  st.base = bm_.state_base();
  st.slot_floats = (long long)bm_.state_slot_floats();
  if (n_want * (size_t)vocab > logits_cap_) {
    if (logits_d_) tha_free(logits_d_);
    logits_cap_ = n_want * (size_t)vocab * 2;
    if (tha_malloc((void**)&logits_d_, logits_cap_ * sizeof(float)) != 0) return fail(tha_last_error());
  }
  const size_t n_taps = taps ? (size_t)model_->device_model()->n_layers * R * model_->device_model()->width : 0;
  if (n_taps > taps_cap_) {
    if (taps_d_) tha_free(taps_d_);
    taps_cap_ = n_taps;
    if (tha_malloc((void**)&taps_d_, taps_cap_ * sizeof(float)) != 0) return fail(tha_last_error());
  }
  const int status = tha_hyb_step(stream_, model_->device_model(), &rows, &kv, &st, (int)n_want, want_d, n_want ? logits_d_ : nullptr,
                                  taps ? taps_d_ : nullptr);
  if (status != 0) return fail(std::string("step failed (status ") + std::to_string(status) + "): " + tha_last_error());
  if (to_host && n_want) {
    if (n_want * (size_t)vocab > logits_h_cap_) {
      if (logits_h_) tha_host_free(logits_h_);
      logits_h_cap_ = n_want * (size_t)vocab * 2;
      if (tha_host_alloc((void**)&logits_h_, logits_h_cap_ * sizeof(float)) != 0) { logits_h_ = nullptr; logits_h_cap_ = 0; return fail(tha_last_error()); }
    }
    if (tha_memcpy_async(logits_h_, logits_d_, n_want * (size_t)vocab * sizeof(float), stream_) != 0) return fail(tha_last_error());
  }
  if (taps) {
    taps->resize(n_taps);
    if (tha_memcpy_async(taps->data(), taps_d_, n_taps * sizeof(float), stream_) != 0) return fail(tha_last_error());
  }
  if (tha_stream_sync(stream_) != 0) return fail(std::string("step failed: ") + tha_last_error());
  for (const StepEntry* e : live) {
    const int s = slot_of_[e->id];
    filled_[s] += (int)e->tokens.size();
    bm_.logical_KV_table[s].second = filled_[s];
  }
  steps_++;
  if (to_host) last_wanted_ = n_want;
  return true;
}

// ---- generation -------------------------------------------------------------------------------------------------------
static unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

bool SequenceEngine::generate(std::vector<GenerationRequest>* requests, const SamplingOptions& opt, int portion) {
  if (!ok_) return false;
  if (portion < 1) portion = 1;
  const int vocab = model_->vocab();
  struct Live { size_t req; std::string id; size_t fed; int next; size_t blocks; };
  std::vector<Live> livev;
  size_t pending = 0, reserved = 0;
  const size_t pool = bm_.num_physical_blocks;
  if (!rng_d_) {
    if (tha_malloc((void**)&rng_d_, max_seqs_ * sizeof(unsigned long long)) != 0 || tha_malloc((void**)&reseed_d_, max_seqs_ * sizeof(unsigned long long)) != 0 ||
        tha_malloc((void**)&next_d_, max_seqs_ * sizeof(int)) != 0 || tha_malloc((void**)&samp_pos_d_, max_seqs_ * sizeof(int)) != 0)
      return fail(tha_last_error());
    tha_memset(rng_d_, 0, max_seqs_ * sizeof(unsigned long long));
    tha_memset(samp_pos_d_, 0, max_seqs_ * sizeof(int));   // position 0: every row handed to the sampler is active
  }
  for (auto& q : *requests) {
    q.output.clear();
    if (q.prompt.empty()) return fail("a request needs at least one prompt token");
  }
  std::vector<float> unused;
  while (pending < requests->size() || !livev.empty()) {
    // admit while slots and blocks allow (a request reserves the blocks of its whole length)
    while (pending < requests->size() && (int)livev.size() < max_seqs_) {
      const GenerationRequest& q = (*requests)[pending];
      const size_t need = bm_.blocks_for((int)q.prompt.size() + q.max_new);
      if (need > pool) return fail("a request is longer than the cache pool");
      if (reserved + need > pool) break;
      livev.push_back({pending, "g" + std::to_string(next_request_id_) + "_" + std::to_string(pending), 0, -1, need});
      reserved += need;
      pending++;
    }
    std::vector<StepEntry> entries;
    std::vector<size_t> wants;   // index into livev of every wanted row, in order
    int budget = portion;
    for (size_t i = 0; i < livev.size(); i++) {
      Live& l = livev[i];
      const GenerationRequest& q = (*requests)[l.req];
      StepEntry e;
      e.id = l.id;
      if (l.fed >= q.prompt.size()) {       // decoding: its last sampled token
        e.tokens.push_back(l.next);
        e.want.push_back(0);
        wants.push_back(i);
      } else if (budget > 0) {              // a portion of its prompt
        const size_t n = std::min((size_t)budget, q.prompt.size() - l.fed);
        e.tokens.assign(q.prompt.begin() + l.fed, q.prompt.begin() + l.fed + n);
        budget -= (int)n;
        if (l.fed + n == q.prompt.size()) { e.want.push_back((int)n - 1); wants.push_back(i); }
      } else {
        continue;
      }
      entries.push_back(e);
    }
    if (entries.empty()) return fail("nothing to run: the scheduler is stuck");
    if (!step(entries, nullptr)) return false;
    for (const StepEntry& e : entries)
      for (Live& l : livev)
        if (l.id == e.id && l.fed < (*requests)[l.req].prompt.size()) l.fed += e.tokens.size();
    if (wants.empty()) continue;
    // sample on the device: one row of logits_d_ per wanted place; the coin of a request's n-th token depends on the seed,
    // the request and n only, not on what else is in the step
    const int nw = (int)wants.size();
    std::vector<unsigned long long> reseed(nw);
    for (int i = 0; i < nw; i++) {
      const Live& l = livev[wants[i]];
      reseed[i] = mix64(opt.seed ^ mix64(l.req * 0x100000001B3ull + (*requests)[l.req].output.size())) | 1ull;
    }
    if (tha_memcpy_async(reseed_d_, reseed.data(), nw * sizeof(unsigned long long), stream_) != 0) return fail(tha_last_error());
    if (tha_sample(stream_, nw, logits_d_, vocab, opt.temperature, opt.topp, rng_d_, reseed_d_, nullptr, samp_pos_d_, next_d_) != 0)
      return fail(std::string("sampler failed: ") + tha_last_error());
    std::vector<int> next(nw);
    if (tha_memcpy_async(next.data(), next_d_, nw * sizeof(int), stream_) != 0 || tha_stream_sync(stream_) != 0) return fail(tha_last_error());
    std::vector<std::string> done;
    for (int i = 0; i < nw; i++) {
      Live& l = livev[wants[i]];
      GenerationRequest& q = (*requests)[l.req];
      q.output.push_back(next[i]);
      l.next = next[i];
      if ((int)q.output.size() >= q.max_new) done.push_back(l.id);
    }
    for (const std::string& id : done) {
      finish(id);
      for (size_t i = 0; i < livev.size(); i++)
        if (livev[i].id == id) { reserved -= livev[i].blocks; livev.erase(livev.begin() + i); break; }
    }
  }
  return true;
}
