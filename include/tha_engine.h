/* tha_engine.h -- C entry points of the layer-program serving path (include/layer_model.hpp, include/sequence_engine.hpp)
 * for callers without C++: open a model folder (config.json + model.safetensors; the "architecture" key picks the
 * registered design), feed scheduler steps, release requests, generate.  Host pointers throughout.
 * Return value: 0 = success; otherwise thaEngineError() / thaEngineOpenError() has the text. */
#ifndef THA_ENGINE_H
#define THA_ENGINE_H
#ifdef __cplusplus
extern "C" {
#endif

typedef struct tha_engine tha_engine_t;

/* dtype: 0 = bf16 matrices with fp32 accumulation, 1 = fp32 throughout */
int thaEngineOpen(const char* model_dir, int dtype, int max_tokens, int max_seqs, tha_engine_t** out);
const char* thaEngineOpenError(void);
const char* thaEngineError(tha_engine_t* e);
void thaEngineClose(tha_engine_t* e);
int thaEngineVocab(tha_engine_t* e);
int thaEngineWidth(tha_engine_t* e);
int thaEngineLayers(tha_engine_t* e);
long long thaEngineFreeBlocks(tha_engine_t* e);
int thaEngineSlot(tha_engine_t* e, const char* id); /* -1: not live */
/* One step.  Entry i: request ids[i] gets counts[i] tokens (consecutive in `tokens`) and asks for the logits at
 * want_counts[i] places (consecutive in `wants`, indices into its own tokens).  logits_out: [sum of want_counts, vocab];
 * taps_out (nullable): residual stream after every layer, [layers, rows, width]. */
int thaEngineStep(tha_engine_t* e, int n_entries, const char* const* ids, const int* counts, const int* tokens,
                  const int* want_counts, const int* wants, float* logits_out, float* taps_out);
/* the logits of the last step in the engine's pinned host buffer, [thaEngineWanted, vocab]; valid until the next step
 * (pass logits_out = NULL to thaEngineStep to skip the copy into a caller's buffer) */
const float* thaEngineLogits(tha_engine_t* e);
long long thaEngineWanted(tha_engine_t* e);
int thaEngineFinish(tha_engine_t* e, const char* id);
/* Generation through the scheduler: request i has prompt_lens[i] prompt tokens (consecutive in `prompts`) and gets
 * max_new[i] tokens, written consecutively to out_tokens.  temperature 0 = greedy. */
int thaEngineGenerate(tha_engine_t* e, int n_requests, const int* prompt_lens, const int* prompts, const int* max_new,
                      float temperature, float topp, unsigned long long seed, int portion, int* out_tokens);
long long thaEngineSteps(tha_engine_t* e);

#ifdef __cplusplus
}
#endif
#endif
