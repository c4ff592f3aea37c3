// ./build/apps/llama -- the inference app of the reference (src/llama.cpp main(), :1514-1638),
// same command line:
//
//   llama <checkpoint> -m test -f <input file> -o <output file> -b <slots per GPU>
//   llama <checkpoint> [-m generate] -i "prompt" -n 256 -t 1.0 -p 0.9 -s seed
//
// Options (reference :1490-1510): -t temperature, -p top-p, -s seed, -n steps, -i prompt,
// -z tokenizer path, -m mode (generate|test), -f/-o files, -b batch size.  Additions: -g <n>
// number of GPUs, -k <file> write the generated token ids, -x 1 ignore stop tokens (timing), -r 0 prompt token by token,
// -q 1 host-side sampler, -c <blocks> paged KV cache,
// and in test mode -t/-p/-s are honoured when given (-t 0 = greedy).  The checkpoint may be a
// v0 fp32 file or a v2 Q8_0 file; the version is detected from the header.
//
// A FOLDER with config.json + model.safetensors is a layer-program model (include/layer_model.hpp): its "architecture"
// key picks the registered design, requests run through the SequenceEngine (continuous batching, prompts in portions
// beside decoding requests) and the same device sampler.  Such models carry no tokenizer: -i and the lines of -f are
// token ids separated by blanks or commas, the output is token ids.  -b = live requests, -d bf16|f32 the number format,
// -j the most prompt tokens per step, -c the cache pool in positions (default: what the requests need).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "layer_model.hpp"
#include "llama_driver.hpp"
#include "sequence_engine.hpp"

static void error_usage() {
  fprintf(stderr, "Usage:   llama <checkpoint> [options]\n");
  fprintf(stderr, "Example: llama model.bin -n 256 -i \"Once upon a time\"\n");
  fprintf(stderr, "Example: llama model.bin -m test -f <input_filename> -o <output_filename> -b <batch>\n");
  fprintf(stderr, "Options:\n");
  fprintf(stderr, "  -t <float>  temperature in [0,inf], default 1.0\n");
  fprintf(stderr, "  -p <float>  p value in top-p (nucleus) sampling in [0,1] default 0.9\n");
  fprintf(stderr, "  -s <int>    random seed, default time(NULL) (test mode: 314028)\n");
  fprintf(stderr, "  -n <int>    number of steps to run for, default 256. 0 = max_seq_len\n");
  fprintf(stderr, "  -i <string> input prompt\n");
  fprintf(stderr, "  -z <string> optional path to custom tokenizer\n");
  fprintf(stderr, "  -m <string> mode: generate|test, default: generate\n");
  fprintf(stderr, "  -f <string> (only for test mode) input filename\n");
  fprintf(stderr, "  -o <string> (only for test mode) output filename\n");
  fprintf(stderr, "  -b <int>    batch size (slots per GPU)\n");
  fprintf(stderr, "  -g <int>    number of GPUs (default: all)\n");
  fprintf(stderr, "  -w <int>    tensor-parallel width: ONE replica split over this many ranks (rank r on GPU r %% n_gpus), greedy only (-t 0)\n");
  fprintf(stderr, "  -k <string> also write the generated token ids to this file\n");
  fprintf(stderr, "  -x <0|1>    ignore stop tokens (fixed-length timing runs)\n");
  fprintf(stderr, "  -c <int>    paged KV cache: the slots of a GPU share this many blocks of 16 positions (-1: what fits; default 0: dense slabs)\n");
  fprintf(stderr, "  -q <0|1>    sampled runs: 1 = sample on the host from B*vocab logits as the reference does (default 0: sampler on the GPU)\n");
  fprintf(stderr, "  -d <bf16|f32> model folders (config.json + model.safetensors): number format, default bf16; -i / -f carry token ids\n");
  fprintf(stderr, "  -j <int>    model folders: the most prompt tokens per scheduler step (default 256)\n");
  fprintf(stderr, "  -r <0|1>    fp32 models: ingest prompts in one tensor-core pass (default 1); 0 = one decode step per prompt token\n");
  exit(EXIT_FAILURE);
}

static std::vector<int> parse_ids(const std::string& text) {
  std::vector<int> out;
  std::string cur;
  for (char c : text + " ") {
    if ((c >= '0' && c <= '9')) cur += c;
    else if (!cur.empty()) { out.push_back(atoi(cur.c_str())); cur.clear(); }
  }
  return out;
}

// generate / test modes for a layer-program model folder
static int run_layer_program(const char* folder, const char* mode, const char* prompt, const char* input_filename, const char* output_filename,
                             int steps, int batch, float temperature, float topp, unsigned long long seed, const char* number_format,
                             int portion, int pool_positions) {
  const int dtype = (!strcmp(number_format, "f32") || !strcmp(number_format, "float32")) ? THA_DT_F32 : THA_DT_BF16;
  std::vector<GenerationRequest> reqs;
  if (!strcmp(mode, "generate")) {
    GenerationRequest q;
    q.prompt = parse_ids(prompt ? prompt : "");
    reqs.push_back(q);
  } else if (!strcmp(mode, "test")) {
    if (!input_filename || !output_filename) error_usage();
    std::ifstream in(input_filename);
    if (!in) { fprintf(stderr, "cannot open %s\n", input_filename); return EXIT_FAILURE; }
    std::string line;
    while (std::getline(in, line)) {
      GenerationRequest q;
      q.prompt = parse_ids(line);
      if (!q.prompt.empty()) reqs.push_back(q);
    }
  } else {
    fprintf(stderr, "unknown mode: %s\n", mode);
    error_usage();
  }
  size_t need = 0, longest = 0;
  for (auto& q : reqs) {
    if (q.prompt.empty()) { fprintf(stderr, "a request needs token ids (-i \"1 2 3\")\n"); return EXIT_FAILURE; }
    q.max_new = steps > 0 ? steps : 256;
    const size_t n = (q.prompt.size() + q.max_new + 63) / 64 * 64;
    longest = n > longest ? n : longest;
  }
  need = longest * (size_t)(batch < (int)reqs.size() ? batch : (int)reqs.size());
  std::string err;
  const long load_start = time_in_ms();
  LayerModel* model = LayerModel::load(folder, dtype, &err);
  if (!model) { fprintf(stderr, "%s\n", err.c_str()); return EXIT_FAILURE; }
  SequenceEngine engine(model, pool_positions > 0 ? pool_positions : (int)need, batch);
  if (!engine.ok()) { fprintf(stderr, "%s\n", engine.error().c_str()); return EXIT_FAILURE; }
  SamplingOptions so;
  so.temperature = temperature; so.topp = topp; so.seed = seed;
  const long start = time_in_ms();
  if (!engine.generate(&reqs, so, portion)) { fprintf(stderr, "%s\n", engine.error().c_str()); return EXIT_FAILURE; }
  const long end = time_in_ms();
  size_t total = 0;
  FILE* out = output_filename ? fopen(output_filename, "w") : stdout;
  if (!out) { fprintf(stderr, "cannot write %s\n", output_filename); return EXIT_FAILURE; }
  for (auto& q : reqs) {
    for (size_t i = 0; i < q.output.size(); i++) fprintf(out, i ? " %d" : "%d", q.output[i]);
    fprintf(out, "\n");
    total += q.output.size();
  }
  if (output_filename) fclose(out);
  fprintf(stderr, "weight upload(s): %f, %lld steps, achieved tok/s: %f\n", (start - load_start) / 1000.0, engine.steps_run(),
          total / (double)(end - start + 1) * 1000);
  delete model;
  return 0;
}

int main(int argc, char* argv[]) {
  const long total_start = time_in_ms();
  char* checkpoint_path = nullptr;
  const char* tokenizer_path = "./assets/tokenizer.bin";
  float temperature = 1.0f, topp = 0.9f;
  int steps = 256, batch = 1, n_gpus = 0, ignore_stop = 0, prefill = 1, tp = 1, host_sampler = 0, kv_blocks = 0;
  const char* prompt = nullptr;
  unsigned long long rng_seed = 0;
  const char* mode = "generate";
  const char *input_filename = nullptr, *output_filename = nullptr, *token_filename = nullptr, *number_format = "bf16";
  int portion = 256;
  bool t_given = false, s_given = false, n_given = false;

  if (argc >= 2) checkpoint_path = argv[1]; else error_usage();
  for (int i = 2; i < argc; i += 2) {
    if (i + 1 >= argc || argv[i][0] != '-' || strlen(argv[i]) != 2) error_usage();
    const char f = argv[i][1];
    const char* v = argv[i + 1];
    if (f == 't') { temperature = atof(v); t_given = true; }
    else if (f == 'p') topp = atof(v);
    else if (f == 's') { rng_seed = strtoull(v, nullptr, 10); s_given = true; }
    else if (f == 'n') { steps = atoi(v); n_given = true; }
    else if (f == 'i') prompt = v;
    else if (f == 'z') tokenizer_path = v;
    else if (f == 'm') mode = v;
    else if (f == 'y') { /* chat system prompt: chat mode is an empty branch in the reference (:1583-1584) */ }
    else if (f == 'f') input_filename = v;
    else if (f == 'o') output_filename = v;
    else if (f == 'b') batch = atoi(v);
    else if (f == 'g') n_gpus = atoi(v);
    else if (f == 'k') token_filename = v;
    else if (f == 'x') ignore_stop = atoi(v);
    else if (f == 'r') prefill = atoi(v);
    else if (f == 'w') tp = atoi(v);
    else if (f == 'q') host_sampler = atoi(v);
    else if (f == 'c') kv_blocks = atoi(v);
    else if (f == 'd') number_format = v;
    else if (f == 'j') portion = atoi(v);
    else error_usage();
  }
  if (rng_seed == 0) rng_seed = (unsigned int)time(nullptr);
  if (temperature < 0.0f) temperature = 0.0f;
  if (topp < 0.0f || 1.0f < topp) topp = 0.9f;
  if (steps < 0) steps = 0;
  if (batch < 1) batch = 1;

  {   // the registry decides which family the path belongs to
    std::string err;
    const ArchitectureEntry* arch = detect_model(checkpoint_path, nullptr, &err);
    if (!arch) { fprintf(stderr, "%s\n", err.c_str()); return EXIT_FAILURE; }
    if (arch->family == ModelFamily::LayerProgram)
      return run_layer_program(checkpoint_path, mode, prompt, input_filename, output_filename, n_given ? steps : 0, batch,
                               t_given ? temperature : 0.0f, topp, rng_seed, number_format, portion, kv_blocks);
  }
  const int version = checkpoint_version(checkpoint_path);
  if (version != 0 && version != 2) { fprintf(stderr, "unreadable checkpoint %s\n", checkpoint_path); return EXIT_FAILURE; }
  Transformer t32;
  TransformerQ8 tq8;
  if (version == 0) build_transformer(&t32, checkpoint_path); else build_transformer_q8(&tq8, checkpoint_path);
  const Config cfg = version == 0 ? t32.config : tq8.config;
  if (steps == 0 || steps > cfg.seq_len) steps = cfg.seq_len;

  Requests requests;
  DriverOptions opt;
  opt.batch_size = batch;
  opt.n_devices = n_gpus;
  opt.ignore_stop = ignore_stop;
  opt.prefill = prefill;
  opt.host_sampler = host_sampler;
  opt.kv_blocks = kv_blocks;
  opt.tp = tp < 1 ? 1 : tp;
  // ranks of one replica that share a GPU hand-shake between concurrent kernels: every rank's stream needs its own
  // hardware queue (set before the CUDA context exists)
  if (opt.tp > 1) setenv("CUDA_DEVICE_MAX_CONNECTIONS", "32", 0);

  if (strcmp(mode, "generate") == 0) {
    // one request through the same driver (the reference's generate() is the single-sequence loop, :1087-1147 of run.cc)
    requests.num_reqs = 1;
    requests.max_seq_len = steps;
    requests.str_reqs.assign(1, prompt ? prompt : "");
    requests.str_gens.assign(1, "");
    requests.tok_gens.assign(1, std::vector<int>());
    opt.batch_size = 1;
    opt.n_devices = opt.tp > 1 ? n_gpus : 1;
    opt.temperature = temperature; opt.topp = topp; opt.seed = rng_seed;
    DriverStats st;
    const long start = time_in_ms();
    run_data_parallel(version == 0 ? &t32 : nullptr, version == 2 ? &tq8 : nullptr, tokenizer_path, &requests, opt, &st);
    const long end = time_in_ms();
    printf("%s", requests.str_gens[0].c_str());
    fprintf(stderr, "achieved tok/s: %f\n", st.gen_tokens / (double)(end - start) * 1000);
  } else if (strcmp(mode, "test") == 0) {
    if (input_filename == nullptr || output_filename == nullptr) error_usage();
    Tokenizer probe;   // max_token_length sizes the request buffers in the reference (:1590)
    build_tokenizer(&probe, tokenizer_path, cfg.vocab_size);
    // the reference always runs a request to seq_len; an explicit -n caps the positions per request (short test runs)
    read_inputfile(input_filename, probe.max_token_length, n_given ? steps : cfg.seq_len, &requests);
    free_tokenizer(&probe);
    if (t_given) { opt.temperature = temperature; opt.topp = topp; }
    if (s_given) opt.seed = rng_seed;
    DriverStats st;
    const long start = time_in_ms();
    const int num_gen_tokens = run_data_parallel(version == 0 ? &t32 : nullptr, version == 2 ? &tq8 : nullptr, tokenizer_path,
                                                 &requests, opt, &st);
    const long end = time_in_ms();
    fprintf(stdout, "Total achieved token: %d\n", num_gen_tokens);
    fprintf(stdout, "elapsed time(s): %f, achieved throughput(tok/s): %f\n", (double)(end - start) / 1000,
            num_gen_tokens / (double)(end - start) * 1000);
    fprintf(stdout, "step loop(s): %f (%lld steps), weight upload(s): %f, loop throughput(tok/s): %f\n", st.loop_seconds,
            st.steps, st.load_seconds, st.loop_seconds > 0 ? num_gen_tokens / st.loop_seconds : 0.0);
    write_outputfile(output_filename, &requests);
    if (token_filename) write_tokenfile(token_filename, &requests);
  } else {
    fprintf(stderr, "unknown mode: %s\n", mode);
    error_usage();
  }

  if (version == 0) free_transformer(&t32); else free_transformer_q8(&tq8);
  fprintf(stdout, "total elapsed time(s): %lf\n", (double)(time_in_ms() - total_start) / 1000);
  return 0;
}
