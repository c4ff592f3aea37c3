// ./build/apps/trace_run -- replays a trace of scheduler steps through the serving path and writes the logits asked for.
//
//   trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-seqs S]
//
// Standard input: one JSON object per line,
//   {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
// `entries` are one batch for SequenceEngine::step (prompt portions beside single decoded tokens); `end` lists the
// requests whose blocks and slot are given back after the step.  For a step with wanted places the logits go to
// DIR/<step>.f32 (little-endian fp32, [wanted, vocab], in entry and want order); every step answers "done <step>".
// It samples nothing.  Exit codes: 0 at end of input, 1 on a failed step or unreadable line, 2 on a bad command line or
// a model that cannot be loaded.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <iostream>
#include <string>

#include "json_min.hpp"
#include "sequence_engine.hpp"

int main(int argc, char** argv) {
  std::string model_dir, out_dir, dtype = "bfloat16";
  int max_tokens = 4096, max_seqs = 4;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--model") model_dir = v;
    else if (k == "--dtype") dtype = v;
    else if (k == "--out") out_dir = v;
    else if (k == "--max-tokens") max_tokens = atoi(v.c_str());
    else if (k == "--max-seqs") max_seqs = atoi(v.c_str());
    else { fprintf(stderr, "trace_run: unknown option %s\n", k.c_str()); return 2; }
  }
  if (model_dir.empty() || out_dir.empty() || (dtype != "bfloat16" && dtype != "float32") || max_tokens < 1 || max_seqs < 1) {
    fprintf(stderr, "usage: trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-seqs S]\n");
    return 2;
  }
  std::string err;
  LayerModel* model = LayerModel::load(model_dir, dtype == "float32" ? THA_DT_F32 : THA_DT_BF16, &err);
  if (!model) { fprintf(stderr, "trace_run: %s\n", err.c_str()); return 2; }
  SequenceEngine engine(model, max_tokens, max_seqs);
  if (!engine.ok()) { fprintf(stderr, "trace_run: %s\n", engine.error().c_str()); return 2; }
  std::string line;
  while (std::getline(std::cin, line)) {
    if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
    long step_no = 0;
    std::vector<StepEntry> entries;
    std::vector<std::string> ends;
    try {
      JsonValue j = JsonValue::parse(line);
      step_no = (long)j.at("step").number();
      for (const JsonValue& e : j.at("entries").arr) {
        StepEntry se;
        se.id = e.at("id").string();
        for (const JsonValue& t : e.at("tokens").arr) se.tokens.push_back(t.integer());
        if (e.has("want"))
          for (const JsonValue& w : e.at("want").arr) se.want.push_back(w.integer());
        entries.push_back(se);
      }
      if (j.has("end"))
        for (const JsonValue& e : j.at("end").arr) ends.push_back(e.string());
    } catch (const std::exception& ex) {
      fprintf(stderr, "trace_run: %s\n", ex.what());
      return 1;
    }
    std::vector<float> logits;
    if (!engine.step(entries, &logits)) { fprintf(stderr, "trace_run: step %ld: %s\n", step_no, engine.error().c_str()); return 1; }
    if (!logits.empty()) {
      const std::string path = out_dir + "/" + std::to_string(step_no) + ".f32";
      FILE* f = fopen(path.c_str(), "wb");
      if (!f || fwrite(logits.data(), sizeof(float), logits.size(), f) != logits.size()) { fprintf(stderr, "trace_run: cannot write %s\n", path.c_str()); return 1; }
      fclose(f);
    }
    for (const std::string& id : ends) engine.finish(id);
    printf("done %ld\n", step_no);
    fflush(stdout);
  }
  return 0;
}
