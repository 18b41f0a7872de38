// Timing driver for the reference arm of bench.py: ember.cpp's own interpreter through its public
// class (ember_ir::Interpreter, graph_ir.h:102-124), on its stock device path, nothing of this
// repository's on the way.  It follows ember.cpp's own tools/ir_decode_bench.cpp (load the GGUF,
// find the graph, build the interpreter on the GPU, prefill, then one-token forwards with the
// argmax of the last logits as the next token), with the prompt length, the number of warm-up and
// timed steps and a whole-prompt timing as arguments:
//
//   ref_bench model.gguf PROMPT WARMUP STEPS PREFILL_TOKENS PREFILL_PROMPTS
//
// The interpreter holds one sequence; a batch is served one sequence after another, so the decode
// rate of a batch is the rate of one sequence.  forward() returns the logits on the host, so every
// call is synchronous and the clock around it is the end-to-end time of a step (token in, a row of
// vocab floats out).  Prints one JSON object.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "gguf_parser.h"
#include "graph_ir.h"

static double now_ms() {
  return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
  if (argc < 7) {
    std::fprintf(stderr, "usage: %s model.gguf prompt warmup steps prefill_tokens prefill_prompts\n", argv[0]);
    return 2;
  }
  const int prompt = std::atoi(argv[2]), warm = std::atoi(argv[3]), steps = std::atoi(argv[4]);
  const int prefill_tokens = std::atoi(argv[5]), prefill_prompts = std::atoi(argv[6]);
  try {
    GGUFData gguf = load_gguf_meta(argv[1], true);
    const std::string ir = ember_ir::find_ir(gguf);
    if (ir.empty()) {
      std::fprintf(stderr, "no graph for %s\n", argv[1]);
      return 2;
    }
    ember_ir::Interpreter interp(ir, gguf, true);
    if (!interp.on_gpu()) {
      std::fprintf(stderr, "the interpreter did not take the device path\n");
      return 3;
    }
    unsigned long long state = 12345;
    auto next_id = [&] {
      state = state * 6364136223846793005ull + 1442695040888963407ull;
      return static_cast<int>((state >> 33) % static_cast<unsigned long long>(interp.vocab()));
    };
    // whole prompts: the median over repeats of `prefill_prompts` forwards of prefill_tokens / prefill_prompts each
    const int per = prefill_tokens / std::max(1, prefill_prompts);
    std::vector<double> pre;
    for (int rep = 0; rep < 5; ++rep) {
      double total = 0;
      for (int q = 0; q < prefill_prompts; ++q) {
        std::vector<int> toks(per);
        for (int& t : toks) t = next_id();
        const double t0 = now_ms();
        interp.forward(toks, 0);
        total += now_ms() - t0;
      }
      if (rep >= 2) pre.push_back(total);
    }
    std::sort(pre.begin(), pre.end());
    // decode: a prompt, then warm + steps single-token forwards; the timed region is exactly `steps` of them
    std::vector<int> toks(prompt);
    for (int& t : toks) t = next_id();
    std::vector<float> logits = interp.forward(toks, 0);
    const int room = interp.max_len() - prompt;
    const int n_warm = std::min(warm, room), n_steps = std::min(steps, room - n_warm);
    double t_start = 0;
    for (int s = 0; s < n_warm + n_steps; ++s) {
      if (s == n_warm) t_start = now_ms();
      const int next = static_cast<int>(std::max_element(logits.begin(), logits.end()) - logits.begin());
      logits = interp.forward({next}, prompt + s);
    }
    const double decode_ms = now_ms() - t_start;
    std::printf("{\"decode_ms_per_step\": %.5f, \"steps\": %d, \"warmup\": %d, \"prompt\": %d, \"context_end\": %d, "
                "\"prefill_ms\": %.4f, \"prefill_tokens\": %d, \"vocab\": %d, \"layers\": %d, \"kv_format\": \"%s\"}\n",
                decode_ms / std::max(1, n_steps), n_steps, n_warm, prompt, prompt + n_warm + n_steps, pre[pre.size() / 2],
                per * prefill_prompts, interp.vocab(), interp.n_layers(), interp.kv_format());
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ember.cpp: %s\n", e.what());
    return 1;
  }
  return 0;
}
