// Drives the reference's own Qwen2 class (scalar attention, scalar kernels, one thread) on a tiny
// float32 GGUF model and dumps logits.  Used only by make_golden.py; links the reference's
// libtge_core.a, which that script builds from an unmodified copy plus two portability shims.
//
//   reference_driver MODEL.gguf SCRIPT.txt OUT.f32 SEQUENCES
//
// SCRIPT lines:   prefill SEQ N t0 .. tN-1          -> 1 row  (logits after the last token)
//                 forward SEQ TOKEN POSITION        -> 1 row
//                 batch N  (TOKEN POSITION SEQ) x N -> N rows (one per row of the mixed batch)
#include <cstdio>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "tge/models/qwen2.hpp"

int main(int argc, char** argv) {
  if (argc != 5) {
    std::fprintf(stderr, "usage: reference_driver MODEL.gguf SCRIPT OUT SEQUENCES\n");
    return 2;
  }
  std::string error;
  const int sequences = std::stoi(argv[4]);
  auto model = tge::models::Qwen2::load(argv[1], error, 0, false, false, false, sequences);
  if (!model) {
    std::fprintf(stderr, "load failed: %s\n", error.c_str());
    return 1;
  }
  model->set_threads(1);
  model->set_prefill_threads(1);
  model->set_attention_mode(tge::models::AttentionMode::Scalar);
  model->set_scalar_kernels(true);
  const int vocab = model->vocab_size();
  std::ifstream script(argv[2]);
  std::FILE* out = std::fopen(argv[3], "wb");
  std::string line;
  long rows = 0;
  while (std::getline(script, line)) {
    std::istringstream in(line);
    std::string what;
    if (!(in >> what)) continue;
    if (what == "prefill") {
      int seq, n;
      in >> seq >> n;
      std::vector<int> tokens(n);
      for (int& t : tokens) in >> t;
      const float* logits = model->prefill(tokens.data(), n, 0, seq);
      std::fwrite(logits, sizeof(float), vocab, out);
      rows += 1;
    } else if (what == "forward") {
      int seq, token, position;
      in >> seq >> token >> position;
      const float* logits = model->forward(seq, token, position);
      std::fwrite(logits, sizeof(float), vocab, out);
      rows += 1;
    } else if (what == "batch") {
      int n;
      in >> n;
      std::vector<int> tokens(n), positions(n), seqs(n);
      for (int i = 0; i < n; ++i) in >> tokens[i] >> positions[i] >> seqs[i];
      const float* logits = model->forward_batch(tokens.data(), positions.data(), n, seqs.data());
      std::fwrite(logits, sizeof(float), static_cast<size_t>(vocab) * n, out);
      rows += n;
    }
  }
  std::fclose(out);
  std::printf("rows %ld vocab %d\n", rows, vocab);
  return 0;
}
