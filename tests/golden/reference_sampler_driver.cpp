// Drives the reference's own sampler (src/models/sampling.cpp: sample_token) on logits read from a file and
// prints what it picks.  Used only by make_golden.py; links the reference's libtge_core.a.
//
//   reference_sampler_driver LOGITS.f32 VOCAB CASES.txt
//
// CASES lines:  ROW DRAWS SEED TEMPERATURE TOP_K TOP_P MIN_P REPEAT_PENALTY PENALTY_WINDOW HISTORY_SIZE h0 .. hN-1
// Output, one line per case: the DRAWS token ids drawn in a row from the generator seeded with SEED
// (0 selects the reference's default seed), every draw seeing the same logits row and history.
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "tge/models/sampling.hpp"

int main(int argc, char** argv) {
  if (argc != 4) {
    std::fprintf(stderr, "usage: reference_sampler_driver LOGITS.f32 VOCAB CASES.txt\n");
    return 2;
  }
  const int vocab = std::stoi(argv[2]);
  std::ifstream raw(argv[1], std::ios::binary);
  std::vector<char> bytes((std::istreambuf_iterator<char>(raw)), std::istreambuf_iterator<char>());
  const float* logits = reinterpret_cast<const float*>(bytes.data());
  const int rows = static_cast<int>(bytes.size() / sizeof(float)) / vocab;
  std::ifstream cases(argv[3]);
  std::string line;
  std::vector<float> scores;
  std::vector<int> order;
  while (std::getline(cases, line)) {
    std::istringstream in(line);
    int row, draws, history_size;
    std::uint32_t seed;
    tge::models::SamplingParams params;
    if (!(in >> row >> draws >> seed >> params.temperature >> params.top_k >> params.top_p >> params.min_p >>
          params.repeat_penalty >> params.penalty_window >> history_size)) {
      continue;
    }
    if (row < 0 || row >= rows) return 1;
    std::vector<int> history(history_size);
    for (int& h : history) in >> h;
    std::uint32_t state = seed != 0 ? seed : 0x9E3779B9u;
    for (int d = 0; d < draws; ++d) {
      const int token = tge::models::sample_token(logits + static_cast<std::size_t>(row) * vocab, vocab, params,
                                                  history.data(), history_size, scores, order, state);
      std::printf(d + 1 < draws ? "%d " : "%d\n", token);
    }
  }
  return 0;
}
