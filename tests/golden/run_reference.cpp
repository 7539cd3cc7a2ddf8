// Drives the reference's own loader and forward pass (src/model.cpp, src/inference.cu and the
// kernels of src/cuda/) on the CPU stand-in for CUDA, and writes the logits it returns.
//
//   run_reference MODEL.gguf PLAN.txt OUT.f32
//
// PLAN.txt: first line "max_seq max_batch", then one forward pass per line:
//   n_seqs  then per token "seq:pos:token"  (the reference's flat tokens / positions / seq_ids,
//   src/inference.h:35-42).  After every pass the last-token logits of each sequence are
//   appended to OUT.f32 (n_seqs rows of n_vocab float32).  The cache is kept between passes.
#include "inference.h"

#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

int main(int argc, char** argv) {
    if (argc != 4) {
        fprintf(stderr, "usage: run_reference MODEL.gguf PLAN.txt OUT.f32\n");
        return 2;
    }
    Qwen3Model model;
    if (!model.load(argv[1])) return 1;
    std::ifstream plan(argv[2]);
    int max_seq = 0, max_batch = 0;
    plan >> max_seq >> max_batch;
    Inference inf;
    if (!inf.init(model, max_seq, max_batch)) return 1;
    FILE* out = fopen(argv[3], "wb");
    if (!out) return 1;
    std::string line;
    std::getline(plan, line);
    int pass = 0;
    while (std::getline(plan, line)) {
        if (line.empty()) continue;
        std::istringstream in(line);
        int n_seqs = 0;
        in >> n_seqs;
        std::vector<int32_t> tokens;
        std::vector<int> positions, seqs;
        std::string item;
        while (in >> item) {
            int s = 0, p = 0, t = 0;
            if (sscanf(item.c_str(), "%d:%d:%d", &s, &p, &t) != 3) return 2;
            seqs.push_back(s);
            positions.push_back(p);
            tokens.push_back(t);
        }
        std::vector<float> logits;
        if (!inf.forward(tokens, positions, seqs, n_seqs, logits)) {
            fprintf(stderr, "forward refused pass %d\n", pass);
            return 1;
        }
        fwrite(logits.data(), sizeof(float), logits.size(), out);
        fprintf(stderr, "pass %d: %zu tokens, %d sequences\n", pass, tokens.size(), n_seqs);
        ++pass;
    }
    fclose(out);
    return 0;
}
