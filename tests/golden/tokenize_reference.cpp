// Tokenizes the lines of a file with the reference's own tokenizer (src/tokenizer.cpp) loaded from
// a GGUF file by its own reader (src/gguf_reader.cpp), the way its command line does
// (src/main.cpp:164-171), and prints the ids of every line; then decodes them back.
//
//   tokenize_reference MODEL.gguf LINES.txt [--special]
//
// In LINES.txt "\n" and "\\" are written as escapes so that a line can hold a newline.
#include "gguf_reader.h"
#include "tokenizer.h"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const bool special = argc > 3 && strcmp(argv[3], "--special") == 0;
    GgufReader reader;
    if (!reader.load(argv[1])) return 1;
    Tokenizer tok;
    if (!tok.load_tokens(reader.get_string_array("tokenizer.ggml.tokens"),
                         reader.get_u32_array("tokenizer.ggml.token_type"))) return 1;
    if (!tok.load_merges(reader.get_string_array("tokenizer.ggml.merges"))) return 1;
    std::ifstream in(argv[2], std::ios::binary);
    std::string line;
    while (std::getline(in, line)) {
        std::string text;
        for (size_t i = 0; i < line.size(); ++i) {
            if (line[i] == '\\' && i + 1 < line.size()) {
                text += line[i + 1] == 'n' ? '\n' : line[i + 1];
                ++i;
            } else {
                text += line[i];
            }
        }
        const auto ids = tok.tokenize(text, false, special);
        std::string back;
        for (size_t i = 0; i < ids.size(); ++i) {
            printf(i ? " %d" : "%d", ids[i]);
            back += tok.token_to_piece(ids[i]);
        }
        printf("\t%s\n", back == text ? "round-trip" : "differs");
    }
    return 0;
}
