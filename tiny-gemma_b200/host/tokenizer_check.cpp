// Drives sentencepiece::Tokenizer the way a parity test needs it; compiles against this directory's
// tokenizer.hpp or, unchanged, against the reference's header of the same name (same class, same interface).
//
//   tokenizer_check <tokenizer.bin> <vocab_size> <chat_format 0|1> <file with one text per line> [--decode]
// per input line prints  ids: <space separated ids>  and, with --decode,  text: <decode(ids)>  and
// pieces: <decode(id, prev) joined by '|'>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <string>

#include "tokenizer.hpp"

int main(int argc, char **argv) {
	if (argc < 5) return 2;
	const bool with_decode = argc > 5 && std::string(argv[5]) == "--decode";
	try {
		sentencepiece::Tokenizer tok(argv[1], 2, 1, std::atoi(argv[2]), std::atoi(argv[3]) != 0);
		std::ifstream f(argv[4]);
		std::string line;
		while (std::getline(f, line)) {
			std::vector<int> ids = tok.encode(line);
			std::printf("ids:");
			for (int v : ids) std::printf(" %d", v);
			std::printf("\n");
			if (!with_decode) continue;
			std::printf("text: %s\npieces: ", tok.decode(ids).c_str());
			int prev = 1;  // exercises the leading-space rule on the first piece
			for (int v : ids) {
				std::printf("%s|", tok.decode(v, prev).c_str());
				prev = v;
			}
			std::printf("\n");
		}
		std::printf("bos %d eos %d eot %d vocab %d\n", tok.get_bos_id(), tok.get_eos_id(), tok.get_eot_id(), tok.get_vocab_size());
	} catch (const std::exception &e) {
		std::fprintf(stderr, "error: %s\n", e.what());
		return 1;
	}
	return 0;
}
