// Text-generation CLI with the flags, defaults and output of the reference's gemma.cpp (:7-61), on the GPU
// library through tiny_gemma.hpp:
//
//   gemma --weights_path W --model_size 270m|1B --prompt "..." --n_dec N [--minp P] --temp T
//         --chat_format 0|1 --terminate_on_eos 0|1 [--tokenizer_path weights/tokenizer_gemma3.bin] [--seed S]
//
// Every option is "--name value"; minp >= 1 (the default 2.0) selects greedy decoding. --seed (not in the
// reference, which seeds from std::random_device) makes a sampled run repeatable.
#include <cstdio>
#include <iostream>
#include <map>
#include <string>

#include "tiny_gemma.hpp"

namespace {
struct Options {
	std::map<std::string, std::string *> strings;
	std::map<std::string, int *> ints;
	std::map<std::string, float *> floats;
	std::map<std::string, std::string> help;
	void usage(const char *prog) const {
		std::cerr << "CLI Application for Gemma 3 text generation.\nUsage: " << prog << " [options]\n\nOptions:\n";
		for (const auto &h : help) std::cerr << "  --" << h.first << "\t" << h.second << '\n';
	}
	// 0 on success, 1 after a usage error (message + option list on stderr); a value that does not parse throws
	int parse(int argc, char **argv) const {
		for (int i = 1; i < argc; i++) {
			const std::string arg = argv[i];
			std::string err;
			if (arg.rfind("--", 0) != 0) {
				err = "unexpected token: " + arg;
			} else {
				const std::string name = arg.substr(2);
				if (!help.count(name)) {
					err = "unknown option: --" + name;
				} else if (i + 1 == argc) {
					err = "missing value for --" + name;
				} else {
					const std::string value = argv[++i];
					try {
						if (strings.count(name)) *strings.at(name) = value;
						if (ints.count(name)) *ints.at(name) = std::stoi(value);
						if (floats.count(name)) *floats.at(name) = std::stof(value);
					} catch (...) {
						throw std::invalid_argument(std::string(ints.count(name) ? "expected integer for " : "expected float for ") + value);
					}
				}
			}
			if (!err.empty()) {
				std::cerr << "Error: " << err << "\n\n";
				usage(argv[0]);
				return 1;
			}
		}
		return 0;
	}
};
}  // namespace

int main(int argc, char **argv) {
	std::string weights_path, model_size, prompt, tokenizer_path = "weights/tokenizer_gemma3.bin";
	int n_decode = 0, chat_format = 0, terminate_on_eos = 0, seed = -1;
	float minp = 2.0f, temp = 1.0f;
	Options app;
	auto opt = [&](const char *name, const char *text) { app.help[name] = text; };
	app.strings = {{"weights_path", &weights_path}, {"model_size", &model_size}, {"prompt", &prompt}, {"tokenizer_path", &tokenizer_path}};
	app.ints = {{"n_dec", &n_decode}, {"chat_format", &chat_format}, {"terminate_on_eos", &terminate_on_eos}, {"seed", &seed}};
	app.floats = {{"minp", &minp}, {"temp", &temp}};
	opt("weights_path", "File path for model weights.");
	opt("model_size", "Model size to load.");
	opt("prompt", "The prompt.");
	opt("n_dec", "Number of tokens to generate.");
	opt("minp", "Minp sampler, defaults to greedy sampling if `minp >= 1`.");
	opt("temp", "Sampler temperature.");
	opt("chat_format", "Flag to enable using chat template.");
	opt("terminate_on_eos", "Flag to enable early termination if model generates an EOS/EOT token.");
	opt("tokenizer_path", "File path for tokenizer.");
	opt("seed", "Seed of the sampler's std::mt19937 (default: std::random_device).");
	try {
		const int rc = app.parse(argc, argv);
		if (rc != 0) return rc;
	} catch (const std::exception &ex) {
		std::cerr << "Parse error: " << ex.what() << '\n';
		return 1;
	}
	try {
		gemma::Config config = gemma::CONFIG_MAP.at(model_size);
		gemma::Transformer t(config);
		gemma::read_weights(&t, weights_path.c_str());
		printf("Weights loaded!\n");
		sentencepiece::Tokenizer tokenizer(tokenizer_path, constants::bos_id, constants::eos_id, constants::vocab, bool(chat_format));
		const unsigned useed = unsigned(seed);
		auto generations = gemma::generate(prompt, n_decode, &tokenizer, &t, minp, temp, bool(terminate_on_eos), seed >= 0 ? &useed : nullptr);
		const int n_generated_tokens = std::get<0>(generations);
		const int n_prompt_tokens = int(tokenizer.encode(prompt).size());
		const float total_s = std::get<2>(generations) + std::get<3>(generations);
		const float prefill_tok_s = n_prompt_tokens / std::get<2>(generations);
		const float decode_tok_s = n_generated_tokens / std::get<3>(generations);
		printf("\n\nGenerating %u tokens took %f seconds. Prefill Tok/s: %f  Decode Tok/s %f ms/token: %f\n", n_generated_tokens, total_s,
		       prefill_tok_s, decode_tok_s, 1e3 * std::get<3>(generations) / n_generated_tokens);
	} catch (const std::exception &e) {  // (the reference lets these escape to std::terminate)
		std::fprintf(stderr, "error: %s\n", e.what());
		return 1;
	}
	return 0;
}
