// Token-level driver over the reference-shaped C++ API (tiny_gemma.hpp): the
// flow of the reference's gemma.cpp / tests/csrc/test_generation.cpp without
// the tokenizer (no tokenizer model is available offline):
//   read weights -> RoPE x2, GeLUTable, DecodeState -> forward_prefill ->
//   sampler -> n_decode x (forward_decode + sampler) -> print ids and tok/s.
//
//   gemma_tokens <weights.bin> <270m|1B> <ids.txt> <n_decode> [minp temp seed] [--device-loop]
// ids.txt: whitespace-separated prompt token ids. minp >= 1 (default 2.0, as
// gemma.cpp:13) selects greedy decoding.
#include <chrono>
#include <fstream>
#include <iostream>

#include "tiny_gemma.hpp"

int main(int argc, char **argv) {
	if (argc < 5) {
		std::fprintf(stderr, "usage: %s weights.bin 270m|1B ids.txt n_decode [minp temp seed] [--device-loop]\n", argv[0]);
		return 2;
	}
	try {
		const std::string weights = argv[1], size = argv[2], ids_path = argv[3];
		const int n_decode = std::atoi(argv[4]);
		const float minp = argc > 5 ? std::atof(argv[5]) : 2.0f;
		const float temp = argc > 6 ? std::atof(argv[6]) : 1.0f;
		const unsigned seed = argc > 7 ? unsigned(std::atol(argv[7])) : 0u;
		const bool device_loop = argc > 8 && std::string(argv[8]) == "--device-loop";

		config::Config cfg = config::CONFIG_MAP.at(size);  // unknown size -> std::out_of_range, as gemma.cpp:38
		gemma::Transformer t(cfg);
		gemma::read_weights(&t, weights.c_str());

		std::vector<int> ids;
		{
			std::ifstream f(ids_path);
			int v;
			while (f >> v) ids.push_back(v);
		}
		if (ids.empty()) throw std::runtime_error("no prompt ids");
		auto tokens_data = tensor::make_unique_aligned<int>(ids.size());
		for (size_t i = 0; i < ids.size(); i++) tokens_data[i] = ids[i];

		auto t0 = std::chrono::high_resolution_clock::now();
		decode::RoPE rope(&cfg, false), rope_sw(&cfg, true);
		lut::GeLUTable table{-4.0, 4.0, 1024};  // transformer.hpp:197
		decode::DecodeState d(1, &cfg);
		tensor::tokens tokens(tokens_data, 1, ids.size());
		tensor::activation o(1, 1, cfg.n_vocab);
		std::mt19937 gen(seed);
		std::uniform_real_distribution<float> unif(0.0, 1.0);

		gemma::forward_prefill(&o, &tokens, &t, &d, &rope, &rope_sw, &table);
		tensor::tokens tok(1, 1);
		if (minp < 1)
			ops::minp_logits(&tok, &o, minp, temp, unif(gen));
		else
			ops::argmax_logits(&tok, &o);
		auto t1 = std::chrono::high_resolution_clock::now();

		std::vector<int> out{tok.data[0]};
		if (device_loop) {
			auto more = gemma::generate_tokens(tok.data[0], n_decode, &t, &d, &rope, &rope_sw, &table, minp, temp, gen);
			out.insert(out.end(), more.begin(), more.end());
		} else {
			for (int step = 0; step < n_decode; step++) {
				gemma::forward_decode(&o, &tok, &t, &d, &rope, &rope_sw, ids.size() + step, &table);
				if (minp < 1)
					ops::minp_logits(&tok, &o, minp, temp, unif(gen));
				else
					ops::argmax_logits(&tok, &o);
				out.push_back(tok.data[0]);
			}
		}
		auto t2 = std::chrono::high_resolution_clock::now();
		for (int v : out) std::printf("%d ", v);
		std::printf("\n");
		const double sp = (t1 - t0).count() / 1e9, sd = (t2 - t1).count() / 1e9;
		std::fprintf(stderr, "prefill %.1f tok/s (%zu tokens, %.3f s incl. table build) | decode %.1f tok/s\n", ids.size() / sp,
		             ids.size(), sp, n_decode / sd);
	} catch (const std::exception &e) {
		std::fprintf(stderr, "error: %s\n", e.what());
		return 1;
	}
	return 0;
}
