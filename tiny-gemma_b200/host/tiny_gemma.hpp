// C++20 host layer: the reference's own API (fattorib/tiny-gemma,
// csrc/include/*.hpp) re-created on top of the C ABI of libtinygemma_b200.so,
// so that code written against the reference — gemma.cpp, a
// test_generation.cpp-style driver — compiles against this header instead.
// Same namespaces, names, argument order and error behaviour; the arithmetic
// runs on the GPU. Not a copy of the reference headers: containers and table
// builders are written from their described behaviour.
//
// Differences a caller can observe:
//   * gemma::Transformer holds no host copy of the weights (they go straight
//     from the file to HBM); its members are `cfg` and the GPU handle.
//   * decode::DecodeState creates its GPU state on the first forward call,
//     because the reference constructor has no model argument.
//   * asserts of the reference that would abort (second prefill on a used
//     cache, decode.hpp:78-79) throw std::runtime_error instead.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <new>
#include <random>
#include <stdexcept>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include <chrono>
#include <iostream>

#include "../../include/tiny_gemma_b200.h"
#include "tokenizer.hpp"

namespace constants {  // reference constants.hpp:4-10
static constexpr size_t simd{8};
static constexpr size_t alignment{32};
static constexpr size_t vocab{262144};
static constexpr int bos_id{2};
static constexpr int eos_id{1};
}  // namespace constants

namespace config {  // reference config.hpp:7-48
struct Config {
	int hidden_size, intermediate_size, n_layers, n_vocab, n_pos, n_pos_local, head_dim, n_head, n_kv;
	float rope_theta, rope_theta_local;
	int window_pattern;
	Config(int hidden_size, int intermediate_size, int n_layers, int n_vocab, int n_pos, int n_pos_local, int head_dim,
	       int n_head, int n_kv, float theta, float theta_local, int window_pattern)
	    : hidden_size(hidden_size), intermediate_size(intermediate_size), n_layers(n_layers), n_vocab(n_vocab),
	      n_pos(n_pos), n_pos_local(n_pos_local), head_dim(head_dim), n_head(n_head), n_kv(n_kv), rope_theta(theta),
	      rope_theta_local(theta_local), window_pattern(window_pattern) {}
};
inline const std::unordered_map<std::string, Config> CONFIG_MAP = {
    {"270m", Config(640, 2048, 18, 262144, 32768, 512, 256, 4, 1, 1000000, 10000, 6)},
    {"1B", Config(1152, 6912, 26, 262144, 32768, 512, 256, 4, 1, 1000000, 10000, 6)}};
}  // namespace config

namespace tensor {  // reference tensor.hpp:13-196 (32-byte aligned owning arrays)
template <typename T>
struct AlignedDeleter {
	void operator()(T *p) const { ::operator delete[](p, std::align_val_t(constants::alignment)); }
};
template <class T>
using AlignedArray = std::unique_ptr<T[], AlignedDeleter<T>>;
template <typename T>
AlignedArray<T> make_unique_aligned(size_t n) {
	return AlignedArray<T>(new (std::align_val_t(constants::alignment)) T[n]);
}
template <typename T>
AlignedArray<T> make_unique_aligned_constant(size_t n, T c) {
	auto p = make_unique_aligned<T>(n);
	for (size_t i = 0; i < n; i++) p[i] = c;
	return p;
}

struct activation {  // 3-D [x,y,z] or 4-D [x,y,z,w] fp32
	AlignedArray<float> data;
	size_t x = 0, y = 0, z = 0, w = 0, ndim = 0;
	activation() = default;
	activation(size_t x, size_t y, size_t z) : x(x), y(y), z(z), w(0), ndim(3) {
		data = make_unique_aligned_constant<float>(x * y * z, 0.0f);
	}
	activation(size_t x, size_t y, size_t z, size_t w) : x(x), y(y), z(z), w(w), ndim(4) {
		data = make_unique_aligned_constant<float>(x * y * z * w, 0.0f);
	}
	activation(AlignedArray<float> &a, size_t x, size_t y, size_t z) : data(std::move(a)), x(x), y(y), z(z), w(0), ndim(3) {}
	size_t numel() const { return ndim < 4 ? x * y * z : x * y * z * w; }
	size_t x_stride() const { return ndim < 4 ? y * z : y * z * w; }
	size_t y_stride() const { return ndim < 4 ? z : z * w; }
	size_t z_stride() const { return ndim < 4 ? 1 : w; }
	void zero() { std::memset(data.get(), 0, sizeof(float) * numel()); }
};

struct tokens {  // [batch, seq] int
	AlignedArray<int> data;
	size_t x = 0, y = 0;
	tokens() = default;
	tokens(size_t x, size_t y) : x(x), y(y) { data = make_unique_aligned_constant<int>(x * y, 0); }
	tokens(AlignedArray<int> &t, size_t x, size_t y) : data(std::move(t)), x(x), y(y) {}
	size_t numel() const { return x * y; }
};

template <typename T>
struct weight {  // [rows, cols] row-major, optional per-column fp32 scales
	AlignedArray<T> data;
	size_t rows = 0, cols = 0, ndim = 0;
	AlignedArray<float> scales = nullptr;
	bool quantized = false;
	weight() = default;
	weight(size_t rows, size_t cols, bool quantized) : rows(rows), cols(cols), ndim(2), quantized(quantized) {
		data = make_unique_aligned_constant<T>(rows * cols, T(0));
		if (quantized) scales = make_unique_aligned_constant<float>(cols, 0.0f);
	}
	weight(size_t rows, size_t cols) : weight(rows, cols, false) {}
	explicit weight(size_t rows) : rows(rows), cols(0), ndim(1) { data = make_unique_aligned_constant<T>(rows, T(0)); }
	size_t numel() const { return ndim == 1 ? rows : rows * cols; }
	size_t row_stride() const { return ndim == 1 ? 1 : cols; }
};
using FloatArray = weight<float>;
using QuantArray = weight<int8_t>;
}  // namespace tensor

namespace tg_detail {
inline void check(int rc) {
	if (rc != TG_OK) throw std::runtime_error(tg_last_error());
}
}  // namespace tg_detail

namespace ops_detail {  // the two samplers on host logits (ops::argmax_logits / ops::minp_logits below forward to these)
inline void argmax(tensor::tokens *toks, tensor::activation *o) {
	tg_detail::check(tg_argmax_logits(o->data.get(), int(constants::vocab), &toks->data[0]));
}
inline void minp(tensor::tokens *toks, tensor::activation *o, float minp, float temp, float randf) {
	tg_detail::check(tg_minp_logits(o->data.get(), int(constants::vocab), minp, temp, randf, &toks->data[0]));
}
}  // namespace ops_detail

namespace lut {  // reference ops.hpp:16-51
struct GeLUTable {
	float min, max;
	size_t table_size;
	tensor::AlignedArray<float> table;
	float eps;
	GeLUTable(float min, float max, size_t table_size) : min(min), max(max), table_size(table_size) {
		table = tensor::make_unique_aligned<float>(table_size);
		eps = float(max - min) / float(table_size);
		for (size_t i = 0; i < table_size; i++) {
			const float a = float(min) + float(i) * eps;
			// tanh-GeLU evaluated in double like the reference expression (its literals are doubles)
			const double inner = double(0.7978845608f) * (double(a) + double(0.044715f) * std::pow(double(a), 3.0));
			table[i] = float((0.5 * double(a)) * (1.0 + std::tanh(inner)));
		}
	}
};
}  // namespace lut

namespace decode {  // reference decode.hpp
struct RoPE {  // decode.hpp:107-134,176-201: cos/sin [n_pos, head_dim], both halves equal
	tensor::weight<float> freqs_cos, freqs_sin;
	int dhead = 0, max_pos = 0;
	float theta = 0;
	RoPE() = default;
	RoPE(config::Config *cfg, bool is_sw) {
		max_pos = cfg->n_pos;
		theta = is_sw ? cfg->rope_theta_local : cfg->rope_theta;
		dhead = cfg->head_dim;
		freqs_cos = tensor::weight<float>(max_pos, dhead);
		freqs_sin = tensor::weight<float>(max_pos, dhead);
		const int half = dhead / 2;
		std::vector<float> freqs(half);
		for (int i = 0; i < half; i++) freqs[i] = float(1.0 / std::pow(theta, float(2 * i) / dhead));
		for (int p = 0; p < max_pos; p++)
			for (int d = 0; d < half; d++) {
				const float outer = p * freqs[d];
				const float c = std::cos(outer), s = std::sin(outer);
				freqs_cos.data[size_t(p) * dhead + d] = freqs_cos.data[size_t(p) * dhead + d + half] = c;
				freqs_sin.data[size_t(p) * dhead + d] = freqs_sin.data[size_t(p) * dhead + d + half] = s;
			}
	}
};

struct DecodeState {  // decode.hpp:215-276: owns the KV caches of one batch of sequences
	int batch;
	config::Config cfg;
	tg_state *gpu = nullptr;
	DecodeState(int batch, config::Config *cfg) : batch(batch), cfg(*cfg) {}
	DecodeState(const DecodeState &) = delete;
	DecodeState &operator=(const DecodeState &) = delete;
	~DecodeState() { tg_state_free(gpu); }
	// KVCache::position_ptr of sequence 0
	int position() const {
		int p = 0;
		if (gpu) tg_state_position(gpu, 0, &p);
		return p;
	}
};
}  // namespace decode

namespace gemma {
using config::Config;
using config::CONFIG_MAP;  // gemma.cpp:38 reads gemma::CONFIG_MAP
using lut::GeLUTable;

struct Transformer {  // transformer.hpp:22-47
	Config cfg;
	tg_model *gpu = nullptr;
	const void *tables_from[3] = {nullptr, nullptr, nullptr};  // what was uploaded last
	explicit Transformer(Config cfg, int device = 0) : cfg(cfg) {
		tg_config k{cfg.hidden_size, cfg.intermediate_size, cfg.n_layers, cfg.n_vocab,     cfg.n_pos,
		            cfg.n_pos_local, cfg.head_dim,          cfg.n_head,   cfg.n_kv,        cfg.rope_theta,
		            cfg.rope_theta_local, cfg.window_pattern};
		tg_detail::check(tg_model_create(&k, device, &gpu));
	}
	Transformer(const Transformer &) = delete;
	Transformer &operator=(const Transformer &) = delete;
	~Transformer() { tg_model_free(gpu); }
};

// transformer.hpp:99-165; a missing file throws std::runtime_error("Could not open file.")
inline void read_weights(Transformer *t, const char *file) { tg_detail::check(tg_model_load_file(t->gpu, file)); }

namespace detail {
inline void ensure(Transformer *t, decode::DecodeState *d, decode::RoPE *r, decode::RoPE *r_sw, GeLUTable *table) {
	if (t->tables_from[0] != r || t->tables_from[1] != r_sw || t->tables_from[2] != table) {
		tg_detail::check(tg_model_set_rope(t->gpu, 0, r->freqs_cos.data.get(), r->freqs_sin.data.get(), r->max_pos));
		tg_detail::check(tg_model_set_rope(t->gpu, 1, r_sw->freqs_cos.data.get(), r_sw->freqs_sin.data.get(), r_sw->max_pos));
		tg_detail::check(tg_model_set_gelu_table(t->gpu, table->min, table->max, table->table.get(), int(table->table_size)));
		t->tables_from[0] = r;
		t->tables_from[1] = r_sw;
		t->tables_from[2] = table;
	}
	if (!d->gpu) tg_detail::check(tg_state_create(t->gpu, d->batch, d->cfg.n_pos, &d->gpu));
}
}  // namespace detail

// transformer.hpp:49-73: logits of the last prompt position into o ([batch,1,V])
inline void forward_prefill(tensor::activation *o, tensor::tokens *toks, Transformer *t, decode::DecodeState *d,
                            decode::RoPE *r, decode::RoPE *r_sw, GeLUTable *table) {
	detail::ensure(t, d, r, r_sw, table);
	tg_detail::check(tg_prefill(d->gpu, toks->data.get(), int(toks->y), o ? o->data.get() : nullptr));
}

// transformer.hpp:75-97: pos_offset is unused there too (the position lives in the cache)
inline void forward_decode(tensor::activation *o, tensor::tokens *toks, Transformer *t, decode::DecodeState *d,
                           decode::RoPE *r, decode::RoPE *r_sw, size_t /*pos_offset*/, GeLUTable *table) {
	detail::ensure(t, d, r, r_sw, table);
	tg_detail::check(tg_decode(d->gpu, toks->data.get(), o ? o->data.get() : nullptr));
}

// The decode loop of generate() (transformer.hpp:226-250) on token ids, run on the device:
// forward_decode + sampler n_decode times, the token never leaving the GPU. minp >= 1 selects
// argmax (transformer.hpp:229). `gen` supplies the uniforms exactly as generate() draws them.
inline std::vector<int> generate_tokens(int first_token, int n_decode, Transformer *t, decode::DecodeState *d,
                                        decode::RoPE *r, decode::RoPE *r_sw, GeLUTable *table, float minp, float temp,
                                        std::mt19937 &gen) {
	detail::ensure(t, d, r, r_sw, table);
	std::uniform_real_distribution<float> unif(0.0, 1.0);
	std::vector<float> randf;
	if (minp < 1) {
		randf.resize(size_t(n_decode) * d->batch);
		for (auto &v : randf) v = unif(gen);
	}
	std::vector<int> first(d->batch, first_token), out(size_t(n_decode) * d->batch);
	tg_detail::check(tg_generate(d->gpu, first.data(), n_decode, minp, temp, minp < 1 ? randf.data() : nullptr, out.data()));
	return out;
}

// transformer.hpp:167-258: tokenize, prefill, sample, n_decode x (forward_decode + sampler), streaming the
// decoded pieces to stdout; returns {decode steps completed, generated text, prefill seconds, decode seconds}.
// The decode steps run on the device in chunks (the token never leaves the GPU inside a chunk); pieces are
// printed chunk by chunk, and with terminate_on_end the first <end_of_turn> ends the text (steps the chunk ran
// past it are dropped). The uniforms are drawn from std::mt19937 in the reference's order: one for the
// token after the prompt, then one per step. seed == nullptr seeds from std::random_device as the reference does.
inline std::tuple<int, std::string, float, float> generate(std::string prompt, int n_decode, sentencepiece::Tokenizer *tokenizer,
                                                           Transformer *t, const float minp, const float temp,
                                                           const bool terminate_on_end, const unsigned *seed = nullptr,
                                                           int chunk = 16) {
	auto t_prefill_s = std::chrono::high_resolution_clock::now();
	std::random_device rd;
	std::mt19937 gen(seed ? *seed : rd());
	std::uniform_real_distribution<float> unif(0.0, 1.0);
	std::vector<int> ids = tokenizer->encode(prompt);
	const size_t prompt_len = ids.size();
	std::string decoded;
	decoded.reserve(size_t(n_decode > 0 ? n_decode : 0));
	printf("Prompt length: %lu\n", (unsigned long)prompt_len);
	std::cout << tokenizer->decode(ids);

	auto tokens_data = tensor::make_unique_aligned<int>(prompt_len);
	for (size_t i = 0; i < prompt_len; i++) tokens_data[i] = ids[i];
	decode::RoPE rope(&(t->cfg), false);
	decode::RoPE rope_sw(&(t->cfg), true);
	lut::GeLUTable table{-4.0, 4.0, 1024};
	decode::DecodeState d(1, &(t->cfg));
	tensor::tokens tokens(tokens_data, 1, prompt_len);
	tensor::activation o(1, 1, t->cfg.n_vocab);
	forward_prefill(&o, &tokens, t, &d, &rope, &rope_sw, &table);
	tensor::tokens tokens_decode(1, 1);
	if (minp < 1)
		ops_detail::minp(&tokens_decode, &o, minp, temp, unif(gen));
	else
		ops_detail::argmax(&tokens_decode, &o);
	int prev_token = ids[ids.size() - 1];
	std::cout << tokenizer->decode(tokens_decode.data[0], prev_token) << std::flush;
	prev_token = tokens_decode.data[0];
	auto t_prefill_e = std::chrono::high_resolution_clock::now();

	auto t_decode_s = std::chrono::high_resolution_clock::now();
	int done = 0;
	bool ended = false;
	while (done < n_decode && !ended) {
		const int n = std::min(chunk, n_decode - done);
		const std::vector<int> out = generate_tokens(prev_token, n, t, &d, &rope, &rope_sw, &table, minp, temp, gen);
		for (int i = 0; i < n; i++) {
			if (terminate_on_end && out[i] == tokenizer->get_eot_id()) {
				ended = true;
				break;
			}
			const std::string piece = tokenizer->decode(out[i], prev_token);
			decoded.append(piece);
			std::cout << piece << std::flush;
			prev_token = out[i];
			done++;
		}
	}
	auto t_decode_e = std::chrono::high_resolution_clock::now();
	const double s_prefill = (t_prefill_e - t_prefill_s).count() / 1e9;
	const double s_decode = (t_decode_e - t_decode_s).count() / 1e9;
	return {done, decoded, float(s_prefill), float(s_decode)};
}
}  // namespace gemma

namespace ops {  // reference ops.hpp: host-buffer operators
using tensor::activation;
using tensor::tokens;
using tensor::weight;

inline void argmax_logits(tokens *toks, activation *o) { ops_detail::argmax(toks, o); }  // ops.hpp:744-760
inline void minp_logits(tokens *toks, activation *o, float minp, float temp, float randf) {  // ops.hpp:762-859
	ops_detail::minp(toks, o, minp, temp, randf);
}
inline void linear_decode(activation *o, activation *a, weight<int8_t> *w) {  // ops.hpp:634-649
	tg_detail::check(tg_qmatvec(o->data.get(), a->data.get(), w->data.get(), w->scales.get(), int(w->rows), int(w->cols)));
}
inline void lm_head_decode(activation *o, activation *a, weight<int8_t> *w) {  // ops.hpp:654-667
	tg_detail::check(tg_qmatvec(o->data.get(), a->data.get(), w->data.get(), w->scales.get(), int(w->rows), int(w->cols)));
}
inline void linear_prefill(activation *o, activation *a, weight<int8_t> *w) {  // ops.hpp:618-632
	tg_detail::check(tg_qgemm(o->data.get(), a->data.get(), w->data.get(), w->scales.get(), int(a->y), int(w->rows), int(w->cols)));
}
inline void rmsnorm(activation *a, weight<float> *w, float /*eps*/ = 1e-06f) {  // ops.hpp:182-222
	const size_t dim = a->ndim == 3 ? a->z : a->w;
	tg_detail::check(tg_rmsnorm(a->data.get(), w->data.get(), int(a->numel() / dim), int(dim)));
}
}  // namespace ops
